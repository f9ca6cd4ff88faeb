"""Compiles the reference project's own W8A8 kernel source (fp8_gemm_kernel.cu, from where it lies
in the reference checkout) with NVRTC for sm_100a, the way the reference's loaders do
(fp8_cuda.py:52-66 and tests/fp8_gemm_host.cpp there: NVRTC, --std=c++17, -default-device), and
writes the cubin to oracle/_ref/ (git-ignored). No source is copied or changed.

TEST INFRASTRUCTURE: tests/test_gpu_w8a8.py loads the cubin on the GPU machine and runs the
reference's kernels beside the new ones, which pins the W8A8 parity to the reference itself.

    python oracle/build_ref_cubin.py <reference checkout> [<cuda include dir>]
"""
import os
import sys


def main():
    ref = sys.argv[1]
    cuda_inc = sys.argv[2] if len(sys.argv) > 2 else "/usr/local/cuda/include"
    src_path = os.path.join(ref, "fp8_gemm_kernel.cu")
    here = os.path.dirname(os.path.abspath(__file__))
    out_path = os.path.join(here, "_ref", "fp8_gemm_kernel.sm_100a.cubin")
    try:
        from cuda.bindings import nvrtc
    except ImportError:
        from cuda import nvrtc

    def ck(res):
        err, *rest = res
        if int(err) != 0:
            raise RuntimeError(f"NVRTC error {err}")
        return rest[0] if len(rest) == 1 else rest

    src = open(src_path, "rb").read()
    prog = ck(nvrtc.nvrtcCreateProgram(src, b"fp8_gemm_kernel.cu", 0, [], []))
    opts = [b"--gpu-architecture=sm_100a", b"--std=c++17", b"-default-device", b"-I" + cuda_inc.encode()]
    err = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)[0]
    if int(err) != 0:
        n = ck(nvrtc.nvrtcGetProgramLogSize(prog))
        log = b" " * n
        nvrtc.nvrtcGetProgramLog(prog, log)
        raise RuntimeError("NVRTC compile failed:\n" + log.decode(errors="replace"))
    n = ck(nvrtc.nvrtcGetCUBINSize(prog))
    cubin = b" " * n
    ck(nvrtc.nvrtcGetCUBIN(prog, cubin) + (None,))
    os.makedirs(os.path.dirname(out_path), exist_ok=True)
    with open(out_path, "wb") as f:
        f.write(cubin)
    print(f"wrote {out_path} ({n} bytes)")


if __name__ == "__main__":
    main()
