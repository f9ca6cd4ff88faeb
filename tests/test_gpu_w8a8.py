"""W8A8 on the GPU: the block quantizer and the FP8 x FP8 GEMM (tcgen05.mma.kind::mxf8f6f4 with
UE8M0 block scales in tensor memory; kind::f8f6f4 for the other scale forms) through the C ABI.

Checked against (i) the numpy oracle -- bit for bit for the quantizer, and for the GEMM with the
reference's own acceptance bound, rel. error < 1e-5 against the float64 product of the dequantized
operands (tests/fp8_gemm_host.cpp:182-183 there), on its six format / scale cases and on shapes
that exercise ragged tiles, many k-tiles and several tiles per CTA; and (ii) the reference's own
kernels: fp8_gemm_kernel.cu compiled unmodified with NVRTC into oracle/_ref/ (oracle/Makefile) and
launched here on the same operands."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import tfp8_oracle as O
from tests.test_w8a8_oracle import CASES, _case_data

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TDT = {"e4m3fn": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


def _rel(y, ref):
    return float(np.abs(y.double().cpu().numpy() - ref).max() / np.abs(ref).max())


@pytest.mark.parametrize("fmt", ("e4m3fn", "e5m2"))
@pytest.mark.parametrize("ue8m0", (False, True))
def test_quantize_k_matches_oracle(fmt, ue8m0):
    from tfp8 import _ext
    x32, _, _ = _case_data(300, 8, 640, 5)
    x32[7, 64:96] = 0.0
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        x = torch.from_numpy(x32).to(dt).cuda()
        q, s = _ext.quantize_k(x, fmt, ue8m0)
        oq, os_ = O.quantize_k(x.float().cpu().numpy(), fmt, ue8m0)
        assert np.array_equal(s.cpu().numpy(), os_), f"{dt} scales"
        assert np.array_equal(q.cpu().numpy(), oq), f"{dt} codes"
        if ue8m0:
            q2, sp = _ext.quantize_k(x, fmt, True, packed=True)
            assert torch.equal(q2, q)
            assert np.array_equal(sp.cpu().numpy(), O.mx_pack_scales(os_))
            assert torch.equal(_ext.mx_pack_scales(s), sp)
    assert _ext.device_status() == 0


def _quantize_case(a, w, a_fmt, w_fmt, ue8m0, rowcol):
    if not rowcol:
        aq, sa = O.quantize_k(a, a_fmt, ue8m0)
        wq, sw = O.quantize_k(w, w_fmt, ue8m0)
        return aq, sa, wq, sw

    def q_rows(x, fmt):
        fmax = O.FORMATS[fmt][4]
        s = (np.abs(x).max(1) / fmax).astype(np.float32)
        if ue8m0:
            e = np.clip(np.ceil(np.log2(s.astype(np.float64))), -127, 127)
            return O.encode((x / np.exp2(e)[:, None]).astype(np.float32), fmt), (e + 127).astype(np.uint8)
        return O.encode(x / s[:, None], fmt), s
    return q_rows(a, a_fmt) + q_rows(w, w_fmt)


def _run_ours(aq, sa, a_fmt, wq, sw, w_fmt, bias, ue8m0, rowcol, out_dtype=torch.float32):
    from tfp8 import _ext
    t = lambda v: torch.from_numpy(np.ascontiguousarray(v)).cuda()
    if rowcol:
        return _ext.gemm_w8a8(t(aq), t(sa), a_fmt, t(wq), t(sw), w_fmt, None if bias is None else t(bias), out_dtype, _ext.W8A8_ROWCOL)
    if ue8m0:
        sa_t, sw_t = _ext.mx_pack_scales(t(sa)), _ext.mx_pack_scales(t(sw))
    else:
        sa_t, sw_t = t(sa), t(sw)
    return _ext.gemm_w8a8(t(aq), sa_t, a_fmt, t(wq), sw_t, w_fmt, None if bias is None else t(bias), out_dtype, _ext.W8A8_BLOCK32)


class _RefKernels:
    """The reference's gemm_{block,rowcol}_{fp32,ue8m0} kernels from the NVRTC-built cubin."""

    def __init__(self):
        path = os.path.join(ROOT, "oracle", "_ref", "fp8_gemm_kernel.sm_100a.cubin")
        if not os.path.exists(path):
            pytest.skip("oracle/_ref/fp8_gemm_kernel.sm_100a.cubin was not built (needs the reference checkout at build time)")
        torch.zeros(1, device="cuda")                              # the primary context, current on this thread
        self.cu = ctypes.CDLL("libcuda.so.1")
        self.mod = ctypes.c_void_p()
        data = open(path, "rb").read()
        assert self.cu.cuModuleLoadData(ctypes.byref(self.mod), data) == 0

    def run(self, aq, sa, a_fmt, wq, sw, w_fmt, bias, ue8m0, rowcol):
        M, K = aq.shape
        N = wq.shape[0]
        assert M % 32 == 0 and N % 32 == 0 and K % 32 == 0
        t = lambda v: torch.from_numpy(np.ascontiguousarray(v)).cuda()
        A, B = t(aq), t(np.ascontiguousarray(wq.T))                  # the reference keeps the weight as [K, N]
        sa_t = t(sa)
        sb_t = t(sw) if rowcol else t(np.ascontiguousarray(sw.T))   # and its block scales as [K/32, N]
        lut = lambda f: torch.arange(256, dtype=torch.uint8, device="cuda").view(TDT[f]).to(torch.float16)
        la, lb = lut(a_fmt), lut(w_fmt)
        b = t(bias.astype(np.float32))
        C = torch.empty(M, N, dtype=torch.float32, device="cuda")
        name = ("gemm_rowcol_" if rowcol else "gemm_block_") + ("ue8m0" if ue8m0 else "fp32")
        fn = ctypes.c_void_p()
        assert self.cu.cuModuleGetFunction(ctypes.byref(fn), self.mod, name.encode()) == 0
        ptrs = [ctypes.c_void_p(x.data_ptr()) for x in (A, B, la, lb, sa_t, sb_t, b, C)]
        ints = [ctypes.c_int(v) for v in (M, N, K)]
        args = (ctypes.c_void_p * 11)(*[ctypes.cast(ctypes.byref(a), ctypes.c_void_p) for a in ptrs + ints])
        torch.cuda.synchronize()
        self.cu.cuLaunchKernel.argtypes = [ctypes.c_void_p] + [ctypes.c_uint] * 7 + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        rc = self.cu.cuLaunchKernel(fn, N // 32, M // 32, 1, 128, 1, 1, 0, None, args, None)
        assert rc == 0, f"cuLaunchKernel failed: {rc}"
        torch.cuda.synchronize()
        return C


@pytest.mark.parametrize("a_fmt,w_fmt,ue8m0,rowcol", CASES)
def test_reference_host_cases(a_fmt, w_fmt, ue8m0, rowcol):
    """M=128, N=96, K=512 in the six combinations of the reference's host test: against the float64
    oracle with its bound, and against the reference's own kernel on the same operands."""
    from tfp8 import _ext
    a, w, bias = _case_data(128, 96, 512, 1234)
    aq, sa, wq, sw = _quantize_case(a, w, a_fmt, w_fmt, ue8m0, rowcol)
    ref = O.w8a8_forward_f64(aq, sa, a_fmt, wq, sw, w_fmt, bias, ue8m0, rowcol)
    y = _run_ours(aq, sa, a_fmt, wq, sw, w_fmt, bias, ue8m0, rowcol)
    assert _rel(y, ref) < 1e-5, f"vs float64 oracle: {_rel(y, ref):.2e}"
    y_ref_kernel = _RefKernels().run(aq, sa, a_fmt, wq, sw, w_fmt, bias, ue8m0, rowcol)
    assert _rel(y_ref_kernel, ref) < 1e-5                                  # the reference passes its own gate here
    d = float((y - y_ref_kernel).abs().max() / np.abs(ref).max())
    assert d < 1e-5, f"vs the reference's kernel: {d:.2e}"
    assert _ext.device_status() == 0


@pytest.mark.parametrize("M,N,K", ((1, 96, 128), (5, 200, 1024), (127, 128, 256), (129, 130, 384), (300, 384, 8192), (640, 2176, 512)))
def test_block_scaled_shapes(M, N, K):
    """Ragged row / column tiles, one to 64 k-tiles, more tiles than SMs (640 x 2176: 85 tiles ... and
    the persistent loop with 2 accumulator buffers), UE8M0 block scales on the tensor cores."""
    from tfp8 import _ext
    a, w, bias = _case_data(M, N, K, M + N + K)
    aq, sa, wq, sw = _quantize_case(a, w, "e4m3fn", "e4m3fn", True, False)
    ref = O.w8a8_forward_f64(aq, sa, "e4m3fn", wq, sw, "e4m3fn", bias, True)
    y = _run_ours(aq, sa, "e4m3fn", wq, sw, "e4m3fn", bias, True, False)
    assert _rel(y, ref) < 1e-5, f"{_rel(y, ref):.2e}"
    ref_nb = ref - bias[None, :]
    for od, tol in ((torch.float16, 2.0 ** -10), (torch.bfloat16, 2.0 ** -7)):
        y16 = _run_ours(aq, sa, "e4m3fn", wq, sw, "e4m3fn", None, True, False, od)
        with np.errstate(over="ignore"):
            fits = np.abs(ref_nb) < 6e4
        err = np.abs(y16.double().cpu().numpy() - ref_nb)
        assert (err[fits] <= tol * np.abs(ref_nb[fits]) + 1e-5 * np.abs(ref_nb).max()).all(), od
    assert _ext.device_status() == 0


@pytest.mark.parametrize("ue8m0", (False, True))
def test_other_scale_forms_many_tiles(ue8m0):
    """Row/column scales (epilogue) and float32 block scales (register accumulation) beyond one tile."""
    from tfp8 import _ext
    a, w, bias = _case_data(260, 300, 1024, 77)
    for rowcol in (True, False):
        if not rowcol and ue8m0:
            continue
        aq, sa, wq, sw = _quantize_case(a, w, "e4m3fn", "e5m2", ue8m0, rowcol)
        ref = O.w8a8_forward_f64(aq, sa, "e4m3fn", wq, sw, "e5m2", bias, ue8m0, rowcol)
        y = _run_ours(aq, sa, "e4m3fn", wq, sw, "e5m2", bias, ue8m0, rowcol)
        assert _rel(y, ref) < 1e-5, f"rowcol={rowcol} ue8m0={ue8m0}: {_rel(y, ref):.2e}"
    assert _ext.device_status() == 0


def test_fp8_cuda_module_mirrors_the_reference_binding():
    """quantize_k / Fp8Weight / fp8_linear / dequant_ref with the reference's names and layouts
    (fp8_cuda.py there): the result against dequant_ref's float64 product, its own definition."""
    import fp8_cuda
    torch.manual_seed(9)
    x = torch.randn(64, 512, device="cuda")
    w = torch.randn(512, 160, device="cuda") * 0.1                      # (K, N) as the reference takes it
    bias = torch.randn(160, device="cuda")
    for fmt in ("e4m3", "e5m2"):
        for ue8m0 in (False, True):
            W = fp8_cuda.Fp8Weight(w, fmt, ue8m0)
            assert W.q.shape == (512, 160) and W.s.shape == (16, 160)
            y = fp8_cuda.fp8_linear(x, W, bias)
            aq, sa = fp8_cuda.quantize_k(x, fmt, ue8m0)
            ref = (fp8_cuda.dequant_ref(aq, sa, fmt, ue8m0, True) @ fp8_cuda.dequant_ref(W.q, W.s, fmt, ue8m0, False)
                   + bias.double())
            rel = float((y.double() - ref).abs().max() / ref.abs().max())
            assert y.dtype == torch.float32 and rel < 1e-5, (fmt, ue8m0, rel)
    with pytest.raises(ValueError):
        fp8_cuda.quantize_k(x.cpu(), "e4m3")


def test_fp8linear_activation_fp8_switch():
    """FP8Config(activation="fp8") / FP8Linear(activation="fp8"): prepare_model builds MX layers
    (32-wide UE8M0 groups) whose forward quantizes the activations per block and multiplies codes by
    codes. Checked against the oracle evaluated on the layer's own codes and scales, and against
    the layer's CPU path (the same arithmetic in torch)."""
    import torch.nn as nn
    from tfp8 import FP8Config, FP8Linear, _ext, prepare_model
    torch.manual_seed(4)
    class Mlp(nn.Module):                                    # names the planner's LLM rule converts
        def __init__(self):
            super().__init__()
            self.up_proj, self.down_proj = nn.Linear(1024, 1536), nn.Linear(1536, 1024, bias=False)

    model = Mlp().half().cuda()
    prepare_model(model, "llm", FP8Config(profile="llm_safe", weight_group=32, scale_format="ue8m0", activation="fp8", nan_check=False))
    layer = model.up_proj
    assert isinstance(layer, FP8Linear) and layer.activation == "fp8" and isinstance(model.down_proj, FP8Linear)
    for M in (1, 8, 40, 300):
        x = torch.randn(M, 1024, device="cuda", dtype=torch.float16)
        y = layer(x)
        aq, sa = O.quantize_k(x.float().cpu().numpy(), "e4m3fn", True)
        e8 = O.ue8m0_encode(layer.weight_scale.cpu().numpy())
        ref = O.w8a8_forward_f64(aq, sa, "e4m3fn", layer.qweight.cpu().numpy(), e8, "e4m3fn", layer.bias_f32.cpu().numpy(), True)
        err = np.abs(y.double().cpu().numpy() - ref)
        assert (err <= 2.0 ** -10 * np.abs(ref) + 1e-5 * np.abs(ref).max()).all(), M          # one fp16 rounding of the output
        cpu = copy_to_cpu(layer)(x.cpu())
        assert (y.cpu().float() - cpu.float()).abs().max() <= 2.0 ** -9 * float(cpu.float().abs().max())
    assert layer.stats["w8a8"] == 4 and layer.stats["gemv"] == 0 and layer.stats["gemm"] == 0
    assert _ext.device_status() == 0


def copy_to_cpu(layer):
    import copy
    return copy.deepcopy(layer).to("cpu")
