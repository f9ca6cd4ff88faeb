"""Operator layer: ctypes bindings of the sm_100a C-ABI library (libtfp8b.so) behind the same
Python functions the reference's launcher exposes (tfp8/_ext.py there: `available`, `last_error`,
`GemvLaunch`, `prepare_activations`, `w8a16`, `gemm_prepared`, `dequant_into`, `epilogue_into`,
`GEMV_MAXM`, `FMT_ID`, `_TAG`), plus `encode`, `decode_codes` and `quantize_weight_cuda`.

The reference compiles its kernels with NVRTC at first use and launches them with
cuLaunchKernel; here the kernels are built ahead of time by nvcc for sm_100a and every call is one
C function call on torch's current stream. There is no torch fallback in this module: if the
library is missing, every operator raises.
"""
import ctypes
import os
import threading

import torch

GEMV_MAXM = 8                      # rows served by the decode GEMV; larger M goes to the tile GEMM
GEMV_MT = (8,)                     # one kernel serves every M <= 8 (the reference had a 1/4/8 ladder)
FMT_ID = {"e4m3fn": 0, "e5m2": 1}
_TAG = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}
_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
SCALE_F32, SCALE_UE8M0 = 0, 1

_LIB_PATH = os.environ.get("TFP8B_LIBRARY") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libtfp8b.so")
_lock = threading.Lock()
_lib = None
_error = None

_P, _I, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
_SIGNATURES = {
    "tfp8b_version": ([], _I),
    "tfp8b_last_error_string": ([], ctypes.c_char_p),
    "tfp8b_device_status": ([_P, _P], _I),
    "tfp8b_encode": ([_P, _I, _P, _L, _I, _I, _P], _I),
    "tfp8b_decode": ([_P, _P, _I, _L, _I, _P], _I),
    "tfp8b_quantize": ([_P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P], _I),
    "tfp8b_dequant": ([_P, _P, _I, _P, _I, _I, _I, _I, _I, _P], _I),
    "tfp8b_prep": ([_P, _I, _P, _P, _I, _I, _P], _I),
    "tfp8b_gemv": ([_P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P], _I),
    "tfp8b_gemv_ex": ([_P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, ctypes.c_uint, _P], _I),
    "tfp8b_gemv_plan_create": ([ctypes.POINTER(_P), _I, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I], _I),
    "tfp8b_gemv_plan_run": ([_P, _P, _P, _I, ctypes.c_uint, _P], _I),
    "tfp8b_gemv_plan_destroy": ([_P], None),
    "tfp8b_allreduce_wait_limit": ([ctypes.c_longlong], ctypes.c_longlong),
    "tfp8b_gemm": ([_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P], _I),
    "tfp8b_gemv_normed": ([_P, _P, _P, _P, ctypes.c_float, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P], _I),
    "tfp8b_gemv_gated": ([_P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P], _I),
    "tfp8b_gemm_w8a8": ([_P, _P, _I, _P, _P, _I, _I, _I, _P, _P, _I, _I, _I, _I, _P], _I),
    "tfp8b_mx_packed_scale_bytes": ([_I, _I], ctypes.c_longlong),
    "tfp8b_mx_pack_scales": ([_P, _P, _I, _I, _P], _I),
    "tfp8b_quantize_k": ([_P, _I, _P, _P, _I, _I, _I, _I, _I, _P], _I),
    "tfp8b_gemm_splitk": ([_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P, ctypes.c_longlong, _P], _I),
    "tfp8b_gemm_scatter": ([_P, _P, _P, _P, _I, _P, _P, _I, ctypes.c_longlong, ctypes.c_longlong, _I, _I, _I, _I, _I, _I, _P], _I),
    "tfp8b_linear_static": ([_P, _I, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P], _I),
    "tfp8b_epilogue": ([_P, _P, _P, _P, _I, _I, _I, _I, _P], _I),
    "tfp8b_rope_kv_store": ([_P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P], _I),
    "tfp8b_silu_mul": ([_P, _P, _I, ctypes.c_longlong, _I, _P], _I),
    "tfp8b_add_rmsnorm": ([_P, _P, _P, _P, _I, ctypes.c_longlong, _I, ctypes.c_float, _P], _I),
    "tfp8b_allreduce_add_rmsnorm": ([_P, _P, _P, _P, _I, _I, _I, ctypes.c_float, _P, _P, _P, _I, _I, _I, _P], _I),
    "tfp8b_attn_decode": ([_P, _P, _P, _P, _P, _P, ctypes.c_longlong, _I, _I, _I, _I, _I, _I, _P], _I),
    "tfp8b_argmax": ([_P, _I, _P, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, _P], _I),
    "tfp8b_rope_kv_store_fp8": ([_P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P], _I),
    "tfp8b_attn_decode_fp8": ([_P, _P, _P, _P, _P, _P, _P, _P, ctypes.c_longlong, _I, _I, _I, _I, _I, _I, _I, _P], _I),
}


def library_path() -> str:
    return _LIB_PATH


def load():
    """The loaded library (ctypes.CDLL). Raises RuntimeError when it is missing or broken."""
    global _lib, _error
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            try:
                lib = ctypes.CDLL(_LIB_PATH)
                for name, (args, res) in _SIGNATURES.items():
                    fn = getattr(lib, name)
                    fn.argtypes, fn.restype = args, res
                _lib = lib
            except (OSError, AttributeError) as e:
                _error = e
                raise RuntimeError(
                    f"tfp8: the CUDA kernel library could not be loaded from {_LIB_PATH} ({e}). "
                    f"Build it with `make -C {os.path.join(os.path.dirname(os.path.dirname(_LIB_PATH)), 'csrc')}`.") from e
    return _lib


def available() -> bool:
    """True when a CUDA device is present and the kernel library loads. Never prints and never
    downgrades anything: callers that hold CUDA tensors and get False must raise."""
    global _error
    if not torch.cuda.is_available():
        return False
    try:
        load()
        return True
    except RuntimeError as e:
        _error = _error or e
        return False


def last_error():
    return _error


def _stream(dev: int) -> int:
    return torch._C._cuda_getCurrentRawStream(dev)


def _check(rc: int, what: str):
    if rc != 0:
        msg = load().tfp8b_last_error_string().decode("utf-8", "replace")
        if rc == -2:
            raise NotImplementedError(f"{what}: {msg}")
        raise RuntimeError(f"{what} failed ({rc}): {msg}")


def _need_cuda(*tensors):
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("tfp8 kernels take CUDA tensors; CPU tensors belong to FP8Linear's torch path")
        d = t.get_device()
        if dev is None:
            dev = d
        elif d != dev:
            raise ValueError(f"tensors on different devices (cuda:{dev} and cuda:{d})")
    return dev


def _scale_kind(ws: torch.Tensor) -> int:
    if ws.dtype == torch.float32:
        return SCALE_F32
    if ws.dtype == torch.uint8:
        return SCALE_UE8M0
    raise ValueError(f"weight scale must be float32 or uint8 (UE8M0), got {ws.dtype}")


def device_status(device=None) -> int:
    """Status word of the kernels' bounded waits on the current device (0 = all fine).
    Synchronises. Raises RuntimeError if a kernel gave up on a wait."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    word = ctypes.c_uint(0)
    with torch.cuda.device(dev):
        rc = load().tfp8b_device_status(ctypes.byref(word), _stream(dev))
    _check(rc, "tfp8b_device_status")
    return word.value


# ------------------------------------------------------------------ codecs
def encode(x: torch.Tensor, fmt="e4m3fn", canonical_nan=False) -> torch.Tensor:
    """uint8 codes of x (f16 / bf16 / f32), RNE + saturate. NaN -> sign|0x7F, or the format's
    canonical NaN with canonical_nan=True."""
    dev = _need_cuda(x)
    x = x.contiguous()
    if x.dtype not in _DT:
        x = x.float()
    out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_encode(x.data_ptr(), _DT[x.dtype], out.data_ptr(), x.numel(), FMT_ID[fmt],
                                 int(canonical_nan), _stream(dev))
    _check(rc, "tfp8b_encode")
    return out


def decode_codes(codes: torch.Tensor, fmt="e4m3fn", dtype=torch.float16) -> torch.Tensor:
    """Values of uint8 codes in `dtype` (exact)."""
    dev = _need_cuda(codes)
    codes = codes.contiguous()
    out = torch.empty(codes.shape, dtype=dtype, device=codes.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_decode(codes.data_ptr(), out.data_ptr(), _DT[dtype], codes.numel(), FMT_ID[fmt], _stream(dev))
    _check(rc, "tfp8b_decode")
    return out


def quantize_weight_cuda(w: torch.Tensor, fmt="e4m3fn", group_size=None, pow2_scale=True, ue8m0=False):
    """One-pass quantizer: w [N,K] -> (codes u8 [N,K], scale [N,K/G] f32 or UE8M0 u8, G)."""
    dev = _need_cuda(w)
    N, K = w.shape
    G = K if group_size is None else group_size
    if K % G:
        raise ValueError(f"K={K} not divisible by group_size={G}")
    w = w.contiguous()
    if w.dtype not in _DT:
        w = w.float()
    q = torch.empty(N, K, dtype=torch.uint8, device=w.device)
    s = torch.empty(N, K // G, dtype=torch.uint8 if ue8m0 else torch.float32, device=w.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_quantize(w.data_ptr(), _DT[w.dtype], q.data_ptr(), s.data_ptr(), int(ue8m0), N, K, G,
                                   FMT_ID[fmt], int(pow2_scale), _stream(dev))
    _check(rc, "tfp8b_quantize")
    return q, s, G


def dequant_into(out16, qweight, lut16, wscale, group_size, fmt="e4m3fn"):
    """out16[n,k] = decode(qweight[n,k]) * wscale[n, k/G], into a caller-provided [n,K] buffer
    (f16, bf16 or f32). `lut16` is accepted for signature compatibility and unused: the kernels
    decode by bit arithmetic."""
    dev = _need_cuda(out16, qweight, wscale)
    N, K = qweight.shape
    if not (out16.is_contiguous() and qweight.is_contiguous() and wscale.is_contiguous()):
        raise ValueError("dequant_into needs contiguous tensors")
    with torch.cuda.device(dev):
        rc = load().tfp8b_dequant(qweight.data_ptr(), wscale.data_ptr(), _scale_kind(wscale), out16.data_ptr(),
                                  _DT[out16.dtype], N, K, group_size, FMT_ID[fmt], _stream(dev))
    _check(rc, "tfp8b_dequant")
    return out16


# ------------------------------------------------------------------ activations
def prepare_activations(x):
    """(x16 fp16 [M,K], xs f32 [M]) in one launch: exact power-of-two row scale that maps the row
    amax into [2^7, 2^8). Unlike the torch twin, fp16 input is rescaled too (as in the reference's
    kernel)."""
    dev = _need_cuda(x)
    M, K = x.shape
    x = x.contiguous()
    x16 = torch.empty(M, K, dtype=torch.float16, device=x.device)
    xs = torch.empty(M, dtype=torch.float32, device=x.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_prep(x.data_ptr(), _DT[x.dtype], x16.data_ptr(), xs.data_ptr(), M, K, _stream(dev))
    _check(rc, "tfp8b_prep")
    return x16, xs


# ------------------------------------------------------------------ GEMV / GEMM
class GemvLaunch:
    """A decode-GEMV call for one layer with everything but (x, y, M) bound once.

    Construction makes a plan in the library (`tfp8b_gemv_plan_create`): shape checks, the
    shared-memory layout, the kernel variant and the tensor map of the weight stream are worked
    out there, once. Per call: one `torch.empty`, a few ctypes values, one C call that launches the
    kernel. The bound tensors are referenced here so their storage outlives the launch; FP8Linear
    rebuilds the object when a buffer object is replaced. Same constructor and call signature as
    the reference's class of this name.
    """
    __slots__ = ("fn", "dev", "device", "plan", "args", "q", "ws", "bias", "lut", "out_dtype", "N", "_stream", "_destroy",
                 "__weakref__")

    def __init__(self, x_dtype, qweight, lut16, wscale, bias, out_dtype, group_size, fmt):
        lib = load()
        self.dev = _need_cuda(qweight, wscale, bias)
        self.device = qweight.device
        N, K = qweight.shape
        self.N = N
        self.fn = lib.tfp8b_gemv_plan_run
        self._destroy = lib.tfp8b_gemv_plan_destroy
        self._stream = torch._C._cuda_getCurrentRawStream
        plan = _P(0)
        with torch.cuda.device(self.dev):
            rc = lib.tfp8b_gemv_plan_create(ctypes.byref(plan), _DT[x_dtype], qweight.data_ptr(), wscale.data_ptr(),
                                            _scale_kind(wscale), bias.data_ptr() if bias is not None else None,
                                            _DT[out_dtype], GEMV_MAXM, N, K, group_size, FMT_ID[fmt])
        _check(rc, "tfp8b_gemv_plan_create")
        self.plan = plan
        self.args = [plan, _P(0), _P(0), _I(0), ctypes.c_uint(0), _P(0)]
        self.q, self.ws, self.bias, self.lut, self.out_dtype = qweight, wscale, bias, lut16, out_dtype

    def __del__(self):
        plan, self.plan = getattr(self, "plan", None), None
        if plan is not None and plan.value:
            self._destroy(plan)

    def __call__(self, x, M, out_shape=None, independent=False):
        """x: contiguous CUDA tensor of the bound dtype on this layer's device holding M rows of K
        (any rank: only its data pointer is used). out_shape: shape of y, default (M, N).
        independent: the caller vouches that x is not produced (and y not used) by the kernel that
        precedes this call in the stream, so the two may run concurrently."""
        y = torch.empty(out_shape or (M, self.N), dtype=self.out_dtype, device=self.device)
        a = self.args
        a[1].value = x.data_ptr()
        a[2].value = y.data_ptr()
        a[3].value = M
        a[4].value = 1 if independent else 0
        a[5].value = self._stream(self.dev)
        rc = self.fn(*a)
        if rc != 0:
            _check(rc, "tfp8b_gemv")
        return y


def _gemv(x, qweight, wscale, bias, y, M, N, K, group_size, fmt, dev):
    rc = load().tfp8b_gemv(x.data_ptr(), _DT[x.dtype], qweight.data_ptr(), wscale.data_ptr(), _scale_kind(wscale),
                           bias.data_ptr() if bias is not None else 0, y.data_ptr(), _DT[y.dtype], M, N, K,
                           group_size, FMT_ID[fmt], _stream(dev))
    _check(rc, "tfp8b_gemv")


SPLITK_MAX_M = 64          # above this the tiles are wide enough that whole-K tiles keep the SMs busy


def _gemm(x16, xs, qweight, wscale, bias, y, M, N, K, group_size, fmt, dev):
    if M <= SPLITK_MAX_M and N * K >= (1 << 24):
        # few, long tiles: let the library split K across SMs (it decides; the workspace is only
        # touched if it does). Partial sums meet in FP32 atomics, so the last bit may vary.
        ws = torch.empty(M * N, dtype=torch.float32, device=y.device)
        rc = load().tfp8b_gemm_splitk(x16.data_ptr(), xs.data_ptr(), qweight.data_ptr(), wscale.data_ptr(), _scale_kind(wscale),
                                      bias.data_ptr() if bias is not None else 0, y.data_ptr(), _DT[y.dtype], M, N, K,
                                      group_size, FMT_ID[fmt], ws.data_ptr(), ws.numel(), _stream(dev))
        _check(rc, "tfp8b_gemm_splitk")
        return
    rc = load().tfp8b_gemm(x16.data_ptr(), xs.data_ptr(), qweight.data_ptr(), wscale.data_ptr(), _scale_kind(wscale),
                           bias.data_ptr() if bias is not None else 0, y.data_ptr(), _DT[y.dtype], M, N, K,
                           group_size, FMT_ID[fmt], _stream(dev))
    _check(rc, "tfp8b_gemm")


def w8a16(x, qweight, lut16, wscale, bias, out_dtype, group_size, fmt="e4m3fn"):
    """y = x @ dequant(qweight).T + bias.

    M <= 8   decode GEMV on x in its own dtype (FP32 accumulate, no prep pass)
    M > 8    activation prep (fp16 + power-of-two row scale) and the tcgen05 tile GEMM
    `lut16` is accepted for signature compatibility and unused.
    """
    dev = _need_cuda(x, qweight, wscale, bias)
    M, K = x.shape
    N = qweight.shape[0]
    y = torch.empty(M, N, dtype=out_dtype, device=x.device)
    if M == 0:
        return y
    x = x.contiguous()
    with torch.cuda.device(dev):
        if M <= GEMV_MAXM:
            _gemv(x, qweight, wscale, bias, y, M, N, K, group_size, fmt, dev)
        else:
            x16, xs = prepare_activations(x)
            _gemm(x16, xs, qweight, wscale, bias, y, M, N, K, group_size, fmt, dev)
    return y


def gemm_prepared(x16, xs, qweight, lut16, wscale, bias, out_dtype, group_size, fmt="e4m3fn"):
    """Tile GEMM on an already prepared fp16 activation (any M >= 1)."""
    dev = _need_cuda(x16, xs, qweight, wscale, bias)
    M, K = x16.shape
    N = qweight.shape[0]
    y = torch.empty(M, N, dtype=out_dtype, device=x16.device)
    if M:
        with torch.cuda.device(dev):
            _gemm(x16.contiguous(), xs, qweight, wscale, bias, y, M, N, K, group_size, fmt, dev)
    return y


def gemm_scatter(x16, xs, qweight, wscale, bias, dst_ptrs, ldy, col0, out_dtype, group_size, fmt="e4m3fn"):
    """Tile GEMM on prepared activations whose N output columns are written at columns
    [col0, col0 + N) of every buffer in `dst_ptrs` (device addresses of [M, ldy] arrays of
    `out_dtype`: this GPU's and, for a fused all-gather, the peers' mapped buffers)."""
    dev = _need_cuda(x16, xs, qweight, wscale, bias)
    M, K = x16.shape
    N = qweight.shape[0]
    if M == 0 or N == 0:
        return
    arr = (ctypes.c_void_p * len(dst_ptrs))(*[int(p) for p in dst_ptrs])
    with torch.cuda.device(dev):
        rc = load().tfp8b_gemm_scatter(x16.contiguous().data_ptr(), xs.data_ptr(), qweight.data_ptr(), wscale.data_ptr(),
                                       _scale_kind(wscale), bias.data_ptr() if bias is not None else 0, arr, len(dst_ptrs),
                                       int(ldy), int(col0), _DT[out_dtype], M, N, K, group_size, FMT_ID[fmt], _stream(dev))
    _check(rc, "tfp8b_gemm_scatter")


def epilogue_into(y, acc, xs, bias, n0=0):
    """y[:, n0:n0+n] = (acc * xs[:, None] + bias[n0:n0+n]).to(y.dtype) in one launch; acc is a
    contiguous FP32 [M, n] block, y a contiguous [M, N] output."""
    dev = _need_cuda(y, acc, xs, bias)
    M, n = acc.shape
    if M == 0 or n == 0:
        return y
    bview = bias[n0:n0 + n] if bias is not None else None
    yv = y[:, n0:] if n0 else y
    with torch.cuda.device(dev):
        rc = load().tfp8b_epilogue(acc.data_ptr(), xs.data_ptr(), bview.data_ptr() if bview is not None else 0,
                                   yv.data_ptr(), _DT[y.dtype], M, n, y.shape[1], _stream(dev))
    _check(rc, "tfp8b_epilogue")
    return y


# ------------------------------------------------------------------ W8A8 (FP8 activations x FP8 weights)
W8A8_BLOCK32, W8A8_ROWCOL = 0, 1


def mx_packed_scale_bytes(rows, K) -> int:
    """Size of the packed UE8M0 scale buffer of a [rows, K] code tensor (512 bytes per 128 rows x 128 K)."""
    return int(load().tfp8b_mx_packed_scale_bytes(rows, K))


def mx_pack_scales(scale_u8):
    """Row-major UE8M0 bytes [rows, K/32] -> the packed chunk layout the MX GEMM reads (uint8, 1-D)."""
    dev = _need_cuda(scale_u8)
    if scale_u8.dtype != torch.uint8 or scale_u8.dim() != 2:
        raise ValueError("mx_pack_scales takes a 2-D uint8 tensor [rows, K/32]")
    rows, kb = scale_u8.shape
    out = torch.empty(mx_packed_scale_bytes(rows, kb * 32), dtype=torch.uint8, device=scale_u8.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_mx_pack_scales(scale_u8.contiguous().data_ptr(), out.data_ptr(), rows, kb * 32, _stream(dev))
    _check(rc, "tfp8b_mx_pack_scales")
    return out


def quantize_k(x, fmt="e4m3fn", ue8m0=False, packed=False):
    """x [R, K] -> (codes u8 [R, K], scales): one scale per row and 32-wide block of K, amax / fmax
    clamped below at 1e-12; with ue8m0 rounded up to a power of two and stored as its exponent byte.
    scales: float32 [R, K/32]; uint8 [R, K/32] (ue8m0); or the packed 1-D uint8 buffer (packed)."""
    dev = _need_cuda(x)
    R, K = x.shape
    if K % 32:
        raise ValueError(f"quantize_k: K={K} must be a multiple of 32")
    x = x.contiguous()
    if x.dtype not in _DT:
        x = x.float()
    q = torch.empty(R, K, dtype=torch.uint8, device=x.device)
    if packed:
        s = torch.empty(mx_packed_scale_bytes(R, K), dtype=torch.uint8, device=x.device)
    else:
        s = torch.empty(R, K // 32, dtype=torch.uint8 if ue8m0 else torch.float32, device=x.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_quantize_k(x.data_ptr(), _DT[x.dtype], q.data_ptr(), s.data_ptr(), R, K, FMT_ID[fmt], int(ue8m0 or packed),
                                     int(packed), _stream(dev))
    _check(rc, "tfp8b_quantize_k")
    return q, s


def gemm_w8a8(a_codes, a_scale, a_fmt, w_codes, w_scale, w_fmt, bias=None, out_dtype=torch.float32, mode=W8A8_BLOCK32):
    """y [M, N] = dec(a_codes [M, K]) @ dec(w_codes [N, K]).T with the scales applied, + bias.
    mode W8A8_BLOCK32: per row and 32-wide block of K -- uint8 scales are UE8M0 in the PACKED
    layout (mx_pack_scales / quantize_k(packed=True)) and run on the block-scaled tensor-core
    path; float32 scales are [rows, K/32] row-major. mode W8A8_ROWCOL: a_scale [M], w_scale [N]."""
    dev = _need_cuda(a_codes, a_scale, w_codes, w_scale, bias)
    M, K = a_codes.shape
    N = w_codes.shape[0]
    if w_codes.shape[1] != K:
        raise ValueError(f"gemm_w8a8: K mismatch ({K} vs {w_codes.shape[1]})")
    if a_scale.dtype != w_scale.dtype:
        raise ValueError("gemm_w8a8: both scale tensors must have the same type")
    y = torch.empty(M, N, dtype=out_dtype, device=a_codes.device)
    if M == 0 or N == 0:
        return y
    with torch.cuda.device(dev):
        rc = load().tfp8b_gemm_w8a8(a_codes.contiguous().data_ptr(), a_scale.contiguous().data_ptr(), FMT_ID[a_fmt],
                                    w_codes.contiguous().data_ptr(), w_scale.contiguous().data_ptr(), FMT_ID[w_fmt], mode,
                                    _scale_kind(a_scale), bias.data_ptr() if bias is not None else None, y.data_ptr(),
                                    _DT[out_dtype], M, N, K, _stream(dev))
    _check(rc, "tfp8b_gemm_w8a8")
    return y


# ------------------------------------------------------------------ decode-step helpers
def rope_kv_store(qkv, pos, cos, sin, k_cache, v_cache, n_heads, n_kv_heads):
    """Rotary embedding + KV-cache write for a fused QKV projection output [B, T, (H + 2 KV) * hd]
    (f16 / bf16, contiguous). Returns Q as [B, H, T, hd]; K and V land in the caches
    [B, KV, max_seq, hd] at positions `pos` (int64 [T], on the device)."""
    dev = _need_cuda(qkv, pos, cos, sin, k_cache, v_cache)
    B, T = qkv.shape[0], qkv.shape[1]
    hd = k_cache.shape[-1]
    q = torch.empty(B, n_heads, T, hd, dtype=qkv.dtype, device=qkv.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_rope_kv_store(qkv.data_ptr(), _DT[qkv.dtype], pos.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), B, T, n_heads, n_kv_heads,
                                        hd, k_cache.shape[2], _stream(dev))
    _check(rc, "tfp8b_rope_kv_store")
    return q


def silu_mul(gate_up):
    """silu(gate) * up for a fused gate/up projection output [..., 2F] (f16 / bf16, contiguous)."""
    dev = _need_cuda(gate_up)
    F = gate_up.shape[-1] // 2
    out = torch.empty(*gate_up.shape[:-1], F, dtype=gate_up.dtype, device=gate_up.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_silu_mul(gate_up.data_ptr(), out.data_ptr(), _DT[gate_up.dtype], gate_up.numel() // (2 * F), F,
                                   _stream(dev))
    _check(rc, "tfp8b_silu_mul")
    return out


def add_rmsnorm(x, delta, weight, eps):
    """x += delta (in place; delta may be None), returns RMSNorm(x) * weight. x, delta [..., dim]
    f16 / bf16 contiguous; weight [dim] of the same dtype."""
    dev = _need_cuda(x, weight) if delta is None else _need_cuda(x, delta, weight)
    dim = x.shape[-1]
    out = torch.empty_like(x)
    with torch.cuda.device(dev):
        rc = load().tfp8b_add_rmsnorm(x.data_ptr(), None if delta is None else delta.data_ptr(), weight.data_ptr(),
                                      out.data_ptr(), _DT[x.dtype], x.numel() // dim, dim, float(eps), _stream(dev))
    _check(rc, "tfp8b_add_rmsnorm")
    return out


def argmax_into(out, logits):
    """out[r] = argmax(logits[r, :]) for a 2-D f16 / bf16 tensor whose rows are contiguous; `out` is
    an int64 tensor with one element per row."""
    dev = _need_cuda(out, logits)
    with torch.cuda.device(dev):
        rc = load().tfp8b_argmax(logits.data_ptr(), _DT[logits.dtype], out.data_ptr(), logits.shape[0], logits.shape[1],
                                 logits.stride(0), _stream(dev))
    _check(rc, "tfp8b_argmax")
    return out


def allreduce_wait_limit(cycles=0) -> int:
    """Sets (cycles > 0) how many SM clock cycles the fused all-reduce waits for a peer before it
    gives up and poisons the row; returns the previous limit. cycles <= 0 only queries."""
    return int(load().tfp8b_allreduce_wait_limit(int(cycles)))


def attn_scratch_floats(batch, n_heads, max_seq, head_dim=128):
    """Size of the split-KV scratch of `attn_decode`: one (max, sum, weighted V) record per head and
    64-position chunk of the cache."""
    return batch * n_heads * ((max_seq + 63) // 64) * (head_dim + 2)


def attn_decode(q, k_cache, v_cache, pos, scratch=None):
    """Attention of one query token per sequence over cache positions [0, pos]: q [B, H, 1, hd] or
    [B, H, hd] (f16 / bf16, contiguous), caches [B, KV, max_seq, hd], pos a one-element int64 device
    tensor. Returns [B, H, hd]. `scratch` (float32, `attn_scratch_floats(B, H, max_seq, hd)` elements)
    is allocated when not given; pass one to stay allocation-free inside a captured step."""
    dev = _need_cuda(q, k_cache, v_cache, pos, scratch)
    B, H, hd = q.shape[0], q.shape[1], q.shape[-1]
    KV, S = k_cache.shape[1], k_cache.shape[2]
    if scratch is None:
        scratch = torch.empty(attn_scratch_floats(B, H, S, hd), dtype=torch.float32, device=q.device)
    out = torch.empty(B, H, hd, dtype=q.dtype, device=q.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_attn_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), pos.data_ptr(), out.data_ptr(),
                                      scratch.data_ptr(), scratch.numel(), _DT[q.dtype], B, H, KV, hd, S, _stream(dev))
    _check(rc, "tfp8b_attn_decode")
    return out


def rope_kv_store_fp8(qkv, pos, cos, sin, k_codes, k_scale, v_codes, v_scale, n_heads, n_kv_heads, fmt="e4m3fn"):
    """`rope_kv_store` into an FP8 KV cache: k_codes / v_codes uint8 [B, KV, max_seq, 128], k_scale /
    v_scale float32 [B, KV, max_seq]. K (rotated) and V are rounded to the activation type and then
    quantized per token and KV head like a row of `quantize_weight` (power-of-two scale). Returns Q
    as [B, H, T, hd]."""
    dev = _need_cuda(qkv, pos, cos, sin, k_codes, k_scale, v_codes, v_scale)
    B, T = qkv.shape[0], qkv.shape[1]
    hd = k_codes.shape[-1]
    q = torch.empty(B, n_heads, T, hd, dtype=qkv.dtype, device=qkv.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_rope_kv_store_fp8(qkv.data_ptr(), _DT[qkv.dtype], pos.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                            q.data_ptr(), k_codes.data_ptr(), k_scale.data_ptr(), v_codes.data_ptr(),
                                            v_scale.data_ptr(), B, T, n_heads, n_kv_heads, hd, k_codes.shape[2], FMT_ID[fmt],
                                            _stream(dev))
    _check(rc, "tfp8b_rope_kv_store_fp8")
    return q


def attn_decode_fp8(q, k_codes, k_scale, v_codes, v_scale, pos, scratch=None, fmt="e4m3fn"):
    """`attn_decode` over an FP8 KV cache (see `rope_kv_store_fp8` for its layout). Returns [B, H, hd]."""
    dev = _need_cuda(q, k_codes, k_scale, v_codes, v_scale, pos, scratch)
    B, H, hd = q.shape[0], q.shape[1], q.shape[-1]
    KV, S = k_codes.shape[1], k_codes.shape[2]
    if scratch is None:
        scratch = torch.empty(attn_scratch_floats(B, H, S, hd), dtype=torch.float32, device=q.device)
    out = torch.empty(B, H, hd, dtype=q.dtype, device=q.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_attn_decode_fp8(q.data_ptr(), k_codes.data_ptr(), k_scale.data_ptr(), v_codes.data_ptr(),
                                          v_scale.data_ptr(), pos.data_ptr(), out.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                          _DT[q.dtype], B, H, KV, hd, S, FMT_ID[fmt], _stream(dev))
    _check(rc, "tfp8b_attn_decode_fp8")
    return out


def allreduce_add_rmsnorm(x, partial, weight, eps, recv_ptrs, flag_ptrs, state, rank, max_rows):
    """x += (sum over ranks of `partial`).to(x.dtype) in place, returns RMSNorm(x) * weight: the
    all-reduce of a row-parallel projection fused with the residual update and the norm, for at
    most `max_rows` rows. partial: this rank's float32 [..., dim]; recv_ptrs / flag_ptrs: device
    addresses of every rank's receive area and flag array (see include/tfp8b.h); state: two int32
    of local device memory. A collective: every rank calls it, in the same order."""
    dev = _need_cuda(x, partial, weight, state)
    dim = x.shape[-1]
    rows = x.numel() // dim
    world = len(recv_ptrs)
    out = torch.empty_like(x)
    rp = (ctypes.c_void_p * world)(*[int(p) for p in recv_ptrs])
    fp = (ctypes.c_void_p * world)(*[int(p) for p in flag_ptrs])
    with torch.cuda.device(dev):
        rc = load().tfp8b_allreduce_add_rmsnorm(x.data_ptr(), partial.data_ptr(), weight.data_ptr(), out.data_ptr(), _DT[x.dtype],
                                                rows, dim, float(eps), rp, fp, state.data_ptr(), rank, world, max_rows, _stream(dev))
    _check(rc, "tfp8b_allreduce_add_rmsnorm")
    return out


def gemv_normed(residual, delta, norm_weight, eps, qweight, wscale, bias, out_dtype, group_size, fmt="e4m3fn"):
    """(residual + delta, RMSNorm(residual + delta) * norm_weight @ W^T) for at most 8 rows in one
    GEMV launch: the activations are computed inside the kernel. residual, delta [..., K] f16 / bf16
    (delta may be None); returns the NEW residual (a fresh tensor) and y [..., N]."""
    dev = _need_cuda(residual, delta, norm_weight, qweight, wscale, bias)
    K = residual.shape[-1]
    M = residual.numel() // K
    N = qweight.shape[0]
    new_res = torch.empty_like(residual) if delta is not None else residual
    y = torch.empty(*residual.shape[:-1], N, dtype=out_dtype, device=residual.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_gemv_normed(new_res.data_ptr() if delta is not None else None, residual.data_ptr(),
                                      None if delta is None else delta.data_ptr(), norm_weight.data_ptr(), float(eps),
                                      _DT[residual.dtype], qweight.data_ptr(), wscale.data_ptr(), _scale_kind(wscale),
                                      bias.data_ptr() if bias is not None else None, y.data_ptr(), _DT[out_dtype], M, N, K,
                                      group_size, FMT_ID[fmt], _stream(dev))
    _check(rc, "tfp8b_gemv_normed")
    return new_res, y


def gemv_gated(gate_up, qweight, wscale, bias, out_dtype, group_size, fmt="e4m3fn"):
    """(silu(gate) * up) @ W^T for a fused gate/up output [..., 2K] (f16 / bf16, at most 8 rows) in one
    GEMV launch."""
    dev = _need_cuda(gate_up, qweight, wscale, bias)
    K = gate_up.shape[-1] // 2
    M = gate_up.numel() // (2 * K)
    N = qweight.shape[0]
    y = torch.empty(*gate_up.shape[:-1], N, dtype=out_dtype, device=gate_up.device)
    with torch.cuda.device(dev):
        rc = load().tfp8b_gemv_gated(gate_up.data_ptr(), _DT[gate_up.dtype], qweight.data_ptr(), wscale.data_ptr(), _scale_kind(wscale),
                                     bias.data_ptr() if bias is not None else None, y.data_ptr(), _DT[out_dtype], M, N, K,
                                     group_size, FMT_ID[fmt], _stream(dev))
    _check(rc, "tfp8b_gemv_gated")
    return y
