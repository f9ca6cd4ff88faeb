"""W8A8 FP8 GEMM with 32-wide K-block scales: the same functions as the reference's root-level
binding of this name (fp8_cuda.py there: `quantize_k`, `Fp8Weight`, `fp8_linear`, `dequant_ref`,
`lut`, `FORMATS`, `BLOCK`), backed by the sm_100a library instead of an NVRTC-compiled WMMA kernel.

    x (M, K) float  --quantize_k-->  FP8 codes + one scale per row and 32-wide block of K
    w (K, N) float  --Fp8Weight-->   FP8 codes + one scale per output column and 32-wide block
    fp8_linear(x, w, bias) = dequant(x) @ dequant(w) + bias, float32, computed from the codes

With UE8M0 scales (`ue8m0=True`) the product runs on tcgen05.mma.kind::mxf8f6f4.block_scale: the
tensor cores take the FP8 codes and the exponent bytes as they are. With float32 scales every
32-wide block's partial product is scaled in FP32 registers, as the reference's kernel does.
The weight is kept K-major ([N, K], the layout FP8Linear uses) -- `Fp8Weight.q` / `.s` expose the
reference's (K, N) / (K/32, N) views of the same data.
"""
import torch

from tfp8 import _ext

FORMATS = {  # name -> (torch dtype, max finite)
    "e4m3": (torch.float8_e4m3fn, 448.0),
    "e5m2": (torch.float8_e5m2, 57344.0),
}
_FMT = {"e4m3": "e4m3fn", "e5m2": "e5m2", "e4m3fn": "e4m3fn"}
BLOCK = 32


def lut(fmt):
    """uint8 -> fp16 table of the format's 256 values (on the current CUDA device)."""
    dt, _ = FORMATS[fmt]
    return torch.arange(256, dtype=torch.uint8, device="cuda").view(dt).to(torch.float16)


def quantize_k(x, fmt, ue8m0=False):
    """Quantize x (R, K) in blocks of 32 along K. Returns uint8 codes (R, K), scales (R, K/32):
    float32, or UE8M0 bytes (value 2^(e-127)) when ue8m0."""
    if not x.is_cuda:
        raise ValueError("quantize_k: x must be a CUDA tensor")
    if x.shape[1] % BLOCK:
        raise ValueError(f"quantize_k: K={x.shape[1]} must be a multiple of {BLOCK}")
    return _ext.quantize_k(x, _FMT[fmt], ue8m0)


class Fp8Weight:
    """B (K, N) quantized along K per output column; `q` (K, N) and `s` (K/32, N) as in the
    reference, stored K-major underneath (`qt` [N, K], `st` [N, K/32])."""

    def __init__(self, w, fmt="e4m3", ue8m0=False):
        if not w.is_cuda:
            raise ValueError("Fp8Weight: w must be a CUDA tensor")
        if w.shape[0] % BLOCK:
            raise ValueError(f"Fp8Weight: K={w.shape[0]} must be a multiple of {BLOCK}")
        self.qt, self.st = quantize_k(w.t().contiguous(), fmt, ue8m0)
        self.fmt, self.ue8m0 = fmt, ue8m0
        self.K, self.N = w.shape
        # what the block-scaled tensor-core path reads: the exponent bytes in their packed order
        self.st_packed = _ext.mx_pack_scales(self.st) if ue8m0 else None

    @property
    def q(self):
        return self.qt.t()

    @property
    def s(self):
        return self.st.t()


def fp8_linear(x, w, bias, act_fmt=None):
    """x (M, K) float -> FP8 GEMM -> (M, N) float32 (+ bias). Activations are quantized dynamically
    per row and 32-wide K block, with the same kind of scale as the weight."""
    act_fmt = act_fmt or w.fmt
    M, K = x.shape
    if not (x.is_cuda and w.qt.is_cuda and bias.is_cuda):
        raise ValueError("fp8_linear: x, weights and bias must all be CUDA tensors")
    if not (x.device == w.qt.device == bias.device):
        raise ValueError(f"fp8_linear: tensors on different devices ({x.device}, {w.qt.device}, {bias.device})")
    if K % 32 or K != w.K:
        raise ValueError(f"fp8_linear: need K a multiple of 32 and K == w.K; got K={K} w.K={w.K}")
    if w.ue8m0:
        aq, sa = _ext.quantize_k(x, _FMT[act_fmt], True, packed=True)
        sw = w.st_packed
    else:
        aq, sa = _ext.quantize_k(x, _FMT[act_fmt], False)
        sw = w.st
    return _ext.gemm_w8a8(aq, sa, _FMT[act_fmt], w.qt, sw, _FMT[w.fmt], bias.float().contiguous(), torch.float32)


def dequant_ref(q, s, fmt, ue8m0, k_axis_last):
    """float64 dequantization used as the reference. q, s as produced above (A layout if k_axis_last)."""
    v = lut(fmt)[q.long()].double()
    sc = torch.exp2(s.double() - 127) if ue8m0 else s.double()
    if k_axis_last:  # (R, K), scales (R, K/32)
        return v * sc.repeat_interleave(BLOCK, dim=1)
    return v * sc.repeat_interleave(BLOCK, dim=0)  # (K, N), scales (K/32, N)
