"""Symmetric FP8 weight quantization, its inverse, and the activation row scale.

    scale = max|w| / FP8_MAX            (rounded up to a power of two by default)
    q     = RNE(clamp(w / scale, -FP8_MAX, FP8_MAX))

Same functions and results as the reference's tfp8/quantize.py. `quantize_weight` on a CUDA
tensor is one fused kernel (amax, scale and codes in a single pass over each row) instead of
five torch passes; on a CPU tensor it is the plain torch expression.
"""
import torch

from .formats import get_format, lut

ACT_TARGET_EXP = 8   # the row amax of a prepared activation lands in [2^7, 2^8)


def pow2_ceil(s: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= s (s > 0), read off the float's exponent and mantissa so that an
    exact power of two maps to itself."""
    m, e = torch.frexp(s.float())
    return torch.ldexp(torch.ones_like(m), torch.where(m == 0.5, e - 1, e))


def quantize_weight(w: torch.Tensor, fmt="e4m3fn", group_size=None, pow2_scale=True):
    """w [N,K] -> (qweight uint8 [N,K], scale f32 [N, K/G], G); group_size None means one scale
    per output channel (G = K). Runs on the device w lives on."""
    f = get_format(fmt)
    N, K = w.shape
    G = K if group_size is None else group_size
    if K % G:
        raise ValueError(f"K={K} not divisible by group_size={G}")
    if w.is_cuda and K % 16 == 0 and G % 16 == 0:
        from . import _ext
        return _ext.quantize_weight_cuda(w, f.name, G, pow2_scale)
    if w.is_cuda:
        from . import _ext
        _ext.load()          # a CUDA tensor without the kernel library is an error, not a downgrade
    blocks = w.float().reshape(N, K // G, G)
    amax = blocks.abs().amax(dim=-1)
    s = (amax / f.max_finite).clamp_min(torch.finfo(torch.float32).tiny)
    if pow2_scale:
        s = pow2_ceil(s)
    s = torch.where(amax == 0, torch.ones_like(s), s)
    scaled = (blocks / s.unsqueeze(-1)).clamp(-f.max_finite, f.max_finite)
    q = scaled.to(f.torch_dtype).view(torch.uint8).reshape(N, K)      # torch's cast is RNE
    return q.contiguous(), s.contiguous(), G


def dequantize_weight(q: torch.Tensor, s: torch.Tensor, fmt, group_size) -> torch.Tensor:
    """float32 [N,K] = table[q] * s, the definition the kernels are checked against."""
    N, K = q.shape
    vals = lut(fmt, q.device)[q.long()].float().reshape(N, K // group_size, group_size)
    return (vals * s.float().unsqueeze(-1)).reshape(N, K)


def scale_to_ue8m0(s: torch.Tensor, strict: bool = True, what: str = "weight scale") -> torch.Tensor:
    """Power-of-two float32 scales -> UE8M0 bytes (value 2^(b-127)).

    A UE8M0 byte can only hold a power of two in [2^-127, 2^127]. With `strict` (the default) any
    other value -- not a power of two, zero, negative, non-finite -- raises ValueError: the bytes
    would otherwise stand for a different number than the float32 scale that the CPU path and
    `dequantized_weight()` keep using. With strict=False such a scale is rounded up to the next
    power of two (and clamped into range)."""
    s = s.float()
    m, e = torch.frexp(s)
    e = torch.where(m == 0.5, e - 1, e)
    b = (e.clamp(-127, 127) + 127).to(torch.uint8)
    if strict:
        bad = ~(ue8m0_to_scale(b) == s)
        if bool(bad.any()):
            v = s[bad].flatten()[0].item()
            raise ValueError(f"{what}: {int(bad.sum())} of {s.numel()} values are not powers of two in [2^-127, 2^127] "
                             f"(first: {v!r}); scale_format='ue8m0' needs power-of-two scales "
                             "(quantize with pow2_scale=True, or keep scale_format='fp32')")
    return b


def ue8m0_to_scale(b: torch.Tensor) -> torch.Tensor:
    v = torch.ldexp(torch.ones(b.shape, dtype=torch.float32, device=b.device), b.to(torch.int32) - 127)
    return torch.where(b == 255, torch.full_like(v, float("nan")), v)


def activation_to_fp16(x: torch.Tensor):
    """Activation rows -> (fp16 [M,K], power-of-two row scale f32 [M]). Dividing by an exact power
    of two loses nothing, so BF16 -> FP16 is exact unless a value lands in fp16's subnormal range.
    FP16 input passes through with scale 1."""
    if x.dtype == torch.float16:
        return x.contiguous(), torch.ones(x.shape[0], dtype=torch.float32, device=x.device)
    amax = x.abs().amax(dim=-1).float()
    e = torch.ceil(torch.log2(amax.clamp_min(2.0 ** -100))) - ACT_TARGET_EXP
    e = torch.where(amax > 0, e, torch.zeros_like(e))
    xs = torch.exp2(e)
    return (x.float() / xs.unsqueeze(1)).half().contiguous(), xs.contiguous()
