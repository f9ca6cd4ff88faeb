"""Helpers shared by the GPU parity tests: torch <-> oracle conversions and the reference's gate."""
import numpy as np
import torch

from oracle import tfp8_oracle as O

DT_NAME = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}


def f32_bits(bits):
    return np.asarray(bits, np.uint32).view(np.float32)


def t_f32(bits, device="cuda"):
    return torch.from_numpy(np.asarray(bits, np.uint32).view(np.float32).copy()).to(device)


def same_bits_or_nan(a: torch.Tensor, b: torch.Tensor) -> bool:
    a, b = a.float().cpu(), b.float().cpu()
    both_nan = torch.isnan(a) & torch.isnan(b)
    eq = (a == b) & (torch.signbit(a) == torch.signbit(b))
    return bool((both_nan | eq).all())


def oracle_reference(x: torch.Tensor, layer, prepared=True):
    """float64 reference of the reference project's kernel gate: the prepared activation
    (fp16 values times the power-of-two row scale) against the dequantized weight, plus bias.
    Computed by the numpy oracle from the layer's codes and scales."""
    x32 = x.detach().float().cpu().numpy()
    if prepared and x.dtype != torch.float16:
        x16, xs = O.activation_to_fp16(x32)
        x64 = x16.astype(np.float64) * xs.astype(np.float64)[:, None]
    else:
        x64 = x32.astype(np.float64)
    q = layer.qweight.cpu().numpy()
    s = layer.weight_scale.cpu().numpy()
    b = layer.bias_f32.cpu().numpy() if layer.bias_f32 is not None else None
    return O.linear_forward_f64(x64, q, s, b, layer.fmt, layer.group_size)


def assert_gate(y: torch.Tensor, ref64: np.ndarray, out_dtype, what=""):
    """Zero violations of eps*|ref| + 1e-4*max|ref| + 1e-6 (eps 2^-11 for fp16 out, else 2^-8)."""
    tol = O.gate_tolerance(ref64, DT_NAME[out_dtype])
    err = np.abs(y.detach().double().cpu().numpy() - ref64)
    bad = int((err > tol).sum())
    assert bad == 0, f"{what}: {bad} of {err.size} outside the gate, worst {(err / tol).max():.2f}x"


def max_rel_err(y: torch.Tensor, ref64: np.ndarray) -> float:
    """max |y - ref| / max |ref|: the headline tolerance (<= 2e-3)."""
    return float(np.abs(y.detach().double().cpu().numpy() - ref64).max() / np.abs(ref64).max())
