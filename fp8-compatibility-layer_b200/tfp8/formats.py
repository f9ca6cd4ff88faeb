"""FP8 formats: bit semantics, the 256-entry decode table and the torch-level encoder.

Same public surface and the same bit-for-bit results as the reference's tfp8/formats.py
(`Fp8Format`, `E4M3FN`, `E5M2`, `get_format`, `decode`, `lut`, `encode`). These are the
numerical definition the CUDA kernels are tested against; on CUDA tensors `encode` and
`decode` run the kernels themselves.
"""
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Fp8Format:
    name: str
    ebits: int
    mbits: int
    bias: int
    has_inf: bool          # E5M2 follows IEEE (inf + NaNs); E4M3FN has one NaN pattern and no inf
    max_finite: float
    torch_dtype: torch.dtype

    @property
    def top_code(self) -> int:
        """Largest finite non-negative code."""
        emax = (1 << self.ebits) - 1
        if self.has_inf:
            return ((emax - 1) << self.mbits) | ((1 << self.mbits) - 1)
        return (emax << self.mbits) | ((1 << self.mbits) - 2)

    def fields(self, c: torch.Tensor):
        c = c.to(torch.int32)
        return (c >> 7) & 1, (c >> self.mbits) & ((1 << self.ebits) - 1), c & ((1 << self.mbits) - 1)

    def is_nan(self, c: torch.Tensor) -> torch.Tensor:
        _, e, m = self.fields(c)
        top = (1 << self.ebits) - 1
        return (e == top) & ((m != 0) if self.has_inf else (m == (1 << self.mbits) - 1))

    def is_inf(self, c: torch.Tensor) -> torch.Tensor:
        _, e, m = self.fields(c)
        return (e == (1 << self.ebits) - 1) & (m == 0) if self.has_inf else torch.zeros_like(e, dtype=torch.bool)


E4M3FN = Fp8Format("e4m3fn", 4, 3, 7, False, 448.0, torch.float8_e4m3fn)
E5M2 = Fp8Format("e5m2", 5, 2, 15, True, 57344.0, torch.float8_e5m2)
FORMATS = {"e4m3fn": E4M3FN, "e5m2": E5M2}


def get_format(fmt) -> Fp8Format:
    if isinstance(fmt, Fp8Format):
        return fmt
    try:
        return FORMATS[fmt]
    except (KeyError, TypeError):
        raise ValueError(f"unsupported FP8 format {fmt!r}; expected one of {sorted(FORMATS)}") from None


def _table(f: Fp8Format) -> torch.Tensor:
    """All 256 values as float32, computed from the bit fields (value = (-1)^s * 2^(e-bias) * 1.m,
    subnormals m * 2^(1-bias-mbits))."""
    vals = []
    for c in range(256):
        s, e, m = c >> 7, (c >> f.mbits) & ((1 << f.ebits) - 1), c & ((1 << f.mbits) - 1)
        top = (1 << f.ebits) - 1
        if e == top and ((f.has_inf and m != 0) or (not f.has_inf and m == (1 << f.mbits) - 1)):
            v = float("nan")
        elif e == top and f.has_inf:
            v = float("inf")
        elif e == 0:
            v = m * 2.0 ** (1 - f.bias - f.mbits)
        else:
            v = (m + (1 << f.mbits)) * 2.0 ** (e - f.bias - f.mbits)
        vals.append(-v if s else v)
    return torch.tensor(vals, dtype=torch.float32)


_TABLES, _LUTS = {}, {}


def decode(codes: torch.Tensor, fmt) -> torch.Tensor:
    """uint8 codes -> float32 values (exact; NaN, inf and -0 preserved)."""
    f = get_format(fmt)
    if codes.is_cuda:
        from . import _ext
        return _ext.decode_codes(codes, f.name, torch.float32)
    t = _TABLES.get(f.name)
    if t is None:
        t = _TABLES[f.name] = _table(f)
    return t[codes.to(torch.int64)]


def lut(fmt, device="cpu") -> torch.Tensor:
    """The 256-entry table in fp16 (every FP8 value is exact in fp16), cached per device."""
    f = get_format(fmt)
    key = (f.name, str(device))
    t = _LUTS.get(key)
    if t is None:
        t = _LUTS[key] = _table(f).to(torch.float16).to(device)
    return t


def encode(x: torch.Tensor, fmt) -> torch.Tensor:
    """float -> uint8 codes: nearest value, ties to the even code, saturating at +-max_finite
    (never inf); NaN -> the format's canonical NaN (0x7F for E4M3FN, 0x7E for E5M2)."""
    f = get_format(fmt)
    if x.is_cuda:
        from . import _ext
        return _ext.encode(x, f.name, canonical_nan=True)
    xd = x.to(torch.float64)
    ax = xd.abs().clamp(max=f.max_finite)
    vals = _table(f)[: f.top_code + 1].to(torch.float64)       # finite non-negative values; index == code
    mids = (vals[:-1] + vals[1:]) / 2
    flat = torch.nan_to_num(ax, nan=0.0).reshape(-1).contiguous()
    idx = torch.bucketize(flat, mids, right=False)             # number of midpoints strictly below
    at_mid = mids[idx.clamp(max=len(mids) - 1)] == flat
    idx = torch.where(at_mid & (idx < len(mids)) & (idx % 2 == 1), idx + 1, idx)
    q = idx.reshape(x.shape) | (torch.signbit(xd).to(torch.int64) << 7)
    q = torch.where(torch.isnan(xd), torch.full_like(q, 0x7E if f.has_inf else 0x7F), q)
    return q.to(torch.uint8)
