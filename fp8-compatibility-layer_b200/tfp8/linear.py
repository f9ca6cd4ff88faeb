"""FP8Linear: a W8A16 Linear whose weight stays resident as FP8 (uint8 codes + scales).

Same constructor, classmethods, buffers (`qweight`, `weight_scale`, `bias_f32`), `stats` keys and
fallback behaviour as the reference's tfp8/linear.py. Routing per call, by M = activation rows:

  CUDA, M <= 8    decode GEMV: FP8 codes streamed once, decoded in registers, FP32 accumulate
  CUDA, M  > 8    activation prep (fp16 + power-of-two row scale) + tcgen05 tile GEMM with the
                  FP8 tile decoded in shared memory; booked as "gemm", or as "chunked" when
                  M >= large_m and large_m_backend == "chunked" (one kernel serves both: no
                  FP16 weight workspace exists any more)
  CPU tensors     dequantize + float32 matmul in torch -- the definition of the result

With activation="fp8" (W8A8: 32-wide UE8M0 K-groups, K a multiple of 128) every M takes one other
route: the activation rows are quantized on the fly to FP8 with one power-of-two scale per 32-wide
block (the reference's quantize_k, fp8_cuda.py:74-91 there) and the product runs on the
block-scaled FP8 tensor cores (tcgen05.mma.kind::mxf8f6f4); booked as "w8a8". On CPU tensors the
same arithmetic is spelled out in torch (quantize, dequantize both operands, float32 matmul).

On CUDA tensors nothing falls back silently: without the kernel library the call raises.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _ext
from .formats import get_format, lut
from .quantize import dequantize_weight, quantize_weight, scale_to_ue8m0

_NAN_CHECKED_CALLS = 3     # failures are structural, so only the first calls pay for the device sync


class FP8Linear(nn.Module):
    precision_owner = "tfp8"

    def __init__(self, in_features, out_features, bias=True, fmt="e4m3fn", group_size=None,
                 out_dtype=torch.bfloat16, large_m=256, large_m_backend="chunked",
                 workspace_mb=32, nan_check=True, device=None, scale_format="fp32", activation="fp16"):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.fmt = get_format(fmt).name
        self.group_size = group_size or in_features
        if in_features % self.group_size:
            raise ValueError(f"K={in_features} not divisible by group_size={self.group_size}")
        if scale_format not in ("fp32", "ue8m0"):
            raise ValueError("scale_format must be 'fp32' or 'ue8m0'")
        self.out_dtype = out_dtype
        self.large_m, self.large_m_backend = large_m, large_m_backend
        self.workspace_mb, self.nan_check = workspace_mb, nan_check
        self.scale_format = scale_format
        if activation not in ("fp16", "fp8"):
            raise ValueError("activation must be 'fp16' or 'fp8'")
        if activation == "fp8" and (self.group_size != 32 or scale_format != "ue8m0" or in_features % 128):
            raise ValueError("activation='fp8' needs group_size=32, scale_format='ue8m0' and in_features % 128 == 0")
        self.activation = activation
        groups = in_features // self.group_size
        self.register_buffer("qweight", torch.zeros(out_features, in_features, dtype=torch.uint8, device=device))
        self.register_buffer("weight_scale", torch.ones(out_features, groups, dtype=torch.float32, device=device))
        self.register_buffer("bias_f32", torch.zeros(out_features, dtype=torch.float32, device=device) if bias else None)
        self._nan_checks = 0
        self.fallback = None
        self.fallback_reason = None
        self.stats = {"gemv": 0, "gemm": 0, "chunked": 0, "torch": 0, "fallback": 0, "w8a8": 0}
        self._shape_ok = in_features % 32 == 0 and self.group_size % 32 == 0
        self._kernels_ok = self._shape_ok and _ext.available()
        self._lut = lut(self.fmt, device) if device is not None else None
        # Set by a model runner for layers whose input is not produced by the kernel launched just
        # before them (K / V after Q, up after gate, the layers of a sweep): the decode GEMV may then
        # overlap that kernel completely instead of only prefetching its weights.
        self.independent_input = False
        self._gemv = {}            # (x dtype, out dtype) -> _ext.GemvLaunch
        self._e8 = None            # (weight_scale object, its version, uint8 tensor) for scale_format="ue8m0"
        self._e8_packed = None     # (the uint8 tensor above, its packed copy) for activation="fp8"

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_linear(cls, lin: nn.Linear, fmt="e4m3fn", group_size=None, pow2_scale=True, **kw):
        if kw.get("scale_format", "fp32") == "ue8m0" and not pow2_scale:
            raise ValueError("scale_format='ue8m0' needs pow2_scale=True")
        q, s, G = quantize_weight(lin.weight.data, fmt, group_size, pow2_scale)
        wd = lin.weight.dtype
        layer = cls(lin.in_features, lin.out_features, lin.bias is not None, fmt, G,
                    out_dtype=wd if wd in (torch.float16, torch.bfloat16) else torch.float16,
                    device=lin.weight.device, **kw)
        layer.qweight.copy_(q)
        layer.weight_scale.copy_(s)
        if lin.bias is not None:
            layer.bias_f32.copy_(lin.bias.data.float())
        return layer

    @classmethod
    def from_fp8_checkpoint(cls, qweight, weight_scale, bias=None, fmt="e4m3fn", **kw):
        """Adopt an existing FP8 checkpoint's codes and scales verbatim. `qweight` is uint8 or a
        torch float8 tensor of the declared format; `weight_scale` is a scalar, [N] or [N, K/G].
        With scale_format="ue8m0" every scale must be an exact power of two (checked here: the
        kernels would otherwise read other values than the float32 buffer holds)."""
        if qweight.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            if qweight.dtype != get_format(fmt).torch_dtype:
                raise ValueError(f"checkpoint dtype {qweight.dtype} does not match declared fmt {fmt}")
            qweight = qweight.view(torch.uint8)
        N, K = qweight.shape
        ws = weight_scale.float()
        ws = ws.reshape(N, -1) if ws.numel() > 1 else ws.expand(N, 1)
        layer = cls(K, N, bias is not None, fmt, K // ws.shape[1], device=qweight.device, **kw)
        layer.qweight.copy_(qweight)
        layer.weight_scale.copy_(ws)
        if bias is not None:
            layer.bias_f32.copy_(bias.float())
        if layer.scale_format == "ue8m0":
            scale_to_ue8m0(layer.weight_scale, what="from_fp8_checkpoint: weight_scale")     # raises unless exact
        return layer

    def __getstate__(self):
        # prepared launches hold handles of the kernel library and device pointers: a copy of the
        # layer (copy.deepcopy, pickle) starts without them and builds its own on first use
        d = self.__dict__.copy()
        d["_gemv"], d["_e8"], d["_e8_packed"] = {}, None, None
        return d

    def extra_repr(self):
        return (f"in={self.in_features}, out={self.out_features}, fmt={self.fmt}, "
                f"group={self.group_size}, out_dtype={self.out_dtype}, scales={self.scale_format}")

    def dequantized_weight(self):
        return dequantize_weight(self.qweight, self.weight_scale, self.fmt, self.group_size)

    # ------------------------------------------------------------------ cached per-device state
    def _lut_for(self):
        dev = self.weight_scale.device
        if self._lut is None or self._lut.device != dev:
            self._lut = lut(self.fmt, dev)
        return self._lut

    def _kernel_scale(self):
        """The scale tensor handed to the kernels: `weight_scale` itself, or its UE8M0 bytes,
        re-derived whenever the float32 buffer was replaced or written in place."""
        ws = self._buffers["weight_scale"]
        if self.scale_format != "ue8m0":
            return ws
        c = self._e8
        if c is None or c[0] is not ws or c[1] != ws._version:
            c = self._e8 = (ws, ws._version,
                            scale_to_ue8m0(ws, what=f"FP8Linear({self.in_features}->{self.out_features}).weight_scale").contiguous())
        return c[2]

    def _packed_scale(self):
        """The weight's UE8M0 bytes in the packed order the block-scaled tensor-core path reads."""
        e8 = self._kernel_scale()
        c = self._e8_packed
        if c is None or c[0] is not e8:
            c = self._e8_packed = (e8, _ext.mx_pack_scales(e8))
        return c[1]

    def _forward_w8a8(self, x2):
        """W8A8: quantize the activation rows per 32-wide block, multiply codes by codes."""
        fmt = self.fmt
        if x2.is_cuda:
            self._require_kernels()
            if x2.dtype not in _ext._TAG:
                x2 = x2.float()
            aq, sa = _ext.quantize_k(x2, fmt, True, packed=True)
            return _ext.gemm_w8a8(aq, sa, fmt, self.qweight, self._packed_scale(), fmt, self.bias_f32, self.out_dtype)
        # CPU tensors: the same arithmetic in torch (the definition)
        f = get_format(fmt)
        M, K = x2.shape
        xb = x2.float().reshape(M, K // 32, 32)
        s = (xb.abs().amax(-1) / f.max_finite).clamp_min(1e-12)
        s = torch.exp2(torch.ceil(torch.log2(s)).clamp(-127, 127))
        xq = (xb / s[..., None]).clamp(-f.max_finite, f.max_finite).to(f.torch_dtype).float() * s[..., None]
        return F.linear(xq.reshape(M, K), self.dequantized_weight(), self.bias_f32).to(self.out_dtype)

    def _gemv_launch(self, x_dtype):
        """Prepared GEMV call for (input dtype, current out_dtype), rebuilt when a buffer object was
        replaced; in-place updates keep the storage and therefore the bound pointers."""
        b = self._buffers
        q, bias = b["qweight"], b.get("bias_f32")
        ws = self._kernel_scale()
        key = (x_dtype, self.out_dtype)
        p = self._gemv.get(key)
        if p is None or p.q is not q or p.ws is not ws or p.bias is not bias:
            if x_dtype not in _ext._TAG or self.out_dtype not in _ext._TAG or not q.is_cuda:
                return None
            p = self._gemv[key] = _ext.GemvLaunch(x_dtype, q, self._lut_for(), ws, bias, self.out_dtype,
                                                   self.group_size, self.fmt)
        return p

    def _require_kernels(self):
        if not self._kernels_ok:
            _ext.load()                       # raises with the reason when the library is missing
            self._kernels_ok = self._shape_ok and _ext.available()
        return self._kernels_ok

    # ------------------------------------------------------------------ forward
    def forward(self, x):
        if self.activation == "fp8" and self.fallback is None:
            lead = x.shape[:-1]
            x2 = x.reshape(-1, x.shape[-1])
            self.stats["w8a8" if x2.is_cuda else "torch"] += 1
            y = self._forward_w8a8(x2.contiguous())
            return y if x.dim() == 2 else y.reshape(*lead, self.out_features)
        # Decode fast path: contiguous CUDA input of at most 8 rows, after the NaN-checked calls.
        # Only x's data pointer and M are needed, so [B, T, K] is neither reshaped in nor out.
        if ((self._nan_checks >= _NAN_CHECKED_CALLS or not self.nan_check) and self.fallback is None
                and self._kernels_ok and x.is_cuda and x.is_contiguous() and x.shape[-1] == self.in_features):
            M = x.numel() // self.in_features
            if 0 < M <= _ext.GEMV_MAXM:
                p = self._gemv_launch(x.dtype)
                if p is not None and x.get_device() == p.dev and torch.cuda.current_device() == p.dev:
                    self.stats["gemv"] += 1
                    return p(x, M, x.shape[:-1] + (self.out_features,), self.independent_input)
        if self.fallback is not None:
            self.stats["fallback"] += 1
            return self.fallback(x)

        lead = x.shape[:-1]
        x2 = x if x.dim() == 2 else x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M = x2.shape[0]
        on_gpu = x2.is_cuda
        if on_gpu and self._shape_ok:
            self._require_kernels()
        if not on_gpu or not self._shape_ok:
            # CPU tensors, and shapes the kernels do not serve (K or G not a multiple of 32):
            # the defining expression, evaluated by torch where the tensors live.
            self.stats["torch"] += 1
            y = F.linear(x2.float(), self.dequantized_weight(), self.bias_f32).to(self.out_dtype)
        elif M <= _ext.GEMV_MAXM:
            self.stats["gemv"] += 1
            p = self._gemv_launch(x2.dtype) if M else None
            if p is not None and x2.get_device() == p.dev and torch.cuda.current_device() == p.dev:
                y = p(x2, M)
            else:
                if x2.dtype not in _ext._TAG:
                    x2 = x2.float()
                y = _ext.w8a16(x2, self.qweight, None, self._kernel_scale(), self.bias_f32, self.out_dtype,
                               self.group_size, self.fmt)
        else:
            self.stats["chunked" if (M >= self.large_m and self.large_m_backend == "chunked") else "gemm"] += 1
            if x2.dtype not in _ext._TAG:
                x2 = x2.float()
            y = _ext.w8a16(x2, self.qweight, None, self._kernel_scale(), self.bias_f32, self.out_dtype,
                           self.group_size, self.fmt)

        if self.nan_check and self._nan_checks < _NAN_CHECKED_CALLS:
            self._nan_checks += 1
            if not torch.isfinite(y).all() and torch.isfinite(x2).all():
                self._back_off(f"non-finite output for input shape {tuple(x2.shape)}")
                return self.forward(x)
        return y if x.dim() == 2 else y.reshape(*lead, self.out_features)

    def _back_off(self, reason):
        """Runtime fallback: an FP32 Linear holding the decoded weights (the same numbers)."""
        lin = nn.Linear(self.in_features, self.out_features, self.bias_f32 is not None,
                        device=self.qweight.device, dtype=torch.float32)
        lin.weight.data.copy_(self.dequantized_weight())
        if self.bias_f32 is not None:
            lin.bias.data.copy_(self.bias_f32)
        self.fallback = _CastLinear(lin, self.out_dtype)
        self.fallback_reason = reason


class _CastLinear(nn.Module):
    def __init__(self, lin, out_dtype):
        super().__init__()
        self.lin, self.out_dtype = lin, out_dtype

    def forward(self, x):
        return self.lin(x.float()).to(self.out_dtype)
