"""Ingestion of existing FP8 checkpoints into FP8Linear layers.

`FP8Linear.from_fp8_checkpoint` (as in the reference, tfp8/linear.py:82-98) adopts a code tensor
and a scale tensor verbatim but knows only the layouts `scalar`, `[N]` and `[N, K/G]`. Community
FP8 checkpoints use a few more, and keep the scales under several names; this module maps them
onto the one layout the kernels read -- `weight_scale f32 [N, K/G]`, a multiplier
(w = decode(code) * scale) -- without touching a single code:

  per tensor        scalar or one-element tensor              -> [N, 1]
  per channel       [N] or [N, 1]                             -> [N, 1]
  per K-group       [N, K/G]                                  -> as is, group G
  2-D blocks        [ceil(N/bn), ceil(K/bk)] (e.g. 128 x 128) -> rows repeated bn times: [N, K/bk], group bk

Names: `<layer>.weight` (torch float8 or uint8 codes) with `<layer>.weight_scale_inv` or
`<layer>.weight_scale` (both hold the multiplier in the checkpoints that use them), optional
`<layer>.bias`. Everything else in the file (norms, embeddings, an FP16 lm_head) is loaded as
ordinary parameters.
"""
import torch
import torch.nn as nn

from .formats import get_format
from .linear import FP8Linear

SCALE_SUFFIXES = ("weight_scale_inv", "weight_scale", "scale")


def normalize_scale(scale, N, K, block=None):
    """Checkpoint scale tensor -> (float32 [N, K/G], G). `block` = (bn, bk) declares a 2-D block
    layout; without it a 2-D tensor whose first dimension is not N is read as blocks whose sizes
    follow from the shapes (they must then divide N and K exactly)."""
    s = scale.detach().float()
    if s.numel() == 1:
        return s.reshape(1, 1).expand(N, 1).contiguous(), K
    if s.dim() == 1 or (s.dim() == 2 and s.shape[1] == 1 and s.shape[0] == N):
        if s.numel() != N:
            raise ValueError(f"per-channel scale has {s.numel()} entries for {N} output channels")
        return s.reshape(N, 1).contiguous(), K
    if s.dim() != 2:
        raise ValueError(f"unsupported scale shape {tuple(scale.shape)}")
    rows, cols = s.shape
    if block is None and rows == N:
        if K % cols:
            raise ValueError(f"K={K} is not a multiple of the {cols} scale groups per row")
        return s.contiguous(), K // cols
    if block is None:
        if N % rows or K % cols:
            raise ValueError(f"scale shape {(rows, cols)} does not tile a {N} x {K} weight; pass block=(bn, bk)")
        block = (N // rows, K // cols)
    bn, bk = block
    if rows != -(-N // bn) or cols != -(-K // bk):
        raise ValueError(f"scale shape {(rows, cols)} does not match {bn} x {bk} blocks of a {N} x {K} weight")
    if K % bk:
        raise ValueError(f"K={K} is not a multiple of the block width {bk}: the last K-group would be ragged")
    return s.repeat_interleave(bn, dim=0)[:N].contiguous(), bk


def linear_from_checkpoint(qweight, scale, bias=None, fmt="e4m3fn", block=None, **kw):
    """One FP8Linear from a checkpoint's code tensor (torch float8 or uint8, [N, K]) and scale
    tensor in any of the layouts above. Codes and scale values are adopted bit for bit.
    `scale_format="ue8m0"` (in **kw) is accepted only for checkpoints whose scales are exact powers
    of two; any other scale raises ValueError instead of being rounded."""
    if qweight.dim() != 2:
        raise ValueError("weight codes must be 2-D [out_features, in_features]")
    N, K = qweight.shape
    ws, _ = normalize_scale(scale, N, K, block)
    return FP8Linear.from_fp8_checkpoint(qweight, ws, bias, fmt, **kw)


def _scale_for(tensors, prefix):
    for suf in SCALE_SUFFIXES:
        t = tensors.get(f"{prefix}.{suf}")
        if t is not None:
            return t
    return None


def load_fp8_state_dict(model: nn.Module, tensors: dict, fmt=None, block=None, strict=True, **kw):
    """Replace every nn.Linear of `model` whose checkpoint weight is stored as FP8 codes by an
    FP8Linear holding those codes, and load all other tensors as ordinary parameters / buffers.

    tensors   name -> tensor (a state dict, or what `safetensors.torch.load_file` returns)
    fmt       "e4m3fn" / "e5m2"; by default read off the torch float8 dtype of each weight (uint8
              codes need it stated)
    block     (bn, bk) for 2-D block scales; inferred from the shapes when they divide exactly
    Returns the list of converted layer names. With strict, a Linear that has FP8 codes but no
    scale tensor, or leftover tensors that match nothing, raise."""
    float8 = {torch.float8_e4m3fn: "e4m3fn", torch.float8_e5m2: "e5m2"}
    used, converted = set(), []
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            if not isinstance(child, nn.Linear):
                continue
            prefix = f"{parent_name}.{child_name}" if parent_name else child_name
            w = tensors.get(f"{prefix}.weight")
            if w is None or (w.dtype not in float8 and w.dtype != torch.uint8):
                continue
            layer_fmt = float8.get(w.dtype, fmt)
            if layer_fmt is None:
                raise ValueError(f"{prefix}.weight holds uint8 codes: state the format (fmt=...)")
            if fmt is not None and get_format(fmt).name != get_format(layer_fmt).name:
                raise ValueError(f"{prefix}.weight is {w.dtype}, declared fmt is {fmt}")
            s = _scale_for(tensors, prefix)
            if s is None:
                if strict:
                    raise KeyError(f"{prefix}: FP8 weight without a scale tensor ({', '.join(SCALE_SUFFIXES)})")
                continue
            if tuple(w.shape) != (child.out_features, child.in_features):
                raise ValueError(f"{prefix}.weight has shape {tuple(w.shape)}, the layer is "
                                 f"{(child.out_features, child.in_features)}")
            b = tensors.get(f"{prefix}.bias")
            dev = child.weight.device if child.weight.device.type != "meta" else w.device
            layer = linear_from_checkpoint(w.to(dev), s.to(dev), None if b is None else b.to(dev), layer_fmt, block, **kw)
            wd = child.weight.dtype
            layer.out_dtype = wd if wd in (torch.float16, torch.bfloat16) else torch.float16
            setattr(parent, child_name, layer)
            converted.append(prefix)
            used.update(k for k in (f"{prefix}.weight", f"{prefix}.bias") if k in tensors)
            used.update(f"{prefix}.{suf}" for suf in SCALE_SUFFIXES if f"{prefix}.{suf}" in tensors)
    rest = {k: v for k, v in tensors.items() if k not in used}
    missing, unexpected = model.load_state_dict(rest, strict=False)
    fp8_state = {f"{p}.{n}" for p in converted for n in ("qweight", "weight_scale", "bias_f32")}
    missing = [k for k in missing if k not in fp8_state]
    if strict and (missing or unexpected):
        raise KeyError(f"checkpoint does not match the model: missing {missing[:5]}, unexpected {list(unexpected)[:5]}")
    return converted


def load_safetensors(model: nn.Module, paths, fmt=None, block=None, strict=True, device="cpu", **kw):
    """`load_fp8_state_dict` on one or several .safetensors files (shards are merged)."""
    from safetensors.torch import load_file
    if isinstance(paths, (str, bytes)) or hasattr(paths, "__fspath__"):
        paths = [paths]
    tensors = {}
    for p in paths:
        tensors.update(load_file(str(p), device=str(device)))
    return load_fp8_state_dict(model, tensors, fmt, block, strict, **kw)
