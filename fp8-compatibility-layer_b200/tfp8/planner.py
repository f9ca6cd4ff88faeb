"""Precision planner: which nn.Linear modules become FP8Linear, and the bookkeeping around it.

The policy is the reference's (tfp8/planner.py:20-88 there), rule for rule and in the same order,
so a model converted here ends up with the same set of FP8 layers:

  already an FP8Linear / already owned  -> left alone (converting twice never re-quantizes)
  image domain: vae / text encoders     -> kept (fp16 / tbf16)
  weight tied to another module         -> kept (never quantize a shared parameter)
  user skip list, sensitive leaf names  -> kept (lm_head, embeddings, routers, LoRA, norms, ...)
  min(out, in) < min_features           -> kept
  in_features % 32 != 0                 -> kept
  name matches the domain's pattern     -> FP8 W8A16
"""
import re
from dataclasses import dataclass

import torch
import torch.nn as nn

from .config import FP8Config
from .linear import FP8Linear

_DOMAIN_RULES = {
    "llm": re.compile(r"(q_proj|k_proj|v_proj|o_proj|qkv|out_proj|gate_proj|up_proj|down_proj|fc1|fc2|w1|w2|w3|mlp)"),
    "image": re.compile(r"(to_q|to_k|to_v|to_out|qkv|proj|attn|ff|mlp|fc1|fc2|linear)"),
}
_SENSITIVE_LEAF = re.compile(
    r"(lm_head|embed|router|gate$|gating|lora|adapter|norm|time|t_embed|adaln|ada_ln|modulation|final|proj_out|head$)",
    re.I)
_IMAGE_COMPONENT_OWNER = {"vae": "fp16", "text_encoder": "tbf16", "text_encoder_2": "tbf16"}


@dataclass
class Decision:
    name: str
    kind: str
    owner: str          # tfp8 | tbf16 | fp16 | native
    reason: str
    shape: tuple = ()


def _tied_parameter_ids(model):
    """ids of parameters that are registered on more than one module."""
    owner, tied = {}, set()
    for mod_name, mod in model.named_modules():
        for _, p in mod.named_parameters(recurse=False):
            first = owner.setdefault(id(p), mod_name)
            if first != mod_name:
                tied.add(id(p))
    return tied


def _decide(name, mod, domain, config, tied):
    """(owner, reason) for one nn.Linear."""
    leaf, top = name.rsplit(".", 1)[-1], name.split(".", 1)[0]
    keep = config.fallback
    if getattr(mod, "precision_owner", None):
        return mod.precision_owner, "already owned"
    if domain == "image" and top in _IMAGE_COMPONENT_OWNER:
        return _IMAGE_COMPONENT_OWNER[top], f"component '{top}' is not quantized in image_safe"
    if id(mod.weight) in tied:
        return keep, "weight shared with another module (tied)"
    if any(re.search(pat, name) for pat in config.extra_skip):
        return keep, "user skip list"
    if _SENSITIVE_LEAF.search(leaf):
        return keep, f"'{leaf}' is precision-sensitive"
    if min(mod.out_features, mod.in_features) < config.min_features:
        return keep, f"small Linear (< {config.min_features})"
    if mod.in_features % 32:
        return keep, "K not a multiple of 32"
    if not _DOMAIN_RULES["llm" if domain == "llm" else "image"].search(name):
        return keep, "not a recognised large Linear"
    return "tfp8", "large Linear -> FP8 W8A16"


def plan(model: nn.Module, domain: str, config: FP8Config):
    tied = _tied_parameter_ids(model)
    decisions = []
    for name, mod in model.named_modules():
        if isinstance(mod, FP8Linear):
            decisions.append(Decision(name, "FP8Linear", "tfp8", "already converted", ()))
        elif isinstance(mod, nn.Linear):
            owner, reason = _decide(name, mod, domain, config, tied)
            decisions.append(Decision(name, type(mod).__name__, owner, reason, (mod.out_features, mod.in_features)))
    return decisions


def _replace_module(root, dotted, new):
    *path, leaf = dotted.split(".")
    for part in path:
        root = getattr(root, part)
    setattr(root, leaf, new)


def prepare_model(model: nn.Module, domain: str = "llm", config: FP8Config | None = None):
    """Quantize, one layer at a time, every module the plan assigns to tfp8 and swap it in place.
    Returns the model; the plan is attached as `model._tfp8_plan`."""
    if config is None:
        config = FP8Config(profile="llm_safe" if domain == "llm" else "image_safe")
    decisions = plan(model, domain, config)
    modules = dict(model.named_modules())
    for d in decisions:
        mod = modules[d.name]
        if isinstance(mod, FP8Linear):
            continue
        if d.owner != "tfp8":
            mod.precision_owner = d.owner
            continue
        new = FP8Linear.from_linear(mod, config.fmt, config.weight_group, config.pow2_scale,
                                    large_m=config.large_m, large_m_backend=config.large_m_backend,
                                    workspace_mb=config.workspace_mb, nan_check=config.nan_check,
                                    scale_format=config.scale_format, activation=config.activation)
        _replace_module(model, d.name, new)
        del mod, modules[d.name]
        if torch.cuda.is_available():
            torch.cuda.empty_cache()       # the full-precision weight of this layer is gone: hand it back
    model._tfp8_plan = decisions
    return model


def report(model, file=None):
    rows = getattr(model, "_tfp8_plan", [])
    lines = [f"{'module':48s} {'shape':>14s}  {'owner':6s}  reason"]
    lines += [f"{r.name:48s} {str(r.shape):>14s}  {r.owner:6s}  {r.reason}" for r in rows]
    lines.append(f"-- {sum(r.owner == 'tfp8' for r in rows)}/{len(rows)} Linear modules on tfp8")
    for name, m in model.named_modules():
        if isinstance(m, FP8Linear) and m.fallback is not None:
            lines.append(f"!! runtime fallback {name}: {m.fallback_reason}")
    text = "\n".join(lines)
    print(text, file=file)
    return text


def weight_bytes(model):
    """Bytes held by parameters and buffers, by dtype name (shared tensors counted once)."""
    totals, seen = {}, set()
    for t in list(model.parameters()) + list(model.buffers()):
        if t is None or id(t) in seen:
            continue
        seen.add(id(t))
        key = str(t.dtype).replace("torch.", "")
        totals[key] = totals.get(key, 0) + t.numel() * t.element_size()
    return totals
