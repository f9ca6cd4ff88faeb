"""`FP8Config`: the knobs of `prepare_model`, field for field those of the reference
(tfp8/config.py:6-34 there), so existing call sites keep working unchanged."""
from dataclasses import dataclass, field

PROFILES = ("llm_safe", "image_safe")
_DEFAULT_MIN_FEATURES = {"llm_safe": 1024, "image_safe": 256}
SCALE_FORMATS = ("fp32", "ue8m0")


@dataclass
class FP8Config:
    fmt: str = "e4m3fn"
    profile: str = "llm_safe"
    weight_group: int | None = None      # None: one scale per output channel; 32 / 128: per K-group
    # "fp16": W8A16, the reference's only implemented mode. "fp8": W8A8 -- activations are quantized
    # per row and 32-wide block of K on the fly and the product runs on the block-scaled FP8 tensor
    # cores; needs weight_group=32 and scale_format="ue8m0" (the MX layout). The reference reserves
    # the field and raises for anything but "fp16" (tfp8/config.py:25-26 there).
    activation: str = "fp16"
    # "fp16": the KV cache of a decoder is left as the model keeps it. "fp8": the serving harness
    # (tfp8.examples.llama) keeps K and V as codes of `fmt` with one power-of-two scale per token and
    # KV head, quantized like a row of quantize_weight, and attends over the codes. prepare_model
    # itself never touches a cache: the field travels with the plan for whoever owns the attention.
    # The reference reserves the field and raises for anything but "fp16" (tfp8/config.py:27-28 there).
    kv_cache: str = "fp16"
    fallback: str = "tbf16"              # owner recorded for modules that are left alone
    min_features: int | None = None      # None: 1024 (llm_safe) / 256 (image_safe)
    pow2_scale: bool = True
    large_m: int = 256
    # The B200 build runs every M > 8 through one tcgen05 tile GEMM. `large_m`, `large_m_backend`
    # and `workspace_mb` are accepted and validated as before and only decide which `stats`
    # counter ("gemm" or "chunked") a call is booked under.
    large_m_backend: str = "chunked"
    workspace_mb: int = 32
    nan_check: bool = True
    extra_skip: list[str] = field(default_factory=list)
    # Addition: how K-group scales are handed to the kernels. "ue8m0" stores one exponent byte per
    # group (needs pow2_scale); the float32 `weight_scale` buffer is kept either way.
    scale_format: str = "fp32"

    def __post_init__(self):
        if self.profile not in PROFILES:
            raise ValueError(f"profile {self.profile!r} not supported; use one of {PROFILES}")
        if self.activation not in ("fp16", "fp8"):
            raise NotImplementedError("activation must be 'fp16' (W8A16) or 'fp8' (W8A8 with 32-wide block scales)")
        if self.activation == "fp8" and (self.weight_group != 32 or self.scale_format != "ue8m0"):
            raise NotImplementedError("activation='fp8' is the MX layout: weight_group=32 and scale_format='ue8m0'")
        if self.kv_cache not in ("fp16", "fp8"):
            raise NotImplementedError("kv_cache must be 'fp16' or 'fp8'")
        if self.large_m_backend not in ("fused", "chunked"):
            raise ValueError("large_m_backend must be 'fused' or 'chunked'")
        if self.scale_format not in SCALE_FORMATS:
            raise ValueError(f"scale_format must be one of {SCALE_FORMATS}")
        if self.scale_format == "ue8m0" and not self.pow2_scale:
            raise ValueError("scale_format='ue8m0' needs pow2_scale=True")
        if self.min_features is None:
            self.min_features = _DEFAULT_MIN_FEATURES[self.profile]
