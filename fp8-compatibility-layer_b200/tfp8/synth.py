"""Seeded synthetic inputs for the benchmark configurations of the FP8Linear hot path.

Everything is generated on the CPU in float32 from a `torch.Generator` with a fixed seed and only
then cast, so a CPU checker and the GPU kernels are handed identical bits. No external data set is
involved anywhere: the shapes are those of Llama-family projection layers.

  config 1   W 4096x4096 fp16, N(0, 0.02^2) with 0.1 % of entries replaced by +-20 sigma,
             x 1x4096 fp16 N(0,1), per-channel power-of-two scales
  config 2   decode sweep, (N,K) in DECODE_SHAPES, M in (1,2,4,8), both formats
  config 3   W 28672x8192 N(0, 0.015^2), 1 % of the 128-wide K-groups multiplied by 8
  config 4   same base weight, 32-wide K-groups, bf16 activations, M in (2048,4096,8192)
  config 5   Llama-3-8B layer shapes (LLAMA3_8B)
"""
import torch

DECODE_SHAPES = ((4096, 4096), (12288, 4096), (11008, 4096), (4096, 11008))
DECODE_M = (1, 2, 4, 8)
GROUP_GEMM_SHAPE = (28672, 8192)
GROUP_GEMM_M = (16, 64, 256, 1024)
PREFILL_M = (2048, 4096, 8192)
LLAMA3_8B = dict(n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, ffn=14336, vocab=128256)


def _gen(seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def outlier_weight(N, K, sigma=0.02, frac=1e-3, k_sigma=20.0, seed=0, dtype=torch.float16):
    """Config-1 weight: Gaussian body, a Bernoulli(frac) mask of entries set to +-k_sigma*sigma."""
    g = _gen(seed)
    w = torch.randn(N, K, generator=g) * sigma
    mask = torch.rand(N, K, generator=g) < frac
    sign = torch.where(torch.rand(N, K, generator=g) < 0.5, -1.0, 1.0)
    w = torch.where(mask, sign * (k_sigma * sigma), w)
    return w.to(dtype)


def gaussian_weight(N, K, sigma=0.02, seed=0, dtype=torch.float16):
    """Config-2 weight."""
    return (torch.randn(N, K, generator=_gen(seed)) * sigma).to(dtype)


def group_outlier_weight(N, K, group=128, sigma=0.015, frac=0.01, gain=8.0, seed=0,
                         dtype=torch.float16):
    """Config-3/4 weight: `frac` of the (row, K-group) blocks of width `group` are scaled by `gain`,
    which gives neighbouring K-groups of one row scales that differ by a few binades."""
    g = _gen(seed)
    w = torch.randn(N, K, generator=g) * sigma
    hot = torch.rand(N, K // group, generator=g) < frac
    w = w.reshape(N, K // group, group) * torch.where(hot, gain, 1.0)[..., None]
    return w.reshape(N, K).to(dtype)


def activations(M, K, seed=1, dtype=torch.float16):
    """N(0,1) activation rows."""
    return torch.randn(M, K, generator=_gen(seed)).to(dtype)


def random_codes(N, K, fmt_dtype, seed=0, finite_only=True):
    """Uniform random FP8 codes (used where only throughput or layout matters). With
    `finite_only` the NaN/inf codes are replaced by 0x10 so a checksum stays finite."""
    q = torch.randint(0, 256, (N, K), generator=_gen(seed), dtype=torch.uint8)
    if finite_only:
        v = q.view(fmt_dtype).float()
        q[~torch.isfinite(v)] = 0x10
    return q
