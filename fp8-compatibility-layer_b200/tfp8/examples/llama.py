"""Llama-architecture decoder used as the serving harness of the benchmark (random weights).

Same role as the reference's examples/demo_llm.py: a plain decoder (RMSNorm, RoPE, grouped-query
attention through torch SDPA, SwiGLU) whose projections `prepare_model` turns into FP8Linear.
Differences that matter on B200: a static KV cache and a device-side position, so that one decode
step can be captured in a CUDA graph and replayed (at batch 1 a token is about a millisecond of
kernels: launch overhead would dominate an eager loop); fused QKV and gate/up projections (one
weight stream and one launch each); and Megatron-style tensor parallelism (heads and FFN columns
split across ranks, one all-reduce after o_proj and one after down_proj).
"""
import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .. import _ext
from ..config import FP8Config
from ..formats import decode as decode_codes
from ..linear import FP8Linear
from ..quantize import quantize_weight
from ..parallel import ColumnParallelFP8Linear, RowParallelFP8Linear


@dataclass
class LlamaConfig:
    n_layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    eps: float = 1e-5
    max_seq: int = 2304

    @property
    def head_dim(self):
        return self.d_model // self.n_heads


LLAMA3_8B = LlamaConfig()
TINY = LlamaConfig(n_layers=2, d_model=256, n_heads=8, n_kv_heads=2, ffn=512, vocab=1000, max_seq=64)
TINY_HD128 = LlamaConfig(n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, ffn=512, vocab=1000, max_seq=64)   # head_dim 128


class RMSNorm(nn.Module):
    def __init__(self, d, eps, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d, device=device, dtype=dtype))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)       # one fused kernel


def _rope(x, cos, sin):
    """x [B, H, T, hd]; cos / sin [T, hd/2] (rotate-half convention)."""
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


# Decode steps of at most FUSE_ROWS rows take the path whose GEMVs compute their own activations
# (norm + residual; SwiGLU up to FUSE_ROWS_GATED rows): up to three kernels fewer per block in
# the dependent chain. Every CTA of such a GEMV recomputes the rows from L2, which stops paying
# as the rows grow -- measured per step at batch 2 / 4 / 8: 2.64 -> 2.45, 2.84 -> 2.70, 2.73 -> 3.06 ms.
FUSE_ROWS = 4
FUSE_ROWS_GATED = 2


def _w8(layer, fn, *args):
    """Call a computed-activation GEMV of the library with an FP8Linear's buffers."""
    layer.stats["gemv"] += 1
    return fn(*args, layer.qweight, layer._kernel_scale(), layer.bias_f32, layer.out_dtype, layer.group_size, layer.fmt)


class _Partial:
    """A row-parallel projection's output still to be summed over the ranks (float32, this rank's part)."""

    def __init__(self, t):
        self.t = t


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig, tp: int, device, dtype):
        super().__init__()
        d, hd = cfg.d_model, cfg.head_dim
        self.cfg, self.tp = cfg, tp
        self.h_local, self.kv_local = cfg.n_heads // tp, max(1, cfg.n_kv_heads // tp)
        mk = lambda i, o: nn.Linear(i, o, bias=False, device=device, dtype=dtype)
        # Fused projections, as most serving stacks store them: one weight stream and one launch for
        # Q, K, V and one for gate, up. Rows are ordered rank by rank ([q_r | k_r | v_r], [gate_r | up_r])
        # so that a column-parallel shard is a contiguous row block.
        self.qkv_proj = mk(d, (cfg.n_heads + 2 * cfg.n_kv_heads) * hd)
        self.o_proj = mk(cfg.n_heads * hd, d)
        self.gate_up_proj, self.down_proj = mk(d, 2 * cfg.ffn), mk(cfg.ffn, d)
        self.input_layernorm = RMSNorm(d, cfg.eps, device, dtype)
        self.post_attention_layernorm = RMSNorm(d, cfg.eps, device, dtype)
        self.k_cache = self.v_cache = None
        self.kv_fmt = None                          # "e4m3fn" / "e5m2": the cache holds FP8 codes + one scale per token and KV head
        self.k_scale = self.v_scale = None
        self.cos_table = self.sin_table = None      # the model's [max_seq, hd/2] tables, shared by all blocks
        self.comm = None                            # FusedAllReduceNorm of a tensor-parallel decode, set by the model

    def alloc_cache(self, batch, device, dtype, kv_fmt=None):
        shape = (batch, self.kv_local, self.cfg.max_seq, self.cfg.head_dim)
        self.kv_fmt = kv_fmt
        if kv_fmt is None:
            self.k_cache = torch.zeros(shape, device=device, dtype=dtype)
            self.v_cache = torch.zeros(shape, device=device, dtype=dtype)
            self.k_scale = self.v_scale = None
        else:               # FP8 codes (zero decodes to 0) and the scale of every (sequence, KV head, position)
            self.k_cache = torch.zeros(shape, device=device, dtype=torch.uint8)
            self.v_cache = torch.zeros(shape, device=device, dtype=torch.uint8)
            self.k_scale = torch.ones(shape[:3], device=device, dtype=torch.float32)
            self.v_scale = torch.ones(shape[:3], device=device, dtype=torch.float32)
        # split-KV partial results of the decode attention; one buffer can serve all blocks
        self.attn_scratch = None

    def _kv_store(self, qkv, pos):
        """Fused rotary embedding + cache write of a QKV projection output; returns head-major Q."""
        if self.kv_fmt is None:
            return _ext.rope_kv_store(qkv, pos, self.cos_table, self.sin_table, self.k_cache, self.v_cache, self.h_local, self.kv_local)
        return _ext.rope_kv_store_fp8(qkv, pos, self.cos_table, self.sin_table, self.k_cache, self.k_scale, self.v_cache,
                                      self.v_scale, self.h_local, self.kv_local, self.kv_fmt)

    def _kv_attend(self, q, pos):
        """One query token per sequence over the cache (the library's split-KV kernel)."""
        if self.kv_fmt is None:
            return _ext.attn_decode(q, self.k_cache, self.v_cache, pos, self.attn_scratch)
        return _ext.attn_decode_fp8(q, self.k_cache, self.k_scale, self.v_cache, self.v_scale, pos, self.attn_scratch, self.kv_fmt)

    def _kv_dense(self, upto=None, dtype=torch.float16):
        """The cache as 16-bit tensors (an FP8 cache decoded: codes * scale, exact in fp32 and then
        rounded to `dtype`), positions [0, upto)."""
        k, v = self.k_cache, self.v_cache
        if upto is not None:
            k, v = k[:, :, :upto], v[:, :, :upto]
        if self.kv_fmt is None:
            return k, v
        ks, vs = self.k_scale, self.v_scale
        if upto is not None:
            ks, vs = ks[:, :, :upto], vs[:, :, :upto]
        return ((decode_codes(k.contiguous(), self.kv_fmt) * ks[..., None]).to(dtype),
                (decode_codes(v.contiguous(), self.kv_fmt) * vs[..., None]).to(dtype))

    def _kv_write_torch(self, pos, k, v):
        """Cache write without the fused kernel (CPU, fp32): k, v [B, KV, T, hd] already rotated."""
        if self.kv_fmt is None:
            self.k_cache.index_copy_(2, pos, k)
            self.v_cache.index_copy_(2, pos, v)
            return
        hd = k.shape[-1]
        for t, codes, scale in ((k, self.k_cache, self.k_scale), (v, self.v_cache, self.v_scale)):
            q8, s8, _ = quantize_weight(t.reshape(-1, hd), self.kv_fmt, None, True)      # one row per token and KV head
            codes.index_copy_(2, pos, q8.view(t.shape))
            scale.index_copy_(2, pos, s8.view(t.shape[:3]))

    def _decode_few_rows(self, x, delta, pos, mask):
        """Block.forward for one or two decode rows on one GPU: 7 kernels instead of 10."""
        B, T, _ = x.shape
        hd, eps = self.cfg.head_dim, self.cfg.eps
        x, qkv = _w8(self.qkv_proj, _ext.gemv_normed, x, delta, self.input_layernorm.weight, eps)
        q = self._kv_store(qkv, pos)
        if mask is False:
            a = self._kv_attend(q, pos).view(B, 1, self.h_local * hd)
        else:
            kd, vd = self._kv_dense(dtype=x.dtype)
            a = F.scaled_dot_product_attention(q, kd, vd, attn_mask=mask, enable_gqa=True)
            a = a.transpose(1, 2).reshape(B, T, self.h_local * hd)
        o = self.o_proj(a)
        x, gu = _w8(self.gate_up_proj, _ext.gemv_normed, x, o, self.post_attention_layernorm.weight, eps)
        if B * T <= FUSE_ROWS_GATED:
            return x, _w8(self.down_proj, _ext.gemv_gated, gu)
        return x, self.down_proj(_ext.silu_mul(gu))

    def forward(self, x, delta, pos, cos, sin, mask):
        """x [B, T, d] the residual stream and delta the previous block's MLP output not yet added
        to it (None for the first block); pos int64 [T] (device) = cache positions of these tokens;
        mask additive [T, max_seq], None (prefill from position 0 uses the causal flag) or False (one
        decode token on the GPU: the split-KV attention kernel reads the position itself).
        Returns (x, delta) in the same convention: the add is fused with the next RMSNorm."""
        B, T, _ = x.shape
        hd = self.cfg.head_dim
        fused = x.is_cuda and x.dtype in (torch.float16, torch.bfloat16)
        if (fused and self.tp == 1 and B * T <= FUSE_ROWS and mask is not None and not isinstance(delta, _Partial)
                and isinstance(self.qkv_proj, FP8Linear) and self.qkv_proj._kernels_ok):
            return self._decode_few_rows(x, delta, pos, mask)
        # tensor-parallel decode: the all-reduce after o_proj / down_proj rides in the add + norm kernel
        comm = self.comm if (fused and self.comm is not None and B * T <= self.comm.max_rows) else None
        if isinstance(delta, _Partial):
            h = self.comm.add_rmsnorm(x, delta.t, self.input_layernorm.weight, self.cfg.eps)
        elif fused:      # one kernel: x += delta (in place), h = RMSNorm(x)
            h = _ext.add_rmsnorm(x, delta, self.input_layernorm.weight, self.cfg.eps)
        else:
            x = x if delta is None else x + delta
            h = self.input_layernorm(x)
        qkv = self.qkv_proj(h).to(x.dtype)
        if fused:      # one kernel: rotate Q and K, write K and V into the cache, lay Q out head-major
            q = self._kv_store(qkv.contiguous(), pos)
        else:
            qkv = qkv.view(B, T, self.h_local + 2 * self.kv_local, hd).transpose(1, 2)
            q, k, v = qkv.split((self.h_local, self.kv_local, self.kv_local), dim=1)
            q, k = _rope(q, cos, sin), _rope(k, cos, sin)
            self._kv_write_torch(pos, k, v)
        if mask is None:
            # prefill starts at position 0 and attends over what the cache now holds (an FP8 cache: the
            # quantized K and V, as every later step will see them)
            k, v = self._kv_dense(T, x.dtype)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
            a = a.transpose(1, 2).reshape(B, T, self.h_local * hd)
        elif mask is False:
            # decode step: split-KV attention over the static cache, [B, H, hd] is already [B, 1, H * hd]
            a = self._kv_attend(q, pos).view(B, 1, self.h_local * hd)
        else:
            kd, vd = self._kv_dense(dtype=x.dtype)
            a = F.scaled_dot_product_attention(q, kd, vd, attn_mask=mask, enable_gqa=True)
            a = a.transpose(1, 2).reshape(B, T, self.h_local * hd)
        if comm is not None:
            h = comm.add_rmsnorm(x, self.o_proj.partial(a), self.post_attention_layernorm.weight, self.cfg.eps)
        else:
            o = self.o_proj(a).to(x.dtype)
            if fused:
                h = _ext.add_rmsnorm(x, o.contiguous(), self.post_attention_layernorm.weight, self.cfg.eps)
            else:
                x = x + o
                h = self.post_attention_layernorm(x)
        gu = self.gate_up_proj(h)
        if comm is not None and B * T <= FUSE_ROWS_GATED and gu.dtype == x.dtype and self.down_proj.bias_f32 is None:
            # this rank's partial of the down projection with SwiGLU computed inside the GEMV
            return x, _Partial(_w8(self.down_proj.local, _ext.gemv_gated, gu.contiguous()))
        if fused and gu.dtype == x.dtype:
            act = _ext.silu_mul(gu.contiguous())
        else:
            f = gu.shape[-1] // 2
            act = F.silu(gu[..., :f]) * gu[..., f:]
        if comm is not None:
            return x, _Partial(self.down_proj.partial(act))
        return x, self.down_proj(act).to(x.dtype)


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig = LLAMA3_8B, device="cpu", dtype=torch.float16, tp=1):
        super().__init__()
        self.cfg, self.tp = cfg, tp
        # decode attention over a 16-bit cache: torch SDPA (cuDNN) by default; True selects the library's
        # split-KV kernel (alone it is faster up to four sequences, inside a full step it ties at one
        # and loses 4 - 6 % at four and eight)
        self.attn_kernel = False
        # None: the KV cache holds activations as they are. "e4m3fn" / "e5m2": FP8 codes + one scale per
        # token and KV head (FP8Config(kv_cache="fp8")); the decode step then always uses the library's
        # attention kernel, which reads the codes (torch's would need the whole cache decoded first).
        self.kv_fmt = None
        self.embed = nn.Embedding(cfg.vocab, cfg.d_model, device=device, dtype=dtype)
        self.layers = nn.ModuleList([Block(cfg, tp, device, dtype) for _ in range(cfg.n_layers)])
        self.norm = RMSNorm(cfg.d_model, cfg.eps, device, dtype)
        self.lm_head = nn.Linear(cfg.d_model, cfg.vocab, bias=False, device=device, dtype=dtype)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=device).float() / cfg.head_dim))
        ang = torch.arange(cfg.max_seq, device=device).float()[:, None] * inv[None, :]
        self.register_buffer("cos", ang.cos(), persistent=False)
        self.register_buffer("sin", ang.sin(), persistent=False)

    def alloc_cache(self, batch):
        p = self.embed.weight
        scratch = None
        if p.is_cuda:
            scratch = torch.empty(_ext.attn_scratch_floats(batch, self.cfg.n_heads // self.tp, self.cfg.max_seq, self.cfg.head_dim),
                                  dtype=torch.float32, device=p.device)
        for l in self.layers:
            l.alloc_cache(batch, p.device, p.dtype, self.kv_fmt)
            l.cos_table, l.sin_table = self.cos, self.sin
            l.attn_scratch = scratch

    def set_comm(self, comm):
        """Fuse the tensor-parallel all-reduces of the decode step into the add + norm kernels
        (comm: tfp8.parallel.FusedAllReduceNorm, or None for NCCL all-reduces)."""
        for l in self.layers:
            l.comm = comm

    def forward(self, tokens, pos, prefill=False, last_only=False):
        """tokens int64 [B, T]; pos int64 [T] on the same device. Returns logits [B, T, vocab], or
        [B, 1, vocab] of the last position with last_only (all a prefill needs to pick a token)."""
        x = self.embed(tokens)
        fused = x.is_cuda and x.dtype in (torch.float16, torch.bfloat16)
        cos, sin = (None, None) if fused else (self.cos[pos], self.sin[pos])     # the fused kernels index the tables
        mask = None
        if not prefill:
            hd, blk = self.cfg.head_dim, self.layers[0]
            if (self.attn_kernel or self.kv_fmt is not None) and fused and tokens.shape[1] == 1 and hd == 128:
                mask = False             # decode attention kernel: reads the position itself, no mask tensor
            else:
                seq = torch.arange(self.cfg.max_seq, device=pos.device)
                mask = torch.where(seq[None, :] <= pos[:, None], 0.0, float("-inf")).to(x.dtype)
        delta = None
        for l in self.layers:
            x, delta = l(x, delta, pos, cos, sin, mask)
        if isinstance(delta, _Partial):
            h = self.layers[0].comm.add_rmsnorm(x, delta.t, self.norm.weight, self.cfg.eps)
            return self.lm_head(h)
        if last_only:
            x, delta = x[:, -1:].contiguous(), delta[:, -1:].contiguous()
        if fused:
            h = _ext.add_rmsnorm(x, delta, self.norm.weight, self.cfg.eps)
        else:
            h = self.norm(x + delta)
        return self.lm_head(h)


def build_fp8_llama(cfg: LlamaConfig, device, dtype=torch.float16, fp8: FP8Config | None = None, group=None, seed=0,
                    sigma=0.02, tp=None):
    """Random-init (N(0, sigma^2)) decoder with every projection quantized to FP8Linear, built one
    layer at a time so the full-precision model never exists. With a process group the layers are
    quantized first and then sharded Megatron-style (every rank draws the same full weights);
    tp=1 builds the unsharded model even when a process group exists."""
    fp8 = fp8 or FP8Config(profile="llm_safe", nan_check=False)
    world = dist.get_world_size(group) if (group is not None or (dist.is_available() and dist.is_initialized())) else 1
    if tp is not None:
        if tp not in (1, world):
            raise ValueError(f"tp={tp}: either 1 (unsharded) or the size of the process group ({world})")
        world = tp
    if cfg.n_heads % world or (cfg.n_kv_heads % world and world % cfg.n_kv_heads) or cfg.ffn % world:
        raise ValueError(f"tensor-parallel size {world} does not divide the model")
    with torch.device("meta"):
        model = Llama(cfg, dtype=dtype, tp=world)
    g = torch.Generator(device=device).manual_seed(seed)
    rnd = lambda *s: (torch.randn(*s, generator=g, device=device) * sigma).to(dtype)

    def quantized(out_f, in_f, kind, independent=False):
        lin = nn.Linear(in_f, out_f, bias=False, device=device, dtype=dtype)
        lin.weight.data = rnd(out_f, in_f)
        q = FP8Linear.from_linear(lin, fp8.fmt, fp8.weight_group, fp8.pow2_scale, nan_check=fp8.nan_check,
                                  scale_format=fp8.scale_format)
        del lin
        if world > 1:
            q = (ColumnParallelFP8Linear.from_full(q, group, gather_output=False) if kind == "col"
                 else RowParallelFP8Linear.from_full(q, group, input_is_parallel=True))
            q.local.independent_input = independent
        else:
            q.independent_input = independent
        return q

    d, hd = cfg.d_model, cfg.head_dim
    for blk in model.layers:
        blk.qkv_proj = quantized((cfg.n_heads + 2 * cfg.n_kv_heads) * hd, d, "col")
        blk.o_proj = quantized(d, cfg.n_heads * hd, "row")
        blk.gate_up_proj = quantized(2 * cfg.ffn, d, "col")
        blk.down_proj = quantized(d, cfg.ffn, "row")
        blk.input_layernorm = RMSNorm(d, cfg.eps, device, dtype)
        blk.post_attention_layernorm = RMSNorm(d, cfg.eps, device, dtype)
    model.embed = nn.Embedding(cfg.vocab, d, device=device, dtype=dtype)
    model.embed.weight.data = rnd(cfg.vocab, d)
    model.norm = RMSNorm(d, cfg.eps, device, dtype)
    model.lm_head = nn.Linear(d, cfg.vocab, bias=False, device=device, dtype=dtype)    # stays fp16 (planner rule)
    model.lm_head.weight.data = rnd(cfg.vocab, d)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=device).float() / hd))
    ang = torch.arange(cfg.max_seq, device=device).float()[:, None] * inv[None, :]
    model.register_buffer("cos", ang.cos(), persistent=False)
    model.register_buffer("sin", ang.sin(), persistent=False)
    model.kv_fmt = fp8.fmt if fp8.kv_cache == "fp8" else None
    return model


def reorder_fused_rows_like_tp(model: Llama, tp: int):
    """Re-orders, in place, the rows of the fused QKV and gate/up projections of an UNSHARDED model
    so that it computes what a `tp`-way tensor-parallel build of the same seed computes.

    The fused projections keep their rows rank by rank ([q_r | k_r | v_r], [gate_r | up_r]), so the
    same random matrix means a different model for every tensor-parallel size: rank r's block of a
    tp-way build holds heads that an unsharded build would read as something else. Gathering the
    q parts of all ranks, then the k parts, then the v parts (and gate parts, then up parts) gives
    the one-GPU model that is mathematically the same as the sharded one -- what a parity check
    between the two needs."""
    cfg = model.cfg
    if model.tp != 1 or cfg.n_heads % tp or cfg.n_kv_heads % tp or cfg.ffn % tp:
        raise ValueError("needs an unsharded model and a tensor-parallel size that divides heads, KV heads and FFN")
    hd = cfg.head_dim
    hq, hk, f = cfg.n_heads // tp * hd, cfg.n_kv_heads // tp * hd, cfg.ffn // tp

    def perm_of(parts, per, dev):
        idx, off = [], 0
        offs = []
        for n in parts:
            offs.append(off)
            off += n
        for o, n in zip(offs, parts):
            for r in range(tp):
                idx.append(torch.arange(r * per + o, r * per + o + n, device=dev))
        return torch.cat(idx)

    for blk in model.layers:
        for lin, parts in ((blk.qkv_proj, (hq, hk, hk)), (blk.gate_up_proj, (f, f))):
            perm = perm_of(parts, sum(parts), lin.qweight.device)
            lin.qweight.copy_(lin.qweight[perm])
            lin.weight_scale.copy_(lin.weight_scale[perm])
            if lin.bias_f32 is not None:
                lin.bias_f32.copy_(lin.bias_f32[perm])
    return model


class DecodeRunner:
    """Prefill, then greedy decode with the whole step (all layers, lm_head, argmax, position bump)
    captured in one CUDA graph."""

    def __init__(self, model: Llama, batch: int, fused_allreduce=True):
        self.model, self.batch = model, batch
        model.alloc_cache(batch)
        dev = model.embed.weight.device
        model.set_comm(None)
        if fused_allreduce and model.tp > 1 and dev.type == "cuda" and model.embed.weight.dtype in (torch.float16, torch.bfloat16):
            from ..parallel import FusedAllReduceNorm
            comm = None
            try:
                comm = FusedAllReduceNorm(model.cfg.d_model, max_rows=max(8, batch), device=dev)
            except Exception as e:               # no peer-mapped memory here: NCCL all-reduces instead
                self.fused_allreduce_error = f"{type(e).__name__}: {e}"
            ok = torch.tensor([0 if comm is None else 1], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)               # every rank takes the same path
            model.set_comm(comm if int(ok) else None)
        self.tok = torch.zeros(batch, 1, dtype=torch.int64, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int64, device=dev)
        self.host_pos = 0            # host-side mirror of self.pos
        self.graph = None
        self.last_logits = None      # logits [B, 1, vocab] of the latest decode step

    def _room(self, more, what):
        """The static KV cache holds cfg.max_seq positions; the position itself lives on the device
        (it is bumped inside the captured graph), so the host keeps its own count and refuses a
        call that would write past the cache instead of letting a kernel find out."""
        if self.host_pos + more > self.model.cfg.max_seq:
            raise ValueError(f"{what}: {self.host_pos} cached positions + {more} more exceed the KV cache "
                             f"(max_seq={self.model.cfg.max_seq})")

    def check_device(self):
        """Raises if a kernel of the step gave up on a bounded wait (a tensor-parallel peer that
        never answered) or skipped an out-of-range position. Synchronises."""
        if self.tok.is_cuda:
            _ext.device_status(self.tok.device)

    @torch.no_grad()
    def prefill(self, tokens):
        T = tokens.shape[1]
        self.host_pos = 0
        self._room(T, "prefill")
        self.host_pos = T
        pos = torch.arange(T, device=tokens.device)
        logits = self.model(tokens, pos, prefill=True, last_only=True)
        self._pick(logits)
        self.pos.fill_(T)
        return logits

    def _pick(self, logits):
        """Greedy choice of the next token from logits [B, 1, vocab] into self.tok."""
        if logits.is_cuda and logits.dtype in (torch.float16, torch.bfloat16):
            _ext.argmax_into(self.tok, logits.view(logits.shape[0], -1))
        else:
            self.tok.copy_(logits[:, -1:].argmax(-1))

    @torch.no_grad()
    def _step(self):
        logits = self.model(self.tok, self.pos, prefill=False)
        self.last_logits = logits            # inside a captured graph: the static tensor every replay rewrites
        self._pick(logits)
        self.pos.add_(1)

    @torch.no_grad()
    def capture(self, warmup=3):
        self._room(max(warmup, 1), "capture (its warm-up steps write cache positions too)")
        keep_tok, keep_pos = self.tok.clone(), self.pos.clone()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(warmup):                  # un-captured calls first (kernel opt-ins, NaN-check calls)
                self._step()
        torch.cuda.current_stream().wait_stream(s)
        self.tok.copy_(keep_tok); self.pos.copy_(keep_pos)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._step()
        self.tok.copy_(keep_tok); self.pos.copy_(keep_pos)

    @torch.no_grad()
    def decode(self, steps, check=True, keep_logits=None):
        """`steps` greedy tokens per sequence, [B, steps]. With `check` the device status word is
        read afterwards (one synchronisation per call, not per step). `keep_logits`: a list that
        receives a copy of every step's logits [B, 1, vocab]."""
        self._room(steps, "decode")
        self.host_pos += steps
        out = []
        for _ in range(steps):
            if self.graph is not None:
                self.graph.replay()
            else:
                self._step()
            out.append(self.tok.clone())
            if keep_logits is not None:
                keep_logits.append(self.last_logits.clone())
        if check:
            self.check_device()
        return torch.cat(out, dim=1)
