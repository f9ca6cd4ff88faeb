"""Tensor-parallel FP8Linear: column- and row-sharded layers over a torch.distributed group.

The reference has no multi-GPU code; single-GPU numerics are the parity target. A layer is
quantized BEFORE it is sharded, so every rank holds a slice of the very codes and scales the
single-GPU layer has:

  column-parallel  rows [r*N/tp, (r+1)*N/tp) of qweight / weight_scale / bias_f32; activations
                   replicated; outputs are the rank's columns, optionally all-gathered.
  row-parallel     columns [r*K/tp, (r+1)*K/tp) of qweight, the matching K-groups of
                   weight_scale (a per-channel scale is replicated); each rank's partial product
                   is computed in float32, summed with one all-reduce, then bias is added and the
                   result rounded once to the output type.

One process per GPU; the collectives are NCCL over NVLink on CUDA tensors (gloo on CPU tensors,
which is how the host logic is tested without GPUs). Summation order differs from one GPU, so
row-parallel results match within the float32 tolerance, not bit for bit.

Fused gather (`gather_output="fused"`, CUDA, more than 8 activation rows): the column-parallel
layer's tile GEMM stores its column shard from the epilogue straight into every rank's full
output buffer -- symmetric memory, plain peer stores over NVLink -- so the all-gather overlaps
the main loop instead of following it as a separate NCCL call; one barrier orders the ranks
before the result is read. Two output buffers alternate, so a call never overwrites a result a
peer may still be reading.
"""
import torch
import torch.distributed as dist
import torch.nn as nn

from .linear import FP8Linear


def _world(group):
    if not dist.is_available() or not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def _slice_layer(full: FP8Linear, rows=None, cols=None, out_dtype=None, bias=True) -> FP8Linear:
    """A new FP8Linear holding rows [r0, r1) and / or input columns [c0, c1) of `full`."""
    N, K, G = full.out_features, full.in_features, full.group_size
    r0, r1 = rows if rows is not None else (0, N)
    c0, c1 = cols if cols is not None else (0, K)
    k_local = c1 - c0
    if G == K:                       # per channel: stays one scale per row on the local K
        g_local, s = k_local, full.weight_scale[r0:r1]
    else:
        if c0 % G or c1 % G:
            raise ValueError(f"row-parallel shard [{c0},{c1}) does not fall on K-group boundaries (G={G})")
        g_local, s = G, full.weight_scale[r0:r1, c0 // G:c1 // G]
    keep_bias = bias and full.bias_f32 is not None
    layer = FP8Linear(k_local, r1 - r0, keep_bias, full.fmt, g_local, out_dtype=out_dtype or full.out_dtype,
                      large_m=full.large_m, large_m_backend=full.large_m_backend, workspace_mb=full.workspace_mb,
                      nan_check=full.nan_check, device=full.qweight.device, scale_format=full.scale_format)
    layer.qweight.copy_(full.qweight[r0:r1, c0:c1])
    layer.weight_scale.copy_(s)
    if keep_bias:
        layer.bias_f32.copy_(full.bias_f32[r0:r1])
    return layer


class ColumnParallelFP8Linear(nn.Module):
    """y[:, shard] = x @ W[shard].T + b[shard]; with gather_output the full [.., N] on every rank."""

    def __init__(self, local: FP8Linear, out_features: int, group=None, gather_output=True):
        super().__init__()
        self.local, self.out_features, self.group, self.gather_output = local, out_features, group, gather_output

    @classmethod
    def from_full(cls, full: FP8Linear, group=None, gather_output=True, rank=None, world=None):
        r, w = _world(group)
        rank, world = (r if rank is None else rank), (w if world is None else world)
        N = full.out_features
        if N % world:
            raise ValueError(f"out_features={N} not divisible by tensor-parallel size {world}")
        per = N // world
        return cls(_slice_layer(full, rows=(rank * per, (rank + 1) * per)), N, group, gather_output)

    # ------------------------------------------------------------------ fused gather
    def _symm_buffers(self, rows, dtype, device):
        """Two [rows, out_features] symmetric-memory outputs and their handles, grown on demand.
        Every rank calls this with the same arguments in the same order (it is a collective)."""
        import torch.distributed._symmetric_memory as symm
        st = getattr(self, "_symm", None)
        if st is None or st["rows"] < rows or st["dtype"] != dtype:
            group = self.group if self.group is not None else dist.group.WORLD
            bufs, hdls = [], []
            for _ in range(2):
                b = symm.empty((rows, self.out_features), dtype=dtype, device=device)
                hdls.append(symm.rendezvous(b, group.group_name))
                bufs.append(b)
            st = self._symm = {"rows": rows, "dtype": dtype, "bufs": bufs, "hdls": hdls, "turn": 0}
        return st

    def _forward_fused(self, x):
        from . import _ext
        loc = self.local
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        M = x2.shape[0]
        rank, world = _world(self.group)
        st = self._symm_buffers(M, loc.out_dtype, x.device)
        turn = st["turn"]
        st["turn"] = turn ^ 1
        buf, hdl = st["bufs"][turn], st["hdls"][turn]
        if x2.dtype not in _ext._TAG:
            x2 = x2.float()
        x16, xs = _ext.prepare_activations(x2)
        ptrs = [int(hdl.buffer_ptrs[r]) for r in range(world)]
        ptrs = ptrs[rank:] + ptrs[:rank]                       # own buffer first
        _ext.gemm_scatter(x16, xs, loc.qweight, loc._kernel_scale(), loc.bias_f32, ptrs, self.out_features,
                          rank * loc.out_features, loc.out_dtype, loc.group_size, loc.fmt)
        loc.stats["gemm"] += 1
        hdl.barrier()                                          # every rank's shard has landed everywhere
        return buf[:M].view(*lead, self.out_features)

    def forward(self, x):
        _, world = _world(self.group)
        if (self.gather_output == "fused" and world > 1 and x.is_cuda and x.numel() // x.shape[-1] > 8
                and self.local._shape_ok and world <= 8):
            return self._forward_fused(x)
        y = self.local(x)
        if not self.gather_output or world == 1:
            return y
        lead = y.shape[:-1]
        y2 = y.reshape(-1, y.shape[-1]).contiguous()
        out = torch.empty(world * y2.shape[0], y2.shape[1], dtype=y.dtype, device=y.device)   # rank-major
        dist.all_gather_into_tensor(out, y2, group=self.group)
        return out.view(world, y2.shape[0], y2.shape[1]).permute(1, 0, 2).reshape(*lead, self.out_features)


class RowParallelFP8Linear(nn.Module):
    """y = sum_r x[:, shard_r] @ W[:, shard_r].T + b: float32 partial products, one all-reduce."""

    def __init__(self, local: FP8Linear, bias_f32, out_dtype, group=None, input_is_parallel=True):
        super().__init__()
        self.local, self.group, self.out_dtype, self.input_is_parallel = local, group, out_dtype, input_is_parallel
        self.register_buffer("bias_f32", bias_f32)

    @classmethod
    def from_full(cls, full: FP8Linear, group=None, input_is_parallel=True, rank=None, world=None):
        r, w = _world(group)
        rank, world = (r if rank is None else rank), (w if world is None else world)
        K = full.in_features
        if K % world or (K // world) % 32:
            raise ValueError(f"in_features={K} cannot be split {world} ways into multiples of 32")
        per = K // world
        local = _slice_layer(full, cols=(rank * per, (rank + 1) * per), out_dtype=torch.float32, bias=False)
        bias = full.bias_f32.detach().clone() if full.bias_f32 is not None else None
        layer = cls(local, bias, full.out_dtype, group, input_is_parallel)
        layer.shard = (rank * per, (rank + 1) * per)
        return layer

    def partial(self, x):
        """This rank's float32 partial product, not reduced (for a caller that fuses the reduction
        with what follows, see FusedAllReduceNorm); the layer must have no bias."""
        if self.bias_f32 is not None:
            raise ValueError("partial() leaves the bias out: use forward() for a layer with bias")
        if not self.input_is_parallel:
            x = x[..., self.shard[0]:self.shard[1]]
        return self.local(x)

    def forward(self, x):
        if not self.input_is_parallel:
            x = x[..., self.shard[0]:self.shard[1]]
        part = self.local(x)                                   # float32 partial sums
        _, world = _world(self.group)
        if world > 1:
            dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
        if self.bias_f32 is not None:
            part = part + self.bias_f32
        return part.to(self.out_dtype)


class FusedAllReduceNorm:
    """Exchange context of `tfp8b_allreduce_add_rmsnorm` for one tensor-parallel group: the
    symmetric-memory receive area and flags of every rank, and the local call-sequence state.
    One context serves every row-parallel layer of a model (calls are ordered by the stream)."""

    def __init__(self, dim, max_rows=8, group=None, device=None):
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.dim, self.max_rows = dim, max_rows
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.recv = symm.empty(2 * self.world * max_rows * dim, dtype=torch.float32, device=device)
        self.flags = symm.empty(2 * self.world * max_rows, dtype=torch.int32, device=device)
        self.recv.zero_()
        self.flags.zero_()
        self._hr = symm.rendezvous(self.recv, group.group_name)
        self._hf = symm.rendezvous(self.flags, group.group_name)
        self.recv_ptrs = [int(self._hr.buffer_ptrs[r]) for r in range(self.world)]
        self.flag_ptrs = [int(self._hf.buffer_ptrs[r]) for r in range(self.world)]
        self.state = torch.zeros(2, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)                      # nobody pushes before every rank has zeroed its flags

    def add_rmsnorm(self, x, partial, weight, eps):
        from . import _ext
        return _ext.allreduce_add_rmsnorm(x, partial, weight, eps, self.recv_ptrs, self.flag_ptrs, self.state, self.rank,
                                          self.max_rows)


def shard_llama_style(model: nn.Module, group=None):
    """Megatron layout for a Llama-style decoder whose projections are FP8Linear modules named
    q_proj / k_proj / v_proj / gate_proj / up_proj (column-parallel, outputs stay sharded) and
    o_proj / down_proj (row-parallel, inputs already sharded). Returns the model."""
    col = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")
    row = ("o_proj", "down_proj")
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, FP8Linear):
                if name in col:
                    setattr(parent, name, ColumnParallelFP8Linear.from_full(child, group, gather_output=False))
                elif name in row:
                    setattr(parent, name, RowParallelFP8Linear.from_full(child, group, input_is_parallel=True))
    return model
