"""Tensor-parallel wrappers on two gloo ranks (CPU): column-parallel with and without the output
gather, row-parallel with the float32 all-reduce, K-group scales split by group, and the
Megatron-style pairing column -> row. Parity target: the unsharded FP8Linear on the same input
(the reference has no multi-GPU code; single-device numerics are the contract)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "fp8-compatibility-layer_b200"))
    from tfp8 import FP8Linear
    from tfp8.parallel import ColumnParallelFP8Linear, RowParallelFP8Linear
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(3)                                   # identical full layers on every rank
        ok = True
        for G in (None, 128):
            up = FP8Linear.from_linear(nn.Linear(512, 768), group_size=G)
            down = FP8Linear.from_linear(nn.Linear(768, 256), group_size=G)
            up.out_dtype = down.out_dtype = torch.float32
            x = torch.randn(5, 512)
            want_up, want = up(x), down(up(x))
            col_g = ColumnParallelFP8Linear.from_full(up, gather_output=True)
            ok &= torch.equal(col_g(x), want_up)               # same codes, same arithmetic per column
            col = ColumnParallelFP8Linear.from_full(up, gather_output=False)
            row = RowParallelFP8Linear.from_full(down, input_is_parallel=True)
            got = row(col(x))                                   # column -> row without a gather in between
            ok &= torch.allclose(got, want, rtol=1e-5, atol=1e-5 * want.abs().max().item())
            row_full = RowParallelFP8Linear.from_full(down, input_is_parallel=False)
            ok &= torch.allclose(row_full(want_up), want, rtol=1e-5, atol=1e-5 * want.abs().max().item())
            ok &= col.local.qweight.shape == (768 // world, 512) and row.local.qweight.shape == (256, 768 // world)
            if G:
                ok &= row.local.weight_scale.shape == (256, 768 // world // G)
        try:
            RowParallelFP8Linear.from_full(FP8Linear.from_linear(nn.Linear(96, 64)))   # 48 per rank: not % 32
            ok = False
        except ValueError:
            pass
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_column_and_row_parallel_match_single_device():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: True, 1: True}
