"""FP8 checkpoint ingestion on the GPU: checkpoints in the four scale layouts that community FP8
models use -- one scale per tensor, per output channel, per K-group, per 2-D block -- are loaded
onto CUDA (as a state dict and from a safetensors file) and the layer's forward through the
kernels (decode GEMV and tile GEMM) is gated against the float64 oracle evaluated on the very
codes and scales the checkpoint holds. `from_fp8_checkpoint` of the reference
(tfp8/linear.py:82-98 there) adopts codes verbatim; this checks that what the kernels compute from
them is the checkpoint's own weight, w = decode(code) * scale, in every layout."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import tfp8_oracle as O
from tests.util import assert_gate, max_rel_err

pytestmark = pytest.mark.gpu

N, K = 384, 512


def _checkpoint(layout, fmt, seed):
    """(codes as torch float8 [N, K], scale tensor in the layout, float32 multiplier [N, K/G], G)"""
    g = torch.Generator().manual_seed(seed)
    f8 = torch.float8_e4m3fn if fmt == "e4m3fn" else torch.float8_e5m2
    fmax = 448.0 if fmt == "e4m3fn" else 57344.0
    w = torch.randn(N, K, generator=g) * 0.05
    if layout == "tensor":
        scale = (w.abs().max() / fmax).reshape(())
        full, G = scale.expand(N, 1), K
    elif layout == "channel":
        scale = w.abs().amax(1) / fmax                                  # [N]
        full, G = scale[:, None], K
    elif layout == "group":
        scale = w.reshape(N, K // 128, 128).abs().amax(-1) / fmax       # [N, K/128]
        full, G = scale, 128
    else:                                                               # 128 x 128 blocks
        scale = w.reshape(N // 128, 128, K // 128, 128).abs().amax((1, 3)) / fmax
        full, G = scale.repeat_interleave(128, 0), 128
    q = (w.reshape(N, K // G, G) / full[..., None]).clamp(-fmax, fmax).reshape(N, K).to(f8)
    return q, scale.contiguous(), full.contiguous().float(), G


@pytest.mark.parametrize("fmt", ("e4m3fn", "e5m2"))
@pytest.mark.parametrize("layout", ("tensor", "channel", "group", "block"))
def test_checkpoint_layouts_forward_on_cuda(layout, fmt):
    from tfp8 import _ext
    from tfp8.checkpoint import linear_from_checkpoint
    q, scale, full, G = _checkpoint(layout, fmt, seed=len(layout))
    bias = torch.randn(N, generator=torch.Generator().manual_seed(1))
    layer = linear_from_checkpoint(q.cuda(), scale.cuda(), bias.cuda(), fmt, block=(128, 128) if layout == "block" else None,
                                   out_dtype=torch.float16)
    assert layer.qweight.is_cuda and layer.group_size == G
    assert torch.equal(layer.qweight.cpu(), q.view(torch.uint8))          # codes adopted verbatim
    assert torch.equal(layer.weight_scale.cpu(), full)                    # the multiplier, bit for bit
    for M in (1, 8, 40, 300):
        x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).half()
        y = layer(x.cuda())
        ref = O.linear_forward_f64(x.double().numpy(), q.view(torch.uint8).numpy(), full.numpy(), bias.numpy(), fmt, G)
        if G != K and M > 8:
            # K-group scales that are not powers of two reach the tile GEMM folded into the decoded
            # fp16 weights (scale / rowmax, one extra fp16 rounding): the reference's own bound for
            # that case is 5e-4 of the row maximum (tests/test_tfp8.py:206 there)
            err = np.abs(y.double().cpu().numpy() - ref)
            assert err.max() <= 5e-4 * np.abs(ref).max() + float(O.gate_tolerance(ref, "f16").max()), f"{layout} {fmt} M={M}"
        else:
            assert_gate(y, ref, torch.float16, f"{layout} {fmt} M={M}")
        assert max_rel_err(y, ref) <= 2e-3
    assert layer.stats["gemv"] == 2 and layer.stats["gemm"] + layer.stats["chunked"] == 2 and layer.stats["torch"] == 0
    assert _ext.device_status() == 0


def test_state_dict_and_safetensors_onto_cuda(tmp_path):
    """A small model whose checkpoint mixes layouts and names (`weight_scale_inv`, `weight_scale`),
    loaded straight onto the GPU from a state dict and from a safetensors file."""
    from safetensors.torch import save_file
    from tfp8 import FP8Linear, _ext
    from tfp8.checkpoint import load_fp8_state_dict, load_safetensors

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(K, N, bias=True)
            self.b = nn.Linear(N, 256, bias=False)
            self.norm = nn.LayerNorm(256)

        def forward(self, x):
            return self.norm(self.b(torch.relu(self.a(x))).float())

    qa, sa, fa, Ga = _checkpoint("block", "e4m3fn", 7)
    g = torch.Generator().manual_seed(8)
    wb = torch.randn(256, N, generator=g) * 0.05
    sb = wb.abs().amax(1) / 448.0
    qb = (wb / sb[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    tensors = {"a.weight": qa, "a.weight_scale_inv": sa, "a.bias": torch.randn(N, generator=g),
               "b.weight": qb, "b.weight_scale": sb,
               "norm.weight": torch.rand(256, generator=g) + 0.5, "norm.bias": torch.randn(256, generator=g)}
    x = torch.randn(5, K, generator=g).half()
    # float64 evaluation of the checkpoint's own numbers
    h = O.linear_forward_f64(x.double().numpy(), qa.view(torch.uint8).numpy(), fa.numpy(), tensors["a.bias"].numpy(), "e4m3fn", Ga)
    h16 = np.maximum(h, 0).astype(np.float16)                              # the activation the second layer sees, as fp16
    want = O.linear_forward_f64(h16.astype(np.float64), qb.view(torch.uint8).numpy(), sb[:, None].numpy(), None, "e4m3fn", N)
    path = tmp_path / "model.safetensors"
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(path))
    for how in ("state_dict", "safetensors"):
        net = Net().half().cuda()
        if how == "state_dict":
            done = load_fp8_state_dict(net, {k: v.cuda() for k, v in tensors.items()}, block=(128, 128))
        else:
            done = load_safetensors(net, path, block=(128, 128), device="cuda")
        assert sorted(done) == ["a", "b"] and isinstance(net.a, FP8Linear) and net.a.qweight.is_cuda
        y_a = net.a(x.cuda())
        assert_gate(y_a, h, torch.float16, f"{how}: layer a")          # 5 rows: the GEMV applies group scales in float32
        hb = torch.from_numpy(h16).cuda()
        assert_gate(net.b(hb), want, torch.float16, f"{how}: layer b")
        assert net.a.stats["gemv"] == 1 and net.b.stats["gemv"] == 1
    assert _ext.device_status() == 0
