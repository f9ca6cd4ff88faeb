"""The benchmark configurations at their FULL sizes. The oracle cannot multiply a 28672 x 8192 weight
in seconds, so these tests check (i) a random sample of output channels against the numpy oracle
with the reference's gate, and (ii) properties that hold at any size: a one-hot activation reads
a column of the dequantized weight back exactly, doubling the activations doubles the output
exactly, raising every UE8M0 scale byte by one doubles it too, and the decode GEMV and the tile
GEMM agree on the same rows."""
import numpy as np
import pytest
import torch

from oracle import tfp8_oracle as O
from tests.util import DT_NAME

pytestmark = pytest.mark.gpu


def _sampled_gate(y, x64, q, s, G, fmt, rows, out_dtype, what):
    """y[:, rows] against the float64 oracle on those output channels."""
    ref = O.linear_forward_f64(x64, q[rows].cpu().numpy(), s[rows].cpu().numpy(), None, fmt, G)
    tol = O.gate_tolerance(ref, DT_NAME[out_dtype])
    err = np.abs(y[:, rows].double().cpu().numpy() - ref)
    assert int((err > tol).sum()) == 0, f"{what}: worst {(err / tol).max():.2f}x of the gate"
    assert np.abs(err).max() <= 2e-3 * np.abs(ref).max(), what


@pytest.mark.parametrize("fmt", ("e4m3fn", "e5m2"))
def test_decode_sweep_full_shapes(fmt):
    """Config 2: the four Llama-7B shapes, M = 1 and 8, per-channel power-of-two scales."""
    from tfp8 import _ext, synth
    g = torch.Generator().manual_seed(11)
    for (N, K) in synth.DECODE_SHAPES:
        w = synth.gaussian_weight(N, K, seed=N + K).cuda()
        q, s, G = _ext.quantize_weight_cuda(w, fmt, None, True)
        rows = torch.randint(0, N, (48,), generator=g).cuda()
        for M in (1, 8):
            x = synth.activations(M, K, seed=M).cuda()
            y = _ext.w8a16(x, q, None, s, None, torch.float16, G, fmt)
            _sampled_gate(y, x.double().cpu().numpy(), q, s, G, fmt, rows, torch.float16, f"{fmt} {N}x{K} M={M}")
            y32 = _ext.w8a16(x, q, None, s, None, torch.float32, G, fmt)     # float32 out: no fp16 subnormals in the way
            assert torch.equal(_ext.w8a16(2 * x, q, None, s, None, torch.float32, G, fmt), 2 * y32)   # exact scaling
        # one-hot probes: y = a column of the dequantized weight, bit for bit (float32 output)
        ks = torch.randint(0, K, (8,), generator=g)
        e = torch.zeros(8, K, dtype=torch.float16, device="cuda")
        e[torch.arange(8), ks] = 1.0
        col = _ext.w8a16(e, q, None, s, None, torch.float32, G, fmt)
        want = _ext.decode_codes(q[:, ks.cuda()].contiguous(), fmt, torch.float32) * s
        assert torch.equal(col, want.t().contiguous())


@pytest.mark.parametrize("G,Ms,xdt", ((128, (16, 64, 256, 1024), torch.float16), (32, (2048, 4096, 8192), torch.bfloat16)))
def test_group_scaled_gemm_full_shape(G, Ms, xdt):
    """The group-scaled layer 28672 x 8192 E4M3FN with UE8M0 K-group scales of 128 (fp16
    activations, 16 .. 1024 rows) and of 32 (bf16 activations, 2048 .. 8192 rows), every M."""
    from tfp8 import _ext, synth
    N, K = synth.GROUP_GEMM_SHAPE
    w = synth.group_outlier_weight(N, K, group=G, seed=G).cuda()
    q, e8, _ = _ext.quantize_weight_cuda(w, "e4m3fn", G, True, ue8m0=True)
    del w
    s32 = torch.from_numpy(O.ue8m0_decode(e8.cpu().numpy())).cuda()
    g = torch.Generator().manual_seed(G)
    rows = torch.randint(0, N, (32,), generator=g).cuda()
    for M in Ms:
        x = synth.activations(M, K, seed=M, dtype=xdt).cuda()
        y = _ext.w8a16(x, q, None, e8, None, torch.float16, G, "e4m3fn")
        mrows = torch.randint(0, M, (min(M, 24),), generator=g)
        x16, xs = O.activation_to_fp16(x[mrows.cuda()].float().cpu().numpy())
        x64 = x16.astype(np.float64) * xs.astype(np.float64)[:, None]
        _sampled_gate(y[mrows.cuda()], x64, q, s32, G, "e4m3fn", rows, torch.float16, f"G={G} M={M}")
        if M == Ms[0]:
            # every scale byte + 1 = every scale doubled = the output doubled, exactly
            y1 = _ext.w8a16(x, q, None, e8, None, torch.float32, G, "e4m3fn")
            y2 = _ext.w8a16(x, q, None, e8 + 1, None, torch.float32, G, "e4m3fn")
            assert torch.equal(y2, 2 * y1)
            # eight of the rows through the decode GEMV: the other kernel, the same numbers
            # (the GEMV reads x in its own type, the GEMM the prepared fp16: one rounding apart)
            yv = _ext.w8a16(x[:8].contiguous(), q, None, e8, None, torch.float16, G, "e4m3fn")
            assert (yv.float() - y[:8].float()).abs().max() <= 2e-3 * float(y[:8].float().abs().max())
    assert _ext.device_status() == 0
