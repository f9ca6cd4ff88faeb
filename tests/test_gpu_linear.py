"""Parity of the decode GEMV and the tcgen05 tile GEMM, through FP8Linear and through the
operator layer, against the numpy oracle. The cases are the reference project's own GPU gates
(tests/test_tfp8.py:75-275, 363-370 there): switch points and tails, ragged K, group scales x
formats x output types, per-block scales, pipeline edges, folded scales, the cached launch,
empty / non-contiguous inputs and the NaN fallback."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import tfp8_oracle as O
from tests.util import assert_gate, max_rel_err, oracle_reference

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _status_clean():
    from tfp8 import _ext
    _ext.load()
    yield
    assert _ext.device_status() == 0          # no kernel ever gave up on a bounded wait


def _layer(N, K, G=None, fmt="e4m3fn", bias=True, seed=0, **kw):
    from tfp8 import FP8Linear
    torch.manual_seed(seed)
    lin = nn.Linear(K, N, bias=bias, device="cuda")
    return FP8Linear.from_linear(lin, fmt=fmt, group_size=G, **kw)


def _check(M, N, K, G, out_dtype, backend="fused", fmt="e4m3fn", bias=True, x_dtype=torch.bfloat16, **kw):
    f = _layer(N, K, G, fmt, bias, seed=M * 7 + N, large_m_backend=backend, **kw)
    f.out_dtype = out_dtype
    x = torch.randn(M, K, device="cuda", dtype=x_dtype)
    y = f(x)
    assert y.dtype == out_dtype and y.shape == (M, N)
    # The GEMV consumes x in its own type; the tile GEMM sees the prepared (fp16 * 2^e) activation.
    ref = oracle_reference(x, f, prepared=M > 8)
    assert_gate(y, ref, out_dtype, f"M={M} N={N} K={K} G={G} {fmt} {out_dtype} {x_dtype}")
    assert max_rel_err(y, ref) <= 2e-3 if out_dtype != torch.bfloat16 else True
    return f


def test_switch_points_and_tails():
    for M in (1, 2, 3, 7, 8, 9, 15, 16, 31, 32, 127, 128, 255, 256, 300):
        f = _check(M, 200, 512, None, torch.float16)              # N=200: tail tile
        assert f.stats["gemv" if M <= 8 else "gemm"] == 1
    for M in (256, 300):
        f = _check(M, 200, 512, None, torch.float16, backend="chunked")
        assert f.stats["chunked"] == 1


def test_ragged_k_tail():
    for K in (528 + 16, 1056, 1152, 1184, 2080):                   # multiples of 32, not of 64 / 1024
        for M in (1, 8, 16, 64):
            _check(M, 200, K, None, torch.float16)


def test_group_scales_formats_dtypes():
    for G in (None, 32, 128):
        for fmt in ("e4m3fn", "e5m2"):
            for od in (torch.float16, torch.bfloat16, torch.float32):
                for M in (1, 40):
                    _check(M, 128, 1024, G, od, fmt=fmt, bias=(G != 32))


def test_input_dtypes_and_ue8m0():
    for xd in (torch.float16, torch.bfloat16, torch.float32):
        for G in (None, 32, 64, 128):
            for M in (1, 5, 8, 24):
                _check(M, 136, 2048, G, torch.float32, x_dtype=xd)
                if G:
                    _check(M, 136, 2048, G, torch.float16, x_dtype=xd, scale_format="ue8m0")


def test_group_scale_applied_per_block():
    K, N = 256, 64
    from tfp8 import FP8Linear
    torch.manual_seed(1)
    lin = nn.Linear(K, N, bias=False, device="cuda")
    with torch.no_grad():
        lin.weight[:, :128] *= 1000.0
    f = FP8Linear.from_linear(lin, group_size=128)
    f.out_dtype = torch.float16
    for M in (4, 33):
        x = torch.randn(M, K, device="cuda") * 1e-3
        ref = oracle_reference(x, f, prepared=False)
        assert max_rel_err(f(x), ref) < 2e-3


def test_gemm_pipeline_edges():
    for K in (32, 64, 96, 160):
        for G in (None, 32):
            for M in (9, 64, 65, 130):
                _check(M, 72, K, G, torch.float16, bias=(G is None))


def test_gemm_many_stages_and_tiles():
    _check(300, 392, 4096, 128, torch.float16)                      # ring reuse, 2 M-tiles, 4 N-tiles
    _check(520, 264, 1024, None, torch.bfloat16)
    _check(64, 1000, 8192, 32, torch.float32)


def test_gemm_scatter_window_and_destinations():
    """The scatter form of the tile GEMM (the fused all-gather of a column-parallel layer): the N
    columns land in a column window of wider outputs, in several buffers at once, bit-identical
    to the plain call, and nothing outside the window is touched."""
    from tfp8 import _ext
    for (M, N, K, G, dt) in ((40, 256, 512, None, torch.float16), (300, 136, 1024, 128, torch.bfloat16)):
        f = _layer(N, K, G, seed=M)
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        x16, xs = _ext.prepare_activations(x)
        want = _ext.gemm_prepared(x16, xs, f.qweight, None, f.weight_scale, f.bias_f32, dt, f.group_size, f.fmt)
        ldy, col0 = 3 * N + 8, N + 8
        bufs = [torch.full((M, ldy), 7.0, dtype=dt, device="cuda") for _ in range(3)]
        _ext.gemm_scatter(x16, xs, f.qweight, f.weight_scale, f.bias_f32, [b.data_ptr() for b in bufs], ldy, col0, dt,
                          f.group_size, f.fmt)
        for b in bufs:
            assert torch.equal(b[:, col0:col0 + N], want)
            assert bool((b[:, :col0] == 7.0).all()) and bool((b[:, col0 + N:] == 7.0).all())
    with pytest.raises(RuntimeError):                               # window wider than the row pitch
        _ext.gemm_scatter(x16, xs, f.qweight, f.weight_scale, f.bias_f32, [bufs[0].data_ptr()], N, 8, dt, f.group_size, f.fmt)


def test_split_k_matches_whole_k():
    """Few rows against few, long weight tiles: the library splits K across SMs (partial tiles meet
    in FP32 atomics). Same gates as every GEMM case, and within float32 rounding of the whole-K
    result; with the environment switch semantics checked through the C entry point: no
    workspace, no split, bit-identical to tfp8b_gemm."""
    from tfp8 import _ext
    for (M, N, K, G) in ((16, 2048, 8192, 128), (64, 4096, 4096, None), (40, 1024, 16384, 32)):
        f = _check(M, N, K, G, torch.float16)                          # FP8Linear routes through the split-K entry
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        x16, xs = _ext.prepare_activations(x)
        y_split = torch.empty(M, N, dtype=torch.float32, device="cuda")
        y_whole = torch.empty(M, N, dtype=torch.float32, device="cuda")
        ws = torch.empty(M * N, dtype=torch.float32, device="cuda")
        lib, st = _ext.load(), torch.cuda.current_stream().cuda_stream
        args = (x16.data_ptr(), xs.data_ptr(), f.qweight.data_ptr(), f.weight_scale.data_ptr(), 0, f.bias_f32.data_ptr())
        tail = (2, M, N, K, f.group_size, 0)
        assert lib.tfp8b_gemm_splitk(*args, y_split.data_ptr(), *tail, ws.data_ptr(), ws.numel(), st) == 0
        assert lib.tfp8b_gemm(*args, y_whole.data_ptr(), *tail, st) == 0
        assert torch.allclose(y_split, y_whole, rtol=2e-5, atol=2e-5 * float(y_whole.abs().max()))
        y_none = torch.empty_like(y_whole)
        assert lib.tfp8b_gemm_splitk(*args, y_none.data_ptr(), *tail, None, 0, st) == 0
        assert torch.equal(y_none, y_whole)


def test_split_k_by_spans_full_width():
    """28672 weight rows are 224 tiles for 148 SMs: with a workspace the library deals the k-blocks
    of all tiles out in equal spans (a tile may get its sum from two CTAs). Against the whole-K
    kernel on the same inputs: within float32 rounding; the same bits on every run (two addends
    commute); a ragged last tile and M that is no multiple of 16 included."""
    from tfp8 import _ext
    lib, st = _ext.load(), torch.cuda.current_stream().cuda_stream
    torch.manual_seed(11)
    K, G = 8192, 128
    for (M, N) in ((16, 28672), (40, 28600), (64, 28672)):
        codes = torch.randint(0, 256, (N, K), dtype=torch.uint8, device="cuda")
        codes[(codes & 0x7F) == 0x7F] = 0x30                           # no NaN codes
        e8 = torch.randint(110, 122, (N, K // G), dtype=torch.uint8, device="cuda")
        bias = torch.randn(N, device="cuda")
        x = torch.randn(M, K, device="cuda", dtype=torch.float16)
        x16, xs = _ext.prepare_activations(x)
        ws = torch.empty(M * N, dtype=torch.float32, device="cuda")
        args = (x16.data_ptr(), xs.data_ptr(), codes.data_ptr(), e8.data_ptr(), 1, bias.data_ptr())
        tail = (2, M, N, K, G, 0)
        outs = [torch.empty(M, N, dtype=torch.float32, device="cuda") for _ in range(3)]
        assert lib.tfp8b_gemm(*args, outs[0].data_ptr(), *tail, st) == 0
        for y in outs[1:]:
            ws.fill_(float("nan"))                                      # the library clears what it uses
            assert lib.tfp8b_gemm_splitk(*args, y.data_ptr(), *tail, ws.data_ptr(), ws.numel(), st) == 0
        torch.cuda.synchronize()
        assert _ext.device_status() == 0
        assert torch.allclose(outs[1], outs[0], rtol=2e-5, atol=2e-5 * float(outs[0].abs().max()))
        assert torch.equal(outs[1], outs[2])


def test_folded_group_scales():
    """Random codes, scales spanning 2^-20: power-of-two scales must stay at FP32-accumulation
    error, arbitrary scales within one fp16 rounding of the folded weight."""
    from tfp8 import FP8Linear
    torch.manual_seed(5)
    N, K, G = 96, 1024, 128
    for fmt, dt in (("e4m3fn", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)):
        for pow2 in (True, False):
            codes = torch.randint(0, 256, (N, K), dtype=torch.uint8, device="cuda")
            codes[~torch.isfinite(codes.view(dt).float())] = 0x10
            ws = torch.exp2(torch.randint(-20, 1, (N, K // G), device="cuda").float()) * 1e-2
            if not pow2:
                ws = ws * (1 + torch.rand(N, K // G, device="cuda"))
            f = FP8Linear.from_fp8_checkpoint(codes, ws, bias=torch.randn(N, device="cuda"), fmt=fmt)
            f.out_dtype = torch.float32
            for M in (1, 8, 16, 100):
                x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
                err = max_rel_err(f(x), oracle_reference(x, f))
                lim = 1e-5 if (pow2 or M <= 8) else 5e-4
                assert err < lim, f"{fmt} pow2={pow2} M={M}: err/max {err}"


def test_special_codes_propagate():
    """NaN and inf codes decode to NaN / inf inside the kernels (bf16 and fp16 decode paths)."""
    from tfp8 import FP8Linear
    for fmt, special in (("e4m3fn", 0x7F), ("e5m2", 0x7C), ("e5m2", 0x7E)):
        codes = torch.full((32, 256), 0x38, dtype=torch.uint8, device="cuda")
        codes[3, 17] = special
        f = FP8Linear.from_fp8_checkpoint(codes, torch.ones(32, device="cuda"), fmt=fmt, nan_check=False)
        for M, xd in ((2, torch.float16), (2, torch.bfloat16), (2, torch.float32), (20, torch.bfloat16)):
            y = f(torch.ones(M, 256, device="cuda", dtype=xd)).float()
            assert not torch.isfinite(y[:, 3]).any(), (fmt, special, M, xd)
            rest = torch.cat([y[:, :3], y[:, 4:]], 1)
            assert torch.isfinite(rest).all()


def test_cached_launch_tracks_layer_state():
    from tfp8 import FP8Linear, _ext
    torch.manual_seed(11)
    f = FP8Linear.from_linear(nn.Linear(512, 200, device="cuda"), group_size=128)
    f.nan_check = False

    def general(x):
        return _ext.w8a16(x.reshape(-1, 512), f.qweight, f._lut_for(), f.weight_scale, f.bias_f32,
                          f.out_dtype, f.group_size, f.fmt)

    for xd in (torch.float16, torch.bfloat16, torch.float32):
        for M in (1, 3, 8):
            x = torch.randn(M, 512, device="cuda", dtype=xd)
            y = f(x)
            assert torch.equal(y, general(x)), (xd, M)
            ref = oracle_reference(x, f, prepared=False)
            assert (np.abs(y.double().cpu().numpy() - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-4 * np.abs(ref).max()).all()
    assert len(f._gemv) == 3
    x = torch.randn(2, 3, 512, device="cuda", dtype=torch.bfloat16)          # N-d input, M = 6
    assert torch.equal(f(x), general(x).reshape(2, 3, 200))
    x = torch.randn(4, 512, device="cuda", dtype=torch.bfloat16)
    f.out_dtype = torch.float16
    assert f(x).dtype == torch.float16 and torch.equal(f(x), general(x))
    other = FP8Linear.from_linear(nn.Linear(512, 200, device="cuda"), group_size=128)
    f.qweight = other.qweight.clone()                                       # replaced buffer objects
    f.weight_scale = other.weight_scale.clone()
    assert torch.equal(f(x), general(x))
    f.load_state_dict(other.state_dict())                                   # in-place copy_
    assert torch.equal(f(x), general(x))
    f.cpu()
    assert f(x.cpu()).device.type == "cpu"
    f.cuda()
    y = f(x)
    assert torch.equal(y, general(x)) and f.stats["gemv"] >= 12


def test_ue8m0_scale_cache_follows_in_place_updates():
    from tfp8 import FP8Linear
    f = FP8Linear.from_linear(nn.Linear(512, 64, device="cuda"), group_size=32, scale_format="ue8m0", nan_check=False)
    x = torch.randn(2, 512, device="cuda", dtype=torch.float16)
    y0 = f(x)
    f.weight_scale.mul_(4.0)
    assert torch.allclose(f(x).float(), 4 * y0.float() - 3 * f.bias_f32.half().float(), rtol=2e-3, atol=1e-3)


def test_empty_and_noncontiguous():
    from tfp8 import FP8Linear
    f = FP8Linear.from_linear(nn.Linear(512, 128, device="cuda"))
    assert f(torch.empty(0, 512, device="cuda")).shape == (0, 128)
    x = torch.randn(512, 20, device="cuda").t()
    assert torch.allclose(f(x).float(), f(x.contiguous()).float())
    assert f(torch.randn(2, 3, 512, device="cuda")).shape == (2, 3, 128)


def test_nan_fallback():
    from tfp8 import FP8Linear
    f = FP8Linear.from_linear(nn.Linear(512, 128, device="cuda"))
    f.out_dtype = torch.float16
    f.weight_scale.fill_(1e30)
    f(torch.randn(4, 512, device="cuda"))
    assert f.fallback is not None and "non-finite" in f.fallback_reason


def test_unsupported_shapes_are_reported():
    from tfp8 import _ext
    q = torch.zeros(16, 48, dtype=torch.uint8, device="cuda")
    s = torch.ones(16, 1, device="cuda")
    with pytest.raises(NotImplementedError):
        _ext.w8a16(torch.zeros(1, 48, device="cuda", dtype=torch.float16), q, None, s, None, torch.float16, 48)
    with pytest.raises(ValueError):
        _ext.w8a16(torch.zeros(1, 48, dtype=torch.float16), q, None, s, None, torch.float16, 48)


def test_config1_golden(golden_c1):
    """The CPU-runnable reference configuration at full size: 4096x4096 outlier weight, per-channel power-of-two scales,
    x 1x4096 fp16: codes and scales bit-exact with the reference, output within fp16 rounding."""
    import hashlib
    from tfp8 import FP8Linear, synth
    w = synth.outlier_weight(4096, 4096, seed=0)
    assert hashlib.sha256(w.numpy().tobytes()).hexdigest() == str(golden_c1["w_sha256"])
    lin = nn.Linear(4096, 4096, bias=False, dtype=torch.float16, device="cuda")
    lin.weight.data.copy_(w)
    f = FP8Linear.from_linear(lin)
    assert hashlib.sha256(f.qweight.cpu().numpy().tobytes()).hexdigest() == str(golden_c1["q_sha256"])
    assert np.array_equal(f.weight_scale.cpu().numpy().view(np.uint32), golden_c1["scale"])
    x = torch.from_numpy(golden_c1["x"].view(np.float16).copy()).cuda()
    y = f(x).float().cpu().numpy()
    want = golden_c1["y"].view(np.float16).astype(np.float32)
    assert np.abs(y - want).max() <= 2.0 ** -10 * np.abs(want).max()
    assert f.stats["gemv"] == 1
