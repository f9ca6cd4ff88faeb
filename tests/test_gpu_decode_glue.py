"""The two fused decode-step helpers (rotary embedding + KV-cache store, silu*mul) against plain
PyTorch float32 references of the same operations, and the serving harness end to end on the GPU
(a decode step through the static cache and the FP8 kernels reproduces a longer prefill)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16))
def test_rope_kv_store_matches_torch(dtype):
    from tfp8 import _ext
    torch.manual_seed(0)
    B, T, H, KV, hd, S = 2, 5, 8, 2, 128, 40
    qkv = torch.randn(B, T, (H + 2 * KV) * hd, device="cuda").to(dtype)
    pos = torch.tensor([7, 8, 9, 20, 3], device="cuda")
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = torch.arange(S, device="cuda").float()[:, None] * inv[None]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    kc = torch.zeros(B, KV, S, hd, device="cuda", dtype=dtype)
    vc = torch.zeros_like(kc)
    q = _ext.rope_kv_store(qkv, pos, cos, sin, kc, vc, H, KV)
    x = qkv.float().view(B, T, H + 2 * KV, hd).transpose(1, 2)
    qr, kr, vr = x.split((H, KV, KV), dim=1)
    c, s = cos[pos], sin[pos]
    rot = lambda t: torch.cat([t[..., :hd // 2] * c - t[..., hd // 2:] * s, t[..., hd // 2:] * c + t[..., :hd // 2] * s], -1)
    # float32 math, one rounding to the 16-bit type (the kernel may contract a*b - c*d into an FMA)
    tol = dict(rtol=2.0 ** -9 if dtype == torch.float16 else 2.0 ** -7, atol=2e-3 if dtype == torch.float16 else 2e-2)
    assert torch.allclose(q.float(), rot(qr), **tol)
    assert torch.allclose(kc[:, :, pos].float(), rot(kr), **tol) and torch.equal(vc[:, :, pos], vr.to(dtype))
    untouched = torch.ones(S, dtype=torch.bool, device="cuda")
    untouched[pos] = False
    assert not kc[:, :, untouched].any() and not vc[:, :, untouched].any()


def test_rope_kv_store_leaves_guard_rows_untouched():
    """The caches sit inside larger buffers whose neighbouring rows hold a pattern: storing at the
    first and the last valid position must leave every guard row as it was (the store offset is
    pos * hd, so an off-by-one at either end would land in a guard row)."""
    from tfp8 import _ext
    torch.manual_seed(3)
    B, T, H, KV, hd, S = 1, 2, 4, 1, 128, 16
    qkv = torch.randn(B, T, (H + 2 * KV) * hd, device="cuda").half()
    pos = torch.tensor([0, S - 1], device="cuda")
    ang = torch.arange(S, device="cuda").float()[:, None] * torch.ones(hd // 2, device="cuda")[None]
    big_k = torch.full((S + 8, hd), 7.0, device="cuda", dtype=torch.float16)
    big_v = torch.full((S + 8, hd), 9.0, device="cuda", dtype=torch.float16)
    kc, vc = big_k[4:4 + S].view(B, KV, S, hd), big_v[4:4 + S].view(B, KV, S, hd)
    _ext.rope_kv_store(qkv, pos, ang.cos().contiguous(), ang.sin().contiguous(), kc, vc, H, KV)
    torch.cuda.synchronize()
    assert (big_k[:4] == 7).all() and (big_k[4 + S:] == 7).all() and (big_v[:4] == 9).all() and (big_v[4 + S:] == 9).all()
    assert (big_k[5:4 + S - 1] == 7).all() and (big_v[5:4 + S - 1] == 9).all()          # positions in between: untouched
    assert not (big_v[4] == 9).all() and not (big_v[4 + S - 1] == 9).all()              # the two positions were written
    assert _ext.device_status() == 0


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16))
def test_silu_mul_matches_torch(dtype):
    from tfp8 import _ext
    torch.manual_seed(1)
    gu = (torch.randn(3, 7, 2 * 1024, device="cuda") * 3).to(dtype)
    got = _ext.silu_mul(gu).float()
    g, u = gu.float()[..., :1024], gu.float()[..., 1024:]
    want = F.silu(g) * u
    tol = 2.0 ** -9 if dtype == torch.float16 else 2.0 ** -7          # one rounding of the output type (+ __expf)
    assert ((got - want).abs() <= tol * want.abs() + 1e-4).all()


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16))
@pytest.mark.parametrize("dim", (256, 4096, 11008))
def test_add_rmsnorm(dtype, dim):
    """Residual update + RMSNorm against the same arithmetic in torch: the sum rounded to the
    activation type (and stored), the norm in FP32 with one final rounding."""
    from tfp8 import _ext
    torch.manual_seed(2)
    x = torch.randn(5, 3, dim, device="cuda").to(dtype)
    d = (torch.randn(5, 3, dim, device="cuda") * 0.5).to(dtype)
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(dtype)
    want_x = (x.float() + d.float()).to(dtype)
    xf = want_x.float()
    want = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float())
    got = _ext.add_rmsnorm(x, d, w, 1e-5)
    assert torch.equal(x, want_x)                                     # in-place residual, bit for bit
    tol = 2.0 ** -9 if dtype == torch.float16 else 2.0 ** -7
    assert ((got.float() - want).abs() <= tol * want.abs() + 1e-5).all()
    # no delta: plain RMSNorm, x untouched
    keep = x.clone()
    got2 = _ext.add_rmsnorm(x, None, w, 1e-5)
    assert torch.equal(x, keep) and torch.equal(got2, got)


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16))
def test_allreduce_add_rmsnorm_single_rank(dtype):
    """The fused all-reduce + residual + RMSNorm with a group of one rank (no peers to wait for):
    the same residual as add_rmsnorm on the partial rounded to the activation type and the same
    norm within a rounding of the output type, call after call (the sequence number advances in device memory), also replayed from a CUDA graph."""
    from tfp8 import _ext
    torch.manual_seed(5)
    dim, rows = 4096, 3
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(dtype)
    recv = torch.zeros(2 * 1 * 8 * dim, dtype=torch.float32, device="cuda")
    flags = torch.zeros(2 * 1 * 8, dtype=torch.int32, device="cuda")
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    for call in range(3):
        x = torch.randn(rows, 1, dim, device="cuda").to(dtype)
        part = torch.randn(rows, 1, dim, device="cuda")
        x_ref = x.clone()
        want = _ext.add_rmsnorm(x_ref, part.to(dtype), w, 1e-5)
        got = _ext.allreduce_add_rmsnorm(x, part, w, 1e-5, [recv.data_ptr()], [flags.data_ptr()], state, 0, 8)
        assert torch.equal(x, x_ref)                                  # the residual, bit for bit
        tol = 2.0 ** -9 if dtype == torch.float16 else 2.0 ** -7        # the sum of squares is grouped differently
        assert ((got.float() - want.float()).abs() <= tol * want.float().abs() + 1e-5).all()
        assert state.tolist() == [call + 1, 0]
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        x.copy_(x_ref)                                              # restore, then capture one call
        with torch.cuda.graph(g, stream=s):
            out = _ext.allreduce_add_rmsnorm(x, part, w, 1e-5, [recv.data_ptr()], [flags.data_ptr()], state, 0, 8)
        g.replay(); g.replay()
    torch.cuda.synchronize()
    assert state.tolist() == [5, 0] and bool(torch.isfinite(out.float()).all())
    assert _ext.device_status() == 0


def test_allreduce_peer_that_never_answers_is_reported_not_summed():
    """Failure detection without a fault: a group of two is described whose second "rank" is just
    another local buffer that no kernel ever writes a flag into. With the wait limit set short the
    kernel must return by itself, raise the status bit, and hand back NaN rows (not a sum that
    silently misses the peer's part); the context stays usable and the next healthy call is right."""
    from tfp8 import _ext
    torch.manual_seed(6)
    dim, rows, world = 1024, 2, 2
    w = torch.ones(dim, device="cuda", dtype=torch.float16)
    recv = [torch.zeros(2 * world * 8 * dim, dtype=torch.float32, device="cuda") for _ in range(world)]
    flags = [torch.zeros(2 * world * 8, dtype=torch.int32, device="cuda") for _ in range(world)]
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    x = torch.randn(rows, 1, dim, device="cuda").half()
    x0 = x.clone()
    part = torch.randn(rows, 1, dim, device="cuda")
    old = _ext.allreduce_wait_limit(2_000_000)                       # about a millisecond of SM clock
    try:
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        out = _ext.allreduce_add_rmsnorm(x, part, w, 1e-5, [r.data_ptr() for r in recv], [f.data_ptr() for f in flags],
                                         state, 0, 8)
        t1.record()
        torch.cuda.synchronize()
    finally:
        _ext.allreduce_wait_limit(old)
    assert t0.elapsed_time(t1) < 500.0                               # it gave up by itself, quickly
    with pytest.raises(RuntimeError, match="peer never answered"):
        _ext.device_status()
    assert bool(torch.isnan(out.float()).all()) and bool(torch.isnan(x.float()).all())
    # what it pushed to the "peer" before waiting is there, with the flag of call 1
    assert torch.equal(recv[1].view(2, world, 8, dim)[1, 0, :rows], part.view(rows, dim))
    assert flags[1].view(2, world, 8)[1, 0, :rows].tolist() == [1] * rows
    assert _ext.device_status() == 0                                 # cleared by the read above
    # a healthy single-rank call afterwards works on the same context
    st1 = torch.zeros(2, dtype=torch.int32, device="cuda")
    x.copy_(x0)
    want = _ext.add_rmsnorm(x0.clone(), part.half(), w, 1e-5)
    got = _ext.allreduce_add_rmsnorm(x, part, w, 1e-5, [recv[0].data_ptr()], [flags[0].data_ptr()], st1, 0, 8)
    assert ((got.float() - want.float()).abs() <= 2.0 ** -9 * want.float().abs() + 1e-5).all()
    assert _ext.device_status() == 0


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16))
@pytest.mark.parametrize("G", (None, 128))
def test_gemv_with_computed_activations(dtype, G):
    """The GEMVs that build their activations inside the kernel (residual + RMSNorm; SwiGLU) against
    the unfused sequence add_rmsnorm / silu_mul -> FP8Linear on the same inputs."""
    import torch.nn as nn
    from tfp8 import FP8Linear, _ext
    torch.manual_seed(6)
    K, N = 4096, 1536
    lin = nn.Linear(K, N, bias=False, device="cuda", dtype=dtype)
    f = FP8Linear.from_linear(lin, group_size=G, nan_check=False)
    w = (1 + 0.1 * torch.randn(K, device="cuda")).to(dtype)
    for M in (1, 2, 5):
        x = torch.randn(M, 1, K, device="cuda").to(dtype)
        d = (torch.randn(M, 1, K, device="cuda") * 0.5).to(dtype)
        x_ref = x.clone()
        h = _ext.add_rmsnorm(x_ref, d, w, 1e-5)
        want = f(h).float()
        new_res, got = _ext.gemv_normed(x, d, w, 1e-5, f.qweight, f.weight_scale, None, f.out_dtype, f.group_size, f.fmt)
        assert torch.equal(new_res, x_ref)                            # the updated residual, bit for bit
        tol = 4e-3 if dtype == torch.float16 else 2e-2                 # the norm may differ by a rounding of the type
        assert (got.float() - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
        # no delta: the residual is only normalised, and not copied
        res2, got2 = _ext.gemv_normed(x_ref, None, w, 1e-5, f.qweight, f.weight_scale, None, f.out_dtype, f.group_size, f.fmt)
        assert res2 is x_ref
        assert (got2.float() - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
        gu = (torch.randn(M, 1, 2 * K, device="cuda") * 2).to(dtype)
        want_g = f(_ext.silu_mul(gu)).float()
        got_g = _ext.gemv_gated(gu, f.qweight, f.weight_scale, None, f.out_dtype, f.group_size, f.fmt).float()
        assert (got_g - want_g).abs().max() <= tol * max(1.0, float(want_g.abs().max()))
    assert _ext.device_status() == 0


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16))
def test_argmax(dtype):
    from tfp8 import _ext
    torch.manual_seed(3)
    for n in (7, 1000, 128256):
        logits = torch.randn(4, n, device="cuda").to(dtype)
        logits[1, n // 2] = 100.0
        logits[2, 3] = logits[2].max()                                # a tie: the lowest index wins
        logits[2, min(5, n - 1)] = logits[2, 3]
        out = torch.empty(4, dtype=torch.int64, device="cuda")
        _ext.argmax_into(out, logits)
        want = torch.stack([(row == row.max()).nonzero()[0, 0] for row in logits.float()])
        assert torch.equal(out, want), n
        logits[3, n - 1] = float("nan")                               # NaN counts as the largest
        _ext.argmax_into(out, logits)
        assert int(out[3]) == n - 1
        sl = logits[:, 1:]                                            # rows no longer 16-byte aligned
        _ext.argmax_into(out, sl)
        assert int(out[1]) == n // 2 - 1 or n < 3


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16))
def test_attn_decode_matches_sdpa(dtype):
    """Split-KV decode attention against torch SDPA in float32 on the same cache contents, for
    several positions (one CTA chunk, many chunks, the last cache slot) and head groupings."""
    from tfp8 import _ext
    torch.manual_seed(4)
    for (B, H, KV, S) in ((2, 8, 2, 300), (1, 32, 8, 2304), (3, 4, 4, 64)):
        q = torch.randn(B, H, 1, 128, device="cuda").to(dtype)
        k = torch.randn(B, KV, S, 128, device="cuda").to(dtype)
        v = torch.randn(B, KV, S, 128, device="cuda").to(dtype)
        for p in (0, 5, S // 2 + 3, S - 1):
            pos = torch.tensor([p], device="cuda")
            got = _ext.attn_decode(q, k, v, pos).float()
            want = F.scaled_dot_product_attention(q.float(), k[:, :, :p + 1].float(), v[:, :, :p + 1].float(),
                                                  enable_gqa=True)[:, :, 0]
            tol = 2e-3 if dtype == torch.float16 else 1.6e-2
            assert (got - want).abs().max() <= tol * max(1.0, float(want.abs().max())), (B, H, KV, S, p)


@pytest.mark.parametrize("cfg_name", ("TINY", "TINY_HD128"))
def test_harness_decode_matches_prefill_on_gpu(cfg_name):
    from tfp8 import FP8Config, _ext
    from tfp8.examples import llama
    from tfp8.examples.llama import DecodeRunner, build_fp8_llama
    TINY = getattr(llama, cfg_name)          # head_dim 32 (torch SDPA decode) and 128 (the decode attention kernel)
    torch.manual_seed(0)
    model = build_fp8_llama(TINY, torch.device("cuda"), torch.float16, fp8=FP8Config(min_features=64, nan_check=False))
    model.attn_kernel = cfg_name == "TINY_HD128"
    toks = torch.randint(0, TINY.vocab, (2, 9), device="cuda")
    full = DecodeRunner(model, 2).prefill(toks).float()
    run = DecodeRunner(model, 2)
    run.prefill(toks[:, :8])
    run.tok.copy_(toks[:, 8:9])
    logits = model(run.tok, run.pos, prefill=False).float()
    assert (logits[:, 0] - full[:, 0]).abs().max() <= 2e-2 * full.abs().max()
    run.capture()
    out = run.decode(4)
    assert out.shape == (2, 4) and int(run.pos) == 8 + 4
    assert model.layers[0].qkv_proj.stats["gemv"] > 0 and model.layers[0].qkv_proj.stats["gemm"] > 0
    assert _ext.device_status() == 0
