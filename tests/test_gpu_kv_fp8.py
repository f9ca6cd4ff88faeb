"""FP8 KV cache on the GPU: the fused rotary + quantizing cache write against the 16-bit cache
write followed by the library's (and the oracle's) row quantizer -- bit for bit --, the attention
over the codes against the oracle's float64 definition, and the serving harness with
`FP8Config(kv_cache="fp8")` against an independent CPU evaluation of the same model."""
import copy

import numpy as np
import pytest
import torch

from oracle import tfp8_oracle as O

pytestmark = pytest.mark.gpu

HD = 128


def _tables(S, dev):
    inv = 1.0 / (10000.0 ** (torch.arange(0, HD, 2, device=dev).float() / HD))
    ang = torch.arange(S, device=dev).float()[:, None] * inv[None, :]
    return ang.cos().contiguous(), ang.sin().contiguous()


@pytest.mark.parametrize("dt", (torch.float16, torch.bfloat16))
@pytest.mark.parametrize("fmt", ("e4m3fn", "e5m2"))
def test_store_equals_16bit_store_then_row_quantizer(dt, fmt):
    from tfp8 import _ext
    dev = torch.device("cuda")
    torch.manual_seed(7)
    B, T, H, KV, S = 2, 5, 8, 2, 40
    qkv = (torch.randn(B, T, (H + 2 * KV) * HD, device=dev) * torch.exp2(torch.randint(-10, 4, (B, T, 1), device=dev).float())).to(dt)
    qkv[1, 2, (H + 1) * HD:(H + 2) * HD] = 0                                  # an all-zero K row: scale 1, codes 0
    pos = torch.tensor([3, 4, 9, 30, 39], device=dev)
    cos, sin = _tables(S, dev)
    k16 = torch.zeros(B, KV, S, HD, device=dev, dtype=dt)
    v16 = torch.zeros_like(k16)
    q16 = _ext.rope_kv_store(qkv, pos, cos, sin, k16, v16, H, KV)
    kc = torch.full((B, KV, S, HD), 0xAA, device=dev, dtype=torch.uint8)
    vc = torch.full_like(kc, 0xAA)
    ks = torch.full((B, KV, S), -1.0, device=dev)
    vs = torch.full_like(ks, -1.0)
    q8 = _ext.rope_kv_store_fp8(qkv, pos, cos, sin, kc, ks, vc, vs, H, KV, fmt)
    torch.cuda.synchronize()
    assert _ext.device_status() == 0
    assert torch.equal(q8, q16)
    untouched = torch.ones(S, dtype=torch.bool, device=dev)
    untouched[pos] = False
    assert bool((kc[:, :, untouched] == 0xAA).all()) and bool((ks[:, :, untouched] == -1.0).all())
    assert bool((vc[:, :, untouched] == 0xAA).all()) and bool((vs[:, :, untouched] == -1.0).all())
    for c16, codes, scale in ((k16, kc, ks), (v16, vc, vs)):
        rows = c16[:, :, pos].float().cpu().numpy()
        want_q, want_s = O.kv_quantize(rows, fmt)
        assert np.array_equal(codes[:, :, pos].cpu().numpy(), want_q)
        assert np.array_equal(scale[:, :, pos].cpu().numpy(), want_s)
        lib_q, lib_s, _ = _ext.quantize_weight_cuda(c16[:, :, pos].reshape(-1, HD).contiguous(), fmt, HD, True)
        assert torch.equal(lib_q.view(B, KV, T, HD), codes[:, :, pos]) and torch.equal(lib_s.view(B, KV, T), scale[:, :, pos])
    assert float(ks[1, 1, 9]) == 1.0 and not bool((kc[1, 1, 9] & 0x7F).any())   # +-0 (the rotation turns some zeros into -0)


def test_store_refuses_other_head_dims():
    from tfp8 import _ext
    dev = torch.device("cuda")
    B, T, S = 1, 1, 8
    qkv = torch.randn(B, T, 12 * 64, device=dev).half()                       # 8 + 2 + 2 heads of 64
    cos, sin = _tables(S, dev)
    kc = torch.zeros(B, 2, S, 64, device=dev, dtype=torch.uint8)
    ks = torch.ones(B, 2, S, device=dev)
    with pytest.raises(NotImplementedError):
        _ext.rope_kv_store_fp8(qkv, torch.tensor([0], device=dev), cos, sin, kc, ks, kc.clone(), ks.clone(), 8, 2)


@pytest.mark.parametrize("dt", (torch.float16, torch.bfloat16))
@pytest.mark.parametrize("fmt", ("e4m3fn", "e5m2"))
def test_attention_over_codes_matches_oracle(dt, fmt):
    from tfp8 import _ext
    dev = torch.device("cuda")
    torch.manual_seed(11)
    B, H, KV, S = 3, 8, 2, 300
    k = torch.randn(B, KV, S, HD) * torch.exp2(torch.randint(-3, 3, (B, KV, S, 1)).float())
    v = torch.randn(B, KV, S, HD) * torch.exp2(torch.randint(-6, 2, (B, KV, S, 1)).float())
    kq, ksc = O.kv_quantize(k.numpy(), fmt)
    vq, vsc = O.kv_quantize(v.numpy(), fmt)
    kc, ks = torch.from_numpy(kq).to(dev), torch.from_numpy(ksc).to(dev)
    vc, vs = torch.from_numpy(vq).to(dev), torch.from_numpy(vsc).to(dev)
    q = (torch.randn(B, H, HD) * 0.5).to(dt)
    scratch = torch.empty(_ext.attn_scratch_floats(B, H, S, HD), dtype=torch.float32, device=dev)
    eps = 2.0 ** -11 if dt == torch.float16 else 2.0 ** -8
    for p in (0, 1, 63, 64, 65, 127, 128, 299):
        pos = torch.tensor([p], device=dev)
        got = _ext.attn_decode_fp8(q.to(dev), kc, ks, vc, vs, pos, scratch, fmt).float().cpu().numpy()
        want = O.attn_decode_fp8_f64(q.float().numpy(), kq, ksc, vq, vsc, p + 1, fmt)
        tol = eps * np.abs(want) + 1e-4 * np.abs(want).max() + 1e-6           # the reference's gate form, tests/test_tfp8.py:87-88
        assert np.all(np.abs(got - want) <= tol), f"pos {p}: worst {np.abs(got - want).max()} of {np.abs(want).max()}"
        # and the 16-bit kernel on the decoded cache gives the same result up to summation order
        kd = (torch.from_numpy(O.decode(kq, fmt)) * torch.from_numpy(ksc)[..., None])
        vd = (torch.from_numpy(O.decode(vq, fmt)) * torch.from_numpy(vsc)[..., None])
        if dt == torch.float16:                                               # every decoded value is exact in fp16 here
            same = _ext.attn_decode(q.to(dev), kd.to(dev, dt), vd.to(dev, dt), pos, scratch).float().cpu().numpy()
            assert np.all(np.abs(got - same) <= 2 * eps * np.abs(want) + 1e-5 * np.abs(want).max())
    assert _ext.device_status() == 0


@pytest.mark.parametrize("batch", (1, 4))
def test_harness_with_fp8_cache_matches_cpu_evaluation(batch):
    """Decoder at head_dim 128 with `kv_cache="fp8"`: prompt + graph-replayed decode steps on the
    GPU against the same model evaluated on the CPU in float32 (its cache quantized by the torch
    path, teacher-forced on the GPU's tokens)."""
    from tfp8 import FP8Config, _ext
    from tfp8.examples.llama import DecodeRunner, LlamaConfig, build_fp8_llama
    from tfp8.linear import FP8Linear
    PROMPT, STEPS = 20, 6
    cfg = LlamaConfig(n_layers=2, d_model=1024, n_heads=8, n_kv_heads=2, ffn=2048, vocab=2048, max_seq=64)
    model = build_fp8_llama(cfg, torch.device("cuda"), torch.float16, fp8=FP8Config(profile="llm_safe", nan_check=False, kv_cache="fp8"),
                            seed=9)
    assert model.kv_fmt == "e4m3fn"
    twin = copy.deepcopy(model).to("cpu").float()
    for m in twin.modules():
        if isinstance(m, FP8Linear):
            m.out_dtype = torch.float32
            m._gemv.clear()
    prompt = torch.randint(0, cfg.vocab, (batch, PROMPT), generator=torch.Generator().manual_seed(batch))
    run = DecodeRunner(model, batch)
    got = [run.prefill(prompt.cuda()).float().cpu()]
    assert model.layers[0].k_cache.dtype == torch.uint8
    first = run.tok.clone().cpu()
    run.capture()
    step_logits = []
    toks = run.decode(STEPS, keep_logits=step_logits).cpu()
    got = torch.cat(got + [l.float().cpu() for l in step_logits], dim=1)
    assert _ext.device_status() == 0
    seq = torch.cat([prompt, first, toks[:, :-1]], dim=1)
    twin.alloc_cache(batch)
    with torch.no_grad():
        ref = twin(seq, torch.arange(seq.shape[1]), prefill=True)[:, PROMPT - 1:].float()
    cos = torch.nn.functional.cosine_similarity(got, ref, dim=-1)
    rel = (got - ref).norm(dim=-1) / ref.norm(dim=-1)
    print(f"fp8 KV cache, batch {batch}: cosine min {cos.min():.6f}, rel L2 max {rel.max():.2e}")
    # The CPU twin quantizes float32 K/V, the GPU the fp16-rounded ones: a value that sits on a
    # rounding boundary may land on the neighbouring code, so the gate is the 16-bit harness's
    # (tests/test_gpu_llama_widths.py) with room for single code flips.
    assert cos.min() >= 0.999, f"cosine {cos.min()}"
    assert rel.max() <= 5e-2, f"relative L2 {rel.max()}"
    assert torch.equal(torch.cat([first, toks], dim=1), got.argmax(-1))
