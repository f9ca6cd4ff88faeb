"""The FP8 KV cache on CPU tensors: the serving harness's torch path (quantize on write, decode
on read) against the numpy oracle's definition, and the config switch that selects it."""
import numpy as np
import torch

from oracle import tfp8_oracle as O


def test_kv_quantize_is_row_quantization():
    rng = np.random.default_rng(3)
    rows = (rng.standard_normal((5, 2, 7, 128)) * np.exp2(rng.integers(-12, 6, (5, 2, 7, 1)))).astype(np.float32)
    rows[0, 0, 0] = 0.0                                                   # an all-zero row: scale 1, codes 0
    for fmt in ("e4m3fn", "e5m2"):
        q, s = O.kv_quantize(rows, fmt)
        assert q.shape == rows.shape and s.shape == rows.shape[:3] and q.dtype == np.uint8
        assert s[0, 0, 0] == 1.0 and not q[0, 0, 0].any()
        assert np.all(np.exp2(np.round(np.log2(s))) == s)                   # powers of two
        back = O.decode(q, fmt) * s[..., None]
        fmax = 448.0 if fmt == "e4m3fn" else 57344.0
        amax = np.abs(rows).max(-1)
        assert np.all(amax <= s * fmax) and np.all((amax > s * fmax / 2) | (amax == 0))   # the smallest such power of two
        step = 2.0 ** (-3 if fmt == "e4m3fn" else -2)
        assert np.all(np.abs(back - rows) <= np.abs(rows) * step / 2 + s[..., None] * 2.0 ** -9 * (1 if fmt == "e4m3fn" else 2.0 ** -8) + 1e-30)


def test_harness_fp8_cache_matches_oracle_attention():
    from tfp8 import FP8Config
    from tfp8.examples.llama import LlamaConfig, build_fp8_llama
    cfg = LlamaConfig(vocab=128, d_model=512, n_layers=1, n_heads=4, n_kv_heads=2, ffn=512, max_seq=24)
    assert cfg.head_dim == 128
    model = build_fp8_llama(cfg, "cpu", torch.float32, FP8Config(nan_check=False, min_features=128, kv_cache="fp8"), seed=2)
    assert model.kv_fmt == "e4m3fn"
    model.alloc_cache(2)
    blk = model.layers[0]
    assert blk.k_cache.dtype == torch.uint8 and blk.k_scale.shape == (2, 2, 24)
    tok = torch.randint(0, 128, (2, 9), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        model(tok, torch.arange(9), prefill=True)
    # what the cache holds is the row quantization of what an unquantized cache would hold
    ref = build_fp8_llama(cfg, "cpu", torch.float32, FP8Config(nan_check=False, min_features=128), seed=2)
    ref.alloc_cache(2)
    with torch.no_grad():
        ref(tok[:, :1], torch.arange(1), prefill=True)                        # position 0 sees no quantized history
    q0, s0 = O.kv_quantize(ref.layers[0].k_cache[:, :, :1].numpy())
    assert np.array_equal(q0, blk.k_cache[:, :, :1].numpy()) and np.array_equal(s0, blk.k_scale[:, :, :1].numpy())
    # one decode step through the masked torch path equals the oracle's attention over the codes
    with torch.no_grad():
        h = blk.input_layernorm(model.embed(tok[:, :1]))
        qkv = blk.qkv_proj(h).view(2, 1, 8, 128).transpose(1, 2)
    qh = qkv[:, :4, 0].float()                                                # un-rotated is fine: any query will do
    want = O.attn_decode_fp8_f64(qh.numpy(), blk.k_cache.numpy(), blk.k_scale.numpy(), blk.v_cache.numpy(),
                                 blk.v_scale.numpy(), 9)
    kd, vd = blk._kv_dense(9, torch.float32)
    got = torch.nn.functional.scaled_dot_product_attention(qh[:, :, None], kd, vd, enable_gqa=True)[:, :, 0]
    assert np.allclose(got.numpy(), want, rtol=1e-4, atol=1e-5)
