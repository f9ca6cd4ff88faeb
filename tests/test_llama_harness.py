"""The serving harness on CPU with a tiny configuration: a decode step through the static KV cache
must reproduce what a longer prefill computes for the same position (cache write, RoPE at the
device-side position and the additive mask are what a CUDA-graph decode loop relies on)."""
import torch

from tfp8 import FP8Config
from tfp8.examples.llama import TINY, DecodeRunner, build_fp8_llama
from tfp8.linear import FP8Linear


def test_decode_step_matches_prefill():
    torch.manual_seed(0)
    model = build_fp8_llama(TINY, "cpu", dtype=torch.float32, fp8=FP8Config(min_features=64, nan_check=False))
    assert sum(isinstance(m, FP8Linear) for m in model.modules()) == 4 * TINY.n_layers
    assert isinstance(model.lm_head, torch.nn.Linear)
    toks = torch.randint(0, TINY.vocab, (2, 9))
    full = DecodeRunner(model, 2).prefill(toks)                      # logits of the last position (8)
    run = DecodeRunner(model, 2)
    run.prefill(toks[:, :8])
    run.tok.copy_(toks[:, 8:9])                                      # feed the true 9th token
    logits = model(run.tok, run.pos, prefill=False)
    assert full.shape == (2, 1, TINY.vocab)
    assert torch.allclose(logits[:, 0], full[:, 0], rtol=1e-3, atol=1e-3)          # fp16 projection outputs
    out = run.decode(3)
    assert out.shape == (2, 3) and int(run.pos) == 8 + 3


def test_decode_step_matches_prefill_with_fp8_kv_cache():
    """The same invariant with `FP8Config(kv_cache="fp8")`: a prefill attends over the quantized K and V
    it has just cached, so a decode step over the cache sees the very same values; and the cache holds
    codes and power-of-two scales."""
    torch.manual_seed(0)
    model = build_fp8_llama(TINY, "cpu", dtype=torch.float32, fp8=FP8Config(min_features=64, nan_check=False, kv_cache="fp8"))
    assert model.kv_fmt == "e4m3fn"
    toks = torch.randint(0, TINY.vocab, (2, 9))
    full = DecodeRunner(model, 2).prefill(toks)
    run = DecodeRunner(model, 2)
    run.prefill(toks[:, :8])
    blk = model.layers[0]
    assert blk.k_cache.dtype == torch.uint8 and blk.v_cache.dtype == torch.uint8
    assert bool((torch.log2(blk.k_scale) == torch.log2(blk.k_scale).round()).all())
    assert not bool(blk.k_cache[:, :, 8:].any()) and bool(blk.k_cache[:, :, :8].any())      # exactly the prompt's positions are written
    run.tok.copy_(toks[:, 8:9])
    logits = model(run.tok, run.pos, prefill=False)
    assert torch.allclose(logits[:, 0], full[:, 0], rtol=1e-3, atol=1e-3)
    # and it is a different function from the 16-bit cache: the quantization is really in the path
    ref = build_fp8_llama(TINY, "cpu", dtype=torch.float32, fp8=FP8Config(min_features=64, nan_check=False))
    ref.load_state_dict(model.state_dict())
    full16 = DecodeRunner(ref, 2).prefill(toks)
    assert not torch.equal(full16, full) and torch.nn.functional.cosine_similarity(full16[:, 0], full[:, 0], dim=-1).min() > 0.98


def test_runner_refuses_to_run_past_the_kv_cache():
    """The cache position lives on the device; the runner's host-side count must stop a prefill, a
    capture or a decode that would write beyond max_seq before any kernel sees such a position."""
    import pytest
    torch.manual_seed(1)
    model = build_fp8_llama(TINY, "cpu", dtype=torch.float32, fp8=FP8Config(min_features=64, nan_check=False))
    run = DecodeRunner(model, 1)
    with pytest.raises(ValueError, match="exceed the KV cache"):
        run.prefill(torch.randint(0, TINY.vocab, (1, TINY.max_seq + 1)))
    run.prefill(torch.randint(0, TINY.vocab, (1, TINY.max_seq - 2)))
    run.decode(2)                                                   # fills the cache exactly
    assert int(run.pos) == TINY.max_seq == run.host_pos
    with pytest.raises(ValueError, match="exceed the KV cache"):
        run.decode(1)
    assert int(run.pos) == TINY.max_seq                             # nothing ran
