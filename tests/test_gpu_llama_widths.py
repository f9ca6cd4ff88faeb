"""The decoder harness at Llama-3-8B layer WIDTHS (d_model 4096, FFN 14336, 32 query / 8 KV heads;
two blocks and a cut-down vocabulary so that it fits a test) against an independent evaluation of
the same weights: every FP8Linear evaluated on CPU tensors in float32 -- the defining expression
of the reference, `F.linear(x.float(), dequantize_weight(q, s), bias)` (tfp8/linear.py:179-181
there) -- with plain torch attention, teacher-forced on the tokens the GPU run produced.

On the GPU side the prompt goes through the tile GEMM (split-K included at batch 1) and the
decode steps are replayed from a CUDA graph: batch 1 takes the GEMVs that compute their own
activations (residual + RMSNorm in front of QKV and gate/up, SwiGLU in front of down), batch 4
the norm form plus the separate SwiGLU helper, batch 8 the plain helpers and the M = 8 GEMVs.
Reported and gated per batch size, as the reference's demo does for its own integration check
(tfp8/examples/demo_llm.py:178-185 there): cosine, relative L2 and top-1 agreement of the logits.
"""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

PROMPT, STEPS = 24, 8


def _cpu_twin(model):
    """The same weights on the CPU, float32 everywhere, FP8Linear on its torch path."""
    from tfp8.linear import FP8Linear
    twin = copy.deepcopy(model).to("cpu").float()
    for m in twin.modules():
        if isinstance(m, FP8Linear):
            m.out_dtype = torch.float32
            m._gemv.clear()
    return twin


@pytest.fixture(scope="module")
def models():
    from tfp8 import FP8Config
    from tfp8.examples.llama import LlamaConfig, build_fp8_llama
    cfg = LlamaConfig(n_layers=2, d_model=4096, n_heads=32, n_kv_heads=8, ffn=14336, vocab=4096, max_seq=64)
    model = build_fp8_llama(cfg, torch.device("cuda"), torch.float16, fp8=FP8Config(profile="llm_safe", nan_check=False), seed=5)
    return cfg, model, _cpu_twin(model)


@pytest.mark.parametrize("batch", (1, 4, 8))
def test_decode_logits_match_cpu_evaluation(models, batch):
    from tfp8 import _ext
    from tfp8.examples.llama import DecodeRunner
    cfg, model, twin = models
    g = torch.Generator().manual_seed(batch)
    prompt = torch.randint(0, cfg.vocab, (batch, PROMPT), generator=g)
    for l in model.layers:
        for lin in (l.qkv_proj, l.o_proj, l.gate_up_proj, l.down_proj):
            for k in lin.stats:
                lin.stats[k] = 0
    run = DecodeRunner(model, batch)
    got = [run.prefill(prompt.cuda()).float().cpu()]                  # logits of position PROMPT - 1
    first = run.tok.clone().cpu()
    run.capture()
    step_logits = []
    toks = run.decode(STEPS, keep_logits=step_logits).cpu()             # replayed from the graph
    got += [l.float().cpu() for l in step_logits]
    got = torch.cat(got, dim=1)                                       # [B, 1 + STEPS, vocab]
    st = model.layers[0].qkv_proj.stats
    assert st["gemm"] + st["chunked"] >= 1 and st["gemv"] >= 1       # prompt through the GEMM, steps through the GEMV
    assert _ext.device_status() == 0

    # teacher-forced CPU evaluation of the very tokens the GPU fed itself
    seq = torch.cat([prompt, first, toks[:, :-1]], dim=1)             # PROMPT + STEPS tokens
    ref_run = DecodeRunner(twin, batch)
    with torch.no_grad():
        ref = twin(seq, torch.arange(seq.shape[1]), prefill=True)[:, PROMPT - 1:].float()
    del ref_run
    assert ref.shape == got.shape
    cos = torch.nn.functional.cosine_similarity(got, ref, dim=-1)
    rel = (got - ref).norm(dim=-1) / ref.norm(dim=-1)
    top_ref = ref.argmax(-1)
    agree = (got.argmax(-1) == top_ref).float().mean().item()
    # where the choice differs the two candidates must be a near-tie in the reference
    pick = ref.gather(-1, got.argmax(-1, keepdim=True))[..., 0]
    slack = (ref.max(-1).values - pick) / ref.abs().max(-1).values
    print(f"batch {batch}: cosine min {cos.min():.6f}, rel L2 max {rel.max():.2e}, top-1 agreement {agree:.3f}, "
          f"worst pick slack {slack.max():.2e}")
    assert cos.min() >= 0.9995, f"cosine {cos.min()}"
    assert rel.max() <= 3e-2, f"relative L2 {rel.max()}"
    assert agree >= 0.75 and slack.max() <= 2e-2, f"top-1 agreement {agree}, slack {slack.max()}"
    # the tokens the GPU chose are the argmax of its own logits (the argmax kernel in the graph)
    assert torch.equal(torch.cat([first, toks], dim=1), got.argmax(-1))
