"""CPU-only gates of the host layer: formats, config validation, planner policy, the CPU tensor
path of FP8Linear, checkpoint-compatibility mode, and that the C-ABI library loads and exports
every symbol include/tfp8b.h declares. Mirrors the reference's CPU gates
(tests/test_tfp8.py:29-72, 278-319 there)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch
import torch.nn as nn

import tfp8
from tfp8 import _ext
from tfp8.formats import E4M3FN, E5M2, decode, encode, lut
from tfp8.linear import FP8Linear
from tfp8.quantize import activation_to_fp16, pow2_ceil, quantize_weight, scale_to_ue8m0, ue8m0_to_scale

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _same(a, b):
    a, b = a.float(), b.float()
    return bool(((torch.isnan(a) & torch.isnan(b)) | ((a == b) & (torch.signbit(a) == torch.signbit(b)))).all())


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "tfp8b.h")).read()
    declared = sorted(set(re.findall(r"TFP8B_API[^;(]*?\b(tfp8b_\w+)\s*\(", header)))
    assert len(declared) >= 11
    lib = ctypes.CDLL(_ext.library_path())
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/tfp8b.h but not exported"
    assert sorted(_ext._SIGNATURES) == declared           # the Python binding covers all of them
    assert _ext.load().tfp8b_version() == int(re.search(r"#define TFP8B_VERSION (\d+)", header).group(1))


def test_argument_validation_needs_no_gpu():
    lib = _ext.load()
    assert lib.tfp8b_gemv(None, 0, None, None, 0, None, None, 0, 9, 16, 64, 64, 0, None) == -2   # M > 8
    assert b"M=9" in lib.tfp8b_last_error_string()
    assert lib.tfp8b_gemv(None, 0, None, None, 0, None, None, 0, 1, 16, 64, 64, 0, None) == -1   # null pointers
    assert lib.tfp8b_encode(None, 7, None, 4, 0, 0, None) == -1
    assert lib.tfp8b_quantize(None, 0, None, None, 1, 4, 64, 64, 0, 0, None) == -1               # UE8M0 without pow2
    assert lib.tfp8b_gemm(None, None, None, None, 0, None, None, 0, 0, 16, 64, 64, 0, None) == 0  # M == 0: nothing to do


def test_formats_match_torch_and_golden(golden):
    for f in (E4M3FN, E5M2):
        codes = torch.arange(256, dtype=torch.uint8)
        ref = codes.view(f.torch_dtype).float()
        assert _same(decode(codes, f), ref) and _same(lut(f).float(), ref)
        assert np.array_equal(decode(codes, f).numpy().view(np.uint32) & 0x7F800000 != 0x7F800000,
                              golden[f"decode32_{f.name}"] & 0x7F800000 != 0x7F800000)
        x = torch.from_numpy(golden[f"enc_x_{f.name}"].view(np.float32).copy())
        assert np.array_equal(encode(x, f).numpy(), golden[f"enc_formats_{f.name}"])
    assert decode(torch.tensor([0x7E], dtype=torch.uint8), E4M3FN).item() == 448.0
    assert decode(torch.tensor([0x01], dtype=torch.uint8), E5M2).item() == 2.0 ** -16
    with pytest.raises(ValueError):
        tfp8.formats.get_format("e3m4")


def test_encode_matches_torch_rne_and_saturates():
    torch.manual_seed(0)
    for f in (E4M3FN, E5M2):
        x = torch.cat([torch.randn(20000) * f.max_finite / 8, torch.randn(2000) * 2.0 ** -10])
        assert torch.equal(encode(x, f), x.to(f.torch_dtype).view(torch.uint8)), f.name
        assert decode(encode(torch.tensor([1e9, -1e9]), f), f).tolist() == [f.max_finite, -f.max_finite]


def test_quantize_weight_cpu_matches_golden(golden):
    dts = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}
    for key in golden["qw_cases"]:
        ci, fmt, G, pow2 = key.split("_")
        w = torch.from_numpy(golden[f"qw_w_{ci}"].view(np.float32).copy()).to(dts[str(golden[f"qw_dtype_{ci}"])])
        q, s, _ = quantize_weight(w, fmt, int(G) or None, bool(int(pow2)))
        assert np.array_equal(q.numpy(), golden[f"qw_q_{key}"]), key
        assert np.array_equal(s.numpy().view(np.uint32), golden[f"qw_s_{key}"]), key
    with pytest.raises(ValueError):
        quantize_weight(torch.zeros(4, 100), group_size=32)
    s = torch.tensor([1.0, 0.75, 2.0 ** -20, 3.0])
    assert pow2_ceil(s).tolist() == [1.0, 1.0, 2.0 ** -20, 4.0]
    assert torch.equal(ue8m0_to_scale(scale_to_ue8m0(pow2_ceil(s))), pow2_ceil(s))


def test_activation_scaling_is_exact_power_of_two():
    x = (torch.randn(5, 256) * 1e3).bfloat16()
    x16, xs = activation_to_fp16(x)
    assert torch.all(torch.log2(xs) == torch.round(torch.log2(xs)))
    assert torch.equal(x16.float() * xs[:, None], x.float())


def test_cpu_reference_path(golden):
    lin = nn.Linear(256, 64)
    f = FP8Linear.from_linear(lin, group_size=128)
    x = torch.randn(3, 256)
    y = f(x)
    ref = x @ f.dequantized_weight().t() + lin.bias
    assert torch.allclose(y.float(), ref, atol=1e-2, rtol=1e-2)
    assert f.stats["torch"] == 1
    # recorded outputs of the reference's own CPU forward
    dts = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}
    for case in golden["fwd_cases"]:
        ci, M, N, K, G, fmt, od, has_bias = case.split("|")
        q = torch.from_numpy(golden[f"fwd_q_{ci}"].copy())
        s = torch.from_numpy(golden[f"fwd_s_{ci}"].view(np.float32).copy())
        b = torch.from_numpy(golden[f"fwd_b_{ci}"].view(np.float32).copy()) if int(has_bias) else None
        layer = FP8Linear.from_fp8_checkpoint(q, s, b, fmt=fmt, out_dtype=dts[od])
        assert layer.group_size == (int(G) or int(K))
        x = torch.from_numpy(golden[f"fwd_x_{ci}"].view(np.int16).copy()).view(torch.bfloat16)
        y = layer(x).float()
        ref = torch.from_numpy(golden[f"fwd_y_{ci}"].view(np.float32).copy())
        assert torch.allclose(y, ref, rtol=2.0 ** -7 if od == "bfloat16" else 2.0 ** -10, atol=1e-5 * ref.abs().max().item())


def test_planner_policy_and_tied_weights():
    class Block(nn.Module):
        def __init__(s):
            super().__init__()
            s.q_proj, s.o_proj = nn.Linear(1024, 1024), nn.Linear(1024, 1024)
            s.gate_proj = nn.Linear(1024, 2048)
            s.input_layernorm = nn.LayerNorm(1024)
            s.lora_A = nn.Linear(1024, 8)
            s.router = nn.Linear(1024, 1024)
            s.odd_proj = nn.Linear(1040 - 8, 1024)      # K % 32 != 0

    class LM(nn.Module):
        def __init__(s):
            super().__init__()
            s.embed = nn.Embedding(100, 1024)
            s.layers = nn.ModuleList([Block()])
            s.lm_head = nn.Linear(1024, 100, bias=False)
            s.lm_head.weight = s.embed.weight

    m = tfp8.prepare_model(LM(), "llm", tfp8.FP8Config(profile="llm_safe"))
    owners = {d.name: d.owner for d in m._tfp8_plan}
    assert owners["layers.0.q_proj"] == "tfp8" and owners["layers.0.gate_proj"] == "tfp8"
    assert owners["layers.0.lora_A"] != "tfp8" and owners["layers.0.router"] != "tfp8"
    assert owners["layers.0.odd_proj"] != "tfp8" and owners["lm_head"] != "tfp8"
    assert m.lm_head.weight is m.embed.weight
    assert isinstance(m.layers[0].q_proj, FP8Linear) and isinstance(m.layers[0].router, nn.Linear)
    again = tfp8.prepare_model(m, "llm", tfp8.FP8Config())
    assert {d.name: d.owner for d in again._tfp8_plan}["layers.0.q_proj"] == "tfp8"
    assert isinstance(again.layers[0].q_proj, FP8Linear)
    text = tfp8.report(m, file=open(os.devnull, "w"))
    assert "3/" in text.splitlines()[-1]
    by = tfp8.weight_bytes(m)
    assert by["uint8"] == 1024 * 1024 * 2 + 2048 * 1024
    skip = tfp8.prepare_model(LM(), "llm", tfp8.FP8Config(extra_skip=[r"o_proj"]))
    assert isinstance(skip.layers[0].o_proj, nn.Linear)


def test_config_validation():
    with pytest.raises(ValueError):
        tfp8.FP8Config(profile="anything")
    with pytest.raises(NotImplementedError):
        tfp8.FP8Config(activation="fp8")
    assert tfp8.FP8Config(kv_cache="fp8").kv_cache == "fp8"           # the serving harness's FP8 KV cache
    with pytest.raises(NotImplementedError):
        tfp8.FP8Config(kv_cache="int4")
    with pytest.raises(ValueError):
        tfp8.FP8Config(large_m_backend="x")
    with pytest.raises(ValueError):
        tfp8.FP8Config(scale_format="ue8m0", pow2_scale=False)
    assert tfp8.FP8Config().min_features == 1024 and tfp8.FP8Config(profile="image_safe").min_features == 256


def test_checkpoint_compat_mode_keeps_codes():
    q = torch.randint(0, 256, (64, 128), dtype=torch.uint8)
    q[E4M3FN.is_nan(q.int())] = 0
    s = torch.rand(64) + 0.5
    f = FP8Linear.from_fp8_checkpoint(q.view(torch.float8_e4m3fn), s, fmt="e4m3fn")
    assert torch.equal(f.qweight, q) and torch.equal(f.weight_scale[:, 0], s)
    with pytest.raises(ValueError):
        FP8Linear.from_fp8_checkpoint(q.view(torch.float8_e4m3fn), s, fmt="e5m2")
    g = FP8Linear.from_fp8_checkpoint(q, torch.tensor(0.5))
    assert g.weight_scale.shape == (64, 1) and g.group_size == 128
    sd = f.state_dict()
    assert set(sd) == {"qweight", "weight_scale"}


def test_operators_refuse_cpu_tensors():
    with pytest.raises(ValueError):
        _ext.prepare_activations(torch.zeros(2, 64))
    with pytest.raises(ValueError):
        _ext.encode(torch.zeros(4))


def test_ue8m0_needs_exact_powers_of_two():
    """UE8M0 bytes can only stand for powers of two: anything else must be refused, not rounded,
    or the kernels would use other scales than the float32 buffer (and the CPU path) holds."""
    import pytest
    from tfp8 import FP8Linear
    from tfp8.quantize import scale_to_ue8m0, ue8m0_to_scale
    s = torch.tensor([[2.0 ** -13, 1.0, 2.0 ** 20, 2.0 ** -127, 2.0 ** 127]])
    assert torch.equal(ue8m0_to_scale(scale_to_ue8m0(s)), s)
    for bad in (3.0, 0.0, -2.0, float("inf"), float("nan"), 2.0 ** -130):
        with pytest.raises(ValueError, match="not powers of two"):
            scale_to_ue8m0(torch.tensor([[1.0, bad]]))
    assert scale_to_ue8m0(torch.tensor([3.0]), strict=False).item() == 129        # rounded up to 4 = 2^(129-127)
    q = torch.zeros(64, 64, dtype=torch.uint8)
    FP8Linear.from_fp8_checkpoint(q, torch.full((64, 2), 0.25), scale_format="ue8m0")
    with pytest.raises(ValueError, match="from_fp8_checkpoint"):
        FP8Linear.from_fp8_checkpoint(q, torch.full((64, 2), 0.3), scale_format="ue8m0")
    layer = FP8Linear.from_fp8_checkpoint(q, torch.full((64, 2), 0.5), scale_format="ue8m0")
    layer.weight_scale[3, 1] = 0.7                                   # a later in-place edit is caught when the bytes are re-derived
    with pytest.raises(ValueError, match="weight_scale"):
        layer._kernel_scale()


def test_plan_argument_validation_needs_no_gpu():
    lib = _ext.load()
    plan = ctypes.c_void_p(0)
    assert lib.tfp8b_gemv_plan_create(ctypes.byref(plan), 0, None, None, 0, None, 0, 9, 16, 64, 64, 0) == -1   # max_M > 8
    assert plan.value is None
    assert lib.tfp8b_gemv_plan_create(ctypes.byref(plan), 0, None, None, 0, None, 0, 8, 16, 64, 64, 0) == -1   # null codes
    assert lib.tfp8b_gemv_plan_run(None, None, None, 1, 0, None) == -1
    lib.tfp8b_gemv_plan_destroy(None)
    old = lib.tfp8b_allreduce_wait_limit(0)
    assert old > 0 and lib.tfp8b_allreduce_wait_limit(12345) == old and lib.tfp8b_allreduce_wait_limit(old) == 12345
