"""Bit-exact parity of the CUDA codecs (encoder, decoder, one-pass quantizer, dequantizer,
activation prep) against fixtures recorded from the reference and against the numpy oracle.
Everything goes through the C ABI (tfp8._ext is a ctypes binding of libtfp8b.so)."""
import numpy as np
import pytest
import torch

from oracle import tfp8_oracle as O
from tests.util import f32_bits, same_bits_or_nan, t_f32

pytestmark = pytest.mark.gpu
FMTS = ("e4m3fn", "e5m2")
TORCH_FP8 = {"e4m3fn": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


@pytest.fixture(scope="module")
def ext():
    from tfp8 import _ext
    _ext.load()
    return _ext


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16, torch.float32))
def test_decode_all_256_codes(ext, golden, fmt, dtype):
    codes = torch.arange(256, dtype=torch.uint8, device="cuda")
    got = ext.decode_codes(codes, fmt, dtype)
    want = t_f32(golden[f"decode32_{fmt}"])
    assert same_bits_or_nan(got, want)
    if dtype == torch.float32:                                                # NaN codes keep their sign
        assert np.array_equal(got.cpu().numpy().view(np.uint32) >> 31, golden[f"decode32_{fmt}"] >> 31)
    assert same_bits_or_nan(got, codes.view(TORCH_FP8[fmt]).float())          # torch.float8_* agrees
    # unaligned / ragged length: the scalar tail path
    rag = torch.arange(256, dtype=torch.uint8, device="cuda").repeat(3)[5:5 + 613]
    assert same_bits_or_nan(ext.decode_codes(rag.clone(), fmt, dtype), want[rag.long()])


@pytest.mark.parametrize("fmt", FMTS)
def test_encode_matches_reference_encoders(ext, golden, fmt):
    x = t_f32(golden[f"enc_x_{fmt}"])
    assert np.array_equal(ext.encode(x, fmt).cpu().numpy(), golden[f"enc_cast_{fmt}"])
    assert np.array_equal(ext.encode(x, fmt, canonical_nan=True).cpu().numpy(), golden[f"enc_formats_{fmt}"])
    big = ext.decode_codes(ext.encode(torch.tensor([1e9, -1e9], device="cuda"), fmt), fmt, torch.float32)
    assert big.tolist() == [O.FORMATS[fmt][4], -O.FORMATS[fmt][4]]            # saturate, never inf


@pytest.mark.parametrize("fmt", FMTS)
def test_encode_exhaustive_16bit_inputs(ext, golden, fmt):
    bits = torch.arange(65536, dtype=torch.int32, device="cuda").to(torch.int16)
    assert np.array_equal(ext.encode(bits.view(torch.float16), fmt).cpu().numpy(), golden[f"enc_all_f16_{fmt}"])
    assert np.array_equal(ext.encode(bits.view(torch.bfloat16), fmt).cpu().numpy(), golden[f"enc_all_bf16_{fmt}"])
    assert np.array_equal(ext.encode(bits.view(torch.float16), fmt, canonical_nan=True).cpu().numpy(),
                          golden[f"enc_all_f16_formats_{fmt}"])


@pytest.mark.parametrize("fmt", FMTS)
def test_encode_random_float32_bit_patterns(ext, fmt):
    """2 Mi random float32 bit patterns (every exponent, NaNs, infs, subnormals) against the oracle,
    and against torch's own clamp-then-cast on the GPU."""
    g = torch.Generator(device="cpu").manual_seed(3)
    bits = torch.randint(-2 ** 31, 2 ** 31 - 1, (1 << 21,), generator=g, dtype=torch.int64).to(torch.int32)
    x = bits.view(torch.float32).cuda()
    got = ext.encode(x, fmt).cpu().numpy()
    assert np.array_equal(got, O.encode(x.cpu().numpy(), fmt, "cast"))
    fmax = O.FORMATS[fmt][4]
    assert np.array_equal(got, x.clamp(-fmax, fmax).to(TORCH_FP8[fmt]).view(torch.uint8).cpu().numpy())
    # empty and odd lengths
    assert ext.encode(x[:0], fmt).numel() == 0
    assert np.array_equal(ext.encode(x[3:1000].clone(), fmt).cpu().numpy(), got[3:1000])


@pytest.mark.parametrize("fmt", FMTS)
def test_encode_float32_rounding_boundaries(ext, fmt):
    """Every midpoint between neighbouring codes (a tie: exact in float32), the float32 values one
    and two ulps either side of it, and the neighbourhoods of every code value, zero, the largest
    finite value and the smallest subnormal, in both signs: where a double rounding or a wrong
    tie rule would show. Checked against the oracle for both NaN conventions."""
    table = O.decode_table(fmt).astype(np.float64)
    pos = np.sort(table[:128][np.isfinite(table[:128])])
    pts = np.concatenate([pos, (pos[:-1] + pos[1:]) / 2, [pos[1] / 2, pos[1] / 4, pos[-1] * 1.03125, pos[-1] * 2]])
    centre = pts.astype(np.float32).view(np.int32).astype(np.int64)
    near = (centre[:, None] + np.arange(-3, 4)[None, :]).clip(0, 0x7F7FFFFF).reshape(-1)
    bits = np.concatenate([near, near | 0x80000000, [0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00000, 0x7F800001]])
    x = bits.astype(np.uint32).view(np.float32)
    x = np.concatenate([x, x[:7]])                    # a ragged tail after the 16-wide body
    xt = torch.from_numpy(x.copy()).cuda()
    for canonical, conv in ((False, "cast"), (True, "canonical")):
        got = ext.encode(xt, fmt, canonical_nan=canonical).cpu().numpy()
        assert np.array_equal(got, O.encode(x, fmt, conv))


def test_round_trip_all_codes(ext, golden_c1):
    for fmt in FMTS:
        codes = torch.arange(256, dtype=torch.uint8, device="cuda")
        rt = ext.encode(ext.decode_codes(codes, fmt, torch.float32), fmt)
        assert np.array_equal(rt.cpu().numpy(), golden_c1[f"roundtrip_{fmt}"])


def test_quantize_matches_reference(ext, golden):
    dts = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}
    for key in golden["qw_cases"]:
        ci, fmt, G, pow2 = key.split("_")
        w = t_f32(golden[f"qw_w_{ci}"]).to(dts[str(golden[f"qw_dtype_{ci}"])])
        q, s, Gr = ext.quantize_weight_cuda(w, fmt, int(G) or None, bool(int(pow2)))
        assert np.array_equal(s.cpu().numpy().view(np.uint32), golden[f"qw_s_{key}"]), key
        assert np.array_equal(q.cpu().numpy(), golden[f"qw_q_{key}"]), key
        if int(pow2):
            q8, s8, _ = ext.quantize_weight_cuda(w, fmt, int(G) or None, True, ue8m0=True)
            assert torch.equal(q8, q)
            assert np.array_equal(O.ue8m0_decode(s8.cpu().numpy()), s.cpu().numpy()), key


@pytest.mark.parametrize("G", (None, 32, 128))
def test_quantize_large_against_oracle(ext, G):
    from tfp8 import synth
    w = synth.outlier_weight(512, 2048, seed=5)
    q, s, Gr = ext.quantize_weight_cuda(w.cuda(), "e4m3fn", G)
    oq, os_, _ = O.quantize_weight(w.float().numpy(), "e4m3fn", G)
    assert np.array_equal(s.cpu().numpy(), os_) and np.array_equal(q.cpu().numpy(), oq)
    # quantize -> dequantize -> quantize -> dequantize reproduces the same values (the second
    # pass may pick a smaller power-of-two scale when a group's largest code is below half range,
    # so the codes may shift by an exponent step, but every value is representable exactly)
    deq = torch.empty(512, 2048, dtype=torch.float32, device="cuda")
    ext.dequant_into(deq, q, None, s, Gr, "e4m3fn")
    assert np.array_equal(deq.cpu().numpy(), O.dequantize_weight(oq, os_, "e4m3fn", Gr))
    q2, s2, _ = ext.quantize_weight_cuda(deq, "e4m3fn", G)
    deq2 = torch.empty_like(deq)
    ext.dequant_into(deq2, q2, None, s2, Gr, "e4m3fn")
    assert torch.equal(deq2, deq)
    # half a quantization step at most: |w - deq| <= s * 2^(e-3) / 2 <= s * 16 for E4M3FN
    err = (w.float().cuda() - deq).abs().reshape(512, -1, Gr)
    assert bool((err <= s.unsqueeze(-1) * 16.0).all())


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("dtype", (torch.float16, torch.float32))
def test_dequant_against_oracle(ext, fmt, dtype):
    g = torch.Generator().manual_seed(9)
    q = torch.randint(0, 256, (40, 512), generator=g, dtype=torch.uint8)
    s = torch.exp2(torch.randint(-12, 3, (40, 4), generator=g).float())
    out = torch.empty(40, 512, dtype=dtype, device="cuda")
    ext.dequant_into(out, q.cuda(), None, s.cuda(), 128, fmt)
    want = torch.from_numpy(O.dequantize_weight(q.numpy(), s.numpy(), fmt, 128)).to(dtype)
    assert same_bits_or_nan(out, want)
    e8 = torch.from_numpy(O.ue8m0_encode(s.numpy()))
    ext.dequant_into(out, q.cuda(), None, e8.cuda(), 128, fmt)
    assert same_bits_or_nan(out, want)


@pytest.mark.parametrize("name", ("bf16", "f32"))
def test_prep_matches_reference(ext, golden, name):
    x = t_f32(golden[f"act_x_{name}"])
    if name == "bf16":
        x = x.bfloat16()
    x16, xs = ext.prepare_activations(x)
    assert np.array_equal(xs.cpu().numpy().view(np.uint32), golden[f"act_xs_{name}"])
    assert same_bits_or_nan(x16, torch.from_numpy(golden[f"act_x16_{name}"].view(np.float16).copy()))


def test_prep_row_amax_is_row_wide(ext):
    """An outlier anywhere in the row decides the scale (reference: tests/test_tfp8.py:210-222)."""
    torch.manual_seed(0)
    x = torch.randn(4, 4096, device="cuda", dtype=torch.bfloat16)
    x[0, 1] = 3e4
    x[1, 4095] = -5e4
    x[2, 300] = 1e5
    x16, xs = ext.prepare_activations(x)
    o16, oxs = O.activation_to_fp16(x.float().cpu().numpy())
    assert torch.isfinite(x16).all()
    assert np.array_equal(xs.cpu().numpy(), oxs)
    assert np.array_equal(x16.cpu().numpy(), o16)
    assert torch.all(torch.log2(xs) == torch.round(torch.log2(xs)))
    assert torch.equal(x16[3].float() * xs[3], x[3].float())          # no outlier in the row: bf16 -> fp16 is lossless


def test_epilogue_window(ext):
    acc = torch.randn(37, 24, device="cuda")
    xs = torch.exp2(torch.randint(-3, 4, (37,), device="cuda").float())
    bias = torch.randn(100, device="cuda")
    for dt in (torch.float16, torch.bfloat16, torch.float32):
        y = torch.zeros(37, 100, dtype=dt, device="cuda")
        ext.epilogue_into(y, acc, xs, bias, 40)
        want = (acc * xs[:, None] + bias[40:64]).to(dt)
        assert torch.equal(y[:, 40:64], want) and not y[:, :40].any() and not y[:, 64:].any()
