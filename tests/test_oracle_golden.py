"""The numpy oracle against fixtures produced by the reference's own code (CPU only).

Every gate mirrors one of the reference's CPU gates (tests/test_tfp8.py:29-72 in the reference
project) or a bit-exactness check of its benchmarks, but reads recorded outputs instead of
importing the reference."""
import math

import numpy as np
import pytest

from oracle import tfp8_oracle as O

FMTS = ("e4m3fn", "e5m2")


def f32(bits):
    return np.asarray(bits, np.uint32).view(np.float32)


def same_floats(a, b):
    """Bitwise equality of float arrays with NaN == NaN and signed zeros kept apart."""
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    both_nan = np.isnan(a) & np.isnan(b)
    return bool(np.all(both_nan | ((a == b) & (np.signbit(a) == np.signbit(b)))))


@pytest.mark.parametrize("fmt", FMTS)
def test_decode_table_matches_reference_and_torch(golden, fmt):
    t = O.decode_table(fmt)
    assert same_floats(t, f32(golden[f"decode32_{fmt}"]))
    assert same_floats(t, f32(golden[f"torchview32_{fmt}"]))
    lut = O.lut16_bits(fmt)
    ref_lut = golden[f"lut16_{fmt}"]
    nan = np.isnan(lut.view(np.float16))
    assert np.array_equal(nan, np.isnan(ref_lut.view(np.float16)))
    assert np.array_equal(lut[~nan], ref_lut[~nan])
    shipped = golden[f"shipped_lut16_{fmt}"]            # lut_<fmt>.bin of the reference
    assert np.array_equal(lut[~nan], shipped[~nan])
    assert np.array_equal(np.isnan(shipped.view(np.float16)), nan)


def test_special_values():
    d = lambda c, f: float(O.decode(np.array([c], np.uint8), f)[0])
    assert d(0x00, "e4m3fn") == 0.0 and not math.copysign(1, d(0x00, "e4m3fn")) < 0
    assert d(0x80, "e4m3fn") == 0.0 and math.copysign(1, d(0x80, "e4m3fn")) < 0
    assert d(0x7E, "e4m3fn") == 448.0
    assert d(0x01, "e4m3fn") == 2.0 ** -9
    assert math.isnan(d(0x7F, "e4m3fn")) and math.isnan(d(0xFF, "e4m3fn"))
    assert d(0x7B, "e5m2") == 57344.0
    assert d(0x7C, "e5m2") == math.inf and d(0xFC, "e5m2") == -math.inf
    assert d(0x01, "e5m2") == 2.0 ** -16
    assert math.isnan(d(0x7D, "e5m2"))


@pytest.mark.parametrize("fmt", FMTS)
def test_encode_matches_both_reference_encoders(golden, fmt):
    x = f32(golden[f"enc_x_{fmt}"])
    assert np.array_equal(O.encode(x, fmt, "canonical"), golden[f"enc_formats_{fmt}"])
    assert np.array_equal(O.encode(x, fmt, "cast"), golden[f"enc_cast_{fmt}"])
    # for finite in-range inputs the raw torch cast agrees too (tests/test_tfp8.py:48-55)
    n = int(golden[f"enc_n_random_{fmt}"])
    assert np.array_equal(O.encode(x[:n], fmt), golden[f"enc_rawcast_{fmt}"][:n])
    big = O.decode(O.encode(np.array([1e9, -1e9], np.float32), fmt), fmt)
    assert big.tolist() == [O.FORMATS[fmt][4], -O.FORMATS[fmt][4]]


@pytest.mark.parametrize("fmt", FMTS)
def test_encode_exhaustive_16bit_inputs(golden, fmt):
    h = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    assert np.array_equal(O.encode(h, fmt, "cast"), golden[f"enc_all_f16_{fmt}"])
    assert np.array_equal(O.encode(h, fmt, "canonical"), golden[f"enc_all_f16_formats_{fmt}"])
    b = O.bf16_bits_to_f32(np.arange(65536, dtype=np.uint16))
    assert np.array_equal(O.encode(b, fmt, "cast"), golden[f"enc_all_bf16_{fmt}"])


def test_round_trip_all_codes(golden_c1):
    for fmt in FMTS:
        rt = O.encode(O.decode_table(fmt), fmt, "cast")
        assert np.array_equal(rt, golden_c1[f"roundtrip_{fmt}"])
    assert np.array_equal(O.encode(O.decode_table("e4m3fn"), "e4m3fn"), np.arange(256, dtype=np.uint8))


def test_quantize_and_dequantize_match_reference(golden):
    for key in golden["qw_cases"]:
        ci, fmt, G, pow2 = key.split("_")
        w = f32(golden[f"qw_w_{ci}"])
        q, s, Gr = O.quantize_weight(w, fmt, int(G) or None, bool(int(pow2)))
        assert np.array_equal(s.view(np.uint32), golden[f"qw_s_{key}"]), key
        assert np.array_equal(q, golden[f"qw_q_{key}"]), key
        if f"qw_deq_{key}" in golden:
            assert same_floats(O.dequantize_weight(q, s, fmt, Gr), f32(golden[f"qw_deq_{key}"])), key


def test_ue8m0_round_trip():
    e = np.arange(-126, 128)
    s = np.ldexp(np.float32(1), e).astype(np.float32)
    b = O.ue8m0_encode(s)
    assert np.array_equal(b, (e + 127).astype(np.uint8))
    assert np.array_equal(O.ue8m0_decode(b), s)
    assert np.isnan(O.ue8m0_decode(np.array([255], np.uint8))[0])
    assert O.ue8m0_encode(np.array([3.0], np.float32))[0] == 129      # ceil(log2 3) = 2


@pytest.mark.parametrize("name", ("bf16", "f32", "f16"))
def test_activation_row_scale(golden, name):
    x = f32(golden[f"act_x_{name}"])
    x16, xs = O.activation_to_fp16(x, is_fp16=(name == "f16"))
    assert np.array_equal(xs.view(np.uint32), golden[f"act_xs_{name}"])
    ref16 = golden[f"act_x16_{name}"].view(np.float16)
    assert same_floats(x16.astype(np.float32), ref16.astype(np.float32))
    fin = np.isfinite(xs) & (xs > 0)
    assert np.all(np.log2(xs[fin]) == np.round(np.log2(xs[fin])))      # exact powers of two


def test_cpu_forward_matches_reference(golden):
    for case in golden["fwd_cases"]:
        ci, M, N, K, G, fmt, od, has_bias = case.split("|")
        K, G = int(K), int(G)
        x = O.bf16_bits_to_f32(golden[f"fwd_x_{ci}"])
        q, s = golden[f"fwd_q_{ci}"], f32(golden[f"fwd_s_{ci}"])
        b = f32(golden[f"fwd_b_{ci}"]) if int(has_bias) else None
        od = {"float16": "f16", "bfloat16": "bf16", "float32": "f32"}[od]
        y = O.linear_forward(x, q, s, b, fmt, G or K, od)
        ref = f32(golden[f"fwd_y_{ci}"])
        # same float32 arithmetic, different summation order inside the BLAS call
        eps = {"f16": 2.0 ** -10, "bf16": 2.0 ** -7, "f32": 2.0 ** -20}[od]
        assert np.all(np.abs(y - ref) <= eps * np.abs(ref) + 1e-5 * np.abs(ref).max()), case


# ------------------------------------------------------------------ C restatement and the reference's fp8.h
def test_c_port_matches_numpy_oracle(golden):
    from oracle import c_port
    for fmt in FMTS:
        assert same_floats(c_port.decode_table(fmt), O.decode_table(fmt))
        x = f32(golden[f"enc_x_{fmt}"])
        assert np.array_equal(c_port.encode(x, fmt, "cast"), golden[f"enc_cast_{fmt}"])
        assert np.array_equal(c_port.encode(x, fmt, "canonical"), golden[f"enc_formats_{fmt}"])
    rng = np.random.default_rng(0)
    q = rng.integers(0, 256, (96, 512), dtype=np.uint8)
    q[np.isnan(O.decode_table("e4m3fn")[q])] = 0x10
    s = np.exp2(rng.integers(-10, 2, (96, 4))).astype(np.float32)
    x = rng.standard_normal((5, 512)).astype(np.float32)
    b = rng.standard_normal(96).astype(np.float32)
    y = c_port.linear_forward(x, q, s, b, "e4m3fn", 128)
    ref = O.linear_forward_f64(x.astype(np.float64), q, s, b, "e4m3fn", 128)
    assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max()


def test_reference_fp8_header_agrees():
    """The reference's own C++ header (compiled where the checkout exists) against the oracle:
    its LUT, its decode and its encoder on every finite code value, midpoint and saturation case."""
    from oracle import c_port
    ref = c_port.load_ref()
    if ref is None:
        pytest.skip("oracle/_ref was not built (no reference checkout at build time)")
    for fi, fmt in enumerate(FMTS):
        lut = np.empty(256, np.uint16)
        ref.ref_fp8_build_lut(fi, lut.ctypes.data_as(__import__("ctypes").c_void_p))
        mine = O.lut16_bits(fmt)
        nan = np.isnan(mine.view(np.float16))
        assert np.array_equal(lut[~nan], mine[~nan]) and np.all(np.isnan(lut.view(np.float16)[nan]))
        table = O.decode_table(fmt)
        for c in range(256):
            v = ref.ref_fp8_decode(c, fi)
            assert (np.isnan(v) and np.isnan(table[c])) or (v == table[c] and np.signbit(v) == np.signbit(table[c]))
        pos = table[:128][np.isfinite(table[:128])].astype(np.float64)
        pts = np.concatenate([pos, (pos[:-1] + pos[1:]) / 2, [1e9, O.FORMATS[fmt][4] * 1.5, np.inf]]).astype(np.float32)
        pts = np.concatenate([pts, -pts])
        want = O.encode(pts, fmt, "cast")
        got = np.array([ref.ref_fp8_encode(float(p), fi) for p in pts], np.uint8)
        assert np.array_equal(got, want)
