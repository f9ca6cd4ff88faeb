"""The W8A8 oracle on the CPU: the block quantizer (quantize_k) against its defining properties and
against torch's float8 casts, the scale packing of the block-scaled tensor-core path, and the six
format / scale cases of the reference's host test (tests/fp8_gemm_host.cpp:205-212 there) evaluated
two ways -- block by block in float32, as the reference's kernel accumulates
(fp8_gemm_kernel.cu:86-103), and as the float64 product of the dequantized operands -- which must
agree within the reference's own bound, rel. error < 1e-5."""
import numpy as np
import pytest
import torch

from oracle import tfp8_oracle as O


def _case_data(M, N, K, seed):
    """Operands of the reference's host test (tests/fp8_gemm_host.cpp:119-133): N(0,1) values whose
    magnitude changes by a power of two in [2^-4, 2^4] from one 32-wide block to the next."""
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, K)).astype(np.float32) * np.exp2(rng.integers(-4, 5, (M, K // 32))).repeat(32, 1).astype(np.float32)
    w = rng.standard_normal((N, K)).astype(np.float32) * np.exp2(rng.integers(-4, 5, (N, K // 32))).repeat(32, 1).astype(np.float32)
    return a, w, rng.standard_normal(N).astype(np.float32)


@pytest.mark.parametrize("fmt,tdt", (("e4m3fn", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)))
@pytest.mark.parametrize("ue8m0", (False, True))
def test_quantize_k_definition(fmt, tdt, ue8m0):
    fmax = O.FORMATS[fmt][4]
    x, _, _ = _case_data(16, 8, 256, 1)
    x[3, 32:64] = 0.0                                            # an all-zero block: scale floor 1e-12
    q, s = O.quantize_k(x, fmt, ue8m0)
    assert q.shape == x.shape and s.shape == (16, 8)
    sv = np.exp2(s.astype(np.float64) - 127) if ue8m0 else s.astype(np.float64)
    amax = np.abs(x.reshape(16, 8, 32)).max(-1)
    assert (sv * fmax >= amax * (1 - 1e-6)).all()                # nothing saturates
    if ue8m0:
        assert (sv <= np.maximum(2 * amax / fmax, 2e-12)).all()  # and the power of two is the next one up
        assert s[3, 1] == int(np.ceil(np.log2(1e-12))) + 127
    else:
        assert np.allclose(sv[amax > 0], amax[amax > 0] / fmax, rtol=1e-6) and np.isclose(sv[3, 1], 1e-12)
    # the codes are torch's RNE cast of x / s
    want = (torch.from_numpy(x.reshape(16, 8, 32)) / torch.from_numpy(sv.astype(np.float32))[..., None]).clamp(-fmax, fmax)
    assert np.array_equal(q, want.to(tdt).view(torch.uint8).reshape(16, 256).numpy())
    assert not q[3, 32:64].any()


def test_pack_scales_layout():
    R, KB = 300, 10                                              # 3 row tiles (the last partial), 3 k tiles (the last partial)
    s = (np.arange(R * KB) % 251).astype(np.uint8).reshape(R, KB)
    p = O.mx_pack_scales(s).reshape(3, 3, 512)
    for r, b in ((0, 0), (31, 3), (32, 0), (127, 3), (128, 4), (299, 9), (45, 6)):
        assert p[r // 128, b // 4, (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4] == s[r, b]
    assert p[2, 0, (300 % 32) * 16 + ((300 % 128) // 32) * 4] == 127        # a row beyond R
    assert p[0, 2, 0 * 16 + 0 * 4 + 2] == 127                                # a block beyond KB
    assert (p == 127).sum() == p.size - R * KB + int((s == 127).sum())


CASES = (("e4m3fn", "e4m3fn", False, False), ("e4m3fn", "e4m3fn", True, False), ("e5m2", "e5m2", False, False),
         ("e4m3fn", "e5m2", True, False), ("e4m3fn", "e4m3fn", False, True), ("e4m3fn", "e4m3fn", True, True))


@pytest.mark.parametrize("a_fmt,w_fmt,ue8m0,rowcol", CASES)
def test_reference_host_cases_blockwise_equals_dequantized_product(a_fmt, w_fmt, ue8m0, rowcol):
    M, N, K = 128, 96, 512
    a, w, bias = _case_data(M, N, K, 1234)
    if rowcol:                                                   # one scale per row / column (tests/fp8_gemm_host.cpp:137-147)
        def q_rows(x, fmt):
            fmax = O.FORMATS[fmt][4]
            s = (np.abs(x).max(1) / fmax).astype(np.float32)
            if ue8m0:
                e = np.clip(np.ceil(np.log2(s.astype(np.float64))), -127, 127)
                return O.encode((x / np.exp2(e)[:, None]).astype(np.float32), fmt), (e + 127).astype(np.uint8)
            return O.encode(x / s[:, None], fmt), s
        aq, sa = q_rows(a, a_fmt)
        wq, sw = q_rows(w, w_fmt)
    else:
        aq, sa = O.quantize_k(a, a_fmt, ue8m0)
        wq, sw = O.quantize_k(w, w_fmt, ue8m0)
    ref = O.w8a8_forward_f64(aq, sa, a_fmt, wq, sw, w_fmt, bias, ue8m0, rowcol)
    # the kernel's order of operations in float32: per-block partial products, scaled, summed
    A, W = O.decode(aq, a_fmt).astype(np.float32), O.decode(wq, w_fmt).astype(np.float32)
    f = (lambda s: np.exp2(s.astype(np.float32) - 127)) if ue8m0 else (lambda s: s.astype(np.float32))
    if rowcol:
        y = (A @ W.T) * f(sa)[:, None] * f(sw)[None, :] + bias
    else:
        y = np.zeros((M, N), np.float32)
        for b in range(K // 32):
            part = A[:, 32 * b:32 * b + 32] @ W[:, 32 * b:32 * b + 32].T
            y += part * (f(sa)[:, b][:, None] * f(sw)[:, b][None, :])
        y += bias
    assert np.abs(y - ref).max() / np.abs(ref).max() < 1e-5
    truth = a.astype(np.float64) @ w.astype(np.float64).T + bias
    assert np.abs(ref - truth).max() / np.abs(truth).max() < 0.15  # FP8 quantization error, for scale
