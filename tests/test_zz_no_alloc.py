"""The allocation-free entry point, tfp8b_linear_static, against the ordinary pair
tfp8b_prep + tfp8b_gemm.

Some users of the library cannot allocate device memory where they call it (a serving loop that
must not stall the device, a process with a fixed device-memory budget, a host runtime without a
CUDA allocator). For them the library keeps the GEMM's prepared activations in a fixed array of its
own. This file checks, through the C ABI and on two calls in a row that leave different contents
in that array, that the result is bit-identical to the path that uses caller-allocated buffers,
and that oversized calls are refused. It is collected last on purpose: a run that stops at the
first failure has then already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, x, q, ws, bias, y, G, fmt_id=0):
    M, K = x.shape
    N = q.shape[0]
    dt = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
    return lib.tfp8b_linear_static(x.data_ptr(), dt[x.dtype], q.data_ptr(), ws.data_ptr(),
                                   0 if ws.dtype == torch.float32 else 1,
                                   bias.data_ptr() if bias is not None else None, y.data_ptr(), dt[y.dtype],
                                   M, N, K, G, fmt_id, torch.cuda.current_stream().cuda_stream)


def test_linear_static_matches_allocating_path_twice():
    from tfp8 import FP8Linear, _ext
    lib = _ext.load()
    torch.manual_seed(21)
    layer = FP8Linear.from_linear(torch.nn.Linear(1024, 392, device="cuda", dtype=torch.float16), group_size=128)
    q, ws, bias = layer.qweight, layer.weight_scale, layer.bias_f32
    # two calls in a row, the second smaller and with another dtype: it must not see the first one's rows
    for M, xd, od in ((300, torch.bfloat16, torch.float16), (40, torch.float32, torch.bfloat16)):
        x = torch.randn(M, 1024, device="cuda", dtype=xd) * 3
        want = _ext.w8a16(x, q, None, ws, bias, od, 128, "e4m3fn")          # prep + gemm, torch-allocated buffers
        got = torch.full((M, 392), float("nan"), device="cuda", dtype=od)
        rc = _call_static(lib, x, q, ws, bias, got, 128)
        assert rc == 0, lib.tfp8b_last_error_string()
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"M={M}: {(got.float() - want.float()).abs().max().item()}"
    assert _ext.device_status() == 0


def test_linear_static_refuses_what_does_not_fit():
    from tfp8 import _ext
    lib = _ext.load()
    q = torch.zeros(64, 8192, dtype=torch.uint8, device="cuda")
    ws = torch.ones(64, 1, device="cuda")
    x = torch.zeros(600, 8192, device="cuda", dtype=torch.float16)          # 600 * 8192 > 4 Mi values
    y = torch.empty(600, 64, device="cuda", dtype=torch.float16)
    assert _call_static(lib, x, q, ws, None, y, 8192) == -2
    assert b"exceeds the built-in scratch" in lib.tfp8b_last_error_string()
    assert _call_static(lib, x[:0], q, ws, None, y[:0], 8192) == 0          # nothing to do


def test_linear_static_allocates_nothing_and_serves_its_limit():
    """What the entry point is named for: free device memory is the same before and after calls
    (torch's caching allocator is not involved either: inputs and outputs exist beforehand), and a
    call of exactly the documented maximum -- 8192 rows x 512 = 4 Mi activation values -- is served,
    here on a layer with UE8M0 scale bytes. Checked against prep + gemm bit for bit."""
    from tfp8 import FP8Linear, _ext
    lib = _ext.load()
    torch.manual_seed(22)
    M, K, N, G = 8192, 512, 256, 128
    layer = FP8Linear.from_linear(torch.nn.Linear(K, N, device="cuda", dtype=torch.bfloat16), group_size=G, scale_format="ue8m0")
    q, e8, bias = layer.qweight, layer._kernel_scale(), layer.bias_f32
    assert e8.dtype == torch.uint8
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    want = _ext.w8a16(x, q, None, e8, bias, torch.bfloat16, G, "e4m3fn")
    got = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    assert _call_static(lib, x[:8], q, e8, bias, got[:8], G) == 0      # first call on the device: the address lookup
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    reserved0 = torch.cuda.memory_reserved()
    for _ in range(3):
        got.fill_(float("nan"))
        rc = _call_static(lib, x, q, e8, bias, got, G)
        assert rc == 0, lib.tfp8b_last_error_string()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0 and torch.cuda.memory_reserved() == reserved0, (free0, free1)
    assert torch.equal(got, want)
    one_more = torch.empty(M + 1, K, device="cuda", dtype=torch.bfloat16)   # one row beyond the limit
    assert _call_static(lib, one_more, q, e8, bias, torch.empty(M + 1, N, device="cuda", dtype=torch.bfloat16), G) == -2
    assert _ext.device_status() == 0
