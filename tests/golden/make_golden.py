"""Generate the golden fixtures from the reference implementation.

Run in a container where the reference checkout is available (it is imported, never copied):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's `tfp8` package and records what its CPU code produces on seeded
inputs: decode tables, both encoders, `quantize_weight`, `dequantize_weight`,
`activation_to_fp16` and `FP8Linear.forward` on CPU tensors. The result is written next to this
script as `tfp8_golden.npz` (about 1 MB) and `config1_golden.npz`. The tests only read the
.npz files, so they run where the reference does not exist.
"""
import hashlib
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else os.path.abspath(os.path.join(HERE, "..", "..", "..", "reference"))   # sibling checkout
sys.path.insert(0, REF)

import tfp8 as ref  # noqa: E402  (the reference package)
from tfp8.formats import E4M3FN, E5M2, decode, encode, lut  # noqa: E402
from tfp8.linear import FP8Linear  # noqa: E402
from tfp8.quantize import activation_to_fp16, dequantize_weight, quantize_weight  # noqa: E402

assert os.path.realpath(ref.__file__).startswith(os.path.realpath(REF)), ref.__file__

_spec = importlib.util.spec_from_file_location(
    "_synth", os.path.join(HERE, "..", "..", "fp8-compatibility-layer_b200", "tfp8", "synth.py"))
synth = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(synth)

out = {}


def bits16(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def bits32(t):
    return t.contiguous().view(torch.int32).numpy().view(np.uint32).copy()


# ---------------------------------------------------------------- decode tables
for f in (E4M3FN, E5M2):
    codes = torch.arange(256, dtype=torch.uint8)
    out[f"lut16_{f.name}"] = bits16(lut(f))
    out[f"decode32_{f.name}"] = bits32(decode(codes, f))
    out[f"torchview32_{f.name}"] = bits32(codes.view(f.torch_dtype).float())
    shipped = np.fromfile(os.path.join(REF, f"lut_{f.name}.bin"), dtype=np.uint16)
    out[f"shipped_lut16_{f.name}"] = shipped

# ---------------------------------------------------------------- encoders
def cast_after_clamp(x, f):
    """What quantize_weight does to an already-scaled value: clamp, then torch's RNE cast."""
    return x.float().clamp(-f.max_finite, f.max_finite).to(f.torch_dtype).view(torch.uint8)


for f in (E4M3FN, E5M2):
    torch.manual_seed(0)
    x = torch.cat([torch.randn(20000) * f.max_finite / 8, torch.randn(2000) * 2.0 ** -10])
    # every finite code value, every midpoint between neighbours, and one float32 ulp either side
    pos = decode(torch.arange(128, dtype=torch.uint8), f).double()
    pos = pos[torch.isfinite(pos)]
    mids = (pos[:-1] + pos[1:]) / 2
    pts = torch.cat([pos, mids]).float()
    nudged = torch.cat([pts, torch.nextafter(pts, torch.full_like(pts, 1e30)),
                        torch.nextafter(pts, torch.full_like(pts, -1e30))])
    edge = torch.tensor([0.0, -0.0, 1e9, -1e9, f.max_finite, -f.max_finite, f.max_finite * 1.03,
                         f.max_finite * 1.0625, f.max_finite * 1.07, 3.4e38, -3.4e38, 1e-30, -1e-30,
                         2.0 ** -9, 2.0 ** -10, 2.0 ** -16, 2.0 ** -17, 2.0 ** -18,
                         float("inf"), float("-inf"), float("nan"), -float("nan")])
    allx = torch.cat([x, nudged, -nudged, edge])
    out[f"enc_x_{f.name}"] = bits32(allx)
    out[f"enc_formats_{f.name}"] = encode(allx, f).numpy()          # canonical-NaN encoder
    out[f"enc_cast_{f.name}"] = cast_after_clamp(allx, f).numpy()   # production path
    out[f"enc_rawcast_{f.name}"] = allx.to(f.torch_dtype).view(torch.uint8).numpy()
    out[f"enc_n_random_{f.name}"] = np.int64(x.numel())
    # fp16 input, exhaustive over all 65536 bit patterns
    h = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.float16)
    out[f"enc_all_f16_{f.name}"] = cast_after_clamp(h, f).numpy()
    out[f"enc_all_f16_formats_{f.name}"] = encode(h.float(), f).numpy()
    bf = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    out[f"enc_all_bf16_{f.name}"] = cast_after_clamp(bf, f).numpy()

# ---------------------------------------------------------------- quantize_weight / dequantize
def weight_case(N, K, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.02
    w[0] = 0                                   # all-zero row -> scale 1
    w[1, :] = 0
    w[1, 5] = 0.4375                           # amax = 7 * 2^-4: amax/448 is an exact power of two
    w[2, 7] = -7.0                             # amax = 7
    w[3, 9] = 7.0 * (1 + 2.0 ** -10)           # one fp16 ulp above 7
    w[4, 11] = 7.0 * (1 - 2.0 ** -11)          # one fp16 ulp below 7
    w[5, 3] = 448.0
    w[6, 0] = 1e-7                             # tiny amax in a group
    w[6, 1:] = 0
    w[7, 13] = 0.4                             # 20-sigma outlier
    return w.to(dtype)


qcases = []
for ci, (N, K, dtype) in enumerate([(24, 256, torch.float16), (24, 256, torch.bfloat16),
                                    (16, 384, torch.float32)]):
    w = weight_case(N, K, dtype, seed=100 + ci)
    out[f"qw_w_{ci}"] = bits32(w.float())
    out[f"qw_dtype_{ci}"] = np.array(str(dtype).replace("torch.", ""))
    for f in (E4M3FN, E5M2):
        for G in (None, 32, 128):
            for pow2 in (True, False):
                q, s, Gr = quantize_weight(w, f.name, G, pow2)
                key = f"{ci}_{f.name}_{G or 0}_{int(pow2)}"
                out[f"qw_q_{key}"] = q.numpy()
                out[f"qw_s_{key}"] = bits32(s)
                if ci == 0:
                    out[f"qw_deq_{key}"] = bits32(dequantize_weight(q, s, f.name, Gr))
                qcases.append(key)
out["qw_cases"] = np.array(qcases)

# ---------------------------------------------------------------- activation row scale
g = torch.Generator().manual_seed(7)
acts = {
    "bf16": (torch.randn(6, 256, generator=g) * 1e3).bfloat16(),
    "f32": torch.randn(6, 256, generator=g) * 3e-3,
    "f16": (torch.randn(6, 256, generator=g)).half(),
}
acts["bf16"][1] = 0
acts["bf16"][2, 17] = 3e38
acts["f32"][3] = 0
acts["f32"][4] *= 1e-30
acts["f32"][5, 0] = 256.0   # amax exactly a power of two
acts["f32"][5, 1:] *= 1e-3
for name, x in acts.items():
    x16, xs = activation_to_fp16(x)
    out[f"act_x_{name}"] = bits32(x.float())
    out[f"act_x16_{name}"] = bits16(x16)
    out[f"act_xs_{name}"] = bits32(xs)

# ---------------------------------------------------------------- FP8Linear on CPU tensors
fcases = []
for ci, (M, N, K, G, fmt, od, bias) in enumerate([
        (1, 64, 256, None, "e4m3fn", torch.float16, True),
        (3, 64, 256, 128, "e4m3fn", torch.bfloat16, True),
        (8, 72, 512, 32, "e5m2", torch.float32, False),
        (40, 96, 1024, 128, "e4m3fn", torch.float16, True),
        (130, 200, 512, None, "e5m2", torch.bfloat16, True),
        (17, 128, 1024, 32, "e4m3fn", torch.float32, True)]):
    torch.manual_seed(1000 + ci)
    lin = torch.nn.Linear(K, N, bias=bias)
    layer = FP8Linear.from_linear(lin, fmt=fmt, group_size=G)
    layer.out_dtype = od
    x = torch.randn(M, K).bfloat16()
    y = layer(x)
    if bias:
        out[f"fwd_b_{ci}"] = bits32(lin.bias.data)
    out[f"fwd_q_{ci}"] = layer.qweight.numpy()
    out[f"fwd_s_{ci}"] = bits32(layer.weight_scale)
    out[f"fwd_x_{ci}"] = bits16(x)
    out[f"fwd_y_{ci}"] = bits32(y.float())
    fcases.append(f"{ci}|{M}|{N}|{K}|{G or 0}|{fmt}|{str(od).replace('torch.', '')}|{int(bias)}")
out["fwd_cases"] = np.array(fcases)

np.savez_compressed(os.path.join(HERE, "tfp8_golden.npz"), **out)

# ---------------------------------------------------------------- config 1 at full size
w = synth.outlier_weight(4096, 4096, seed=0)
x = synth.activations(1, 4096, seed=1)
lin = torch.nn.Linear(4096, 4096, bias=False, dtype=torch.float16)
lin.weight.data.copy_(w)
layer = FP8Linear.from_linear(lin, fmt="e4m3fn", group_size=None)
y = layer(x)
c1 = {
    "w_sha256": np.array(hashlib.sha256(w.numpy().tobytes()).hexdigest()),
    "q_sha256": np.array(hashlib.sha256(layer.qweight.numpy().tobytes()).hexdigest()),
    "q_rowsum": layer.qweight.long().sum(1).numpy(),
    "scale": bits32(layer.weight_scale),
    "x": bits16(x),
    "y": bits16(y),
    "roundtrip_e4m3fn": cast_after_clamp(decode(torch.arange(256, dtype=torch.uint8), E4M3FN), E4M3FN).numpy(),
    "roundtrip_e5m2": cast_after_clamp(decode(torch.arange(256, dtype=torch.uint8), E5M2), E5M2).numpy(),
}
np.savez_compressed(os.path.join(HERE, "config1_golden.npz"), **c1)
print("wrote", {k: os.path.getsize(os.path.join(HERE, k)) for k in ("tfp8_golden.npz", "config1_golden.npz")})
