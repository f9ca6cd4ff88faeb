"""Benchmark of the FP8Linear hot path on B200.

    python bench.py --gpus N --steps K --warmup W            this build (CUDA kernels through the C ABI)
    python bench.py --impl reference --gpus N ...            the reference's CPU path, timed on the host cores

Headline metric (BASELINE.json, configs[1]): weight-streaming bandwidth of the M = 1 decode GEMV
over Llama-7B-shaped FP8 E4M3FN layers with per-channel scales. One "step" is one pass over
DECODE_COPIES x the four layer shapes -- 314 MB of distinct codes, more than twice the L2, so
every pass streams from HBM. `value` is algorithmic bytes / time with everything resident in
HBM and the launches replayed from a CUDA graph; `e2e` is the same pass through
`FP8Linear.forward` with pinned HOST activations copied in and results copied out every layer.
With N > 1 ranks (torchrun) every rank streams its own copy of the layer set (independent
layers, no data-path collective: weak scaling); extra keys report the tensor-parallel GEMM.

One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "fp8-compatibility-layer_b200"), ROOT):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402
import torch  # noqa: E402

DECODE_COPIES = 2
METRIC = "fp8linear_gemv_m1_weight_stream_bandwidth"
UNIT = "GB/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# dram__bytes_read.sum + dram__bytes_write.sum of one M=1 12288x4096 GEMV launch (50.42 MB + 0.04 MB)
# over its algorithmic bytes (50 413 568: codes + scales + x + y): profiles/gemv_m1_12288x4096_ncu_full.md
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = (50.42e6 + 0.04e6) / 50413568.0


def gemv_bytes(M, N, K, G, xsz=2, ysz=2, scale_bytes=4, bias=False):
    """Algorithmic bytes of one GEMV: codes + scales + activations in + results out (+ bias)."""
    return N * K + scale_bytes * N * (K // G) + M * K * xsz + M * N * ysz + (4 * N if bias else 0)


# ---------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()          # the exact child this object started
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------- CPU baseline
def cpu_baseline(budget_s=12.0):
    """The reference's CPU path (dequantize the whole weight to float32, then a float32 matmul;
    tfp8/linear.py:179-181 in the reference) restated in C with OpenMP, on all host threads.
    Sample: the M = 1 forward of the 4096x4096 and 11008x4096 layers, repeated for ~budget_s."""
    from oracle import c_port
    from tfp8 import synth
    lib = c_port.load()
    shapes = [(4096, 4096), (11008, 4096)]
    layers = []
    for i, (N, K) in enumerate(shapes):
        q = synth.random_codes(N, K, torch.float8_e4m3fn, seed=i).numpy()
        s = np.full((N, 1), 2.0 ** -13, np.float32)
        x = synth.activations(1, K, seed=7).float().numpy()
        layers.append((x, q, s, np.empty((N, K), np.float32)))
    for x, q, s, work in layers:                       # warm-up, page in
        c_port.linear_forward(x, q, s, None, "e4m3fn", q.shape[1], work, lib)
    nbytes, t0, reps = 0, time.perf_counter(), 0
    while time.perf_counter() - t0 < budget_s:
        for x, q, s, work in layers:
            c_port.linear_forward(x, q, s, None, "e4m3fn", q.shape[1], work, lib)
            nbytes += gemv_bytes(1, q.shape[0], q.shape[1], q.shape[1], xsz=4, ysz=4)
        reps += 1
    dt = time.perf_counter() - t0
    return {"value": nbytes / dt / 1e9, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
            "sample": f"{reps} x M=1 forward of FP8 layers 4096x4096 and 11008x4096 (dequantize to f32 + f32 matmul, "
                      f"C/OpenMP restatement of the reference's torch CPU path), {dt:.1f} s",
            "threads": int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))}


# ---------------------------------------------------------------------------------- workloads
def build_decode_layers(device, fmt="e4m3fn", copies=DECODE_COPIES, seed=0):
    """copies x the four Llama-7B projection shapes as FP8Linear layers (config 2): Gaussian
    N(0, 0.02^2) weights, per-channel power-of-two scales, quantized on the GPU by the fused kernel."""
    from tfp8 import FP8Linear, synth
    layers = []
    g = torch.Generator(device=device).manual_seed(seed)
    for c in range(copies):
        for (N, K) in synth.DECODE_SHAPES:
            w = (torch.randn(N, K, generator=g, device=device) * 0.02).half()
            lin = torch.nn.Linear(K, N, bias=False, device=device, dtype=torch.float16)
            lin.weight.data = w
            layers.append(FP8Linear.from_linear(lin, fmt=fmt, nan_check=False))
            del lin, w
    return layers


STEPS_PER_GRAPH = 25


def time_steps_in_graphs(fn, steps, warmup, per_graph=STEPS_PER_GRAPH):
    """Time exactly `steps` calls of fn(), captured as CUDA graphs of up to `per_graph` consecutive
    steps each (a serving loop replays graphs of hundreds of kernels, not eight), after at least
    `warmup` untimed steps. Returns seconds per step (CUDA events on the replay stream)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()                                   # warm (allocations, lazy module state)
        torch.cuda.synchronize()

        def capture(n):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                for _ in range(n):
                    fn()
            return g
        per_graph = max(1, min(per_graph, steps))
        full, rest = divmod(steps, per_graph)
        g_full = capture(per_graph)
        g_rest = capture(rest) if rest else None
        for _ in range(-(-max(1, warmup) // per_graph)):
            g_full.replay()
        if g_rest is not None:
            g_rest.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(s)
        for _ in range(full):
            g_full.replay()
        if g_rest is not None:
            g_rest.replay()
        e1.record(s)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3 / steps


def time_eager(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3 / steps


def barrier(world):
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x, world, device):
    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device=device)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


# ---------------------------------------------------------------------------------- main arms
def run_ours(args, rank, world, local_rank):
    from tfp8 import _ext, synth
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    _ext.load()
    peaks = measured_peaks()
    layers = build_decode_layers(device)
    xs = [synth.activations(1, l.in_features, seed=11 + i).to(device) for i, l in enumerate(layers)]
    launches = [_ext.GemvLaunch(torch.float16, l.qweight, None, l.weight_scale, None, torch.float16,
                                l.group_size, l.fmt) for l in layers]
    outs = [torch.empty(1, l.out_features, dtype=torch.float16, device=device) for l in layers]
    step_bytes = sum(gemv_bytes(1, l.out_features, l.in_features, l.group_size) for l in layers)
    weight_bytes = sum(l.out_features * l.in_features for l in layers)
    lib = _ext.load()

    def make_step(flags):
        # the C-ABI entry point itself, outputs preallocated: nothing but kernels in the timed region
        def step():
            st = torch.cuda.current_stream().cuda_stream
            for l, x, y in zip(layers, xs, outs):
                rc = lib.tfp8b_gemv_ex(x.data_ptr(), 0, l.qweight.data_ptr(), l.weight_scale.data_ptr(), 0, None,
                                       y.data_ptr(), 0, 1, l.out_features, l.in_features, l.group_size, 0, flags, st)
                assert rc == 0, lib.tfp8b_last_error_string()
        return step

    # The layers of the sweep are independent of one another (own activations, own outputs), which
    # each call states with TFP8B_GEMV_INDEPENDENT_IO; `chain` repeats the pass without the flag,
    # i.e. as if every layer consumed the output of the one before it.
    barrier(world)
    with ClockSampler(local_rank) as clk:
        barrier(world)
        sec = time_steps_in_graphs(make_step(1), args.steps, args.warmup)
        barrier(world)
    sec = max_over_ranks(sec, world, device)
    sec_chain = max_over_ranks(time_steps_in_graphs(make_step(0), args.steps, args.warmup), world, device)
    value = world * step_bytes / sec / 1e9

    # end to end: pinned host activations in, results out, through FP8Linear.forward
    for l in layers:
        l.independent_input = True       # each layer of the sweep has its own activations and outputs
    hx = [x.cpu().pin_memory() for x in xs]
    hy = [torch.empty(1, l.out_features, dtype=torch.float16).pin_memory() for l in layers]
    dx = [torch.empty_like(x) for x in xs]

    def step_e2e():
        for l, h, d, o in zip(layers, hx, dx, hy):
            d.copy_(h, non_blocking=True)
            o.copy_(l(d), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    barrier(world)
    e2e_sec = max_over_ranks(time_eager(step_e2e, args.steps, args.warmup), world, device)
    e2e = {"value": world * step_bytes / e2e_sec / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": sum(h.numel() * 2 for h in hx), "d2h_bytes_per_step": sum(h.numel() * 2 for h in hy),
           "ms_per_step": e2e_sec * 1e3}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "impl": "tfp8_b200",
        "config": {"workload": "decode GEMV sweep (BASELINE configs[1]): M=1 fp16 activations x FP8 E4M3FN weights, "
                               "per-channel pow2 f32 scales, (N,K) in (4096,4096),(12288,4096),(11008,4096),(4096,11008), "
                               f"{DECODE_COPIES} distinct copies per rank; the layers are independent and each call says so "
                               "(TFP8B_GEMV_INDEPENDENT_IO)", "layers_per_step": len(layers),
                   "weight_bytes_per_step": weight_bytes, "algorithmic_bytes_per_step": step_bytes,
                   "l2": "inputs larger than L2: 314 MB of distinct codes per pass", "launch": f"CUDA graphs of up to {STEPS_PER_GRAPH} consecutive steps each, replayed back to back"},
        "gpu_launches": 2 * args.steps * len(layers),
        "e2e": e2e,
        "clocks": clk.summary(),
        "roofline": {"bound": "hbm", "achieved": step_bytes / sec / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": step_bytes / sec / 1e9 / peaks["hbm_gbs"],
                     # DRAM read + write bytes per launch. One ncu capture of this kernel (the
                     # 12288 x 4096 layer: 50.42 MB read + 0.04 MB written for 50.41 MB of algorithmic
                     # bytes) shows every byte crossing DRAM exactly once, and traffic grows with
                     # N*K, so the sweep's average launch is scaled by that measured ratio.
                     "traffic": NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * step_bytes / len(layers),
                     "traffic_source": "ncu capture of gemv:1,12288,4096 (profiles/), scaled by algorithmic bytes",
                     "algorithmic_bytes_per_launch": step_bytes / len(layers),
                     "peak_source": peaks["source"], "kernel": "gemv_kernel<__half, E4M3FN, per-channel>",
                     "avg_launch_us": sec / len(layers) * 1e6,
                     "weights_only_gbs": weight_bytes / sec / 1e9,
                     "dependent_chain": {"achieved": step_bytes / sec_chain / 1e9,
                                         "frac": step_bytes / sec_chain / 1e9 / peaks["hbm_gbs"],
                                         "avg_launch_us": sec_chain / len(layers) * 1e6,
                                         "note": "same pass without TFP8B_GEMV_INDEPENDENT_IO: every call waits for "
                                                 "its predecessor before it reads activations"}},
    }
    if not args.quick:
        line["extra"] = extra_measurements(args, device, peaks, world) if world == 1 else {}
        del layers, launches, xs, outs, hx, hy, dx
        torch.cuda.empty_cache()
        # the extras must never cost the headline line: an error that every rank meets alike
        # (a shape the tensor-parallel size does not divide, no peer memory) is recorded instead
        if world > 1:
            try:
                line["extra"]["tp_gemm"] = tp_gemm_measurements(device, peaks, world, rank)
            except Exception as e:
                line["extra"]["tp_gemm"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        if not args.no_llama:
            try:
                line["extra"]["llama_decode"] = llama_decode_measurements(device, peaks, world)
            except Exception as e:
                line["extra"]["llama_decode"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    if rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_baseline(args.cpu_seconds)
    return line


def extra_measurements(args, device, peaks, world):
    """Per-shape GEMV table (M = 1..8, both formats), the group-scaled and prefill GEMMs
    (configs 3 and 4) and the encoder, each timed with CUDA events over inputs larger than L2 or
    rotated over distinct buffers."""
    from tfp8 import FP8Linear, _ext, synth
    lib = _ext.load()
    out = {"gemv": [], "gemm": [], "codec": []}
    st = lambda: torch.cuda.current_stream().cuda_stream
    # --- GEMV per shape / M / format: rotate over enough copies to exceed 2x L2
    for fmt_id, fmt in ((0, "e4m3fn"), (1, "e5m2")):
        for (N, K) in synth.DECODE_SHAPES:
            copies = max(2, int(np.ceil(2.2 * 126e6 / (N * K))))
            qs = [synth.random_codes(N, K, torch.float8_e4m3fn if fmt_id == 0 else torch.float8_e5m2, seed=c).to(device)
                  for c in range(copies)]
            sc = torch.full((N, 1), 2.0 ** -13, device=device)
            for M in synth.DECODE_M:
                x = synth.activations(M, K).to(device)
                y = torch.empty(M, N, dtype=torch.float16, device=device)

                def step():
                    for q in qs:
                        lib.tfp8b_gemv_ex(x.data_ptr(), 0, q.data_ptr(), sc.data_ptr(), 0, None, y.data_ptr(), 0, M, N, K, K,
                                          fmt_id, 1, st())
                sec = time_steps_in_graphs(step, 20, 3) / copies
                b = gemv_bytes(M, N, K, K)
                out["gemv"].append({"fmt": fmt, "N": N, "K": K, "M": M, "us": sec * 1e6, "gbs": b / sec / 1e9,
                                    "frac_hbm": b / sec / 1e9 / peaks["hbm_gbs"]})
            del qs
    # --- the comparison the reference's own benches make (tests/perf_decode.py, bench_transcode.py):
    # a cached fp16 copy of the weights through cuBLAS (torch F.linear), same shapes, same rotation
    # over distinct buffers. Twice the bytes per weight at M = 1; the fp16 tensor-core ceiling at M = 4096.
    out["fp16_cublas"] = []
    for (N, K) in synth.DECODE_SHAPES:
        copies = max(2, int(np.ceil(2.2 * 126e6 / (2 * N * K))))
        ws = [(torch.randn(N, K, device=device) * 0.02).half() for _ in range(copies)]
        x = synth.activations(1, K).to(device)

        def step16():
            for w in ws:
                torch.nn.functional.linear(x, w)
        sec = time_steps_in_graphs(step16, 20, 3) / copies
        out["fp16_cublas"].append({"M": 1, "N": N, "K": K, "us": sec * 1e6, "gbs_fp16_bytes": 2 * N * K / sec / 1e9})
        del ws
    N, K = synth.GROUP_GEMM_SHAPE
    w16 = (torch.randn(N, K, device=device) * 0.015).half()
    x16c = synth.activations(4096, K).to(device)
    sec = time_eager(lambda: torch.nn.functional.linear(x16c, w16), 10, 3)
    out["fp16_cublas"].append({"M": 4096, "N": N, "K": K, "us": sec * 1e6, "tflops": 2.0 * 4096 * N * K / sec / 1e12})
    del w16, x16c
    # --- tile GEMM: config 3 (G=128 UE8M0, fp16 x) and config 4 (G=32 UE8M0, bf16 x)
    N, K = synth.GROUP_GEMM_SHAPE
    q = synth.random_codes(N, K, torch.float8_e4m3fn, seed=3).to(device)
    for G, Ms, xdt in ((128, synth.GROUP_GEMM_M, torch.float16), (32, synth.PREFILL_M, torch.bfloat16)):
        e8 = torch.randint(110, 118, (N, K // G), dtype=torch.uint8, device=device)
        for M in Ms:
            x = synth.activations(M, K, dtype=xdt).to(device)
            y = torch.empty(M, N, dtype=torch.float16, device=device)
            x16 = torch.empty(M, K, dtype=torch.float16, device=device)
            xsc = torch.empty(M, dtype=torch.float32, device=device)

            ws = torch.empty(M * N, dtype=torch.float32, device=device) if M <= _ext.SPLITK_MAX_M else None

            def step(with_prep=True, split=True):
                if with_prep:
                    lib.tfp8b_prep(x.data_ptr(), 0 if xdt == torch.float16 else 1, x16.data_ptr(), xsc.data_ptr(), M, K, st())
                if ws is not None and split:        # what FP8Linear calls for few rows: K may be split across SMs
                    rc = lib.tfp8b_gemm_splitk(x16.data_ptr(), xsc.data_ptr(), q.data_ptr(), e8.data_ptr(), 1, None, y.data_ptr(), 0,
                                               M, N, K, G, 0, ws.data_ptr(), ws.numel(), st())
                else:
                    rc = lib.tfp8b_gemm(x16.data_ptr(), xsc.data_ptr(), q.data_ptr(), e8.data_ptr(), 1, None, y.data_ptr(), 0,
                                        M, N, K, G, 0, st())
                assert rc == 0, lib.tfp8b_last_error_string()
            iters = 10 if M <= 1024 else 4
            sec = time_eager(step, iters, 3)
            sec_mm = time_eager(lambda: step(False), iters, 2)
            sec_whole_k = time_eager(lambda: step(False, False), iters, 2) if ws is not None else None
            fl = 2.0 * M * N * K
            byt = N * K + N * (K // G) + M * K * 2 + M * N * 2
            bound_s = max(fl / (peaks["bf16_tflops"] * 1e12), byt / (peaks["hbm_gbs"] * 1e9))
            out["gemm"].append({"M": M, "N": N, "K": K, "G": G, "x": str(xdt).replace("torch.", ""),
                                "ms_prep_plus_gemm": sec * 1e3, "ms_gemm": sec_mm * 1e3, "tflops": fl / sec / 1e12,
                                "tflops_gemm_only": fl / sec_mm / 1e12,
                                "frac_tensor_peak": fl / sec_mm / 1e12 / peaks["bf16_tflops"],
                                # launches of a millisecond or more, timed back to back, run under the
                                # power cap: the seconds-long cuBLAS loop is the like-for-like peak there
                                "frac_tensor_peak_sustained": (fl / sec_mm / 1e12 / peaks["bf16_tflops_sustained"]
                                                               if peaks.get("bf16_tflops_sustained") else None),
                                "frac_of_bound": bound_s / sec_mm,
                                "ms_gemm_without_split_k": sec_whole_k * 1e3 if sec_whole_k else None})
            del x, y, x16, ws
    del q
    # --- encoder and fused quantizer on a 256 Mi-element fp16 tensor (512 MB in, 256 MB out)
    n = 1 << 28
    w = (torch.randn(n // 8192, 8192, device=device) * 0.02).half()
    codes = torch.empty(w.shape, dtype=torch.uint8, device=device)
    sec = time_eager(lambda: lib.tfp8b_encode(w.data_ptr(), 0, codes.data_ptr(), n, 0, 0, st()), 5, 3)
    out["codec"].append({"op": "encode f16->e4m3fn", "elements": n, "gelem_s": n / sec / 1e9, "gbs": 3 * n / sec / 1e9,
                         "frac_hbm": 3 * n / sec / 1e9 / peaks["hbm_gbs"]})
    sc = torch.empty(w.shape[0], 1, device=device)
    sec = time_eager(lambda: lib.tfp8b_quantize(w.data_ptr(), 0, codes.data_ptr(), sc.data_ptr(), 0, w.shape[0], 8192, 8192, 0, 1,
                                                st()), 5, 3)
    out["codec"].append({"op": "quantize_weight f16 per-channel", "elements": n, "gelem_s": n / sec / 1e9,
                         "gbs": 3 * n / sec / 1e9, "frac_hbm": 3 * n / sec / 1e9 / peaks["hbm_gbs"]})
    sec = time_eager(lambda: lib.tfp8b_decode(codes.data_ptr(), w.data_ptr(), 0, n, 0, st()), 5, 3)
    out["codec"].append({"op": "decode e4m3fn->f16", "elements": n, "gelem_s": n / sec / 1e9, "gbs": 3 * n / sec / 1e9,
                         "frac_hbm": 3 * n / sec / 1e9 / peaks["hbm_gbs"]})
    return out


def llama_decode_measurements(device, peaks, world, batches=(1, 4, 8), prompt=2048, new_tokens=256):
    """Config 5: Llama-3-8B architecture, random weights, every projection FP8Linear (E4M3FN,
    per-channel); a `prompt`-token prefill, then `new_tokens` greedy decode steps replayed from a
    CUDA graph, per batch size. With world > 1 the model is tensor-parallel over all ranks
    (Megatron layout, NCCL all-reduce after o_proj and down_proj)."""
    from tfp8.examples.llama import LLAMA3_8B, DecodeRunner, build_fp8_llama
    from tfp8.linear import FP8Linear
    t0 = time.perf_counter()
    model = build_fp8_llama(LLAMA3_8B, device, torch.float16)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    code_bytes = sum(m.qweight.numel() for m in model.modules() if isinstance(m, FP8Linear))
    stream_bytes = code_bytes + model.lm_head.weight.numel() * 2 // 1          # per rank, per decoded token
    rows = []
    warm = DecodeRunner(model, 1)        # one-time costs at the real shapes (kernel opt-ins, cuDNN attention plans)
    warm.prefill(torch.randint(0, LLAMA3_8B.vocab, (1, prompt), device=device))
    del warm
    for B in batches:
        g = torch.Generator(device=device).manual_seed(100 + B)
        toks = torch.randint(0, LLAMA3_8B.vocab, (B, prompt), generator=g, device=device)
        run = DecodeRunner(model, B)
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); run.prefill(toks); e1.record(); torch.cuda.synchronize()
        prefill_s = max_over_ranks(e0.elapsed_time(e1) / 1e3, world, device)
        run.capture()
        barrier(world)
        e0.record(); out = run.decode(new_tokens); e1.record(); torch.cuda.synchronize()
        dec_s = max_over_ranks(e0.elapsed_time(e1) / 1e3, world, device)
        ms_tok = dec_s / new_tokens * 1e3
        rows.append({"batch": B, "tp": world,
                     "allreduce": None if world == 1 else ("fused into add+norm (peer stores)" if model.layers[0].comm is not None
                                                            else "nccl"),
                     "prefill_tokens": prompt, "prefill_ms": prefill_s * 1e3,
                     "prefill_tok_s": B * prompt / prefill_s, "decode_tokens": new_tokens, "ms_per_step": ms_tok,
                     "decode_tok_s": B * new_tokens / dec_s,
                     "hbm_bound_ms_per_step": stream_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3,
                     "frac_of_hbm_bound": stream_bytes / (peaks["hbm_gbs"] * 1e9) / (dec_s / new_tokens),
                     "finite": bool(torch.isfinite(out.float()).all())})
        del run
        torch.cuda.empty_cache()
    return {"model": "Llama-3-8B architecture, random N(0,0.02^2) fp16 weights, FP8 E4M3FN per-channel projections",
            "fp8_code_bytes_per_rank": code_bytes, "bytes_streamed_per_token_per_rank": stream_bytes,
            "build_seconds": build_s, "runs": rows}


def tp_gemm_measurements(device, peaks, world, rank):
    """Config 4: 28672 x 8192 E4M3FN weight with 32-wide UE8M0 K-groups, column-sharded across the
    ranks, bf16 activations replicated. TFLOP/s of the whole job three ways: shard only, shard +
    NCCL all-gather, and the gather fused into the GEMM epilogue (peer stores into every rank's
    symmetric-memory output, then one barrier)."""
    from tfp8 import _ext, synth
    lib = _ext.load()
    N, K = synth.GROUP_GEMM_SHAPE
    Nl = N // world
    q = synth.random_codes(N, K, torch.float8_e4m3fn, seed=3)[rank * Nl:(rank + 1) * Nl].contiguous().to(device)
    e8 = torch.randint(110, 118, (Nl, K // 32), dtype=torch.uint8, device=device)
    st = lambda: torch.cuda.current_stream().cuda_stream
    rows = []
    # fused gather: two symmetric-memory outputs (alternating), written by every rank's epilogue
    import ctypes
    fused_error = None
    try:
        import torch.distributed._symmetric_memory as symm
        Mmax = max(synth.PREFILL_M)
        sbufs = [symm.empty((Mmax, N), dtype=torch.float16, device=device) for _ in range(2)]
        shdls = [symm.rendezvous(b, torch.distributed.group.WORLD) for b in sbufs]
    except Exception as e:                       # no peer-mapped memory on this box: NCCL numbers only
        fused_error = f"{type(e).__name__}: {e}"[:200]
    # every rank must take the same branch
    flag = torch.tensor([1 if fused_error else 0], device=device)
    torch.distributed.all_reduce(flag)
    if int(flag) and not fused_error:
        fused_error = "symmetric memory unavailable on another rank"
    turn = [0]
    for M in synth.PREFILL_M:
        x = synth.activations(M, K, dtype=torch.bfloat16).to(device)
        x16 = torch.empty(M, K, dtype=torch.float16, device=device)
        xs = torch.empty(M, dtype=torch.float32, device=device)
        y = torch.empty(M, Nl, dtype=torch.float16, device=device)
        full = torch.empty(world * M, Nl, dtype=torch.float16, device=device)

        def step_fused():
            t = turn[0]
            turn[0] = t ^ 1
            ptrs = [int(shdls[t].buffer_ptrs[r]) for r in range(world)]
            ptrs = ptrs[rank:] + ptrs[:rank]
            arr = (ctypes.c_void_p * world)(*ptrs)
            lib.tfp8b_prep(x.data_ptr(), 1, x16.data_ptr(), xs.data_ptr(), M, K, st())
            rc = lib.tfp8b_gemm_scatter(x16.data_ptr(), xs.data_ptr(), q.data_ptr(), e8.data_ptr(), 1, None, arr, world, N,
                                        rank * Nl, 0, M, Nl, K, 32, 0, st())
            assert rc == 0, lib.tfp8b_last_error_string()
            shdls[t].barrier()
            return sbufs[t]

        def step(gather):
            lib.tfp8b_prep(x.data_ptr(), 1, x16.data_ptr(), xs.data_ptr(), M, K, st())
            rc = lib.tfp8b_gemm(x16.data_ptr(), xs.data_ptr(), q.data_ptr(), e8.data_ptr(), 1, None, y.data_ptr(), 0,
                                M, Nl, K, 32, 0, st())
            assert rc == 0, lib.tfp8b_last_error_string()
            if gather and world > 1:
                torch.distributed.all_gather_into_tensor(full, y)
        barrier(world)
        t_g = max_over_ranks(time_eager(lambda: step(True), 4, 3), world, device)
        barrier(world)
        t_n = max_over_ranks(time_eager(lambda: step(False), 4, 3), world, device)
        fl = 2.0 * M * N * K
        row = {"M": M, "N": N, "K": K, "G": 32, "tp": world, "ms_with_gather": t_g * 1e3, "ms_without_gather": t_n * 1e3,
               "tflops_with_gather": fl / t_g / 1e12, "tflops_without_gather": fl / t_n / 1e12,
               "frac_tensor_peak_all_gpus": fl / t_g / 1e12 / (world * peaks["bf16_tflops"])}
        if fused_error is None:
            barrier(world)
            t_f = max_over_ranks(time_eager(step_fused, 4, 3), world, device)
            # the fused result must be what NCCL gathers: rank r's shard in columns [r*Nl, (r+1)*Nl)
            step(True)
            got = step_fused()[:M]
            torch.cuda.synchronize()
            want = full.view(world, M, Nl).permute(1, 0, 2).reshape(M, N)
            row.update({"ms_fused_gather": t_f * 1e3, "fused_equals_nccl": bool(torch.equal(got, want)),
                        "tflops_fused_gather": fl / t_f / 1e12,
                        "frac_tensor_peak_all_gpus_fused": fl / t_f / 1e12 / (world * peaks["bf16_tflops"])})
            barrier(world)
        else:
            row["fused_gather_unavailable"] = fused_error
        rows.append(row)
        del x, x16, y, full
    return rows


def run_probe(args):
    """`--probe gemm:M,N,K,G` / `--probe gemv:M,N,K,G`: a few launches of one kernel on one shape
    (a small, self-ending case for profiler captures). Prints one JSON line with the timing."""
    from tfp8 import _ext, synth
    kind, dims = args.probe.split(":")
    M, N, K, G = (int(v) for v in dims.split(","))
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    lib = _ext.load()
    copies = max(1, min(8, int(2.2 * 126e6 / (N * K)) + 1))
    qs = [synth.random_codes(N, K, torch.float8_e4m3fn, seed=c).to(device) for c in range(copies)]
    ng = K // G
    sc = torch.randint(110, 118, (N, ng), dtype=torch.uint8, device=device) if ng > 1 else torch.full((N, 1), 2.0 ** -13, device=device)
    skind = 1 if ng > 1 else 0
    x = synth.activations(M, K).to(device)
    y = torch.empty(M, N, dtype=torch.float16, device=device)
    x16 = torch.empty(M, K, dtype=torch.float16, device=device)
    xs = torch.empty(M, dtype=torch.float32, device=device)
    st = lambda: torch.cuda.current_stream().cuda_stream
    lib.tfp8b_prep(x.data_ptr(), 0, x16.data_ptr(), xs.data_ptr(), M, K, st())
    ws = torch.empty(M * N, dtype=torch.float32, device=device) if M <= _ext.SPLITK_MAX_M else None   # as FP8Linear calls it

    def step():
        for q in qs:
            if kind == "gemm" and ws is not None:
                rc = lib.tfp8b_gemm_splitk(x16.data_ptr(), xs.data_ptr(), q.data_ptr(), sc.data_ptr(), skind, None, y.data_ptr(), 0,
                                           M, N, K, G, 0, ws.data_ptr(), ws.numel(), st())
            elif kind == "gemm":
                rc = lib.tfp8b_gemm(x16.data_ptr(), xs.data_ptr(), q.data_ptr(), sc.data_ptr(), skind, None, y.data_ptr(), 0,
                                    M, N, K, G, 0, st())
            else:
                rc = lib.tfp8b_gemv_ex(x.data_ptr(), 0, q.data_ptr(), sc.data_ptr(), skind, None, y.data_ptr(), 0, M, N, K, G, 0,
                                       0, st())
            assert rc == 0, lib.tfp8b_last_error_string()
    sec = time_eager(step, args.steps, args.warmup) / copies
    fl = 2.0 * M * N * K
    print(json.dumps({"probe": args.probe, "copies": copies, "us_per_launch": sec * 1e6, "tflops": fl / sec / 1e12,
                      "gbs": gemv_bytes(M, N, K, G) / sec / 1e9}))


def run_reference(args, rank, world):
    """The reference's own CPU implementation of the path on the host cores, same metric."""
    if rank != 0:
        return None
    steps = max(1, args.steps)
    base = cpu_baseline(budget_s=min(60.0, max(5.0, 1.0 * steps)))
    return {"metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "impl": "reference",
            "config": {"workload": "decode GEMV sweep (BASELINE configs[1]), bounded sample on the host cores"},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--quick", action="store_true", help="headline only: skip the per-shape / GEMM / codec tables")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-llama", action="store_true", help="skip the Llama-3-8B decode measurement")
    ap.add_argument("--probe", default=None, help="gemm:M,N,K,G or gemv:M,N,K,G -- a few launches of one kernel (profiling)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.probe:
        run_probe(args)
        return
    # The result is ONE line on stdout. Libraries write there too (NCCL prints a version banner
    # when NCCL_DEBUG asks for it), so during the run file descriptor 1 points at stderr and the
    # line goes to the saved descriptor at the end.
    sys.stdout.flush()
    result_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(line):
        sys.stdout.flush()
        os.write(result_fd, (json.dumps(line) + "\n").encode())

    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            emit(line)
        return
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    line = run_ours(args, rank, world, local_rank)
    if rank == 0:
        emit(line)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
