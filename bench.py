"""Benchmark of the FP8Linear hot path on B200.

    python bench.py --gpus N --steps K --warmup W            this build (CUDA kernels through the C ABI)
    python bench.py --impl reference --gpus N ...            the reference's CPU path, timed on the host cores
    python bench.py --impl reference-gpu                     the reference's own NVRTC kernels on this GPU (A/B table)

Headline metric: weight-streaming bandwidth of the M = 1 decode GEMV over Llama-7B-shaped FP8
E4M3FN layers with per-channel scales (the decode sweep of the benchmark configurations). One "step" is one pass over
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


# dram__bytes_read.sum + dram__bytes_write.sum of one M=1 12288x4096 GEMV launch under ncu
# (50.42 MB + 0.04 MB) over its algorithmic bytes (50 413 568: codes + scales + x + y)
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
def reference_package():
    """The reference project's own Python package (an unmodified copy staged under oracle/_ref/ by
    `make -C oracle` where the reference checkout exists; it is git-ignored). None when absent."""
    path = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isfile(os.path.join(path, "tfp8_reference", "linear.py")):
        return None
    if path not in sys.path:
        sys.path.insert(0, path)
    import tfp8_reference
    return tfp8_reference


def cpu_baseline(budget_s=12.0):
    """The reference's CPU path for the headline workload -- M = 1 fp16 activations through each of
    the four layer shapes, `FP8Linear.forward` on CPU tensors = dequantize the whole weight to
    float32, then a float32 matmul (tfp8/linear.py:179-181 there) -- timed on the host cores.
    kind "reference": the reference's own package (torch, all threads). The C/OpenMP restatement
    of the same arithmetic is timed beside it (`port_value`), and is the number reported when the
    reference package is not staged (kind "port")."""
    from oracle import c_port
    from tfp8 import synth
    lib = c_port.load()
    shapes = list(synth.DECODE_SHAPES)
    layers = []
    for i, (N, K) in enumerate(shapes):
        q = synth.random_codes(N, K, torch.float8_e4m3fn, seed=i)
        s = torch.full((N, 1), 2.0 ** -13)
        x = synth.activations(1, K, seed=7)                      # fp16
        layers.append((x, q, s))
    pass_bytes = sum(gemv_bytes(1, q.shape[0], q.shape[1], q.shape[1]) for _, q, _ in layers)
    cores = os.cpu_count() or 1

    def timed(fn, budget):
        fn()                                                     # warm-up, page in
        t0, reps = time.perf_counter(), 0
        while reps < 2 or time.perf_counter() - t0 < budget:
            fn()
            reps += 1
        return reps, time.perf_counter() - t0

    work = [np.empty(tuple(q.shape), np.float32) for _, q, _ in layers]
    xs32 = [x.float().numpy() for x, _, _ in layers]

    def port_pass():
        for (x, q, s), w, x32 in zip(layers, work, xs32):
            c_port.linear_forward(x32, q.numpy(), s.numpy(), None, "e4m3fn", q.shape[1], w, lib)

    ref = reference_package()
    port_budget = budget_s if ref is None else max(2.0, 0.25 * budget_s)
    reps_p, dt_p = timed(port_pass, port_budget)
    port_value = reps_p * pass_bytes / dt_p / 1e9
    out = {"unit": UNIT, "cores": cores, "port_value": port_value,
           "port_sample": f"{reps_p} passes, C/OpenMP restatement (float32 activations), {dt_p:.1f} s",
           "threads": int(os.environ.get("OMP_NUM_THREADS", cores))}
    if ref is None:
        out.update({"value": port_value, "kind": "port",
                    "sample": f"{reps_p} x M=1 forward of the four FP8 layers {shapes} (dequantize to f32 + f32 matmul, "
                              f"C/OpenMP restatement of the reference's torch CPU path), {dt_p:.1f} s"})
        return out
    del work
    rl = [ref.FP8Linear.from_fp8_checkpoint(q, s, None, "e4m3fn", out_dtype=torch.float16) for _, q, s in layers]

    def ref_pass():
        with torch.no_grad():
            for l, (x, _, _) in zip(rl, layers):
                l(x)

    reps_r, dt_r = timed(ref_pass, budget_s - port_budget)
    assert all(l.stats["torch"] > 0 and l.stats["gemv"] == 0 for l in rl)
    out.update({"value": reps_r * pass_bytes / dt_r / 1e9, "kind": "reference", "cores": torch.get_num_threads(),
                "sample": f"{reps_r} x M=1 fp16 forward of the four FP8 layers {shapes} through the reference's own "
                          f"FP8Linear on CPU tensors (torch {torch.__version__}, {torch.get_num_threads()} threads of "
                          f"{cores} cores), {dt_r:.1f} s"})
    return out


# ---------------------------------------------------------------------------------- workloads
def build_decode_layers(device, fmt="e4m3fn", copies=DECODE_COPIES, seed=0):
    """copies x the four Llama-7B projection shapes as FP8Linear layers (the decode sweep): Gaussian
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
        # the C-ABI entry point itself (the layer's prepared plan), outputs preallocated: nothing but
        # kernels in the timed region
        def step():
            st = torch.cuda.current_stream().cuda_stream
            for pl, x, y in zip(launches, xs, outs):
                rc = lib.tfp8b_gemv_plan_run(pl.plan, x.data_ptr(), y.data_ptr(), 1, flags, st)
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

    # end to end through FP8Linear.forward with HOST buffers: the step's activations (one pinned
    # buffer holding every layer's row) go to the device in one copy, each layer's result comes back
    # into its pinned host row as soon as the layer is enqueued, one synchronisation ends the step --
    # the way a serving loop feeds a step, instead of a copy-launch-copy-sync round trip per layer.
    for l in layers:
        l.independent_input = True       # each layer of the sweep has its own activations and outputs
    offs = np.cumsum([0] + [l.in_features for l in layers])
    hx_all = torch.cat([x.reshape(-1).cpu() for x in xs]).pin_memory()
    dx_all = torch.empty_like(hx_all, device=device)
    dx = [dx_all[offs[i]:offs[i + 1]].view(1, -1) for i in range(len(layers))]
    youts = np.cumsum([0] + [l.out_features for l in layers])
    hy_all = torch.empty(int(youts[-1]), dtype=torch.float16).pin_memory()
    hy = [hy_all[youts[i]:youts[i + 1]].view(1, -1) for i in range(len(layers))]

    def enqueue_e2e():
        # one copy in, the layers back to back (a copy between two layers would end the overlap of
        # consecutive kernels), their results gathered on the device, one copy out
        dx_all.copy_(hx_all, non_blocking=True)
        ys = [l(d).view(-1) for l, d in zip(layers, dx)]
        hy_all.copy_(torch.cat(ys), non_blocking=True)

    # the step is captured once (copies and layer calls alike, as the decode runner captures its
    # step) and replayed: per step one graph launch and one synchronisation on the host side
    e2e_stream = torch.cuda.Stream()
    e2e_stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(e2e_stream):
        for _ in range(4):
            enqueue_e2e()                                   # past the layers' checked first calls
        torch.cuda.synchronize()
        e2e_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(e2e_graph, stream=e2e_stream):
            enqueue_e2e()

    def step_e2e():
        e2e_graph.replay()                                  # on the current stream
        torch.cuda.current_stream().synchronize()

    hy_all.zero_()
    step_e2e()
    for l, x, o in zip(layers, xs, hy):                     # the host rows hold the layers' results
        assert torch.equal(o, l(x).cpu()), "e2e path does not reproduce the layer's output"
    barrier(world)
    with ClockSampler(local_rank) as clk_e2e:
        e2e_sec = max_over_ranks(time_eager(step_e2e, args.steps, args.warmup), world, device)
    e2e = {"value": world * step_bytes / e2e_sec / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": hx_all.numel() * 2, "d2h_bytes_per_step": hy_all.numel() * 2,
           "ms_per_step": e2e_sec * 1e3, "clocks": clk_e2e.summary(),
           "how": "FP8Linear.forward per layer (prepared GEMV plan), captured once in a CUDA graph together with the pinned "
                  "H2D copy of the step's activations, a device-side gather of the layers' results and one D2H copy "
                  "into pinned host memory; per step one replay and one stream synchronisation"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "impl": "tfp8_b200",
        "config": {"workload": "decode GEMV sweep: M=1 fp16 activations x FP8 E4M3FN weights, "
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
                     "traffic_source": "one ncu capture of this kernel on the 12288x4096 layer, scaled by algorithmic bytes",
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
    clocks = {}                                   # one nvidia-smi record per timed section of the extras
    if not args.quick:
        line["extra"] = extra_measurements(args, device, peaks, world, clocks, local_rank) if world == 1 else {}
        line["extra"]["clocks"] = clocks
        del layers, launches, xs, outs, hx_all, hy, hy_all, dx, dx_all
        torch.cuda.empty_cache()
        # the extras must never cost the headline line: an error that every rank meets alike
        # (a shape the tensor-parallel size does not divide, no peer memory) is recorded instead
        if world > 1:
            try:
                with ClockSampler(local_rank) as c:
                    line["extra"]["tp_gemm"] = tp_gemm_measurements(device, peaks, world, rank)
                clocks["tp_gemm"] = c.summary()
            except Exception as e:
                line["extra"]["tp_gemm"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        if world == 1:
            try:        # one layer's decode attention at Llama-3-8B shapes: library kernels (16-bit and FP8 cache) and torch's
                with ClockSampler(local_rank) as c:
                    line["extra"]["attention"] = [attention_row(device, k, B, 2304, 20, 3) for B in (1, 4, 8) for k in ("sdpa", "attn", "attn8")]
                clocks["attention"] = c.summary()
            except Exception as e:
                line["extra"]["attention"] = {"error": f"{type(e).__name__}: {e}"[:300]}
            torch.cuda.empty_cache()
        if not args.no_llama:
            try:
                with ClockSampler(local_rank) as c:
                    line["extra"]["llama_decode"] = llama_decode_measurements(device, peaks, world)
                clocks["llama_decode"] = c.summary()
            except Exception as e:
                line["extra"]["llama_decode"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    if world > 1 and "extra" in line:
        # the sharded configurations in named keys: whole-job numbers on `world` GPUs, the one-GPU
        # figures measured by the same processes, and the efficiency = speed-up / world
        sh = {"tp": world}
        tg = line["extra"].get("tp_gemm")
        if isinstance(tg, list):
            sh["prefill_gemm_28672x8192_g32"] = [
                {"M": r["M"], "tflops_fused_gather": r.get("tflops_fused_gather"), "tflops_nccl_gather": r["tflops_with_gather"],
                 "tflops_one_gpu": r["tflops_one_gpu_same_process"], "efficiency_fused_gather": r.get("efficiency_fused_gather"),
                 "efficiency_nccl_gather": r["efficiency_nccl_gather"], "fused_equals_nccl": r.get("fused_equals_nccl")} for r in tg]
        ld = line["extra"].get("llama_decode")
        if isinstance(ld, dict) and "scaling" in ld:
            sh["llama3_8b_decode"] = ld["scaling"]
            sh["llama3_8b_decode_parity"] = ld.get("parity")
        line["sharded"] = sh
    if rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_baseline(args.cpu_seconds)
    return line


def extra_measurements(args, device, peaks, world, clocks, local_rank):
    """Per-shape GEMV table (M = 1..8, both formats), the group-scaled and prefill GEMMs and the
    codecs, each timed with CUDA events over inputs larger than L2 or rotated over distinct
    buffers; `clocks` receives one clock / throttle record per section."""
    from tfp8 import FP8Linear, _ext, synth
    lib = _ext.load()
    out = {"gemv": [], "gemm": [], "codec": []}
    st = lambda: torch.cuda.current_stream().cuda_stream
    sampler = ClockSampler(local_rank).__enter__()

    def section_done(name):
        nonlocal sampler
        sampler.__exit__(None, None, None)
        clocks[name] = sampler.summary()
        sampler = ClockSampler(local_rank).__enter__()
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
    section_done("gemv_table")
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
    section_done("fp16_cublas")
    # --- tile GEMM on the 28672 x 8192 layer: 128-wide UE8M0 K-groups with fp16 activations (16 .. 1024
    # rows) and 32-wide groups with bf16 activations (2048 .. 8192 rows). The weight is the
    # configuration's own distribution -- N(0, 0.015^2) with 1 % of the K-groups multiplied by 8 --
    # quantized by the fused quantizer, so neighbouring groups of a row differ by several binades
    # and the decode warps' scale fold sees real exponent differences, not a constant.
    N, K = synth.GROUP_GEMM_SHAPE
    for G, Ms, xdt in ((128, synth.GROUP_GEMM_M, torch.float16), (32, synth.PREFILL_M, torch.bfloat16)):
        w = synth.group_outlier_weight(N, K, group=G, seed=G).to(device)
        q, e8, _ = _ext.quantize_weight_cuda(w, "e4m3fn", G, True, ue8m0=True)
        del w
        spread = int(e8.max()) - int(e8.min())
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
            iters = 40 if M <= 1024 else 20
            sec = time_eager(step, iters, 3)
            sec_mm = time_eager(lambda: step(False), iters, 3)
            sec_whole_k = time_eager(lambda: step(False, False), iters, 3) if ws is not None else None
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
                                "frac_of_bound": bound_s / sec_mm, "iterations": iters,
                                "ue8m0_exponent_spread": spread,
                                "ms_gemm_without_split_k": sec_whole_k * 1e3 if sec_whole_k else None})
            del x, y, x16, ws
        del q, e8
        section_done(f"gemm_g{G}")
    # --- W8A8: the MX layer (32-wide UE8M0 blocks on both operands) on the block-scaled FP8 tensor cores
    out["w8a8"] = []
    for M in synth.PREFILL_M:
        row = w8a8_row(device, M, N, K, 20, 3)
        row.update({"frac_measured_bf16_peak": row["tflops_gemm_only"] / peaks["bf16_tflops"],
                    "frac_nominal_fp8_peak": row["tflops_gemm_only"] / 4500.0,
                    "note": "FP8 x FP8 with tensor-core block scaling; the measured denominator is the cuBLAS bf16 GEMM "
                            "(no FP8 peak is measured on this pool), the nominal dense FP8 peak is 4500 TFLOP/s"})
        out["w8a8"].append(row)
    section_done("w8a8")
    # --- encoder and fused quantizer on a 256 Mi-element fp16 tensor (512 MB in, 256 MB out)
    n = 1 << 28
    w = (torch.randn(n // 8192, 8192, device=device) * 0.02).half()
    codes = torch.empty(w.shape, dtype=torch.uint8, device=device)
    sec = time_eager(lambda: lib.tfp8b_encode(w.data_ptr(), 0, codes.data_ptr(), n, 0, 0, st()), 20, 3)
    out["codec"].append({"op": "encode f16->e4m3fn", "elements": n, "gelem_s": n / sec / 1e9, "gbs": 3 * n / sec / 1e9,
                         "frac_hbm": 3 * n / sec / 1e9 / peaks["hbm_gbs"]})
    sc = torch.empty(w.shape[0], 1, device=device)
    sec = time_eager(lambda: lib.tfp8b_quantize(w.data_ptr(), 0, codes.data_ptr(), sc.data_ptr(), 0, w.shape[0], 8192, 8192, 0, 1,
                                                st()), 20, 3)
    out["codec"].append({"op": "quantize_weight f16 per-channel", "elements": n, "gelem_s": n / sec / 1e9,
                         "gbs": 3 * n / sec / 1e9, "frac_hbm": 3 * n / sec / 1e9 / peaks["hbm_gbs"]})
    sec = time_eager(lambda: lib.tfp8b_decode(codes.data_ptr(), w.data_ptr(), 0, n, 0, st()), 20, 3)
    out["codec"].append({"op": "decode e4m3fn->f16", "elements": n, "gelem_s": n / sec / 1e9, "gbs": 3 * n / sec / 1e9,
                         "frac_hbm": 3 * n / sec / 1e9 / peaks["hbm_gbs"]})
    section_done("codec")
    sampler.__exit__(None, None, None)
    return out


def _decode_rows(model, device, peaks, world, batches, prompt, new_tokens, stream_bytes, keep=None):
    """Prefill + graph-replayed greedy decode per batch size on `model`; one row of numbers each.
    `keep` (a dict) receives, per batch size, the prefill logits and the decoded token ids."""
    from tfp8.examples.llama import LLAMA3_8B, DecodeRunner
    rows = []
    for B in batches:
        g = torch.Generator(device=device).manual_seed(100 + B)
        toks = torch.randint(0, LLAMA3_8B.vocab, (B, prompt), generator=g, device=device)
        run = DecodeRunner(model, B)
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); pre = run.prefill(toks); e1.record(); torch.cuda.synchronize()
        prefill_s = max_over_ranks(e0.elapsed_time(e1) / 1e3, world, device)
        run.capture()
        barrier(world)
        e0.record(); out = run.decode(new_tokens, check=False); e1.record(); torch.cuda.synchronize()
        dec_s = max_over_ranks(e0.elapsed_time(e1) / 1e3, world, device)
        run.check_device()                       # raises if a kernel gave up on a wait or skipped a position
        if keep is not None:
            keep[B] = (pre.float().cpu(), out.cpu())
        rows.append({"batch": B, "tp": model.tp,
                     "allreduce": None if model.tp == 1 else ("fused into add+norm (peer stores)" if model.layers[0].comm is not None
                                                               else "nccl"),
                     "prefill_tokens": prompt, "prefill_ms": prefill_s * 1e3,
                     "prefill_tok_s": B * prompt / prefill_s, "decode_tokens": new_tokens, "ms_per_step": dec_s / new_tokens * 1e3,
                     "decode_tok_s": B * new_tokens / dec_s,
                     "hbm_bound_ms_per_step": stream_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3,
                     "frac_of_hbm_bound": stream_bytes / (peaks["hbm_gbs"] * 1e9) / (dec_s / new_tokens),
                     "finite": bool(torch.isfinite(out.float()).all())})
        del run
        torch.cuda.empty_cache()
    return rows


def llama_decode_measurements(device, peaks, world, batches=(1, 4, 8), prompt=2048, new_tokens=256):
    """The full decoder configuration: Llama-3-8B architecture, random weights, every projection
    FP8Linear (E4M3FN, per-channel); a `prompt`-token prefill, then `new_tokens` greedy decode
    steps replayed from a CUDA graph, per batch size. With world > 1 the model is tensor-parallel
    over all ranks (Megatron layout, the all-reduce after o_proj and down_proj fused into the
    add + norm kernel). In that case every rank first runs the UNSHARDED model on its own GPU, in
    the same process: that gives the one-GPU tokens/s the scaling figures are taken against, and
    the logits / tokens the tensor-parallel run is checked against; a second tensor-parallel run
    with NCCL all-reduces must produce the same greedy tokens as the fused one."""
    from tfp8.examples.llama import LLAMA3_8B, DecodeRunner, build_fp8_llama, reorder_fused_rows_like_tp
    from tfp8.linear import FP8Linear

    def bytes_per_token(model):
        code = sum(m.qweight.numel() for m in model.modules() if isinstance(m, FP8Linear))
        return code, code + model.lm_head.weight.numel() * 2

    def warm(model):        # one-time costs at the real shapes (kernel opt-ins, cuDNN attention plans)
        w = DecodeRunner(model, 1)
        w.prefill(torch.randint(0, LLAMA3_8B.vocab, (1, prompt), device=device))
        del w

    result = {"model": "Llama-3-8B architecture, random N(0,0.02^2) fp16 weights, FP8 E4M3FN per-channel projections"}
    one_rows, one_keep = None, {}
    if world > 1:
        # same seed = same random matrices; the fused rows re-ordered as the sharded build reads them,
        # so that the two models are the same function and their logits can be compared
        one = reorder_fused_rows_like_tp(build_fp8_llama(LLAMA3_8B, device, torch.float16, tp=1), world)
        torch.cuda.synchronize()
        warm(one)
        _, sb1 = bytes_per_token(one)
        one_rows = _decode_rows(one, device, peaks, 1, batches, prompt, new_tokens, sb1, keep=one_keep)
        del one
        torch.cuda.empty_cache()
        result["one_gpu_runs_same_process"] = one_rows
    t0 = time.perf_counter()
    model = build_fp8_llama(LLAMA3_8B, device, torch.float16)
    torch.cuda.synchronize()
    result["build_seconds"] = time.perf_counter() - t0
    code_bytes, stream_bytes = bytes_per_token(model)
    result.update({"fp8_code_bytes_per_rank": code_bytes, "bytes_streamed_per_token_per_rank": stream_bytes})
    warm(model)
    keep = {}
    rows = _decode_rows(model, device, peaks, world, batches, prompt, new_tokens, stream_bytes, keep=keep)
    result["runs"] = rows
    if world == 1:
        # The same model and workload with the KV cache held as FP8 codes + one scale per token and KV
        # head (FP8Config(kv_cache="fp8")): the decode attention then reads half the bytes. Beside it,
        # for a like-for-like comparison of the cache formats, the library's attention kernel over the
        # 16-bit cache (the default rows above use torch's attention).
        cfg = LLAMA3_8B
        def kv_bytes(B, per_elem):        # K and V of every layer, read once per step at mid-run length
            return 2 * cfg.n_layers * cfg.n_kv_heads * (prompt + new_tokens // 2) * B * (cfg.head_dim * per_elem + (4 if per_elem == 1 else 0))
        model.attn_kernel = True
        result["runs_attn_kernel_fp16_cache"] = _decode_rows(model, device, peaks, world, batches, prompt, new_tokens, stream_bytes)
        model.attn_kernel, model.kv_fmt = False, "e4m3fn"
        keep8 = {}
        result["runs_kv_cache_fp8"] = _decode_rows(model, device, peaks, world, batches, prompt, new_tokens, stream_bytes, keep=keep8)
        model.kv_fmt = None
        for r16, r8 in zip(result["runs_attn_kernel_fp16_cache"], result["runs_kv_cache_fp8"]):
            r16["kv_bytes_per_step"], r8["kv_bytes_per_step"] = kv_bytes(r16["batch"], 2), kv_bytes(r8["batch"], 1)
            pre16, _ = keep[r8["batch"]]
            pre8, _ = keep8[r8["batch"]]
            r8["prefill_logits_cosine_vs_fp16_cache"] = float(torch.nn.functional.cosine_similarity(pre8, pre16, dim=-1).min())
    if world > 1:
        # scaling against the one-GPU run of this process
        result["scaling"] = [{"batch": r["batch"], "tp": world, "decode_tok_s": r["decode_tok_s"], "one_gpu_decode_tok_s": o["decode_tok_s"],
                              "speedup": r["decode_tok_s"] / o["decode_tok_s"], "efficiency": r["decode_tok_s"] / o["decode_tok_s"] / world}
                             for r, o in zip(rows, one_rows)]
        # parity: (i) the NCCL decoder picks the same greedy tokens as the fused one; (ii) the
        # tensor-parallel logits agree with the unsharded model's within the tolerance of a
        # different float32 summation order (stated: 2e-2 of the largest logit)
        B = batches[0]
        g = torch.Generator(device=device).manual_seed(100 + B)
        toks = torch.randint(0, LLAMA3_8B.vocab, (B, prompt), generator=g, device=device)
        run = DecodeRunner(model, B, fused_allreduce=False)
        pre_nccl = run.prefill(toks).float().cpu()
        run.capture()
        ids_nccl = run.decode(64).cpu()
        del run
        pre_f, ids_f = keep[B]
        pre_1, ids_1 = one_keep[B]
        scale = float(pre_1.abs().max())
        n_same = int((ids_f[:, :64] == ids_1[:, :64]).int().cumprod(1).sum(1).min())
        n_same_nccl = int((ids_f[:, :64] == ids_nccl).int().cumprod(1).sum(1).min())
        result["parity"] = {"batch": B, "fused_tokens_equal_nccl_tokens": bool(torch.equal(ids_f[:, :64], ids_nccl)),
                            "leading_greedy_tokens_equal_nccl_of_64": n_same_nccl,
                            "fused_prefill_logits_equal_nccl": bool(torch.equal(pre_f, pre_nccl)),
                            "prefill_logits_max_abs_diff_vs_one_gpu_over_max_logit": float((pre_f - pre_1).abs().max() / scale),
                            "tolerance": 2e-2, "within_tolerance": bool(float((pre_f - pre_1).abs().max() / scale) <= 2e-2),
                            "first_token_equal_one_gpu": bool(torch.equal(pre_f.argmax(-1), pre_1.argmax(-1))),
                            "leading_greedy_tokens_equal_one_gpu": n_same,
                            "note": "the fused and the NCCL decoder add the same float32 partials in the same order; their norm "
                                    "kernels group the sum of squares differently, a last-bit difference that greedy decoding "
                                    "of a random-weight model (near-uniform logits) amplifies into a different token sooner or "
                                    "later; prefill logits are compared exactly, token runs are reported"}
    return result


def tp_gemm_measurements(device, peaks, world, rank):
    """Config 4: 28672 x 8192 E4M3FN weight with 32-wide UE8M0 K-groups, column-sharded across the
    ranks, bf16 activations replicated. TFLOP/s of the whole job three ways: shard only, shard +
    NCCL all-gather, and the gather fused into the GEMM epilogue (peer stores into every rank's
    symmetric-memory output, then one barrier)."""
    from tfp8 import _ext, synth
    lib = _ext.load()
    N, K = synth.GROUP_GEMM_SHAPE
    Nl = N // world
    w = synth.group_outlier_weight(N, K, group=32, seed=32).to(device)          # the same full weight on every rank
    q_full, e8_full, _ = _ext.quantize_weight_cuda(w, "e4m3fn", 32, True, ue8m0=True)
    del w
    q = q_full[rank * Nl:(rank + 1) * Nl].contiguous()
    e8 = e8_full[rank * Nl:(rank + 1) * Nl].contiguous()
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
        # the whole layer on ONE GPU, in this process: what the sharded runs are scaled against
        y1 = torch.empty(M, N, dtype=torch.float16, device=device)

        def step_one():
            lib.tfp8b_prep(x.data_ptr(), 1, x16.data_ptr(), xs.data_ptr(), M, K, st())
            rc = lib.tfp8b_gemm(x16.data_ptr(), xs.data_ptr(), q_full.data_ptr(), e8_full.data_ptr(), 1, None, y1.data_ptr(), 0,
                                M, N, K, 32, 0, st())
            assert rc == 0, lib.tfp8b_last_error_string()
        barrier(world)
        t_1 = max_over_ranks(time_eager(step_one, 10, 3), world, device)
        del y1
        barrier(world)
        t_g = max_over_ranks(time_eager(lambda: step(True), 10, 3), world, device)
        barrier(world)
        t_n = max_over_ranks(time_eager(lambda: step(False), 10, 3), world, device)
        fl = 2.0 * M * N * K
        row = {"M": M, "N": N, "K": K, "G": 32, "tp": world, "ms_one_gpu_same_process": t_1 * 1e3,
               "tflops_one_gpu_same_process": fl / t_1 / 1e12,
               "ms_with_gather": t_g * 1e3, "ms_without_gather": t_n * 1e3,
               "tflops_with_gather": fl / t_g / 1e12, "tflops_without_gather": fl / t_n / 1e12,
               "efficiency_nccl_gather": t_1 / t_g / world,
               "frac_tensor_peak_all_gpus": fl / t_g / 1e12 / (world * peaks["bf16_tflops"])}
        if fused_error is None:
            barrier(world)
            t_f = max_over_ranks(time_eager(step_fused, 10, 3), world, device)
            # the fused result must be what NCCL gathers: rank r's shard in columns [r*Nl, (r+1)*Nl)
            step(True)
            got = step_fused()[:M]
            torch.cuda.synchronize()
            want = full.view(world, M, Nl).permute(1, 0, 2).reshape(M, N)
            row.update({"ms_fused_gather": t_f * 1e3, "fused_equals_nccl": bool(torch.equal(got, want)),
                        "tflops_fused_gather": fl / t_f / 1e12, "efficiency_fused_gather": t_1 / t_f / world,
                        "frac_tensor_peak_all_gpus_fused": fl / t_f / 1e12 / (world * peaks["bf16_tflops"])})
            barrier(world)
        else:
            row["fused_gather_unavailable"] = fused_error
        rows.append(row)
        del x, x16, y, full
    return rows


def w8a8_row(device, M, N, K, iters=20, warmup=3):
    """One W8A8 measurement: bf16 activations [M, K] quantized per 32-wide block (quantize_k, packed
    UE8M0 scales) and multiplied with an MX weight [N, K] on tcgen05.mma.kind::mxf8f6f4. The weight
    buffers are rotated so that the stripe is not already in L2 from the previous iteration."""
    from tfp8 import _ext, synth
    copies = max(1, min(4, int(2.2 * 126e6 / (N * K)) + 1))
    g = torch.Generator(device=device).manual_seed(K)
    ws = []
    for _ in range(copies):
        w = (torch.randn(N, K, generator=g, device=device) * 0.015).bfloat16()
        q, s = _ext.quantize_k(w, "e4m3fn", True, packed=True)
        ws.append((q, s))
        del w
    x = synth.activations(M, K, dtype=torch.bfloat16).to(device)
    aq, sa = _ext.quantize_k(x, "e4m3fn", True, packed=True)
    y = torch.empty(M, N, dtype=torch.bfloat16, device=device)
    lib = _ext.load()
    st = lambda: torch.cuda.current_stream().cuda_stream
    turn = [0]

    def step(with_quant=True):
        q, s = ws[turn[0] % copies]
        turn[0] += 1
        if with_quant:
            rc = lib.tfp8b_quantize_k(x.data_ptr(), 1, aq.data_ptr(), sa.data_ptr(), M, K, 0, 1, 1, st())
            assert rc == 0, lib.tfp8b_last_error_string()
        rc = lib.tfp8b_gemm_w8a8(aq.data_ptr(), sa.data_ptr(), 0, q.data_ptr(), s.data_ptr(), 0, 0, 1, None, y.data_ptr(), 1, M, N, K, st())
        assert rc == 0, lib.tfp8b_last_error_string()
    sec = time_eager(step, iters, warmup)
    sec_mm = time_eager(lambda: step(False), iters, warmup)
    fl = 2.0 * M * N * K
    return {"M": M, "N": N, "K": K, "ms_quantize_plus_gemm": sec * 1e3, "ms_gemm": sec_mm * 1e3, "tflops": fl / sec / 1e12,
            "tflops_gemm_only": fl / sec_mm / 1e12, "iterations": iters}


def attention_row(device, kind, B, S, steps, warmup):
    """One decode-attention call of a Llama-3-8B block (32 query / 8 KV heads of 128) over a cache of S
    positions, the query at position S - 200: kind "attn" = the library kernel over a 16-bit cache,
    "attn8" = over an FP8 cache, "sdpa" = torch's attention with a mask over the 16-bit cache. Eight
    distinct caches in turn so that L2 does not hold them."""
    from tfp8 import _ext
    H, KV, hd = 32, 8, 128
    pos = torch.tensor([S - 200], device=device)
    scratch = torch.empty(_ext.attn_scratch_floats(B, H, S, hd), dtype=torch.float32, device=device)
    if kind == "attn8":
        q = torch.randn(B, H, hd, device=device).half()
        ks = [torch.randint(0, 120, (B, KV, S, hd), device=device, dtype=torch.uint8) for _ in range(8)]
        vs = [torch.randint(0, 120, (B, KV, S, hd), device=device, dtype=torch.uint8) for _ in range(8)]
        sc = torch.full((B, KV, S), 2.0 ** -6, device=device)
        call = lambda i: _ext.attn_decode_fp8(q, ks[i], sc, vs[i], sc, pos, scratch)
        per_pos = 2 * (hd + 4)
    else:
        ks = [torch.randn(B, KV, S, hd, device=device).half() for _ in range(8)]
        vs = [torch.randn(B, KV, S, hd, device=device).half() for _ in range(8)]
        per_pos = 4 * hd
        if kind == "attn":
            q = torch.randn(B, H, hd, device=device).half()
            call = lambda i: _ext.attn_decode(q, ks[i], vs[i], pos, scratch)
        else:
            q = torch.randn(B, H, 1, hd, device=device).half()
            mask = torch.where(torch.arange(S, device=device)[None, :] <= pos[:, None], 0.0, float("-inf")).half()
            call = lambda i: torch.nn.functional.scaled_dot_product_attention(q, ks[i], vs[i], attn_mask=mask, enable_gqa=True)

    def step():
        for i in range(8):
            call(i)
    sec = time_steps_in_graphs(step, steps, warmup) / 8
    byt = B * KV * (S - 199) * per_pos
    return {"kind": kind, "batch": B, "cache_positions": S - 199, "us_per_call": sec * 1e6, "kv_bytes": byt, "gbs": byt / sec / 1e9}


def run_probe(args):
    """`--probe gemm:M,N,K,G` / `--probe gemv:M,N,K,G`: a few launches of one kernel on one shape
    (a small, self-ending case for profiler captures). Prints one JSON line with the timing."""
    from tfp8 import _ext, synth
    kind, dims = args.probe.split(":")
    M, N, K, G = (int(v) for v in (dims.split(",") + ["32", "32", "32"])[:4])
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    lib = _ext.load()
    if kind == "w8a8":
        print(json.dumps({"probe": args.probe, **w8a8_row(device, M, N, K, args.steps, args.warmup)}))
        return
    if kind in ("attn", "attn8", "sdpa"):
        # attn:B,S / attn8:B,S / sdpa:B,S -- one decode-attention call, see attention_row
        print(json.dumps({"probe": args.probe, **attention_row(device, kind, M, N, args.steps, args.warmup)}))
        return
    if kind == "decode":
        # decode:B,layers,prompt -- a Llama-3-8B-shaped decoder cut to `layers` blocks: prefill, capture,
        # then `steps` graph-replayed decode steps (a launch list of one step under a profiler)
        from tfp8.examples.llama import LlamaConfig, DecodeRunner, build_fp8_llama
        B, layers, prompt = M, N, K
        cfg = LlamaConfig(n_layers=layers, max_seq=prompt + max(64, args.steps + 8))
        model = build_fp8_llama(cfg, device, torch.float16)
        # TFP8_PROBE_ATTN=kernel: the library's decode attention instead of torch's; =fp8: that kernel over an FP8 KV cache
        mode = os.environ.get("TFP8_PROBE_ATTN", "")
        model.attn_kernel = mode == "kernel"
        model.kv_fmt = "e4m3fn" if mode == "fp8" else None
        run = DecodeRunner(model, B)
        run.prefill(torch.randint(0, cfg.vocab, (B, prompt), device=device))
        run.capture()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); run.decode(args.steps); e1.record(); torch.cuda.synchronize()
        print(json.dumps({"probe": args.probe, "batch": B, "layers": layers, "ms_per_step": e0.elapsed_time(e1) / args.steps}))
        return
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
            "config": {"workload": "decode GEMV sweep (M=1, the four Llama-7B layer shapes), bounded sample on the host cores"},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def run_reference_gpu(args):
    """The reference's OWN GPU kernels on this GPU, beside this build's: its Python package is
    imported unmodified from oracle/_ref/tfp8_reference (staged by `make -C oracle` where the
    reference checkout exists) and compiles its sm_75-era kernels with NVRTC for the device it
    finds, exactly as it does on the authors' machine. Same inputs, same rotation over distinct
    weight buffers (> 2x L2), CUDA-event loops, interleaved A/B as the reference's own benches do
    (tests/perf_decode.py:32-48 there). Prints one JSON line; not part of the default run."""
    ref = reference_package()
    if ref is None:
        print(json.dumps({"impl": "reference-gpu", "unavailable": "oracle/_ref/tfp8_reference is not staged (build where the reference checkout exists)"}))
        return
    import tfp8
    from tfp8 import synth
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    if not ref._ext.available():
        print(json.dumps({"impl": "reference-gpu", "unavailable": f"the reference's NVRTC kernels did not load: {ref._ext.last_error()}"[:300]}))
        return
    peaks = measured_peaks()
    rows = []

    def ab(make_ref, make_ours, x, copies, rounds=7, inner=20):
        """Median over rounds of the per-call time of each side, the sides alternating."""
        ref_layers, our_layers = [make_ref(c) for c in range(copies)], [make_ours(c) for c in range(copies)]
        for l in ref_layers + our_layers:
            for _ in range(4):                       # past the NaN-checked calls, kernels compiled
                l(x)
        tr, to = [], []
        for _ in range(rounds):
            for side, layers, acc in (("ref", ref_layers, tr), ("ours", our_layers, to)):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                for _ in range(inner):
                    for l in layers:
                        l(x)
                e1.record()
                torch.cuda.synchronize()
                acc.append(e0.elapsed_time(e1) / 1e3 / (inner * copies))
        return float(np.median(tr)), float(np.median(to))

    for (N, K) in synth.DECODE_SHAPES:
        copies = max(2, int(np.ceil(2.2 * 126e6 / (N * K))))
        qs = [synth.random_codes(N, K, torch.float8_e4m3fn, seed=c).to(device) for c in range(copies)]
        sc = torch.full((N, 1), 2.0 ** -13, device=device)
        for M in (1, 8):
            x = synth.activations(M, K).to(device)
            t_ref, t_ours = ab(lambda c: ref.FP8Linear.from_fp8_checkpoint(qs[c], sc, None, "e4m3fn", out_dtype=torch.float16),
                               lambda c: tfp8.FP8Linear.from_fp8_checkpoint(qs[c], sc, None, "e4m3fn", out_dtype=torch.float16), x, copies)
            b = gemv_bytes(M, N, K, K)
            rows.append({"op": "FP8Linear.forward", "M": M, "N": N, "K": K, "reference_us": t_ref * 1e6, "ours_us": t_ours * 1e6,
                         "reference_gbs": b / t_ref / 1e9, "ours_gbs": b / t_ours / 1e9, "speedup": t_ref / t_ours,
                         "note": "eager calls through each package's own FP8Linear (Python launch overhead included on both sides)"})
        del qs
    # prefill-size GEMM: the reference's fused WMMA kernel and its chunked dequant + cuBLAS path
    N, K, M = 4096, 4096, 2048
    q = synth.random_codes(N, K, torch.float8_e4m3fn, seed=1).to(device)
    sc = torch.full((N, 1), 2.0 ** -13, device=device)
    x = synth.activations(M, K).to(device)
    for backend in ("fused", "chunked"):
        t_ref, t_ours = ab(lambda c: ref.FP8Linear.from_fp8_checkpoint(q, sc, None, "e4m3fn", out_dtype=torch.float16, large_m_backend=backend),
                           lambda c: tfp8.FP8Linear.from_fp8_checkpoint(q, sc, None, "e4m3fn", out_dtype=torch.float16), x, 1, rounds=5, inner=10)
        fl = 2.0 * M * N * K
        rows.append({"op": f"FP8Linear.forward (reference large_m_backend={backend})", "M": M, "N": N, "K": K,
                     "reference_ms": t_ref * 1e3, "ours_ms": t_ours * 1e3, "reference_tflops": fl / t_ref / 1e12,
                     "ours_tflops": fl / t_ours / 1e12, "speedup": t_ref / t_ours})
    print(json.dumps({"impl": "reference-gpu", "device": torch.cuda.get_device_name(0), "peaks": peaks, "rows": rows}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference", "reference-gpu"))
    ap.add_argument("--quick", action="store_true", help="headline only: skip the per-shape / GEMM / codec tables")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-llama", action="store_true", help="skip the Llama-3-8B decode measurement")
    ap.add_argument("--probe", default=None, help="gemm:M,N,K,G, gemv:M,N,K,G, w8a8:M,N,K, attn:B,S, attn8:B,S or decode:B,layers,prompt -- a few launches of one kernel (profiling)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.probe:
        run_probe(args)
        return
    if args.impl == "reference-gpu":
        run_reference_gpu(args)
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
