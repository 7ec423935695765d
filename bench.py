#!/usr/bin/env python
"""Benchmark of the W4A32 quantized-linear path on B200.

Headline workload ("qwen2-1.5b-decode-linears"): one decode token's worth of quantized linears of
the Qwen2-1.5B architecture - 28 decoder layers x the seven linears q,k,v,o,gate,up,down at M=1
(BASELINE config 1 at decode, once per layer) - every layer with its own weights (737 MB of
int4+scales per step, larger than the 126 MB L2, so no flush is needed between steps) and every
linear with its own input and output buffer.  A step is one pass over those 196 linears through the
C ABI, replayed as a CUDA graph.  Three call structures are measured in every run:
  layer   (default headline) one mllmb200_w4a32_linear_forward_multi call per layer: the seven
          independent linears of config 1 in ONE launch (28 launches per step);
  grouped the calls a decoder makes: (q,k,v) (o) (gate,up) (down), linears that share their
          activations sharing a call (mllmb200_w4a32_linear_forward_grouped; 112 launches per step);
  per-op  one mllmb200_w4a32_linear_forward per linear, as the reference's engine dispatches ops
          (196 launches per step).
`--calls grouped|per-op` makes one of the others the headline; all three are always reported
(`call_structures`).  The metric is algorithmic HBM bytes per second: nibbles + scales + bias +
fp32 x + fp32 y of every linear, divided by the device time (CUDA events on the launching stream,
median over at least 5 timed regions of --steps steps each, max over ranks).

Extra objects in the JSON line: `roofline` (GEMV kernel vs the measured HBM copy bandwidth),
`prefill` (the same seven linears at M=512, TFLOP/s), `e2e` (host buffers in, host buffers out),
`cpu_baseline` (the reference's X86 int4 kernels on the host cores), `per_shape`, `clocks`, and on one GPU
`config4` (the 28672 x 8192 matrix: GEMV at M=1, GEMM at M=2048), `w4a16` (the W4A16 sibling path on the same
shapes) and `decoder` (512-token prefill + 128 greedy steps of the whole model).

With N > 1 ranks (torchrun) every rank serves its own token (independent replicas, weak scaling,
no collective on the data path), and rank 0 adds a `tp` object: the column-sharded large linear of
BASELINE config 4 with an NCCL all-gather of y.

`--impl reference` times the reference's CPU path for the same workload on the host cores.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "mllm-advanced_b200"))

LAYERS = 28
# name, K, N, has_bias  (mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:38-44,86-93 of the reference project)
LINEARS = [("q", 1536, 1536, True), ("k", 1536, 256, True), ("v", 1536, 256, True), ("o", 1536, 1536, False),
           ("gate", 1536, 8960, False), ("up", 1536, 8960, False), ("down", 8960, 1536, False)]
PREFILL_M = 512
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def algorithmic_bytes(m, k, n, has_bias):
    return n * k // 2 + n * (k // 32) * 2 + m * k * 4 + m * n * 4 + (n * 4 if has_bias else 0)


def workload_config():
    """The `config` object both arms print: it names the workload, nothing arm-specific."""
    step_bytes = LAYERS * sum(algorithmic_bytes(1, k, n, hb) for _, k, n, hb in LINEARS)
    return {"workload": "qwen2-1.5b-decode-linears", "layers": LAYERS, "linears_per_layer": len(LINEARS), "M": 1,
            "weight_bytes_per_step": LAYERS * 26320896, "algorithmic_bytes_per_step": step_bytes,
            "l2": "737 MB of weights per step > 126 MB L2: no flush between steps"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d.get("bf16_tflops"))), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.samples, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass

    def summary(self, t0, t1):
        sm, mx, reasons = [], 0.0, set()
        for t, line in self.samples:
            if t < t0 - 0.05 or t > t1 + 0.05:
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:  # region shorter than the sampling period: use every sample we have
            for _, line in self.samples:
                parts = [p.strip() for p in line.split(",")]
                try:
                    sm.append(float(parts[0]))
                    mx = max(mx, float(parts[1]))
                except (ValueError, IndexError):
                    pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------ CPU baselines
def cpu_has(flag):
    try:
        return flag in open("/proc/cpuinfo").read()
    except Exception:
        return False


def load_x86_ref():
    d = os.path.join(ROOT, "oracle", "_ref")
    names = (["libx86q4k_ref_avx512.so"] if cpu_has("avx512f") and cpu_has("avx512bw") else []) + ["libx86q4k_ref_avx2.so"]
    for n in names:
        p = os.path.join(d, n)
        if os.path.exists(p):
            L = C.CDLL(p)
            L.x86ref_q4k_row_bytes.restype = C.c_size_t
            L.x86ref_q8k_row_bytes.restype = C.c_size_t
            L.x86ref_quantize_weights.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
            L.x86ref_linear.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                        C.c_int, C.c_void_p]
            return L, n
    return None, None


def time_reference_cpu(budget_s=12.0, steps=None, warmup=1, max_threads=None):
    """One decoder layer's seven linears at M=1 on the reference's X86 int4 kernels (Q4_K x Q8_K -
    a different int4 format from the Arm W4A32 path, same 0.5625 bytes per weight), all host threads.
    Returns (GB/s over the algorithmic W4A32 bytes of those linears, info dict)."""
    L, libname = load_x86_ref()
    if L is None:
        return None, {"why": "oracle/_ref/libx86q4k_ref_*.so not built"}
    rng = np.random.default_rng(0)
    threads = L.x86ref_max_threads()
    if max_threads:
        threads = min(threads, max_threads)
    variant = 1 if L.x86ref_has_avx512() else 0
    mats = []
    for name, k, n, hb in LINEARS:
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        wq = np.empty(n * L.x86ref_q4k_row_bytes(k), np.uint8)
        L.x86ref_quantize_weights(w.ctypes.data, n, k, wq.ctypes.data)
        x = rng.standard_normal((1, k)).astype(np.float32)
        y = np.empty((1, n), np.float32)
        ws = np.empty(L.x86ref_q8k_row_bytes(k) + 64, np.uint8)
        mats.append((k, n, hb, wq, x, y, ws))

    def one_pass():
        for k, n, hb, wq, x, y, ws in mats:
            L.x86ref_linear(x.ctypes.data, wq.ctypes.data, y.ctypes.data, 1, n, k, threads, variant, ws.ctypes.data)

    for _ in range(max(1, warmup)):
        one_pass()
    t0 = time.perf_counter()
    one_pass()
    dt1 = time.perf_counter() - t0
    reps = steps if steps else int(max(3, min(2000, budget_s / max(dt1, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(reps):
        one_pass()
    dt = (time.perf_counter() - t0) / reps
    nbytes = sum(algorithmic_bytes(1, k, n, hb) for _, k, n, hb in LINEARS)
    return nbytes / dt / 1e9, {"cores": threads, "lib": libname, "variant": "avx512f" if variant else "avx2",
                              "ms_per_layer": dt * 1e3, "reps": reps,
                              "sample": f"one decoder layer (7 linears, M=1) x {reps} passes, Q4_K x Q8_K kernels of the "
                                        "reference X86 backend, OpenMP over output rows"}


def time_oracle_port(budget_s=6.0):
    """The same sample on the C restatement of the W4A32 arithmetic (same format as the GPU path)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import Oracle
    o = Oracle()
    rng = np.random.default_rng(0)
    mats = []
    for name, k, n, hb in LINEARS:
        q = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
        s = ((np.abs(rng.standard_normal((n, k // 32))) * 0.02 / 7).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
        x = rng.standard_normal((1, k)).astype(np.float32)
        mats.append((x, q, s))
    t0 = time.perf_counter()
    for x, q, s in mats:
        o.linear(x, q, s)
    dt1 = time.perf_counter() - t0
    reps = int(max(2, min(200, budget_s / max(dt1, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(reps):
        for x, q, s in mats:
            o.linear(x, q, s)
    dt = (time.perf_counter() - t0) / reps
    nbytes = sum(algorithmic_bytes(1, k, n, hb) for _, k, n, hb in LINEARS)
    return nbytes / dt / 1e9, o.lib.oracle_num_threads(), dt * 1e3


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # a multi-process launcher pins every rank to one OpenMP thread; this arm runs on rank 0 alone and
    # is meant to use all the host threads (the variable is read when the OpenMP runtime starts, i.e.
    # when the kernels' library is loaded below)
    if os.environ.get("OMP_NUM_THREADS") == "1" and "LOCAL_RANK" in os.environ:
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    val, info = time_reference_cpu(budget_s=20.0, steps=None, warmup=max(1, args.warmup))
    if val is None:
        print(json.dumps({"impl": "reference", "unavailable": info["why"]}))
        return
    step_bytes = LAYERS * sum(algorithmic_bytes(1, k, n, hb) for _, k, n, hb in LINEARS)
    ms_per_step = step_bytes / (val * 1e9) * 1e3
    line = {"impl": "reference", "metric": "W4A32 decode-linear HBM GB/s", "value": val, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int4 -> int32 -> f32",
            "data": "synthetic",
            "config": workload_config(),
            "run": {"note": "each step of this arm is a bounded sample: one layer's 7 linears; ms_per_step scales it to 28 layers"},
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": info["cores"], "kind": "reference",
                             "sample": info["sample"], "variant": info["variant"]},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------ GPU side
def make_random_weights(mb, torch, n, k, has_bias, gen, scale_mode=0):
    """Random int4 (uniform in -7..7) + scales |N(0, 0.02)| / 7 (BASELINE config 0 distributions), assembled as a blob
    on the device and repacked there: no host quantization of 1.3 G weights."""
    dev = "cuda"
    total = mb.prepack_size(n, k, has_bias)
    blob = torch.zeros(total, dtype=torch.uint8, device=dev)
    # section offsets of a blob of this shape (the repack takes the shape as arguments, not from the header)
    a, b, c = C.c_size_t(), C.c_size_t(), C.c_size_t()
    mb.lib().mllmb200_w4a32_blob_offsets(n, k, int(has_bias), C.byref(a), C.byref(b), C.byref(c))
    # int4 values uniform in -7..7 (stored +8): zero-mean rows, as a symmetric quantizer leaves them.  With the full
    # 0..15 range every row has mean -0.5 scale units, and the common-mode term that gives a 28-layer random stack
    # (the same all-negative vector added by every layer) drowns the token embedding in the residual stream.
    lo = torch.randint(1, 16, (n * (k // 2),), dtype=torch.uint8, device=dev, generator=gen)
    hi = torch.randint(1, 16, (n * (k // 2),), dtype=torch.uint8, device=dev, generator=gen)
    nib = lo | (hi << 4)
    del lo, hi
    sc = (torch.randn((n * (k // 32),), device=dev, generator=gen).abs() * (0.02 / 7.0))
    sc16 = (sc.view(torch.int32) >> 16).to(torch.int16)
    blob[a.value:a.value + nib.numel()] = nib
    blob[b.value:b.value + sc16.numel() * 2] = sc16.view(torch.uint8)
    if has_bias:
        bias = torch.randn((n,), device=dev, generator=gen) * 0.02
        blob[c.value:c.value + n * 4] = bias.view(torch.uint8)
    tiled = torch.empty(mb.tiled_size(n, k), dtype=torch.uint8, device=dev)
    st = mb.lib().mllmb200_w4a32_repack_device(blob.data_ptr(), n, k, scale_mode, int(has_bias), 0, n, tiled.data_ptr(),
                                               C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0, mb.status_str(st)
    torch.cuda.synchronize()
    return mb.W4A32Weights(tiled, n, k, scale_mode, int(has_bias))


def event_time_ms(torch, fn, iters):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def run_gpu(args):
    import torch
    import mllm_b200 as mb

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    mb.lib()  # fails loudly when the CUDA library is missing
    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)

    if args.prefill_only:
        lw = [make_random_weights(mb, torch, n, k, hb, gen) for _, k, n, hb in LINEARS]
        ws = torch.empty(mb.workspace_size(PREFILL_M, 8960), dtype=torch.uint8, device="cuda")
        xp = {k: torch.randn((PREFILL_M, k), device="cuda", generator=gen) for k in (1536, 8960)}
        kern = mb.KERNEL_TC_F16 if args.prefill_f16 else mb.KERNEL_AUTO
        for _ in range(max(1, args.steps)):
            if args.prefill_grouped:  # the call structure of prefill_fastest_grouped: 4 quantizations + 4 GEMM launches
                mb.linear_forward_grouped(xp[1536], lw[0:3], workspace=ws, policy=mb.KERNEL_FASTEST)
                mb.linear_forward(xp[1536], lw[3], workspace=ws, kernel=mb.KERNEL_FASTEST)
                mb.linear_forward_grouped(xp[1536], lw[4:6], workspace=ws, policy=mb.KERNEL_FASTEST)
                mb.linear_forward(xp[8960], lw[6], workspace=ws, kernel=mb.KERNEL_FASTEST)
                continue
            for w in lw:
                mb.linear_forward(xp[w.k], w, workspace=ws, kernel=kern)
        torch.cuda.synchronize()
        mb.check_device_status()
        print(json.dumps({"prefill_only": True, "M": PREFILL_M, "passes": max(1, args.steps)}))
        return

    if args.config4_only:
        print(json.dumps({"config4": run_config4(args, torch, mb, gen, hbm_peak, tensor_peak, peak_kind)}), flush=True)
        return
    if args.w4a16_only:
        print(json.dumps({"w4a16": run_w4a16(args, torch, mb, gen, hbm_peak, tensor_peak, peak_kind)}), flush=True)
        return

    # ---- weights: 28 layers x 7 linears, each its own tiled buffer
    if args.batched_only:
        # the batched decode section alone on a model of --decoder-layers layers (small captures under a profiler)
        few = [[make_random_weights(mb, torch, n, k, hb, gen) for _, k, n, hb in LINEARS] for _ in range(args.decoder_layers)]
        print(json.dumps({"batched": run_decoder(args, torch, mb, few, gen, hbm_peak, peak_kind, batched_only=True)}), flush=True)
        return
    layers = [[make_random_weights(mb, torch, n, k, hb, gen) for _, k, n, hb in LINEARS] for _ in range(LAYERS)]
    if args.decoder_only:
        print(json.dumps({"decoder": run_decoder(args, torch, mb, layers, gen, hbm_peak, peak_kind)}), flush=True)
        return
    # every linear of a layer has its own activations and output (BASELINE config 1); they are slices of one
    # buffer each so that the end-to-end leg can move a layer's inputs and outputs with one copy per direction
    x_all = torch.randn((sum(k for _, k, _, _ in LINEARS),), device="cuda", generator=gen)
    y_all = torch.empty((sum(n for _, _, n, _ in LINEARS),), device="cuda")
    xs7, ys7, xo, yo = [], [], 0, 0
    for _, k, n, _ in LINEARS:
        xs7.append(x_all[xo:xo + k].view(1, k))
        ys7.append(y_all[yo:yo + n].view(1, n))
        xo, yo = xo + k, yo + n
    xs = {1536: xs7[0], 8960: xs7[6]}
    ys = {1536: ys7[0], 256: ys7[1], 8960: ys7[4]}
    stream = torch.cuda.Stream()
    pdl = not args.no_pdl
    ws = torch.empty(mb.workspace_size(PREFILL_M, 8960), dtype=torch.uint8, device="cuda")

    def layer_pass():  # one call per layer: the seven independent linears in one launch
        for lw in layers:
            mb.linear_forward_multi(xs7, lw, outs=ys7, stream=stream, pdl=pdl)

    def grouped_pass():  # linears that read the same activations share a call: (q,k,v) (o) (gate,up) (down)
        for lw in layers:
            mb.linear_forward_grouped(xs7[0], lw[0:3], outs=ys7[0:3], workspace=ws, stream=stream, pdl=pdl)
            mb.linear_forward(xs7[3], lw[3], out=ys7[3], workspace=ws, stream=stream, pdl=pdl)
            mb.linear_forward_grouped(xs7[4], lw[4:6], outs=ys7[4:6], workspace=ws, stream=stream, pdl=pdl)
            mb.linear_forward(xs7[6], lw[6], out=ys7[6], workspace=ws, stream=stream, pdl=pdl)

    def per_op_pass():  # one C-ABI call per linear: 7 per layer
        for lw in layers:
            for i, w in enumerate(lw):
                mb.linear_forward(xs7[i], w, out=ys7[i], workspace=ws, stream=stream, pdl=pdl)

    structures = {"layer": (layer_pass, 1, "one call per layer: the seven independent linears of BASELINE config 1 in one launch"),
                  "grouped": (grouped_pass, 4, "calls per layer: (q,k,v) (o) (gate,up) (down) - linears sharing their activations share a call"),
                  "per-op": (per_op_pass, len(LINEARS), "one call per linear (7 per layer), as the reference's engine dispatches ops")}
    decode_pass, calls_per_layer, structure_note = structures[args.calls]
    calls_per_step = LAYERS * calls_per_layer
    launches_per_step = calls_per_step  # every call is ONE launch: the GEMV quantizes the activations itself
    step_bytes = LAYERS * sum(algorithmic_bytes(1, k, n, hb) for _, k, n, hb in LINEARS)

    def capture(fn):
        with torch.cuda.stream(stream):
            fn()  # configures kernel attributes before capture
        stream.synchronize()
        mb.check_device_status(stream)
        if args.no_graph:
            return None
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
        return g

    graph = capture(decode_pass)

    def step():
        if graph is not None:
            graph.replay()
        else:
            with torch.cuda.stream(stream):
                decode_pass()

    sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    # graph.replay() launches on torch's current stream: time on that stream
    timing_stream = torch.cuda.current_stream() if graph is not None else stream
    # Timed regions of exactly --steps steps each, bracketed by a barrier and a synchronize on both sides.  At
    # least 5 of them, and as many more as it takes to keep the GPU under this load for ~0.7 s, so that the clock
    # sampler (one sample per 50 ms) sees the timed work at least ten times.  The reported time is the median region.
    regions = []
    t_wall0 = time.time()
    while len(regions) < 5 or (time.time() - t_wall0 < 0.7 and len(regions) < 400):
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(timing_stream)
        for _ in range(args.steps):
            step()
        e1.record(timing_stream)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        ms_region = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms_region, float(len(regions) >= 4 and time.time() - t_wall0 >= 0.7)], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)  # the slowest rank's time; and every rank stops in the same round
            ms_region = float(t[0].item())
            regions.append(ms_region)
            if t[1].item() > 0:
                break
        else:
            regions.append(ms_region)
    t_wall1 = time.time()
    ms_total = float(np.median(regions))
    ms_per_step = ms_total / args.steps
    mb.check_device_status()
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- everything below is extra reporting, outside the headline timed region
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "frac_of_8TBs_spec": achieved / 8000.0, "peak_kind": f"of {peak_kind}", "traffic": None,
                "kernel": "w4a32_gemv_stream_kernel<1>", "gemv_launches_per_step": launches_per_step,
                "avg_gemv_launch_us": ms_per_step * 1e3 / launches_per_step,
                "algorithmic_bytes_per_gemv_launch": step_bytes / launches_per_step,
                "note": "achieved = algorithmic bytes of the step / device time of the step; a launch quantizes its "
                        "activations itself (no separate kernel)"}
    # dram__bytes_read + dram__bytes_write per launch of the layer call, from the ncu capture summarized in
    # profiles/gemv_decode_qwen2_1p5b.md (kept as numbers in the .json beside it)
    try:
        prof = json.load(open(os.path.join(ROOT, "profiles", "gemv_decode_qwen2_1p5b.json")))
        if args.calls in prof.get("dram_bytes_per_launch", {}):
            roofline["traffic"] = prof["dram_bytes_per_launch"][args.calls]
            roofline["traffic_note"] = prof.get("note")
    except Exception as ex:
        roofline["traffic_note"] = f"profiles/gemv_decode_qwen2_1p5b.json unreadable: {str(ex)[:80]}"

    line = {"metric": "W4A32 decode-linear HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int4 -> int32 -> f32", "data": "synthetic",
            "config": workload_config(),
            "run": {"calls": args.calls, "calls_per_step": calls_per_step,
                    "launch": ("cuda-graph replay" if graph is not None else "stream launches") + (", PDL" if pdl else "")
                              + ", " + structure_note,
                    "timing": f"median of {len(regions)} regions of {args.steps} steps",
                    "parallelism": "replicas (one token per GPU)" if world > 1 else "single GPU"},
            "roofline": roofline, "gpu_launches": args.steps * launches_per_step,
            "timed_regions_ms": [round(r, 4) for r in regions[:12]],
            "tokens_per_s_linears_only": world * 1e3 / ms_per_step}

    if rank == 0:
        sampler.stop()
        line["clocks"] = sampler.summary(t_wall0, t_wall1)

    if rank == 0:
        # the other call structures over the same weights (device time, graph replay, median of 5 x 10 steps)
        cs = {args.calls: {"calls_per_layer": calls_per_layer, "ms_per_step": ms_per_step, "GBs": achieved,
                           "frac": achieved / hbm_peak}}
        for name, (fn, cpl, _) in structures.items():
            if name == args.calls or (args.quick and not args.all_structures):
                continue
            gg = capture(fn)
            run = gg.replay if gg is not None else (lambda fn=fn: fn())
            for _ in range(3):
                run()
            ms_g = float(np.median([event_time_ms(torch, run, 10) for _ in range(5)]))
            cs[name] = {"calls_per_layer": cpl, "ms_per_step": ms_g, "GBs": step_bytes / (ms_g * 1e-3) / 1e9,
                        "frac": step_bytes / (ms_g * 1e-3) / 1e9 / hbm_peak}
            del gg
        line["call_structures"] = cs
        for name, v in cs.items():
            roofline[f"frac_{name.replace('-', '_')}_calls"] = v["frac"]

    # ---- end to end, on every rank at the same time (N replicas, as the headline)
    e2e_line = None
    if not args.quick:
        if dist is not None:
            dist.barrier()
        # e2e: the same step with HOST buffers (pinned) through the C ABI: one cudaMemcpyAsync H2D of the step's inputs
        # (every layer's seven x), the 28 layer calls on their slices, one cudaMemcpyAsync D2H of the step's outputs
        # (every layer's seven y); one CUDA graph per step and a host synchronize after every step because the host
        # reads y.  Host wall clock: launch and synchronize included.
        nx, ny = x_all.numel(), y_all.numel()
        hx_all = torch.randn((LAYERS, nx)).pin_memory()
        hy_all = torch.empty((LAYERS, ny)).pin_memory()
        dx_all = torch.empty((LAYERS, nx), device="cuda")
        dy_all = torch.empty((LAYERS, ny), device="cuda")
        xs_l, ys_l = [], []
        for l in range(LAYERS):
            xo = yo = 0
            xs_l.append([])
            ys_l.append([])
            for _, k, n, _ in LINEARS:
                xs_l[l].append(dx_all[l, xo:xo + k].view(1, k))
                ys_l[l].append(dy_all[l, yo:yo + n].view(1, n))
                xo += k
                yo += n

        def e2e_pass():
            dx_all.copy_(hx_all, non_blocking=True)
            for l, lw in enumerate(layers):
                xs, ys = xs_l[l], ys_l[l]
                if args.calls == "layer":
                    mb.linear_forward_multi(xs, lw, outs=ys, stream=stream, pdl=pdl)
                elif args.calls == "grouped":
                    mb.linear_forward_grouped(xs[0], lw[0:3], outs=ys[0:3], workspace=ws, stream=stream, pdl=pdl)
                    mb.linear_forward(xs[3], lw[3], out=ys[3], workspace=ws, stream=stream, pdl=pdl)
                    mb.linear_forward_grouped(xs[4], lw[4:6], outs=ys[4:6], workspace=ws, stream=stream, pdl=pdl)
                    mb.linear_forward(xs[6], lw[6], out=ys[6], workspace=ws, stream=stream, pdl=pdl)
                else:
                    for i, w in enumerate(lw):
                        mb.linear_forward(xs[i], w, out=ys[i], workspace=ws, stream=stream, pdl=pdl)
            hy_all.copy_(dy_all, non_blocking=True)

        h2d = LAYERS * x_all.numel() * 4
        d2h = LAYERS * y_all.numel() * 4
        try:
            with torch.cuda.stream(stream):
                e2e_pass()
            stream.synchronize()
            mb.check_device_status(stream)
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, stream=stream):
                e2e_pass()
            for _ in range(3):
                g2.replay()
            torch.cuda.synchronize()
            iters = max(5, args.steps)
            samples = []
            for _ in range(5):
                t0 = time.perf_counter()
                for _ in range(iters):
                    g2.replay()
                    torch.cuda.current_stream().synchronize()  # the host reads y after every step
                    _ = float(hy_all[LAYERS - 1, 0])
                samples.append((time.perf_counter() - t0) * 1e3 / iters)
            ms_serial = float(np.median(samples))
            hy_serial = hy_all.clone()
            del g2
            # The same steps two deep: while the GPU computes step i, step i + 1's inputs go up on a copy stream and step
            # i - 1's outputs come down on another (PCIe is full duplex), each step in its own device and host buffers;
            # the host reads step i - 1's y while step i runs.  Every step still makes its own H2D and D2H copy and
            # the host still reads every step's result - one step later.
            DEPTH = 2
            cin, cout = torch.cuda.Stream(), torch.cuda.Stream()
            hx_s = [hx_all] + [torch.randn((LAYERS, nx)).pin_memory() for _ in range(DEPTH - 1)]
            hy_s = [hy_all] + [torch.empty((LAYERS, ny)).pin_memory() for _ in range(DEPTH - 1)]
            slots = [(dx_all, dy_all, xs_l, ys_l)]
            for _ in range(DEPTH - 1):
                dxa = torch.empty((LAYERS, nx), device="cuda")
                dya = torch.empty((LAYERS, ny), device="cuda")
                xl, yl = [], []
                for l in range(LAYERS):
                    xo = yo = 0
                    xl.append([])
                    yl.append([])
                    for _, k, n, _ in LINEARS:
                        xl[l].append(dxa[l, xo:xo + k].view(1, k))
                        yl[l].append(dya[l, yo:yo + n].view(1, n))
                        xo += k
                        yo += n
                slots.append((dxa, dya, xl, yl))

            def compute_pass(xl, yl):
                for l, lw in enumerate(layers):
                    xs, ys = xl[l], yl[l]
                    if args.calls == "layer":
                        mb.linear_forward_multi(xs, lw, outs=ys, stream=stream, pdl=pdl)
                    elif args.calls == "grouped":
                        mb.linear_forward_grouped(xs[0], lw[0:3], outs=ys[0:3], workspace=ws, stream=stream, pdl=pdl)
                        mb.linear_forward(xs[3], lw[3], out=ys[3], workspace=ws, stream=stream, pdl=pdl)
                        mb.linear_forward_grouped(xs[4], lw[4:6], outs=ys[4:6], workspace=ws, stream=stream, pdl=pdl)
                        mb.linear_forward(xs[6], lw[6], out=ys[6], workspace=ws, stream=stream, pdl=pdl)
                    else:
                        for i, w in enumerate(lw):
                            mb.linear_forward(xs[i], w, out=ys[i], workspace=ws, stream=stream, pdl=pdl)

            graphs = []
            for (_, _, xl, yl) in slots:
                with torch.cuda.stream(stream):
                    compute_pass(xl, yl)
                stream.synchronize()
                gs = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gs, stream=stream):
                    compute_pass(xl, yl)
                graphs.append(gs)
            up = [torch.cuda.Event() for _ in range(DEPTH)]
            done = [torch.cuda.Event() for _ in range(DEPTH)]
            down = [torch.cuda.Event() for _ in range(DEPTH)]

            def issue(i):
                sl = i % DEPTH
                dxa, dya, _, _ = slots[sl]
                with torch.cuda.stream(cin):
                    cin.wait_event(done[sl])       # the step that last read this slot's x has finished
                    dxa.copy_(hx_s[sl], non_blocking=True)
                    up[sl].record(cin)
                with torch.cuda.stream(stream):
                    stream.wait_event(up[sl])
                    stream.wait_event(down[sl])    # this slot's y of two steps ago has been copied out
                    graphs[sl].replay()
                    done[sl].record(stream)
                with torch.cuda.stream(cout):
                    cout.wait_event(done[sl])
                    hy_s[sl].copy_(dya, non_blocking=True)
                    down[sl].record(cout)

            def pipelined(n_steps):
                for i in range(n_steps):
                    issue(i)
                    if i >= 1:                     # the host reads the previous step's y while this one runs
                        down[(i - 1) % DEPTH].synchronize()
                        _ = float(hy_s[(i - 1) % DEPTH][LAYERS - 1, 0])
                down[(n_steps - 1) % DEPTH].synchronize()
                _ = float(hy_s[(n_steps - 1) % DEPTH][LAYERS - 1, 0])

            pipelined(4)
            torch.cuda.synchronize()
            mb.check_device_status(stream)
            samples = []
            for _ in range(5):
                t0 = time.perf_counter()
                pipelined(iters)
                samples.append((time.perf_counter() - t0) * 1e3 / iters)
            ms_e2e = float(np.median(samples))
            torch.cuda.synchronize()
            # the pipelined step's outputs against the serial graph's (same inputs in slot 0)
            e2e_same = bool(torch.equal(hy_s[0], hy_serial)) and bool(torch.isfinite(hy_s[DEPTH - 1]).all())
            del graphs
        except Exception as ex:
            ms_e2e, ms_serial, e2e_same, e2e_err = -1.0, -1.0, False, str(ex)[:200]
        else:
            e2e_err = None if e2e_same else "the pipelined steps' outputs differ from the serial step's"
        if dist is not None:  # every rank ran its own copy of the step at the same time: the slowest one counts
            t = torch.tensor([ms_e2e, 1.0 if e2e_err is None else 0.0, ms_serial], device="cuda")
            tmax, tmin = t.clone(), t.clone()
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
            ms_e2e = float(tmax[0].item())
            ms_serial = float(tmax[2].item())
            if float(tmin[1].item()) == 0.0 and e2e_err is None:
                e2e_err = "another rank failed"
        if e2e_err is None:
            e2e_line = {"value": world * step_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e,
                        "h2d_bytes_per_step": world * h2d, "d2h_bytes_per_step": world * d2h,
                        "transfer": "cudaMemcpyAsync, pinned host memory", "pipeline_depth": 2,
                        "serial": {"ms_per_step": ms_serial, "value": world * step_bytes / (ms_serial * 1e-3) / 1e9,
                                   "how": "the same step with nothing overlapped: H2D, the 28 calls, D2H and the host's read "
                                          "one after the other (one CUDA graph, one stream)"},
                        "how": "per step and rank: every layer's seven x in pinned host memory -> ONE H2D copy -> the 28 C-ABI "
                               "layer calls on their slices (one CUDA graph) -> ONE D2H copy of every layer's seven y into pinned "
                               "host memory -> the host reads y; steps run two deep: step i+1's H2D and step i-1's D2H and host "
                               "read overlap step i's calls (copy streams, events, two sets of buffers); host wall clock, median "
                               "of 5 x %d steps, max over ranks; value = all ranks' bytes / that time" % max(5, args.steps)}
        else:
            e2e_line = {"error": e2e_err}

    if rank == 0 and not args.quick:
        # per-shape GEMV numbers, each over its 28 distinct weight copies
        per_shape = {}
        for idx, (name, k, n, hb) in enumerate(LINEARS):
            def shape_pass(idx=idx, k=k, n=n):
                for lw in layers:
                    mb.linear_forward(xs[k], lw[idx], out=ys[n], workspace=ws, stream=stream, pdl=pdl)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                shape_pass()
            for _ in range(3):
                g.replay()
            ms = event_time_ms(torch, g.replay, 10)
            by = algorithmic_bytes(1, k, n, hb)
            per_shape[f"{name}_{k}x{n}"] = {"us": ms * 1e3 / LAYERS, "GBs": by * LAYERS / (ms * 1e-3) / 1e9}
            del g
        line["per_shape"] = per_shape
        line["e2e"] = e2e_line

        # prefill: the same seven linears at M=512 (one layer after another, all 28 layers)
        xp = {k: torch.randn((PREFILL_M, k), device="cuda", generator=gen) for k in (1536, 8960)}
        yp = {n: torch.empty((PREFILL_M, n), device="cuda") for n in (1536, 256, 8960)}
        n_pf_layers = LAYERS if not args.fast_prefill else 2

        def prefill_pass():
            for lw in layers[:n_pf_layers]:
                for w in lw:
                    mb.linear_forward(xp[w.k], w, out=yp[w.n], workspace=ws, stream=stream)
        with torch.cuda.stream(stream):
            prefill_pass()
        stream.synchronize()
        with torch.cuda.stream(stream):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(3):
                prefill_pass()
            e1.record(stream)
        stream.synchronize()
        ms_pf = e0.elapsed_time(e1) / 3
        flops = n_pf_layers * sum(2 * PREFILL_M * k * n for _, k, n, _ in LINEARS)
        kern = {1: "gemv", 2: "simt-dp4a", 3: "tcgen05"}[mb.lib().mllmb200_w4a32_select_kernel(PREFILL_M, 1536, 8960)]
        line["prefill"] = {"M": PREFILL_M, "layers": n_pf_layers, "ms": ms_pf, "tflops": flops / (ms_pf * 1e-3) / 1e12,
                           "kernel": kern, "unit": "TOP/s (2*M*N*K int8 ops)",
                           "frac_of_bf16_peak": flops / (ms_pf * 1e-3) / 1e12 / tensor_peak, "peak_kind": f"of {peak_kind}"}
        mb.check_device_status()

        # the same prefill pass with the fp16 tensor-core path (exact fp16 operands, fp32 accumulation over
        # all of K in tensor memory; same 1e-3 * rms bound): kernel 4 everywhere, and kernel 5 = the "fastest"
        # policy (the fp16 path for M >= 128, the default paths below)
        for key, kern_id, label in (("prefill_f16", mb.KERNEL_TC_F16, "tcgen05 kind::f16 on every linear (kernel 4)"),
                                    ("prefill_fastest", mb.KERNEL_FASTEST, "fastest policy (kernel 5): kind::f16 for M >= 128")):
            try:
                def pf_pass(kern_id=kern_id):
                    for lw in layers[:n_pf_layers]:
                        for w in lw:
                            mb.linear_forward(xp[w.k], w, out=yp[w.n], workspace=ws, stream=stream, kernel=kern_id)
                with torch.cuda.stream(stream):
                    pf_pass()
                stream.synchronize()
                with torch.cuda.stream(stream):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                    for _ in range(3):
                        pf_pass()
                    e1.record(stream)
                stream.synchronize()
                ms_v = e0.elapsed_time(e1) / 3
                line[key] = {"M": PREFILL_M, "layers": n_pf_layers, "ms": ms_v, "tflops": flops / (ms_v * 1e-3) / 1e12,
                             "kernel": label, "unit": "TOP/s (2*M*N*K)",
                             "frac_of_bf16_peak": flops / (ms_v * 1e-3) / 1e12 / tensor_peak, "peak_kind": f"of {peak_kind}"}
                mb.check_device_status()
            except Exception as ex:
                line[key] = {"error": str(ex)[:160]}

        # and the call structure a decoder uses: (q,k,v) and (gate,up) through the grouped call, sharing one
        # quantization of their common input, with the fastest policy
        try:
            def pf_grouped(pdl=True):
                for lw in layers[:n_pf_layers]:
                    mb.linear_forward_grouped(xp[1536], lw[0:3], outs=[yp[1536], yp[256], yp256b], workspace=ws, stream=stream,
                                              policy=mb.KERNEL_FASTEST, pdl=pdl)
                    mb.linear_forward(xp[1536], lw[3], out=yp[1536], workspace=ws, stream=stream, kernel=mb.KERNEL_FASTEST, pdl=pdl)
                    mb.linear_forward_grouped(xp[1536], lw[4:6], outs=[yp[8960], yp8960b], workspace=ws, stream=stream,
                                              policy=mb.KERNEL_FASTEST, pdl=pdl)
                    mb.linear_forward(xp[8960], lw[6], out=yp[1536], workspace=ws, stream=stream, kernel=mb.KERNEL_FASTEST, pdl=pdl)
            yp256b = torch.empty((PREFILL_M, 256), device="cuda")
            yp8960b = torch.empty((PREFILL_M, 8960), device="cuda")
            with torch.cuda.stream(stream):
                pf_grouped()
            stream.synchronize()
            mb.check_device_status(stream)
            # one CUDA graph of the whole pass (8 launches per layer, programmatic dependent launch between them)
            gpf = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gpf, stream=stream):
                pf_grouped()
            for _ in range(2):
                gpf.replay()
            ms_v = event_time_ms(torch, gpf.replay, 5)
            del gpf
            line["prefill_fastest_grouped"] = {"M": PREFILL_M, "layers": n_pf_layers, "ms": ms_v,
                                               "tflops": flops / (ms_v * 1e-3) / 1e12, "unit": "TOP/s (2*M*N*K)",
                                               "kernel": "fastest policy, (q,k,v) and (gate,up) as grouped calls (shared quantization); CUDA graph, programmatic dependent launch",
                                               "frac_of_bf16_peak": flops / (ms_v * 1e-3) / 1e12 / tensor_peak,
                                               "peak_kind": f"of {peak_kind}"}
            mb.check_device_status()
        except Exception as ex:
            line["prefill_fastest_grouped"] = {"error": str(ex)[:160]}

        # CPU baselines on this box's host cores (single-process runs only: under a multi-process launcher
        # every rank is pinned to one OpenMP thread, which would misstate the host)
        val, info = time_reference_cpu(budget_s=10.0) if world == 1 else (None, {})
        if val is not None:
            line["cpu_baseline"] = {"value": val, "unit": "GB/s", "cores": info["cores"], "kind": "reference",
                                    "sample": info["sample"], "variant": info["variant"],
                                    "ms_per_layer": info["ms_per_layer"]}
            # the reference engine's default is 4 threads (mllm/Engine/Context.cpp:29): the same sample with 4
            v4, i4 = time_reference_cpu(budget_s=4.0, max_threads=4)
            if v4 is not None:
                line["cpu_baseline"]["value_4_threads"] = v4
                line["cpu_baseline"]["ms_per_layer_4_threads"] = i4["ms_per_layer"]
        try:
            if world != 1:
                raise RuntimeError("single-process runs only")
            pv, pc, pms = time_oracle_port(budget_s=6.0)
            line["cpu_port"] = {"value": pv, "unit": "GB/s", "cores": pc, "kind": "port", "ms_per_layer": pms,
                                "sample": "same sample on oracle/w4a32_oracle.c (W4A32 format, OpenMP over output rows)"}
            if "cpu_baseline" not in line:
                line["cpu_baseline"] = dict(line["cpu_port"])
        except Exception as ex:  # the oracle is optional for the bench
            line["cpu_port"] = {"unavailable": str(ex)[:100]}
        if "cpu_baseline" not in line:
            line["cpu_baseline"] = None
        if world == 1 and not args.no_config4:
            try:
                line["config4"] = run_config4(args, torch, mb, gen, hbm_peak, tensor_peak, peak_kind)
            except Exception as ex:
                line["config4"] = {"error": str(ex)[:200]}
        if world == 1 and not args.no_w4a16:
            try:
                line["w4a16"] = run_w4a16(args, torch, mb, gen, hbm_peak, tensor_peak, peak_kind)
            except Exception as ex:
                line["w4a16"] = {"error": str(ex)[:200]}
        if not args.no_decoder and world == 1:
            try:
                cpu_ms = line.get("cpu_baseline", {}).get("ms_per_layer")
                line["decoder"] = run_decoder(args, torch, mb, layers, gen, hbm_peak, peak_kind, cpu_ms)
            except Exception as ex:
                line["decoder"] = {"error": str(ex)[:200]}
    elif rank == 0:
        line["e2e"] = None

    if world > 1:
        tp = run_tp(args, torch, mb, dist, rank, world, gen)
        if rank == 0 and tp is not None:
            line["tp"] = tp
    if rank == 0:
        # compact copies of the secondary results inside `roofline`, next to the headline fraction
        def pick(obj, *path):
            for key in path:
                if not isinstance(obj, dict) or key not in obj:
                    return None
                obj = obj[key]
            return obj
        extras = {"config4_gemv_frac": pick(line, "config4", "gemv_M1", "frac"),
                  "config4_gemm_fp16_frac_of_bf16": pick(line, "config4", "gemm_M2048_fp16", "frac_of_bf16_peak"),
                  "prefill_frac_of_bf16": max([v for v in (pick(line, key, "frac_of_bf16_peak") for key in
                                                          ("prefill", "prefill_f16", "prefill_fastest", "prefill_fastest_grouped"))
                                               if v is not None], default=None),
                  "decode_tokens_per_s": pick(line, "decoder", "decode_tokens_per_s"),
                  "decode_distinct_tokens": pick(line, "decoder", "distinct_tokens"),
                  "e2e_GBs": pick(line, "e2e", "value"),
                  "tp_checked": pick(line, "tp", "checked"),
                  "tp_gemm_speedup_vs_1gpu": pick(line, "tp", "gemm", "speedup_vs_1gpu"),
                  "tp_gemv_speedup_vs_1gpu": pick(line, "tp", "gemv", "speedup_vs_1gpu")}
        roofline.update({k: v for k, v in extras.items() if v is not None})
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_decoder(args, torch, mb, layers, gen, hbm_peak, peak_kind, cpu_ms_per_layer=None, batched_only=False):
    """BASELINE config 2: the whole 28-layer decoder with random-init W4A32 weights, batch 1,
    512-token prompt of uniform random ids, 128 greedy decode steps, fp32 KV cache, fp16 lm_head."""
    cfg = dict(mb.QWEN2_1P5B, max_ctx=1024, layers=len(layers))
    prompt_len, steps = args.decoder_prompt, args.decoder_steps  # BASELINE config 2: 512 and 128
    dec = mb.Qwen2Decoder(cfg)
    for l, lw in enumerate(layers):
        for (name, _, _, _), w in zip(LINEARS, lw):
            dec.set_linear_tiled(l, name, w)
        dec.set_norm(0, l, np.ones(cfg["hidden"], np.float32))
        dec.set_norm(1, l, np.ones(cfg["hidden"], np.float32))
    dec.set_norm(2, 0, np.ones(cfg["hidden"], np.float32))
    # embedding rows ~ N(0, 16^2): the current token stays the largest component of the residual stream through all 28
    # random-init layers (each adds a vector of rms < 1).  lm_head = a row permutation of the embedding table (x 0.02):
    # the largest logit then belongs to the row that matches the current token's embedding, so greedy decoding walks
    # the permutation instead of collapsing onto one token as a fully random head does (`distinct_tokens` below)
    emb = torch.randn((cfg["vocab"], cfg["hidden"]), device="cuda", generator=gen) * 16.0
    perm = torch.randperm(cfg["vocab"], device="cuda", generator=gen)
    head = (emb[perm] * 0.02).to(torch.float16)
    del perm
    dec.set_tables(emb, head)
    if batched_only:
        out = run_batched_decode(args, torch, mb, dec, cfg, emb, gen, hbm_peak, peak_kind)
        dec.close()
        return out
    host_prompt = np.random.default_rng(7).integers(0, cfg["vocab"], prompt_len).astype(np.int32)
    ds = dec.stream()
    modes = {"persistent": mb.DECODE_PERSISTENT, "graph": mb.DECODE_GRAPH}
    if args.decoder_mode != "both":
        modes = {args.decoder_mode: modes[args.decoder_mode]}
    res = {}
    toks_by_mode = {}
    for mname, mode in modes.items():
        try:
            dec.prefill(host_prompt)
            dec.decode(min(4, steps), mode)  # first call builds the plan / captures the step graph
            ds.synchronize()
            mb.check_device_status(ds)
        except Exception as ex:
            res[mname] = {"error": str(ex)[:160]}
            continue
        pf, dc, wall = [], [], []
        for _ in range(max(1, args.decoder_reps)):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            t0 = time.perf_counter()
            tokens_dev = torch.from_numpy(host_prompt).to("cuda")  # H2D of the prompt, inside the e2e region
            torch.cuda.current_stream().synchronize()
            ev[0].record(ds)
            dec.prefill_device(tokens_dev)
            ev[1].record(ds)
            dec.decode(steps, mode)
            ev[2].record(ds)
            toks = dec.generated(steps)  # synchronizes, D2H of the sampled tokens
            wall.append(time.perf_counter() - t0)
            pf.append(ev[0].elapsed_time(ev[1]))
            dc.append(ev[1].elapsed_time(ev[2]))
        mb.check_device_status(ds)
        if mname == "persistent":
            try:
                dec.set_profiling(True)   # one more run with the cycle counters on (not timed)
                dec.prefill_device(tokens_dev)
                dec.decode(steps, mode)
                dec.set_profiling(False)
                cyc = dec.phase_cycles().astype(np.float64) / steps  # cycles per decode step
                names = ["P1 norm+quant", "P1 qkv gemv", "wait", "P2 attention", "wait", "P2b merge", "wait", "P3 quant",
                         "P3 o gemv", "wait", "P4 norm+quant", "P4 gate/up gemv", "wait", "P5 quant", "P5 down gemv", "wait",
                         "final norm", "lm_head", "wait", "sample", "gemv: wait for weights", "gemv: cells + loop",
                         "gemv: run flush", "probe: 8 dependent L2 loads (x steps)", "probe: 4 empty grid barriers (x steps)", "-"]
                phase_prof = {"unit": "SM clock cycles per decode step (28 layers), thread 0 of each CTA",
                              "names": names, "mean_over_ctas": [round(float(v)) for v in cyc.mean(0)],
                              "max_over_ctas": [round(float(v)) for v in cyc.max(0)],
                              "min_over_ctas": [round(float(v)) for v in cyc.min(0)]}
            except Exception as ex:
                phase_prof = {"error": str(ex)[:120]}
        toks_by_mode[mname] = toks.tolist()
        res[mname] = {"prefill_ms": min(pf), "decode_ms": min(dc), "wall_s": min(wall)}
    good = [m for m in res if "error" not in res[m]]
    if not good:
        raise RuntimeError(f"decoder: {res}")
    best_mode = min(good, key=lambda m: res[m]["decode_ms"])
    pf_ms, dc_ms, wall_s = res[best_mode]["prefill_ms"], res[best_mode]["decode_ms"], res[best_mode]["wall_s"]
    toks = np.asarray(toks_by_mode[best_mode])
    # algorithmic bytes of one decode step at the mean context of the run
    lin = LAYERS * sum(algorithmic_bytes(1, k, n, hb) for _, k, n, hb in LINEARS)
    head_b = cfg["vocab"] * cfg["hidden"] * 2
    ctx_mean = prompt_len + steps / 2
    kv_b = LAYERS * 2 * cfg["kv_heads"] * cfg["head_dim"] * 4 * ctx_mean
    step_b = lin + head_b + kv_b
    out = {"config": "28 layers, hidden 1536, 12q/2kv heads x128, inter 8960, vocab 151936, rope 1e6; batch 1, "
                     "512-token prompt, 128 greedy steps, fp32 KV cache, fp16 lm_head, random-init weights",
           "prefill_ms": pf_ms, "prefill_tokens_per_s": prompt_len / (pf_ms * 1e-3),
           "decode_ms_per_token": dc_ms / steps, "decode_tokens_per_s": steps / (dc_ms * 1e-3),
           "e2e_wall_s": wall_s, "e2e_decode_tokens_per_s": steps / wall_s,
           "prompt_len": prompt_len, "steps": steps,
           "e2e_note": "host prompt -> H2D -> prefill -> greedy steps -> D2H of the sampled tokens, host wall clock; "
                       "tokens/s counts the generated tokens over the whole wall time (prefill included)",
           "bytes_per_decode_step": step_b,
           "decode_roofline": {"bound": "hbm", "achieved": step_b / (dc_ms / steps * 1e-3) / 1e9, "peak": hbm_peak,
                               "unit": "GB/s", "frac": step_b / (dc_ms / steps * 1e-3) / 1e9 / hbm_peak,
                               "peak_kind": f"of {peak_kind}"},
           "decode_mode": best_mode,
           "decode_ms_per_token_by_mode": {m: (res[m]["decode_ms"] / steps if "error" not in res[m] else res[m]) for m in res},
           "modes_agree": (len(good) < 2 or toks_by_mode[good[0]] == toks_by_mode[good[1]]),
           "launches_per_decode_step": {"persistent": "1 cooperative launch for all steps", "graph": 1 + LAYERS * 9 + 3},
           "distinct_tokens": int(len(set(toks.tolist())))}
    if "persistent" in good:
        out["persistent_phase_cycles"] = phase_prof
    if cpu_ms_per_layer:
        out["cpu_reference_linears_only_tokens_per_s"] = 1e3 / (cpu_ms_per_layer * LAYERS)
        out["cpu_note"] = ("upper bound for the host-CPU reference: only the 28x7 linears of a step, timed with the "
                           "reference X86 Q4_K x Q8_K kernels; attention, norms and lm_head not included")
    if not args.no_batched_decode:
        try:
            out["batched"] = run_batched_decode(args, torch, mb, dec, cfg, emb, gen, hbm_peak, peak_kind)
        except Exception as ex:  # e.g. out of memory on a shared device: the batch-1 numbers stand
            out["batched"] = {"error": str(ex)[:200]}
    dec.close()
    del emb, head
    return out


def run_batched_decode(args, torch, mb, dec, cfg, emb, gen, hbm_peak, peak_kind):
    """BASELINE config 3: 64 concurrent sequences on the same weights, every quantized linear at M = 64.  Each
    sequence is prefilled with 512 positions - 256 synthetic vision-patch embeddings (~N(0,1), width 1536) followed by
    256 looked-up text tokens - then all decode together up to a 1024-token context.  Timed: device time of the
    greedy steps at the start (context 512) and at the end (context ~1000) of that range."""
    B, ctx_end, steps_t = args.batch_sequences, cfg["max_ctx"], args.batch_timed_steps
    n_vis, n_txt = 256, 256
    bd = mb.Qwen2BatchDecoder(dec, B)
    if args.batch_policy:
        bd.set_policy(args.batch_policy)
    ds = dec.stream()
    rng = np.random.default_rng(11)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record(ds)
    for b in range(B):
        vis = torch.randn((n_vis, cfg["hidden"]), device="cuda", generator=gen)
        txt = emb[torch.from_numpy(rng.integers(0, cfg["vocab"], n_txt)).cuda()]
        bd.prefill(b, embeds=torch.cat([vis, txt]).contiguous())
    ev[1].record(ds)
    ds.synchronize()
    prefill_ms = ev[0].elapsed_time(ev[1])
    n0 = n_vis + n_txt
    bd.decode(2)  # builds the step graph
    ds.synchronize()
    mb.check_device_status(ds)

    def timed(steps):
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(ds)
        bd.decode(steps)
        b_.record(ds)
        ds.synchronize()
        return a.elapsed_time(b_) / steps

    ms_start = timed(steps_t)
    done = 2 + steps_t
    room = (args.batch_context or ctx_end - 1) - n0 - done - steps_t
    if room > 0:
        bd.decode(room)  # untimed: walk to the end of the context
        done += room
    ctx_late = n0 + done
    ms_end = timed(steps_t)
    done += steps_t
    mb.check_device_status(ds)
    toks = np.stack([bd.generated(b, done) for b in range(B)])
    lin = cfg["layers"] * sum(algorithmic_bytes(B, k, n, hb) for _, k, n, hb in LINEARS)
    head_b = cfg["vocab"] * cfg["hidden"] * 2

    def step_bytes(ctx):
        return lin + head_b + cfg["layers"] * B * 2 * cfg["kv_heads"] * cfg["head_dim"] * 4 * ctx

    def entry(ms, ctx):
        by = step_bytes(ctx)
        return {"context": int(ctx), "ms_per_step": ms, "tokens_per_s": B / (ms * 1e-3), "bytes_per_step": by,
                "GBs": by / (ms * 1e-3) / 1e9, "frac_hbm": by / (ms * 1e-3) / 1e9 / hbm_peak}

    out = {"config": f"BASELINE config 3: {B} sequences x {ctx_end}-token context on the Qwen2-1.5B language tower, prefill of "
                     f"{n_vis} vision-patch embeddings + {n_txt} text tokens per sequence, fp32 KV cache, every linear at M = {B}, "
                     f"kernel policy {args.batch_policy} (5: gate / up on the fp16 tile GEMM, the other linears on the exact streaming GEMM; 0: all exact)",
           "policy": args.batch_policy,
           "prefill_ms_all_sequences": prefill_ms, "prefill_tokens_per_s": B * n0 / (prefill_ms * 1e-3),
           "at_start": entry(ms_start, n0 + 2 + steps_t / 2), "at_end": entry(ms_end, ctx_late + steps_t / 2),
           "timed_steps": steps_t, "peak_kind": f"of {peak_kind}",
           "distinct_tokens_per_sequence_min": int(min(len(set(r.tolist())) for r in toks)),
           "sequences_differ": bool(len({tuple(r.tolist()) for r in toks}) > 1),
           "bytes_note": "per step: the 196 linears at M = 64 (weights once), fp16 lm_head once, every sequence's K and V rows once"}
    bd.close()
    return out


def make_random_weights_a16(mb, torch, n, k, gen):
    """Random W4A16 weights (nibbles uniform, scales |N(0, 0.02)|/7, zero terms within +-8 scales), assembled as a
    blob on the device and repacked there."""
    from mllm_b200 import w4a16
    dev = "cuda"
    blob = torch.zeros(w4a16.prepack_size(n, k, False), dtype=torch.uint8, device=dev)
    a, b, z, c = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_size_t()
    mb.lib().mllmb200_w4a16_blob_offsets(n, k, 0, C.byref(a), C.byref(b), C.byref(z), C.byref(c))
    nb = k // 32
    blob[a.value:a.value + n * (k // 2)] = torch.randint(0, 256, (n * (k // 2),), dtype=torch.uint8, device=dev, generator=gen)
    sc = torch.randn((n * nb,), device=dev, generator=gen).abs() * (0.02 / 7.0)
    zr = (torch.rand((n * nb,), device=dev, generator=gen) * 16 - 8).round() * sc
    blob[b.value:b.value + n * nb * 4] = sc.view(torch.uint8)
    blob[z.value:z.value + n * nb * 4] = zr.view(torch.uint8)
    tiled = torch.empty(w4a16.tiled_size(n, k), dtype=torch.uint8, device=dev)
    st = mb.lib().mllmb200_w4a16_repack_device(blob.data_ptr(), n, k, 0, 0, n, tiled.data_ptr(),
                                               C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0, mb.status_str(st)
    torch.cuda.synchronize()
    return w4a16.W4A16Weights(tiled, n, k, 0)


def run_w4a16(args, torch, mb, gen, hbm_peak, tensor_peak, peak_kind):
    """The W4A16 sibling path (fp16 activations in, fp16 out) on the same shapes: the 7 linears of the 28 layers
    at M=1 (CUDA graph, distinct weights per layer) and at M=512, and BASELINE config 4's matrix."""
    from mllm_b200 import w4a16

    def a16_bytes(m, k, n):  # nibbles + fp32 scale and zero per group + fp16 x and y
        return n * k // 2 + n * (k // 32) * 8 + m * k * 2 + m * n * 2

    out = {"workload": "W4A16: 28 layers x 7 linears of Qwen2-1.5B at M=1 and M=512; config 4 matrix at M=1 and M=2048",
           "dtype": "int4 weights (fp32 scale + zero per group of 32), int8 per-block activations, fp16 in/out"}
    stream = torch.cuda.Stream()
    layers = [[make_random_weights_a16(mb, torch, n, k, gen) for _, k, n, _ in LINEARS] for _ in range(LAYERS)]
    for m, key in ((1, "decode_M1"), (PREFILL_M, "prefill_M512")):
        xs = {k: torch.randn((m, k), device="cuda", generator=gen).half() for k in (1536, 8960)}
        ys = {n: torch.empty((m, n), device="cuda", dtype=torch.float16) for n in (1536, 256, 8960)}
        ws = torch.empty(max(w4a16.workspace_size(m, k, n) for _, k, n, _ in LINEARS), dtype=torch.uint8, device="cuda")

        def one_pass():
            for lw in layers:
                for w in lw:
                    w4a16.linear_forward(xs[w.k], w, out=ys[w.n], workspace=ws, stream=stream, pdl=not args.no_pdl)
        with torch.cuda.stream(stream):
            one_pass()
        stream.synchronize()
        if args.w4a16_once:  # launch-list runs under ncu: one eager pass per section, nothing timed
            out[key] = {"passes": 1}
            continue
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            one_pass()
        for _ in range(3):
            g.replay()
        ms = event_time_ms(torch, g.replay, 10 if m == 1 else 3)
        by = sum(a16_bytes(m, k, n) for _, k, n, _ in LINEARS) * LAYERS
        fl = sum(2.0 * m * k * n for _, k, n, _ in LINEARS) * LAYERS
        out[key] = {"ms": ms, "GBs": by / (ms * 1e-3) / 1e9, "tflops": fl / (ms * 1e-3) / 1e12,
                    "frac_hbm": by / (ms * 1e-3) / 1e9 / hbm_peak, "frac_of_bf16_peak": fl / (ms * 1e-3) / 1e12 / tensor_peak,
                    "peak_kind": f"of {peak_kind}", "how": "CUDA graph of 196 calls (activation quantization + kernel each)"}
        del g
        if not args.w4a16_once:
            # the same step with (q,k,v) and (gate,up) as grouped calls: 4 calls per layer (M=1: 4 launches)
            ysb = {n: torch.empty((m, n), device="cuda", dtype=torch.float16) for n in (256, 8960)}

            def grouped_pass():
                for q, kk, v, o, gate, up, down in layers:
                    w4a16.linear_forward_grouped(xs[1536], [q, kk, v], outs=[ys[1536], ys[256], ysb[256]], workspace=ws,
                                                 stream=stream, pdl=not args.no_pdl)
                    w4a16.linear_forward(xs[1536], o, out=ys[1536], workspace=ws, stream=stream, pdl=not args.no_pdl)
                    w4a16.linear_forward_grouped(xs[1536], [gate, up], outs=[ys[8960], ysb[8960]], workspace=ws,
                                                 stream=stream, pdl=not args.no_pdl)
                    w4a16.linear_forward(xs[8960], down, out=ys[1536], workspace=ws, stream=stream, pdl=not args.no_pdl)
            with torch.cuda.stream(stream):
                grouped_pass()
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                grouped_pass()
            for _ in range(3):
                g.replay()
            msg = event_time_ms(torch, g.replay, 10 if m == 1 else 3)
            out[key + "_grouped"] = {"ms": msg, "GBs": by / (msg * 1e-3) / 1e9, "frac_hbm": by / (msg * 1e-3) / 1e9 / hbm_peak,
                                     "tflops": fl / (msg * 1e-3) / 1e12, "frac_of_bf16_peak": fl / (msg * 1e-3) / 1e12 / tensor_peak,
                                     "peak_kind": f"of {peak_kind}",
                                     "how": "CUDA graph of 112 calls: (q,k,v) (o) (gate,up) (down) per layer; M=1: one launch per "
                                            "call; M=512: one quantization + one tensor-core launch per call"}
            del g
    del layers
    n, k = 28672, 8192
    copies = [make_random_weights_a16(mb, torch, n, k, gen) for _ in range(3)]  # 3 x 176 MB > L2
    for m, key in ((1, "config4_M1"), (2048, "config4_M2048")):
        x = torch.randn((m, k), device="cuda", generator=gen).half()
        y = torch.empty((m, n), device="cuda", dtype=torch.float16)
        ws = torch.empty(w4a16.workspace_size(m, k, n), dtype=torch.uint8, device="cuda")

        def big_pass():
            for w in copies:
                w4a16.linear_forward(x, w, out=y, workspace=ws, stream=stream)
        with torch.cuda.stream(stream):
            big_pass()
        stream.synchronize()
        if args.w4a16_once:
            out[key] = {"passes": 1}
            continue
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            big_pass()
        for _ in range(3):
            g.replay()
        ms = event_time_ms(torch, g.replay, 10 if m == 1 else 3) / len(copies)
        by, fl = a16_bytes(m, k, n), 2.0 * m * k * n
        out[key] = {"ms": ms, "GBs": by / (ms * 1e-3) / 1e9, "tflops": fl / (ms * 1e-3) / 1e12,
                    "frac_hbm": by / (ms * 1e-3) / 1e9 / hbm_peak, "frac_of_bf16_peak": fl / (ms * 1e-3) / 1e12 / tensor_peak,
                    "peak_kind": f"of {peak_kind}"}
        del g
    mb.check_device_status()
    return out


def run_config4(args, torch, mb, gen, hbm_peak, tensor_peak, peak_kind):
    """BASELINE config 4 on one GPU: W [28672, 8192] int4 g32 (132 MB).  The same kernels as the
    headline, at a size where fixed latencies no longer dominate: GEMV at M=1 (HBM roofline) and the
    GEMM at M=2048 rows of x per call (4 calls = the config's 8192 rows), per kernel policy."""
    n, k = 28672, 8192
    copies = [make_random_weights(mb, torch, n, k, False, gen) for _ in range(4)]  # 4 x 132 MB > L2
    out = {"workload": "config4: W[28672,8192] int4 g32; GEMV M=1 over 4 weight copies, GEMM M=2048"}
    stream = torch.cuda.Stream()
    x1 = torch.randn((1, k), device="cuda", generator=gen)
    y1 = torch.empty((1, n), device="cuda")
    ws1 = torch.empty(mb.workspace_size(1, k), dtype=torch.uint8, device="cuda")

    def gemv_pass():
        for w in copies:
            mb.linear_forward(x1, w, out=y1, workspace=ws1, stream=stream, pdl=True)
    with torch.cuda.stream(stream):
        gemv_pass()
    stream.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        gemv_pass()
    for _ in range(3):
        g.replay()
    ms = event_time_ms(torch, g.replay, 20) / len(copies)
    by = algorithmic_bytes(1, k, n, False)
    out["gemv_M1"] = {"us": ms * 1e3, "GBs": by / (ms * 1e-3) / 1e9, "frac": by / (ms * 1e-3) / 1e9 / hbm_peak,
                      "peak_kind": f"of {peak_kind}", "how": "graph of 4 single-launch GEMV calls over 4 weight copies, programmatic dependent launch"}
    del g
    m = 2048
    xm = torch.randn((m, k), device="cuda", generator=gen)
    ym = torch.empty((m, n), device="cuda")
    wsm = torch.empty(mb.workspace_size(m, k), dtype=torch.uint8, device="cuda")
    flops = 2.0 * m * n * k
    for key, kern in (("gemm_M2048_int8", mb.KERNEL_AUTO), ("gemm_M2048_fp16", mb.KERNEL_TC_F16)):
        def gemm_pass(kern=kern):
            with torch.cuda.stream(stream):
                for w in copies[:2]:
                    mb.linear_forward(xm, w, out=ym, workspace=wsm, stream=stream, kernel=kern)
        gemm_pass()
        stream.synchronize()
        with torch.cuda.stream(stream):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(3):
                gemm_pass()
            e1.record(stream)
        stream.synchronize()
        msg = e0.elapsed_time(e1) / 6
        out[key] = {"ms": msg, "tflops": flops / (msg * 1e-3) / 1e12, "frac_of_bf16_peak": flops / (msg * 1e-3) / 1e12 / tensor_peak,
                    "peak_kind": f"of {peak_kind}", "unit": "TOP/s (2*M*N*K), activation quantization included"}
    mb.check_device_status()
    return out


def run_tp(args, torch, mb, dist, rank, world, gen):
    """BASELINE config 4 through the C ABI's tensor-parallel entry points (mllmb200_w4a32_tp_*): W [28672, 8192]
    column-sharded over the ranks, x replicated, every rank ends with the full fp32 y.  The GEMV at M = 1 and the GEMM
    at M = 2048 rows of x per call (four such calls are the config's 8192 rows), each with the fused gather (the
    kernels' epilogues store into every rank's y over NVLink), with the NCCL baseline (ncclAllGather + re-assembly)
    and against ONE GPU running the unsharded matrix in the same process.  Device time, max over ranks.  The gathered
    result is compared on every rank with the unsharded one."""
    from mllm_b200 import tp
    n, k = 28672, 8192
    if n % (world * 32) != 0:
        return None
    g = torch.Generator(device="cuda").manual_seed(99)  # the same matrix and activations on every rank
    nib = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    sc = torch.randn((n, k // 32), device="cuda", generator=g).abs() * (0.02 / 7.0)
    s16 = (sc.view(torch.int32) >> 16).to(torch.int16).cpu().numpy().view(np.uint16)
    blob_host = mb.prepack_from_quantized(nib.cpu().numpy(), s16, n, k)  # int4 + bf16 scales drawn directly (config 0's distributions)
    del nib, sc, s16
    m_gemm = 2048
    full = mb.W4A32Weights.from_blob(blob_host)  # the unsharded matrix, for the one-GPU time and the check
    tpl = tp.TensorParallelLinear(blob_host, m_gemm)
    del blob_host
    ws_full = torch.empty(mb.workspace_size(m_gemm, k), dtype=torch.uint8, device="cuda")
    out = {"workload": "config4: W[28672,8192] int4 g32 column-sharded over the ranks; fused gather (peer stores from the "
                       "kernels' epilogues) vs NCCL all-gather vs one GPU, same process, device time, max over ranks",
           "world": world}
    checked = True

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        ms = float(np.median([event_time_ms(torch, fn, iters) for _ in range(3)]))
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for key, m, kern, iters in (("gemv", 1, mb.KERNEL_AUTO, 50), ("gemm", m_gemm, mb.KERNEL_FASTEST, 10)):
        x = torch.randn((m, k), device="cuda", generator=g)
        y1 = torch.empty((m, n), device="cuda")
        res = {"M": m}
        res["one_gpu_ms"] = timed(lambda: mb.linear_forward(x, full, out=y1, workspace=ws_full, kernel=kern), iters)
        res["tp_fused_ms"] = timed(lambda: tpl.forward(x, gather=tp.GATHER_PEER_STORES, kernel=kern), iters)
        res["tp_nccl_ms"] = timed(lambda: tpl.forward(x, gather=tp.GATHER_NCCL, kernel=kern), iters)
        res["tp_compute_only_ms"] = timed(lambda: tpl.forward(x, gather=tp.GATHER_NONE, kernel=kern), iters)
        res["speedup_vs_1gpu"] = res["one_gpu_ms"] / res["tp_fused_ms"]
        res["speedup_vs_1gpu_nccl"] = res["one_gpu_ms"] / res["tp_nccl_ms"]
        recv_bytes = (world - 1) / world * m * n * 4
        res["nvlink_bound_ms"] = recv_bytes / 770e9 * 1e3  # every rank receives the other ranks' blocks; 770 GB/s measured peer copy
        res["tflops" if m > 1 else "GBs_weights_alg"] = (2.0 * m * k * n / (res["tp_fused_ms"] * 1e-3) / 1e12 if m > 1 else
                                                         algorithmic_bytes(m, k, n, False) / (res["tp_fused_ms"] * 1e-3) / 1e9)
        # the gathered result against the unsharded one computed here, within 1e-5 * rms (GEMV; the shard splits K over
        # its CTAs differently) or 1e-4 * rms (GEMM, K = 8192: either launch splits K in two on the tiles left over after
        # its own last full wave - other orders of the same fp32 additions; measured 1.2e-5), and bit for bit between
        # the ranks and between the two gather modes
        mb.linear_forward(x, full, out=y1, workspace=ws_full, kernel=kern)
        ok = True
        for mode in (tp.GATHER_PEER_STORES, tp.GATHER_NCCL):
            tpl.output(m).zero_()
            torch.cuda.synchronize()
            dist.barrier()
            y = tpl.forward(x, gather=mode, kernel=kern)
            torch.cuda.synchronize()
            mb.check_device_status()
            rms = float(y1.pow(2).mean().sqrt())
            rel = float((y - y1).abs().max()) / rms
            res["max_diff_over_rms"] = max(res.get("max_diff_over_rms", 0.0), rel)
            digest = y.view(torch.int32).to(torch.int64).sum().reshape(1)  # same bits on every rank <=> same digest
            lo, hi = digest.clone(), digest.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            res["ranks_agree"] = res.get("ranks_agree", True) and int(lo.item()) == int(hi.item())
            if mode == tp.GATHER_PEER_STORES:
                y_fused = y.clone()
            elif m > 1:
                res["modes_agree"] = bool(torch.equal(y, y_fused))
            ok = ok and rel <= (1e-5 if m == 1 else 1e-4) and res["ranks_agree"] and res.get("modes_agree", True)
            dist.barrier()
        flag = torch.tensor([1.0 if ok else 0.0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        res["checked"] = bool(flag.item() > 0.5)
        checked = checked and res["checked"]
        out[key] = res
        del y1
    out["checked"] = checked
    dist.barrier()
    tpl.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch on the stream instead of replaying a CUDA graph")
    ap.add_argument("--no-pdl", action="store_true", help="disable programmatic dependent launch between linears")
    ap.add_argument("--calls", default="layer", choices=["layer", "grouped", "per-op"],
                    help="call structure of the headline step: one multi call per layer, the decoder's four calls per layer, or one call per linear")
    ap.add_argument("--all-structures", action="store_true", help="with --quick: still time the other two call structures")
    ap.add_argument("--config4-only", action="store_true", help="only the section on BASELINE config 4's large matrix")
    ap.add_argument("--no-config4", action="store_true", help="skip the single-GPU section on BASELINE config 4's large matrix")
    ap.add_argument("--w4a16-only", action="store_true", help="only the section on the W4A16 sibling path")
    ap.add_argument("--no-w4a16", action="store_true", help="skip the section on the W4A16 sibling path")
    ap.add_argument("--w4a16-once", action="store_true", help="with --w4a16-only: one untimed eager pass per section (for ncu launch lists)")
    ap.add_argument("--decoder-only", action="store_true", help="only the whole-model prefill + decode section")
    ap.add_argument("--decoder-prompt", type=int, default=512, help="prompt length of the decoder section")
    ap.add_argument("--decoder-steps", type=int, default=128, help="greedy steps of the decoder section (small values for ncu)")
    ap.add_argument("--decoder-mode", default="both", choices=["both", "persistent", "graph"])
    ap.add_argument("--decoder-reps", type=int, default=3, help="timed repetitions of prefill + 128 steps")
    ap.add_argument("--no-decoder", action="store_true", help="skip the whole-model prefill + decode section")
    ap.add_argument("--no-batched-decode", action="store_true", help="skip the 64-sequence batched decode of the decoder section")
    ap.add_argument("--batched-only", action="store_true", help="only the batched decode section, on --decoder-layers layers")
    ap.add_argument("--decoder-layers", type=int, default=LAYERS, help="layers of the model of --batched-only (small values for profiler captures)")
    ap.add_argument("--batch-policy", type=int, default=5,
                    help="kernel policy of the batched decoder's linears: 5 fastest (gate / up on the fp16 tile GEMM: exact "
                         "products, fp32 accumulation; the rest exact int32 group sums), 0 exact int32 group sums everywhere")
    ap.add_argument("--batch-context", type=int, default=0, help="with --batched-only: stop the untimed walk at this context (0 = the full 1024)")
    ap.add_argument("--batch-sequences", type=int, default=64, help="sequences of the batched decode section (BASELINE config 3: 64)")
    ap.add_argument("--batch-timed-steps", type=int, default=16, help="timed greedy steps at either end of the batched decode")
    ap.add_argument("--quick", action="store_true", help="headline number only (used under ncu)")
    ap.add_argument("--prefill-only", action="store_true",
                    help="run one decoder layer's seven linears at M=512 once and exit (small target for ncu)")
    ap.add_argument("--prefill-grouped", action="store_true",
                    help="with --prefill-only: (q,k,v) and (gate,up) as grouped calls, fastest policy")
    ap.add_argument("--prefill-f16", action="store_true", help="with --prefill-only: use the fp16 tensor-core path (kernel 4)")
    ap.add_argument("--fast-prefill", action="store_true", help="time the prefill linears on 2 layers instead of 28")
    args = ap.parse_args()
    # Libraries write to file descriptor 1 behind Python's back (NCCL prints its version banner there when a
    # communicator is created); stdout must carry the result lines only, so everything that is not printed
    # through `print` in this file goes to stderr.
    sys.stdout.flush()
    result_fd = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(result_fd, "w", buffering=1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)
    sys.stdout.flush()


if __name__ == "__main__":
    main()
