#!/usr/bin/env python
"""Benchmark of the quantized linear-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W]            this build (prism_b200)
    python bench.py --impl reference [--gpus N] ...                 the reference's CPU arithmetic on the host cores
    python bench.py --detail                                        per-shape table (GEMM TOPS / decode GB/s), no JSON line

Workload (config "w8a8-27b-layer-set"): 4 decoder layers of the 27B-class linear set (q|k|v 7168x5120, o 5120x5120,
gate|up 34816x5120, down 5120x17408; W8A8 with one scale per token and per output row, the engine's mode) over M = 8192
rows, every GEMM fed by its activation quantizer (prism_b200.linear_stack).  A step is one pass.  The metric is int8
GEMM throughput in TOPS = 2 * M * sum(N * K) * layers / time (the quantizers' work is not counted as ops).
With --gpus N the same pass runs tensor-parallel over N ranks (column- / row-parallel, int32 all-reduce): total work
is fixed, so scaling is "strong".  Weights (1.3 GB) and activations exceed the 126 MB L2, so nothing is served from a
warm cache between steps.  Synthetic data: seeded N(0, 0.02^2) weights through Q8_0, N(0, 1) residual rows.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = 4
M_DEFAULT = 8192
METRIC = "w8a8_int8_gemm_throughput"
UNIT = "TOPS"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], bf16=p["bf16_tflops_sustained"], bf16_burst=p["bf16_tflops"], src="measured")
    return dict(hbm=6650.0, bf16=1400.0, bf16_burst=1590.0, src="fallback")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 9 and r[5 + i].lower().startswith("active")
                                                         for r in self.rows)]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------------------------ CPU arm
_CPU = {}


def cpu_layer_pass(rows):
    """One layer of the same linear set through the reference's CPU emulation (oracle/emulation.py: fake-quantized
    operands multiplied in fp32 by torch on every host core) for `rows` of the workload's rows.  Returns
    (seconds, ops, threads)."""
    import torch

    from oracle import emulation
    if "set" not in _CPU:
        _CPU["set"] = emulation.LayerSet()
    ls = _CPU["set"]
    h = torch.randn(rows, 5120, generator=torch.Generator().manual_seed(rows))
    dt, ops, _ = ls.run(h)
    return dt, ops, ls.threads


CPU_SAMPLE_ROWS = 256


def reference_gpu_kernels(rows):
    """The reference's own GPU kernel for this path on this GPU, when a checkout of its package travelled with the
    repository (baseline/_ref, never committed): its Triton W8A8 kernel (kernels/w8a8.py:31-98, what a B200 runs there:
    it has no dispatch table for this GPU and its wgmma kernels are sm_90a-only) on the four projections at `rows`
    rows, CUDA events, weights rotated over copies larger than L2.  Reported beside the CPU number; never the
    measured product.  Any failure is reported as the reason it is unavailable."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "startlux_prism")):
        return {"unavailable": "no reference checkout under baseline/_ref on this machine"}
    try:
        import torch
        if not torch.cuda.is_available():
            return {"unavailable": "no GPU"}
        sys.path.insert(0, ref)
        os.environ["STARTLUX_PRISM_GEMM"] = "triton"
        import triton
        if tuple(int(v) for v in triton.__version__.split(".")[:2]) < (3, 8):
            # the reference pins Triton 3.8, whose tl.dot takes its result type from the accumulator; older Tritons
            # default out_dtype to float32 and reject the reference's int32 accumulator (kernels/w8a8.py:58,70).  Only
            # that default is adapted; the reference's source runs as it is.
            import triton.language as tl
            from triton.language import core as tl_core
            dot = tl.dot

            @tl_core.builtin
            def dot_typed_by_acc(input, other, acc=None, input_precision=None, allow_tf32=None,
                                 max_num_imprecise_acc=None, out_dtype=None, _semantic=None):
                if out_dtype is None:
                    out_dtype = acc.dtype if acc is not None else tl.float32
                return dot(input, other, acc, input_precision, allow_tf32, max_num_imprecise_acc, out_dtype,
                           _semantic=_semantic)
            tl.dot = tl_core.dot = dot_typed_by_acc
        from startlux_prism.kernels import w8a8 as RW8
        dev = torch.device("cuda", 0)
        gen = torch.Generator(device=dev).manual_seed(3)
        out = {}
        tot_ops = tot_s = 0.0
        for name, (N, K, epi) in SHAPES.items():
            copies = max(2, -(-2 * (126 << 20) // (N * K)))
            ws = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev, generator=gen) for _ in range(copies)]
            a = torch.randint(-127, 128, (rows, K), dtype=torch.int8, device=dev, generator=gen)
            sa = torch.rand(rows, 1, device=dev, generator=gen) * 1e-2
            sw = torch.rand(N, 1, device=dev, generator=gen) * 1e-3
            o = torch.zeros(rows, N, dtype=torch.float32 if epi else torch.bfloat16, device=dev)
            nr = torch.tensor([rows], dtype=torch.int32, device=dev)
            cfg = RW8.pick(rows, N, K, epi)
            for c in range(copies):
                RW8.gemm(a, sa, ws[c], sw, o, nr, K, epi=epi, cfg=cfg)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for c in range(copies):
                RW8.gemm(a, sa, ws[c], sw, o, nr, K, epi=epi, cfg=cfg)
            e1.record()
            torch.cuda.synchronize()
            sec = e0.elapsed_time(e1) * 1e-3 / copies
            out[name] = round(2.0 * rows * N * K / sec / 1e12, 1)
            tot_ops += 2.0 * rows * N * K
            tot_s += sec
            del ws, a, o
            torch.cuda.empty_cache()
        return {"kernel": "the reference's Triton _w8a8_kernel (kernels/w8a8.py:31-98), unmodified", "rows": rows,
                "tops_per_projection": out, "tops_layer_set": round(tot_ops / tot_s / 1e12, 1), "unit": UNIT}
    except Exception as e:                              # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}


def run_reference(args):
    """The reference arm: the reference's CPU emulation of the path (restated in oracle/emulation.py; the reference's own
    is Python that needs its model files) on every host core, a bounded sample of the workload per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = CPU_SAMPLE_ROWS                              # sample: 256 of the 8192 rows through one of the 4 layers
    for _ in range(args.warmup):
        cpu_layer_pass(rows)
    t = []
    for _ in range(args.steps):
        dt, ops, cores = cpu_layer_pass(rows)
        t.append(dt)
    sec = sum(t) / len(t)
    val = ops / sec / 1e12
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
            "config": {"workload": "w8a8-27b-layer-set", "rows": M_DEFAULT, "layers": LAYERS, "graph": False,
                       "parallelism": f"tp{args.gpus}", "l2": "inputs larger than L2 (1.3 GB of weights per pass)"},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"{rows} of {M_DEFAULT} rows through 1 of {LAYERS} layers per step"},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    if not args.no_ref_gpu:
        line["reference_gpu_kernels"] = reference_gpu_kernels(args.rows)
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------ GPU arm
def run_gpu(args):
    import torch
    import torch.distributed as dist

    from prism_b200 import _lib, linear_stack as LS, tp
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    _lib.lib()
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG", "WARN")            # NCCL's version banner goes to stdout otherwise
        group = tp.Group(rank, world, backend="nccl", local_rank=local)
    M = args.rows
    layers = []
    for i in range(LAYERS):
        whole = LS.make_layer_weights(i, dev)
        layers.append(LS.shard_layer(whole, world, rank))
        del whole
    torch.cuda.empty_cache()
    stack = LS.LinearStack(layers, M, dev, group)
    gen = torch.Generator(device=dev).manual_seed(5)
    h0 = torch.randn(M, LS.HIDDEN, generator=gen, device=dev)
    ops = LS.OPS_PER_ROW_LAYER * M * LAYERS

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        stack(h0)
    sync()
    code, where = _lib.device_status()
    if code:
        raise SystemExit(f"device status {code} at {where:#x}")
    int8_peak = measure_int8_peak() if rank == 0 else None
    step = lambda: stack(h0)                                      # noqa: E731
    if args.graph:
        # the whole pass (collectives included) as one CUDA graph: what a decode loop replays per token
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            stack(h0)
        step = graph.replay
        for _ in range(3):
            step()
        sync()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # ---- device-resident timing
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    sync()
    e0.record()
    for i in range(args.steps):
        step()
        marks[i].record()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1) / args.steps
    per_step = sorted(a.elapsed_time(b) for a, b in zip([e0] + marks[:-1], marks))
    ms_median = per_step[len(per_step) // 2]
    # the step's result as a checksum: every GPU count must print the same one (tensor-parallel bit-identity)
    import zlib
    final = stack(h0)
    torch.cuda.synchronize()
    crc = zlib.crc32(final.cpu().numpy().tobytes()) if rank == 0 else 0
    # ---- per-GEMM durations for the roofline (events around each launch, same stream)
    gemm_ms = time_gemms(stack, h0, args.steps)
    # ---- end to end: host buffers, copies inside the timed region, pipelined over three streams
    e2e_ms, h2d, d2h = time_e2e(stack, h0, args.steps, sync)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    if rank == 0:
        pk = peaks()
        value = ops / (ms * 1e-3) / 1e12
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "s8", "data": "synthetic",
                "config": {"workload": "w8a8-27b-layer-set", "rows": M, "layers": LAYERS, "graph": bool(args.graph),
                           "parallelism": f"tp{world}", "l2": "inputs larger than L2 (1.3 GB of weights per pass)"},
                "e2e": {"value": ops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
                "gpu_launches": launches_per_step(world) * args.steps, "clocks": clocks,
                "ms_per_step_median": ms_median, "value_at_median_step": ops / (ms_median * 1e-3) / 1e12,
                "check": {"residual_crc32": f"{crc:08x}", "of": "fp32 residual [rows, 5120] after one pass of the seeded "
                          "input; identical at every GPU count"}}
        if gemm_ms is not None:
            achieved = ops / world / (gemm_ms * 1e-3) / 1e12    # per GPU: this rank's share of the products / its GEMM time
            peak, peak_mean = int8_peak
            # DRAM bytes per launch of the dominant kernel (the gate|up GEMM): its algorithmic bytes (weights once +
            # activations + bf16 output) times the ratio ncu measured on the one-launch capture at M = 2048 (300 MB of
            # DRAM traffic against 332 MB algorithmic: part of the output was still in L2 when the capture ended)
            n_gu, k_gu = 34816 // world, 5120
            algorithmic = n_gu * k_gu + M * k_gu + 2 * M * n_gu
            line["roofline"] = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                                "frac": achieved / peak, "traffic": int(algorithmic * 0.90),
                                "kernel": "w8a8_tile_kernel<256>", "gemm_ms_per_step": gemm_ms,
                                "algorithmic_bytes": algorithmic,
                                "peak_note": "int8 tensor-core rate measured in this process before the timed region: "
                                             "tcgen05 kind::i8 128x256x32 on shared-memory-resident random operands, "
                                             f"one CTA per SM, 0.3 s of launches; highest launch {peak:.0f} (used), "
                                             f"mean {peak_mean:.0f}.  For context: 2 x {pk['src']} bf16 burst = "
                                             f"{2 * pk['bf16_burst']:.0f}, 2 x sustained = {2 * pk['bf16']:.0f}, nominal "
                                             "dense int8 4500",
                                "frac_of_nominal_4500": achieved / 4500.0,
                                "traffic_note": "algorithmic bytes x 0.90, the DRAM / algorithmic ratio of the ncu "
                                                "capture at M = 2048; not measured at this M"}
            if achieved > peak:
                line["roofline"]["flag"] = "achieved above the measured peak: the probe ran at a lower clock than the step"
        if world == 1 and not args.no_detail:
            line["detail"] = quick_detail(dev, pk)
        if world == 1 and not args.no_cpu:
            rows = CPU_SAMPLE_ROWS
            cpu_layer_pass(rows)
            dt, cops, cores = min(cpu_layer_pass(rows) for _ in range(3))
            line["cpu_baseline"] = {"value": cops / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"{rows} of {M} rows through 1 of {LAYERS} layers"}
        print(json.dumps(line), flush=True)
    if args.graph:
        # a live graph holds the communicator's kernels: it goes before the process group does
        step = None
        del graph
        torch.cuda.synchronize()
    if group is not None:
        sync()
        stack.close()
        group.close()


def measure_int8_peak(seconds=0.3):
    """The int8 tensor-core ceiling of THIS GPU in THIS process: pb_int8_peak_probe (128 x 256 x 32 tcgen05 MMAs on
    shared-memory-resident pseudo-random operands, one CTA per SM, no memory traffic) launched back to back for
    `seconds`; returns (highest, mean) TOPS over the launches.  The highest is used as the roofline's denominator."""
    import torch

    from prism_b200 import _lib
    L = _lib.lib()
    iters = 4000
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    ops = 2.0 * 128 * 256 * 128 * iters * sms
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.pb_int8_peak_probe(200, 1, 256, None, st), "peak probe")
    torch.cuda.synchronize()
    rates, t_end = [], time.time() + seconds
    while time.time() < t_end:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _lib.check(L.pb_int8_peak_probe(iters, 1, 256, None, st), "peak probe")
        e1.record()
        torch.cuda.synchronize()
        rates.append(ops / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return max(rates), sum(rates) / len(rates)


def launches_per_step(world):
    # per layer: 2 rows_q8 + rows_q8(attn) + swiglu + 4 GEMMs (+ fold per row-parallel projection and second quantizer
    # passes when tensor parallel)
    per_layer = 8 + (4 if world > 1 else 0)
    return per_layer * LAYERS


def time_gemms(stack, h0, steps):
    """Sum of the GEMM kernels' durations per step: CUDA events around each w8a8.gemm / gemm_i32 / gemm_scatter call of
    a pass."""
    import torch

    from prism_b200 import w8a8
    events = []
    orig, orig_i32, orig_sc = w8a8.gemm, w8a8.gemm_i32, w8a8.gemm_scatter

    def wrap(fn):
        def timed(*a, **k):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            r = fn(*a, **k)
            e.record()
            events.append((s, e))
            return r
        return timed
    w8a8.gemm, w8a8.gemm_i32, w8a8.gemm_scatter = wrap(orig), wrap(orig_i32), wrap(orig_sc)
    try:
        for _ in range(steps):
            stack(h0)
        torch.cuda.synchronize()
    finally:
        w8a8.gemm, w8a8.gemm_i32, w8a8.gemm_scatter = orig, orig_i32, orig_sc
    return sum(s.elapsed_time(e) for s, e in events) / steps


def time_e2e(stack, h0, steps, sync):
    """Host -> device copy of every step's input rows from pinned memory and device -> host copy of its result, inside
    the timed region; copies of neighbouring steps overlap the compute on their own streams (two device buffers)."""
    import torch
    dev = h0.device
    # several ranks on the row-split pass: a rank needs only its own M / n rows in and gives only those back (the
    # int8 inputs of the column-parallel projections are what the ranks exchange), so the host copies shrink with n
    own = bool(getattr(stack, "by_rows", False))
    src = h0[stack.r0:stack.r0 + stack.Ml] if own else h0
    host_in = src.cpu().pin_memory()
    host_out = torch.empty_like(host_in).pin_memory()
    d_in = [torch.empty_like(src) for _ in range(2)]
    d_out = [torch.empty_like(src) for _ in range(2)]
    s_in, s_out, s_c = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.current_stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_c = [torch.cuda.Event() for _ in range(2)]
    ev_free_in = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    sync()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(s_c)
    s_in.wait_stream(s_c)
    s_out.wait_stream(s_c)
    for i in range(steps):
        b = i & 1
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_free_in[b])
            d_in[b].copy_(host_in, non_blocking=True)
            ev_in[b].record(s_in)
        s_c.wait_event(ev_in[b])
        if i >= 2:
            s_c.wait_event(ev_out[b])
        out = stack(d_in[b], own_rows=True) if own else stack(d_in[b])
        ev_free_in[b].record(s_c)
        d_out[b].copy_(out, non_blocking=True)
        ev_c[b].record(s_c)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_c[b])
            host_out.copy_(d_out[b], non_blocking=True)
            ev_out[b].record(s_out)
    s_c.wait_stream(s_out)
    s_c.wait_stream(s_in)
    t1.record(s_c)
    sync()
    nbytes = src.numel() * src.element_size()
    return t0.elapsed_time(t1) / steps, nbytes, nbytes



# ------------------------------------------------------------------------------------------------------ detail table
SHAPES = {"qkv": (7168, 5120, 0), "o": (5120, 5120, 1), "gate_up": (34816, 5120, 0), "down": (5120, 17408, 1)}


def graph_time(fn_of_copy, copies, iters=None, reps=5):
    """Microseconds per call: a CUDA graph of back-to-back calls cycling over `copies` operand sets (so weights
    stream from HBM, not from L2), best of `reps` replays, CUDA events around each replay."""
    import torch
    iters = iters or max(copies, 8)
    for c in range(copies):
        fn_of_copy(c)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn_of_copy(i % copies)
    best = 1e30
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / iters)
    return best


def quick_detail(dev, pk):
    """The rest of the metric in the contract line, a few seconds in all: per format (W8A8 one group / per-32 groups,
    W4A8 on the Q4_K_M assignment, MXFP4) the GEMM rate at 8192 and 2048 rows and the algorithmic HBM rate at 16 rows
    on the four projection shapes, config 0 itself (Q8_0 groups, 5120 x 5120, 16 rows), and the FP4 tensor-core ceiling.
    Graph-timed with weight copies rotating through more than L2 (graph_time)."""
    import torch

    from prism_b200 import _lib, mxfp4, quant, w4a8, w8a8
    L2 = 126 << 20
    gen = torch.Generator(device=dev).manual_seed(11)
    hbm = pk["hbm"]
    out = {"hbm_peak_gbs": hbm, "note": "tops at M = 8192 / 2048 (prefill), us and fraction of the measured HBM copy rate "
           "at M = 16 (decode; weights at GGUF density); o and down include the fp32 residual add; 'chained': every "
           "launch a programmatic dependent of the one before it, as the few-row pass runs them"}
    u8 = lambda *sh, lo=0, hi=256: torch.randint(lo, hi, sh, dtype=torch.uint8, device=dev, generator=gen)   # noqa: E731
    i8 = lambda *sh: torch.randint(-127, 128, sh, dtype=torch.int8, device=dev, generator=gen)               # noqa: E731
    f = lambda *sh, m=1e-3: torch.rand(*sh, device=dev, generator=gen) * m                                    # noqa: E731
    kinds = {"qkv": [("q4k", 6144), ("q6k", 1024)], "o": [("q4k", 5120)], "gate_up": [("q4k", 34816)], "down": [("q6k", 5120)]}

    def rand_w4(kind, n, k):
        if kind == "q4k":
            return w4a8.W4("q4k", u8(n, k // 2), u8(k // 256, n, 8, hi=64), u8(k // 256, n, 8, hi=64), f(k // 256, n),
                           f(k // 256, n), n, k)
        return w4a8.W4("q6k", torch.randint(-32, 32, (n, k), dtype=torch.int8, device=dev, generator=gen),
                       torch.randint(-128, 128, (k // 256, n, 16), dtype=torch.int8, device=dev, generator=gen), None,
                       f(k // 256, n), None, n, k)
    for name, (N, K, epi) in SHAPES.items():
        row = {}
        odt = torch.bfloat16 if epi == 0 else torch.float32
        # ---- W8A8, one scale group (the engine's mode) and Q8_0's own groups
        copies = max(4, -(-3 * L2 // (N * K)))
        ws = [i8(N, K) for _ in range(copies)]
        sw1, sw32 = f(N), f(N, K // 32)
        for M in (8192, 2048, 16):
            a, sa1, nr = i8(M, K), f(M, m=1e-2), torch.tensor([M], dtype=torch.int32, device=dev)
            o = torch.zeros(M, N, dtype=odt, device=dev)
            slots = torch.zeros(4, M, N, dtype=torch.int32, device=dev) if (epi == 1 and M <= 64) else None
            pend = {}

            def call(c):
                pend[0] = w8a8.gemm(a, sa1, ws[c], sw1, o, nr, K, epi=epi, slots=slots)
            us = graph_time(call, copies, reps=3)
            if M > 64:
                row[f"w8a8_tops_M{M}"] = round(2.0 * M * N * K / us / 1e6)
            else:
                if pend[0] is not None:
                    us += graph_time(lambda c: quant.fold(o, slots, pend[0], nr, M), 1, iters=8, reps=3)
                nbytes = N * K + 4 * N + M * K + 4 * M + (2 if epi == 0 else 8) * M * N
                row["w8a8_M16_us"], row["w8a8_M16_hbm_frac"] = round(us, 1), round(nbytes / us / 1e3 / hbm, 3)

                # the same product as LinearStack runs it at few rows: every launch a programmatic dependent of the one
                # before it (set-up and first weight reads overlap the predecessor's tail), the deferred fold in the chain
                def chained(c):
                    pd = w8a8.gemm(a, sa1, ws[c], sw1, o, nr, K, epi=epi, slots=slots)
                    if pd is not None:
                        quant.fold(o, slots, pd, nr, M)
                before = _lib.lib().pb_set_pdl(1)
                try:
                    us = graph_time(chained, copies, reps=3)
                finally:
                    _lib.lib().pb_set_pdl(before)
                row["w8a8_M16_chained_us"], row["w8a8_M16_chained_hbm_frac"] = round(us, 1), round(nbytes / us / 1e3 / hbm, 3)
                sa32 = f(M, K // 32, m=1e-2)
                us = graph_time(lambda c: w8a8.gemm(a, sa32, ws[c], sw32, o, nr, 32, epi=epi), copies, reps=3)
                nbytes = N * K * 34 / 32 + M * K * 36 / 32 + (2 if epi == 0 else 8) * M * N
                row["w8a8_q8_0_groups_M16_us"], row["w8a8_q8_0_groups_M16_hbm_frac"] = round(us, 1), round(nbytes / us / 1e3 / hbm, 3)
                before = _lib.lib().pb_set_pdl(1)
                try:
                    us = graph_time(lambda c: w8a8.gemm(a, sa32, ws[c], sw32, o, nr, 32, epi=epi), copies, reps=3)
                finally:
                    _lib.lib().pb_set_pdl(before)
                row["w8a8_q8_0_groups_M16_chained_us"] = round(us, 1)
                row["w8a8_q8_0_groups_M16_chained_hbm_frac"] = round(nbytes / us / 1e3 / hbm, 3)
            del a, o, slots
        del ws
        torch.cuda.empty_cache()
        # ---- W4A8
        wbytes = sum(n * K * (144 if kind == "q4k" else 210) // 256 for kind, n in kinds[name])
        copies = max(2, -(-2 * L2 // wbytes))
        segsets = []
        for _ in range(copies):
            segs, off = [], 0
            for kind, n in kinds[name]:
                segs.append((rand_w4(kind, n, K), off))
                off += n
            segsets.append(segs)
        for M in (8192, 16):
            x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
            q = torch.empty(M, K, dtype=torch.int8, device=dev)
            sa = torch.empty(K // 256, M, device=dev)
            xs = torch.empty(K // 256, M, 16, dtype=torch.int8, device=dev)
            nr = torch.tensor([M], dtype=torch.int32, device=dev)
            quant.rows_g(x, q, sa, xs, nr, M)
            o = torch.zeros(M, N, dtype=odt, device=dev)
            us = graph_time(lambda c: w4a8.gemm_segs(q, sa, xs, segsets[c], o, nr, epi), copies, reps=3)
            if M > 64:
                row[f"w4a8_tops_M{M}"] = round(2.0 * M * N * K / us / 1e6)
            else:
                nbytes = wbytes + M * K * (1 + 20 / 256) + (2 if epi == 0 else 8) * M * N
                row["w4a8_M16_us"], row["w4a8_M16_hbm_frac"] = round(us, 1), round(nbytes / us / 1e3 / hbm, 3)
            del x, q, o
        del segsets
        torch.cuda.empty_cache()
        # ---- MXFP4
        copies = max(2, -(-2 * L2 // (N * K * 17 // 32)))
        wms = [mxfp4.prepare(mxfp4.MX4(u8(N, K // 2), u8(N, K // 32, lo=118, hi=126), N, K)) for _ in range(copies)]
        for M in (8192, 16):
            x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
            q = torch.empty(M, K // 2, dtype=torch.uint8, device=dev)
            sc = torch.empty(M, K // 32, dtype=torch.uint8, device=dev)
            mxfp4.quantize_act(x, q, sc)
            o = torch.zeros(M, N, dtype=odt, device=dev)
            mxfp4.gemm(q, sc, wms[0], o, M, epi=epi)
            us = graph_time(lambda c: mxfp4.gemm(q, sc, wms[c], o, M, epi=epi), copies, reps=3)
            if M > 64:
                row[f"mxfp4_tflops_M{M}"] = round(2.0 * M * N * K / us / 1e6)
            else:
                nbytes = (N + M) * K * 17 / 32 + (2 if epi == 0 else 8) * M * N
                row["mxfp4_M16_us"], row["mxfp4_M16_hbm_frac"] = round(us, 1), round(nbytes / us / 1e3 / hbm, 3)
            del x, q, o
        del wms
        torch.cuda.empty_cache()
        out[name] = row
    out["config0_q8_0_5120x5120_M16_us"] = out["o"].get("w8a8_q8_0_groups_M16_us")
    out["config0_q8_0_5120x5120_M16_chained_us"] = out["o"].get("w8a8_q8_0_groups_M16_chained_us")
    L = _lib.lib()
    if hasattr(L, "pb_mxf4_peak_probe"):
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        iters = 4000
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(L.pb_mxf4_peak_probe(200, 1, None, st), "mxf4 peak probe")
        torch.cuda.synchronize()
        rates, t_end = [], time.time() + 0.3
        while time.time() < t_end:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _lib.check(L.pb_mxf4_peak_probe(iters, 1, None, st), "mxf4 peak probe")
            e1.record()
            torch.cuda.synchronize()
            rates.append(2.0 * 128 * 256 * 256 * iters * sms / (e0.elapsed_time(e1) * 1e-3) / 1e12)
        out["fp4_peak_tflops_measured"] = round(max(rates))
        out["fp4_peak_note"] = ("tcgen05 kind::mxf4.block_scale 128x256x64 on shared-memory-resident operands, one CTA per "
                                f"SM, 0.3 s: highest launch {max(rates):.0f}, mean {sum(rates) / len(rates):.0f}; nominal "
                                "dense FP4 9000")
        for name in SHAPES:
            if "mxfp4_tflops_M8192" in out[name]:
                out[name]["mxfp4_frac_of_measured_fp4_peak"] = round(out[name]["mxfp4_tflops_M8192"] / max(rates), 3)
    code, where = _lib.device_status()
    out["device_status"] = code
    return out


def run_detail(args):
    """Per projection shape and row count: time, TOPS, algorithmic GB/s (weights at GGUF Q8_0 density for gk = 32, int8
    + one fp32 scale per row for gk = K) and the fractions of the measured peaks.  One JSON object per line."""
    import torch

    from prism_b200 import _lib, quant, w8a8
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    pk = peaks()
    L2 = 126 << 20
    rows_list = [int(x) for x in (args.detail_rows or "1,8,16,64,256,2048,8192").split(",")]
    only = args.detail_shapes.split(",") if args.detail_shapes else list(SHAPES)
    gks = [int(x) for x in (args.detail_gk or "0").split(",")]            # 0 = one group (gk == K)
    gen = torch.Generator(device=dev).manual_seed(1)
    for name in ([] if args.detail_formats and "w8a8" not in args.detail_formats else only):
        N, K, epi = SHAPES[name]
        copies = max(4, -(-3 * L2 // (N * K)))
        ws = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev, generator=gen) for _ in range(copies)]
        for gk in gks:
            G = 1 if gk == 0 else K // gk
            sw = torch.rand(N, G, device=dev, generator=gen) * 1e-3
            for M in rows_list:
                if gk and M > 256:
                    continue
                a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev, generator=gen)
                sa = torch.rand(M, G, device=dev, generator=gen) * 1e-2
                nr = torch.tensor([M], dtype=torch.int32, device=dev)
                out = torch.zeros(M, N, dtype=torch.bfloat16 if epi == 0 else torch.float32, device=dev)
                slots = torch.zeros(4, M, N, dtype=torch.int32, device=dev) if (epi == 1 and M <= 64 and not gk) else None
                pend = {}

                def call(c):
                    pend[0] = w8a8.gemm(a, sa, ws[c], sw, out, nr, gk or K, epi=epi, slots=slots,
                                        cfg=args.detail_split, pdl=args.detail_pdl)
                call(0)
                us = graph_time(call, copies)
                fold_us = 0.0
                if pend[0] is not None:
                    fold_us = graph_time(lambda c: quant.fold(out, slots, pend[0], nr, M), 1, iters=8)
                ops = 2.0 * M * N * K
                wbytes = N * K * 34 / 32 if gk == 32 else N * K + 4 * N
                obytes = (2 if epi == 0 else 8) * M * N if pend[0] is None else 4 * pend[0].n * M * N
                abytes = M * K + 4 * M * G
                gbs = (wbytes + abytes + obytes) / us / 1e3
                print(json.dumps({"shape": name, "N": N, "K": K, "M": M, "gk": gk or K, "epi": epi,
                                  "split": None if pend[0] is None else pend[0].n, "us": round(us, 2),
                                  "fold_us": round(fold_us, 2), "tops": round(ops / us / 1e6, 1),
                                  "gbs": round(gbs, 1), "frac_hbm_measured": round(gbs / pk["hbm"], 3),
                                  "frac_int8_2x_bf16_sustained": round(ops / us / 1e6 / (2 * pk["bf16"]), 3)}),
                      flush=True)
        del ws
        torch.cuda.empty_cache()
    # W4A8 (Q4_K_M assignment: q|k Q4_K + v Q6_K, o and gate|up Q4_K, down Q6_K) and MXFP4, same shapes and row counts
    from prism_b200 import mxfp4, w4a8
    if args.detail_formats:
        fmts = args.detail_formats.split(",")
        kinds = {"qkv": [("q4k", 6144), ("q6k", 1024)], "o": [("q4k", 5120)], "gate_up": [("q4k", 34816)],
                 "down": [("q6k", 5120)]}

        def rand_w4(kind, n, k):
            u8 = lambda *sh, hi=256: torch.randint(0, hi, sh, dtype=torch.uint8, device=dev, generator=gen)   # noqa: E731
            f = lambda *sh: torch.rand(*sh, device=dev, generator=gen) * 1e-3                                # noqa: E731
            if kind == "q4k":
                return w4a8.W4("q4k", u8(n, k // 2), u8(k // 256, n, 8, hi=64), u8(k // 256, n, 8, hi=64),
                               f(k // 256, n), f(k // 256, n), n, k)
            return w4a8.W4("q6k", torch.randint(-32, 32, (n, k), dtype=torch.int8, device=dev, generator=gen),
                           torch.randint(-128, 128, (k // 256, n, 16), dtype=torch.int8, device=dev, generator=gen),
                           None, f(k // 256, n), None, n, k)
        for name in only:
            N, K, epi = SHAPES[name]
            if "w4a8" in fmts:
                segs, off = [], 0
                for kind, n in kinds[name]:
                    segs.append((rand_w4(kind, n, K), off))
                    off += n
                wbytes = sum(n * K * (144 if kind == "q4k" else 210) // 256 for kind, n in kinds[name])
                for M in rows_list:
                    x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
                    q = torch.empty(M, K, dtype=torch.int8, device=dev)
                    sa = torch.empty(K // 256, M, device=dev)
                    xs = torch.empty(K // 256, M, 16, dtype=torch.int8, device=dev)
                    nr = torch.tensor([M], dtype=torch.int32, device=dev)
                    quant.rows_g(x, q, sa, xs, nr, M)
                    out = torch.zeros(M, N, dtype=torch.bfloat16 if epi == 0 else torch.float32, device=dev)
                    us = graph_time(lambda c: w4a8.gemm_segs(q, sa, xs, segs, out, nr, epi), 1, iters=4)
                    ops = 2.0 * M * N * K
                    nbytes = wbytes + M * K * (1 + 20 / 256) + (2 if epi == 0 else 8) * M * N
                    print(json.dumps({"format": "w4a8", "shape": name, "kinds": [k for k, _ in kinds[name]], "M": M,
                                      "us": round(us, 2), "tops": round(ops / us / 1e6, 1),
                                      "gbs_gguf_density": round(nbytes / us / 1e3, 1),
                                      "frac_hbm_measured": round(nbytes / us / 1e3 / pk["hbm"], 3)}), flush=True)
            if "mxfp4" in fmts:
                wq = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=gen)
                wsc = torch.randint(118, 126, (N, K // 32), dtype=torch.uint8, device=dev, generator=gen)
                wm = mxfp4.prepare(mxfp4.MX4(wq, wsc, N, K))
                for M in rows_list:
                    x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
                    q = torch.empty(M, K // 2, dtype=torch.uint8, device=dev)
                    sc = torch.empty(M, K // 32, dtype=torch.uint8, device=dev)
                    mxfp4.quantize_act(x, q, sc)
                    out = torch.zeros(M, N, dtype=torch.bfloat16 if epi == 0 else torch.float32, device=dev)
                    msplit = "auto" if args.detail_mx_split else None
                    mxfp4.gemm(q, sc, wm, out, M, epi=epi, split=msplit)
                    us = graph_time(lambda c: mxfp4.gemm(q, sc, wm, out, M, epi=epi, split=msplit), 1, iters=4)
                    ops = 2.0 * M * N * K
                    nbytes = (N + M) * K * 17 / 32 + (2 if epi == 0 else 8) * M * N
                    print(json.dumps({"format": "mxfp4", "shape": name, "M": M, "us": round(us, 2),
                                      "tflops": round(ops / us / 1e6, 1), "gbs": round(nbytes / us / 1e3, 1),
                                      "frac_hbm_measured": round(nbytes / us / 1e3 / pk["hbm"], 3),
                                      "frac_fp4_4x_bf16_sustained": round(ops / us / 1e6 / (4 * pk["bf16"]), 3)}),
                          flush=True)
            torch.cuda.empty_cache()
    # activation quantizers
    for T, K in ((8192, 5120), (8192, 17408), (64, 5120)):
        x = torch.randn(T, K, device=dev, generator=gen).to(torch.bfloat16)
        q = torch.empty(T, K, dtype=torch.int8, device=dev)
        s = torch.empty(T, device=dev)
        nr = torch.tensor([T], dtype=torch.int32, device=dev)
        us = graph_time(lambda c: quant.rows_q8(x, None, q, s, nr, T), 1, iters=8)
        b = 3.0 * T * K + 4 * T
        print(json.dumps({"kernel": "rows_q8", "T": T, "K": K, "us": round(us, 2), "gbs": round(b / us / 1e3, 1),
                          "frac_hbm_measured": round(b / us / 1e3 / pk["hbm"], 3)}), flush=True)
    for T, K in ((8192, 5120), (64, 5120)):
        h = torch.randn(T, K, device=dev, generator=gen)
        wn = torch.rand(K, device=dev, generator=gen) + 0.5
        q = torch.empty(T, K, dtype=torch.int8, device=dev)
        s = torch.empty(T, device=dev)
        nr = torch.tensor([T], dtype=torch.int32, device=dev)
        us = graph_time(lambda c: quant.norm_q8(h, wn, q, s, nr, T, 1e-6), 1, iters=8)
        b = 5.0 * T * K + 4 * T
        print(json.dumps({"kernel": "norm_q8", "T": T, "K": K, "us": round(us, 2), "gbs": round(b / us / 1e3, 1),
                          "frac_hbm_measured": round(b / us / 1e3 / pk["hbm"], 3)}), flush=True)
    FF = 17408
    gu = torch.randn(8192, 2 * FF, device=dev, generator=gen).to(torch.bfloat16)
    q = torch.empty(8192, FF, dtype=torch.int8, device=dev)
    s = torch.empty(8192, device=dev)
    nr = torch.tensor([8192], dtype=torch.int32, device=dev)
    us = graph_time(lambda c: quant.swiglu_q8(gu, None, q, s, nr, 8192), 1, iters=8)
    b = 5.0 * 8192 * FF
    print(json.dumps({"kernel": "swiglu_q8", "T": 8192, "FF": FF, "us": round(us, 2), "gbs": round(b / us / 1e3, 1),
                      "frac_hbm_measured": round(b / us / 1e3 / pk["hbm"], 3)}), flush=True)
    if args.detail_head:
        # the vocabulary head (Q8_0, per-32 groups, N = 248,320): 1.27 GB of weights + 159 MB of group scales per step
        from prism_b200 import decode
        N, K = 248320, 5120
        w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev, generator=gen)
        ws = torch.rand(N, K // 32, device=dev, generator=gen) * 1e-3
        for M in (1, 16, 64):
            a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev, generator=gen)
            sa = torch.rand(M, K // 32, device=dev, generator=gen) * 1e-2
            out = torch.zeros(M, N, device=dev)
            nr = torch.tensor([M], dtype=torch.int32, device=dev)
            us = graph_time(lambda c: decode.head_q8(a, sa, w, ws, out, nr, M), 1, iters=4)
            b = N * K * 34.0 / 32 + M * K + 4.0 * M * N
            print(json.dumps({"kernel": "head_q8", "M": M, "N": N, "K": K, "us": round(us, 2),
                              "gbs": round(b / us / 1e3, 1), "frac_hbm_measured": round(b / us / 1e3 / pk["hbm"], 3)}),
                  flush=True)
        del w, ws
        torch.cuda.empty_cache()
    code, where = _lib.device_status()
    print(json.dumps({"device_status": code, "where": where}))


# ------------------------------------------------------------------------------------------------------ probes
def run_probe(args):
    """A few eager launches of one kernel on a case larger than L2 but small in memory: the command ncu captures
    (`ncu --clock-control none --metrics gpu__time_duration.sum -k regex:<kernel> -c 3 python bench.py --probe <case>`;
    sections or more metrics only with `-c 1`, and only after the same command has exited 0 without ncu); also prints
    the CUDA-event time per launch."""
    import torch

    from prism_b200 import _lib, mxfp4, quant, synth, w4a8, w8a8
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev).manual_seed(2)
    case = args.probe
    if case == "peak":
        return run_peak(dev)
    ri = lambda *s: torch.randint(-127, 128, s, dtype=torch.int8, device=dev, generator=gen)     # noqa: E731
    if case in ("tile", "tile_add", "decode", "decode32", "config0"):
        M = 2048 if case.startswith("tile") else 16
        N, K = (34816, 5120) if case in ("tile", "decode32") else (5120, 17408)
        if case == "tile_add":
            N, K = 5120, 17408
        if case == "config0":                              # BASELINE config 0: Q8_0 groups, 5120 x 5120, 16 rows
            N, K = 5120, 5120
        gk = 32 if case in ("decode32", "config0") else K
        a, w = ri(M, K), ri(N, K)
        sa = torch.rand(M, K // gk, device=dev, generator=gen) * 1e-2
        sw = torch.rand(N, K // gk, device=dev, generator=gen) * 1e-3
        epi = 1 if case in ("tile_add", "decode") else 0
        out = torch.zeros(M, N, dtype=torch.float32 if epi else torch.bfloat16, device=dev)
        slots = torch.zeros(4, M, N, dtype=torch.int32, device=dev) if case == "decode" else None
        nr = torch.tensor([M], dtype=torch.int32, device=dev)
        fn = lambda: w8a8.gemm(a, sa, w, sw, out, nr, gk, epi=epi, slots=slots)                   # noqa: E731
        ops, nbytes = 2.0 * M * N * K, N * K + M * K
    elif case in ("w4a8_q4k", "w4a8_q6k", "w4a8_q4k_decode", "w4a8_q6k_decode"):
        M, N, K = (args.probe_rows or 16, 34816, 5120) if case.endswith("decode") else (2048, 8192, 5120)
        wcpu = synth.weights(N, K, 3)
        w = w4a8.repack((synth.q4_k if "q4k" in case else synth.q6_k)(wcpu)).to(dev)
        x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
        q = torch.empty(M, K, dtype=torch.int8, device=dev)
        s = torch.empty(K // 256, M, device=dev)
        xs = torch.empty(K // 256, M, 16, dtype=torch.int8, device=dev)
        nr = torch.tensor([M], dtype=torch.int32, device=dev)
        quant.rows_g(x, q, s, xs, nr, M)
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        fn = lambda: w4a8.gemm(q, s, xs, w, out, nr)                                              # noqa: E731
        ops, nbytes = 2.0 * M * N * K, w.nbytes() + M * K
    elif case == "mxfp4":
        M, N, K = 2048, 34816, 5120
        wq = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=gen)
        ws = torch.randint(118, 126, (N, K // 32), dtype=torch.uint8, device=dev, generator=gen)
        w = mxfp4.prepare(mxfp4.MX4(wq, ws, N, K))
        x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
        q = torch.empty(M, K // 2, dtype=torch.uint8, device=dev)
        s = torch.empty(M, K // 32, dtype=torch.uint8, device=dev)
        mxfp4.quantize_act(x, q, s)
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        fn = lambda: mxfp4.gemm(q, s, w, out, M)                                                  # noqa: E731
        ops, nbytes = 2.0 * M * N * K, N * K * 17 // 32 + M * K * 17 // 32
    elif case in ("rows_q8", "swiglu_q8"):
        T, K = 8192, 17408
        nr = torch.tensor([T], dtype=torch.int32, device=dev)
        q = torch.empty(T, K, dtype=torch.int8, device=dev)
        s = torch.empty(T, device=dev)
        if case == "rows_q8":
            x = torch.randn(T, K, device=dev, generator=gen).to(torch.bfloat16)
            fn = lambda: quant.rows_q8(x, None, q, s, nr, T)                                      # noqa: E731
            ops, nbytes = 0.0, 3 * T * K
        else:
            x = torch.randn(T, 2 * K, device=dev, generator=gen).to(torch.bfloat16)
            fn = lambda: quant.swiglu_q8(x, None, q, s, nr, T)                                    # noqa: E731
            ops, nbytes = 0.0, 5 * T * K
    else:
        raise SystemExit(f"unknown probe {case}")
    fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(5)]
    for a0, a1 in ev:
        a0.record()
        fn()
        a1.record()
    torch.cuda.synchronize()
    us = min(a0.elapsed_time(a1) for a0, a1 in ev) * 1e3
    code, where = _lib.device_status()
    print(json.dumps({"probe": case, "us": round(us, 2), "tops": round(ops / us / 1e6, 1),
                      "gbs": round(nbytes / us / 1e3, 1), "device_status": code}), flush=True)


def run_peak(dev):
    """The int8 tensor-core ceiling: pb_int8_peak_probe for ~2 s per operand pattern with the SM clock and power sampled,
    next to the same loop over a real GEMM (gate|up, M = 8192)."""
    import torch

    from prism_b200 import _lib, w8a8
    L = _lib.lib()
    iters = 20000
    ops = 2.0 * 128 * 256 * 128 * iters * 148
    st = lambda: torch.cuda.current_stream().cuda_stream                  # noqa: E731
    for pattern in (0, 1):
        L.pb_int8_peak_probe(200, pattern, 256, None, st())
        torch.cuda.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        best, t_end = 0.0, time.time() + 2.0
        rates = []
        while time.time() < t_end:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _lib.check(L.pb_int8_peak_probe(iters, pattern, 256, None, st()), "peak probe")
            e1.record()
            torch.cuda.synchronize()
            rates.append(ops / (e0.elapsed_time(e1) * 1e-3) / 1e12)
        clocks = sampler.stop()
        print(json.dumps({"probe": "int8_peak", "pattern": "random" if pattern else "zeros", "tops_first": round(rates[0], 1),
                          "tops_last": round(rates[-1], 1), "tops_max": round(max(rates), 1), "launches": len(rates),
                          "clocks": clocks}), flush=True)
    # issue cost of one MMA against its N: small-N instructions have a floor (what bounds the few-rows kernels)
    cyc = torch.zeros(148, dtype=torch.int64, device=dev)
    for n in (16, 32, 64, 128, 256):
        _lib.check(L.pb_int8_peak_probe(2000, 0, n, cyc.data_ptr(), st()), "peak probe")
        torch.cuda.synchronize()
        print(json.dumps({"probe": "mma_issue", "mma": f"128x{n}x32", "cycles_per_mma": round(float(cyc.float().mean()) / 8000, 1)}),
              flush=True)
    gen = torch.Generator(device=dev).manual_seed(2)
    M, N, K = 8192, 34816, 5120
    a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev, generator=gen)
    w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev, generator=gen)
    g = (torch.randn(M, K, device=dev, generator=gen) * 25).round().clamp(-127, 127).to(torch.int8)
    sa, sw = torch.rand(M, device=dev) * 1e-2, torch.rand(N, device=dev) * 1e-3
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    nr = torch.tensor([M], dtype=torch.int32, device=dev)
    for name, act in (("uniform int8 activations", a), ("gaussian int8 activations (sigma 25)", g)):
        w8a8.gemm(act, sa, w, sw, out, nr, K)
        torch.cuda.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        rates, t_end = [], time.time() + 2.0
        while time.time() < t_end:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                w8a8.gemm(act, sa, w, sw, out, nr, K)
            e1.record()
            torch.cuda.synchronize()
            rates.append(10 * 2.0 * M * N * K / (e0.elapsed_time(e1) * 1e-3) / 1e12)
        print(json.dumps({"probe": "gemm_sustained", "case": name, "tops_first": round(rates[0], 1),
                          "tops_last": round(rates[-1], 1), "clocks": sampler.stop()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="prism_b200", choices=["prism_b200", "reference"])
    ap.add_argument("--rows", type=int, default=M_DEFAULT)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-ref-gpu", action="store_true", help="reference arm: skip timing the reference's Triton kernel")
    ap.add_argument("--no-detail", action="store_true", help="skip the short per-format detail object of the JSON line")
    ap.add_argument("--graph", action="store_true", help="time the pass as a replayed CUDA graph (decode rows)")
    ap.add_argument("--detail", action="store_true", help="per-shape GEMM table instead of the JSON line")
    ap.add_argument("--probe", default=None, help="one kernel case, a few eager launches (for ncu)")
    ap.add_argument("--probe-rows", type=int, default=None, help="activation rows of the W4A8 decode probes")
    ap.add_argument("--detail-rows", default=None)
    ap.add_argument("--detail-head", action="store_true", help="add the vocabulary head (head_q8) to --detail")
    ap.add_argument("--detail-shapes", default=None)
    ap.add_argument("--detail-gk", default=None, help="comma list; 0 = one group per row (gk == K), 32 = Q8_0 blocks")
    ap.add_argument("--detail-split", type=int, default=None)
    ap.add_argument("--detail-mx-split", action="store_true", help="MXFP4 GEMMs with split=\"auto\" (K slices per tile)")
    ap.add_argument("--detail-formats", default=None, help="comma list of extra formats: w4a8,mxfp4")
    ap.add_argument("--detail-pdl", action="store_true", help="few-rows GEMMs as programmatic dependent launches")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.probe:
        run_probe(args)
    elif args.detail:
        run_detail(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
