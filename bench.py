#!/usr/bin/env python
"""Benchmark of the quantized-weight decode GEMV path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload): the Q4_K decode GEMV set with Llama-2-7B layer shapes, batch 1:
per layer four matmuls (N x K) 4096x4096, 11008x4096, 11008x4096, 4096x11008, weights Q4_K,
activations f32 ~ N(0,1), outputs f32. One STEP is one decode token's pass over all 32 layers
(128 GEMV launches, 2.74 GB of distinct quantized weights), so every weight byte is read once
per step and the working set is ~22x the 126 MB L2: the numbers are HBM numbers. Weights are
seeded synthetic blocks with the value distributions of the real format (no checkpoint).

value   = quantized weight bytes read per second over all GPUs, device-timed with CUDA events,
          inputs resident in HBM.
e2e     = the same, measured through the host-buffer boundary (CudaBackend: upload of the
          step's activations from pinned host memory, 128 gemm() calls, download of the outputs).
roofline= the streaming GEMV kernel against the measured HBM copy bandwidth.
cpu_baseline = Kraken's own CPU backend (compiled reference sources when available, else the
          in-repo restatement) on a bounded sample of the same workload.

With N > 1 every rank runs its own replica of the workload (these dense layers do not shard;
the sharded head / expert configs are reported under "sharded"), timing is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from kraken_b200 import synth  # noqa: E402

LAYER_SHAPES = [(4096, 4096), (11008, 4096), (11008, 4096), (4096, 11008)]   # (n_out, n_in)
N_LAYERS = 32
WT = synth.Q4_K
METRIC = "quant GEMV weight GB/s"
UNIT = "GB/s"
WORKLOAD = "q4_k_decode_gemv_llama2_7b_layer_set_x32"


def layer_weight_bytes() -> int:
    return sum(n * synth.row_bytes(WT, k) for n, k in LAYER_SHAPES)


def layer_algorithmic_bytes() -> int:
    # weights once + x + y per matmul
    return sum(n * synth.row_bytes(WT, k) + 4 * k + 4 * n for n, k in LAYER_SHAPES)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---- clocks ---------------------------------------------------------------------------------

class ClockSampler:
    """SM clock and throttle reasons of one GPU, read through NVML from a thread of this process every few
    milliseconds (read-only queries). `mark()` brackets the timed region: only samples taken inside it are
    reported, so a short run still carries a few. Falls back to an `nvidia-smi -lms` child when the NVML
    binding is missing."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, uuid: str = None):
        self.index, self.uuid = index, uuid
        self.proc = self.path = self.thread = None
        self.samples = []          # (time, sm_mhz, reasons bitmask)
        self.t0 = self.t1 = None
        self.sm_max = None
        self._stop = False

    def start(self):
        try:
            import threading
            import pynvml
            pynvml.nvmlInit()
            handle = None
            if self.uuid:
                try:
                    handle = pynvml.nvmlDeviceGetHandleByUUID(self.uuid)
                except Exception:
                    handle = None
            if handle is None:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons

            def loop():
                while not self._stop:
                    try:
                        mhz = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                        self.samples.append((time.perf_counter(), mhz, int(reasons_fn(handle))))
                    except Exception:
                        pass
                    time.sleep(0.004)
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def mark(self):
        """First call: the timed region starts; second call: it has ended."""
        if self.t0 is None:
            self.t0 = time.perf_counter()
        else:
            self.t1 = time.perf_counter()

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=2)
            inside = [s for s in self.samples if self.t0 is None or self.t1 is None or self.t0 <= s[0] <= self.t1]
            # NVML bit masks of the reasons that invalidate (or annotate) a measurement
            bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20}
            if inside:
                mask = 0
                for _, _, r in inside:
                    mask |= r
                out.update(sm_mhz=statistics.median(s[1] for s in inside), sm_max_mhz=self.sm_max,
                           reasons=sorted(n for n, b in bits.items() if mask & b), samples=len(inside), source="nvml")
            return out
        if not self.proc:
            return out
        self.proc.terminate()          # our own child, by handle
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(smax), reasons=sorted(reasons), samples=len(sm),
                       source="nvidia-smi")
        return out


# ---- our arm ------------------------------------------------------------------------------------

def device_weights(torch, n_out: int, n_in: int, gen):
    """Q4_K blocks made on the device: payload bytes uniform (so every nibble and every packed
    6-bit scale/min is uniform, as in the spec), d in [1e-3, 1e-2], dmin in [0, 5e-3] as f16."""
    nblk = n_in // 256
    w = torch.randint(0, 256, (n_out, nblk, 144), dtype=torch.uint8, device="cuda", generator=gen)
    d = (1e-3 + 9e-3 * torch.rand((n_out, nblk), device="cuda", generator=gen)).to(torch.float16)
    dm = (5e-3 * torch.rand((n_out, nblk), device="cuda", generator=gen)).to(torch.float16)
    w[..., 0:2] = d.view(torch.uint8).view(n_out, nblk, 2)
    w[..., 2:4] = dm.view(torch.uint8).view(n_out, nblk, 2)
    return w.view(n_out, nblk * 144)


def workload_config(layers: int, world: int) -> dict:
    """The `config` of the bench line: the same dictionary from both arms."""
    return {"workload": WORKLOAD, "weight_type": "Q4_K", "batch": 1, "layers": layers,
            "matmuls_per_layer": [list(s) for s in LAYER_SHAPES],
            "weight_bytes_per_step": layer_weight_bytes() * layers, "parallelism": f"replicas x{world}",
            "l2": "inputs larger than L2: every layer of a step has its own weights in memory, each byte read once per step"}


def layer_shift(li: int, n_out: int) -> int:
    """Rows by which layer li's matrices are rotated against layer 0's (layer li row r = layer 0 row r + shift)."""
    return (li * 1031) % n_out


def check_step(torch, layers, base, grouped):
    """What the timed step computes, against the CPU checker, before anything is timed: the four outputs of
    layer 0 and of the last layer within 1e-4 * ||w_row|| * ||x|| of the exact scalar chain on the same bytes
    (the last layer's rows are layer 0's rotated, so the checker multiplies layer 0's matrix by that layer's x)."""
    from oracle.krk_oracle import Oracle
    orc = Oracle()
    worst = 0.0
    for li in sorted({0, len(layers) - 1}):
        for mi, (w_np, _, n_out, n_in) in enumerate(base):
            _, x, y, _, _ = layers[li][mi]
            if grouped and mi == 2:
                x = layers[li][1][1]          # gate and up leave in one launch on the gate's activation row
            x_np = x.cpu().numpy().reshape(1, -1)
            ref = orc.gemm(x_np, w_np, WT, n_out, n_in, threads=os.cpu_count() or 1)[0]
            wd = orc.dequant_rows(w_np, WT, n_out, n_in).astype(np.float64)
            lim = 1e-4 * np.sqrt((wd ** 2).sum(axis=1)) * np.sqrt((x_np.astype(np.float64) ** 2).sum())
            got = np.roll(y.cpu().numpy().astype(np.float64), layer_shift(li, n_out))
            err = np.abs(got - ref)
            if not (err <= lim).all():
                raise AssertionError(f"bench step differs from the CPU checker: layer {li} matmul {mi}, "
                                     f"worst {float((err / lim).max()):.3g} of the bound")
            worst = max(worst, float((err / np.maximum(lim, 1e-300)).max()))
    return {"layers_checked": sorted({0, len(layers) - 1}), "bound": "1e-4 * ||w_row|| * ||x||",
            "worst_fraction_of_bound": round(worst, 5)}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from kraken_b200 import capi

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    gen = torch.Generator(device="cuda")
    gen.manual_seed(synth.BASE_SEED % (2 ** 63) + 2 + 1000 * rank)
    # Layer 0 is the seeded synthetic layer the CPU legs use, byte for byte (synth.weights / synth.activations
    # with the same seed and streams). The other layers hold the same rows rotated by a layer-specific count:
    # every row keeps the format's field distributions, every layer has its own 85 MB in HBM (2.74 GB of distinct
    # addresses per step), and any layer's output is layer 0's rotated, so the checker can vouch for all of them.
    base = cpu_layer()
    layers = []
    for li in range(args.layers):
        mats = []
        for mi, (w0, _, n_out, n_in) in enumerate(base):
            # rotated on the host and uploaded: setting the workload up launches no kernel
            w = torch.from_numpy(w0 if li == 0 else np.ascontiguousarray(np.roll(w0, -layer_shift(li, n_out), axis=0))).cuda()
            x = torch.from_numpy(synth.activations(1, n_in, synth.BASE_SEED + 2, stream=200 + mi + 10 * li)).cuda().view(-1)
            y = torch.empty(n_out, device="cuda")
            mats.append((w, x, y, n_out, n_in))
        layers.append(mats)
    stream = torch.cuda.current_stream()

    # Gate and up read the same activation row and leave in ONE grouped launch, which is how Kraken's engine
    # issues them (Backend::gemm_group, include/krk/backend.hpp:1040-1056); --ungrouped launches all four apart.
    grouped = not args.ungrouped
    assert LAYER_SHAPES[1] == LAYER_SHAPES[2]

    def launch_layer(mats, st):
        (w0, x0, y0, n0, k0), (wg, xg, yg, ng, kg), (wu, _, yu, nu, _), (wd, xd, yd, nd, kd) = mats
        capi.gemv(x0, w0, WT, n0, k0, out=y0.view(1, -1), stream=st)
        if grouped:
            capi.gemv_group([xg, xg], [wg, wu], [WT, WT], [ng, nu], kg, outs=[yg, yu], stream=st)
        else:
            capi.gemv(xg, wg, WT, ng, kg, out=yg.view(1, -1), stream=st)
            capi.gemv(xg, wu, WT, nu, kg, out=yu.view(1, -1), stream=st)
        capi.gemv(xd, wd, WT, nd, kd, out=yd.view(1, -1), stream=st)

    def step():
        for mats in layers:
            launch_layer(mats, stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    assert capi.device_status() == 0, "a device-side wait gave up during warm-up"
    assert all(torch.isfinite(m[2]).all() for m in layers[0])
    checked = check_step(torch, layers, base, grouped) if rank == 0 and not args.no_check else None

    # The step's launches are captured once into a CUDA graph and replayed: same kernels, same
    # order, without a host round trip per launch (a decode loop replays a fixed launch sequence).
    launches_per_step = (3 if grouped else 4) * args.layers
    replay = step
    graph_holder = []
    if not args.no_graph:
        cap_stream = torch.cuda.Stream()
        cap_stream.wait_stream(stream)
        c0 = capi.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(cap_stream):
            graph.capture_begin()
            for mats in layers:
                launch_layer(mats, cap_stream)
            graph.capture_end()
        launches_per_step = capi.launch_count() - c0
        stream = cap_stream
        graph_holder.append(graph)

        def replay():
            graph.replay()
        with torch.cuda.stream(cap_stream):
            for _ in range(3):
                replay()
        barrier()

    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        uuid = None
    sampler = ClockSampler(local, uuid)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark()
    with torch.cuda.stream(stream):
        ev0.record(stream)
        for _ in range(args.steps):
            replay()
        ev1.record(stream)
    barrier()
    sampler.mark()
    ms = ev0.elapsed_time(ev1)
    launches = launches_per_step * args.steps
    clocks = sampler.stop() if rank == 0 else None
    assert capi.device_status() == 0, "a device-side wait gave up during the timed region"

    # ---- end to end through the host-buffer boundary (CudaBackend) ----
    be = capi.Backend(local)
    x_host = torch.randn(sum(k for _, k in LAYER_SHAPES) * args.layers, generator=torch.Generator().manual_seed(7)).pin_memory()
    y_host = torch.empty(sum(n for n, _ in LAYER_SHAPES) * args.layers).pin_memory()
    d_x = be.alloc(x_host.numel() * 4)
    d_y = be.alloc(y_host.numel() * 4)

    # The step's calls into the C shim of CudaBackend, with their argument arrays built once: what a C++ host (the
    # engine) passes per call is a handful of pointers, and a Python loop that rebuilt ctypes arrays for every
    # one of the 96 calls would time the interpreter instead of the boundary.
    import ctypes as C
    calls = []
    xo = yo = 0
    for mats in layers:
        i = 0
        while i < len(mats):
            w, _, _, n_out, n_in = mats[i]
            if grouped and i == 1:      # gate and up: one gemm_group call on the gate's activation row
                wu = mats[2][0]
                outs = (C.c_void_p * 2)(d_y + 4 * yo, d_y + 4 * (yo + n_out))
                ws2 = (C.c_void_p * 2)(w.data_ptr(), wu.data_ptr())
                nouts = (C.c_int64 * 2)(n_out, n_out)
                fused = C.c_int(0)
                calls.append((capi.lib.krk_cuda_backend_gemm_group,
                              (be.h, outs, d_x + 4 * xo, ws2, WT, nouts, n_in, 2, 1, 0, C.byref(fused))))
                xo += 2 * n_in
                yo += 2 * n_out
                i += 2
                continue
            calls.append((capi.lib.krk_cuda_backend_gemm, (be.h, d_y + 4 * yo, d_x + 4 * xo, w.data_ptr(), WT, n_out, n_in, 1)))
            xo += n_in
            yo += n_out
            i += 1

    def e2e_step():
        be.upload(d_x, x_host.data_ptr(), x_host.numel() * 4)
        for fn, a in calls:
            fn(*a)
        be.download(y_host.data_ptr(), d_y, y_host.numel() * 4)      # synchronises

    e2e_steps = 0 if args.no_e2e else args.steps
    for _ in range(3 if e2e_steps else 0):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(torch.cuda.default_stream())
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(torch.cuda.default_stream())
    barrier()
    e2e_ms = e0.elapsed_time(e1) if e2e_steps else float("nan")
    assert args.no_e2e or torch.isfinite(y_host).all()
    be.release(d_x)
    be.release(d_y)
    be.close()

    def reduce_max(v):
        if world == 1:
            return v
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms, e2e_ms = reduce_max(ms), reduce_max(e2e_ms)
    extras = set() if args.no_extras else {e for e in args.extras.split(",") if e}
    sharded = None if "sharded" not in extras else sharded_extra(torch, dist, capi, gen, rank, world, barrier, reduce_max)

    if rank == 0:
        wbytes = layer_weight_bytes() * args.layers
        abytes = layer_algorithmic_bytes() * args.layers
        per_step_ms = ms / args.steps
        value = wbytes * world / (per_step_ms * 1e-3) / 1e9
        peak, peak_kind = measured_peaks()
        n_launch = launches_per_step
        achieved = abytes / (per_step_ms * 1e-3) / 1e9          # = (bytes per launch) / (avg launch duration)
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(per_step_ms, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "s8 quants x 23-bit fixed-point activations, f32 scales",
            "data": "synthetic",
            "config": workload_config(args.layers, world),
            "run": {"launch": "host launches" if args.no_graph else "CUDA graph replay of the step's launches",
                    "launches_per_layer": ("3: gemm(4096x4096), gemm_group(gate, up), gemm(4096x11008) - the engine's call pattern"
                                           if grouped else "4: one gemm per matrix")},
            "e2e": {"value": round(wbytes * world / (e2e_ms / args.steps * 1e-3) / 1e9, 2), "unit": UNIT,
                    "h2d_bytes_per_step": x_host.numel() * 4, "d2h_bytes_per_step": y_host.numel() * 4,
                    "ms_per_step": round(e2e_ms / args.steps, 5)},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "gemv_stream_kernel<Q4_K, 1 activation row>", "achieved": round(achieved, 2),
                         "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": round(achieved / peak, 4),
                         "launches_per_step": n_launch, "avg_launch_us": round(per_step_ms * 1e3 / n_launch, 3),
                         "algorithmic_bytes_per_launch": abytes // n_launch, "traffic": ((TRAFFIC_BYTES_PER_LAYER_GROUPED if grouped else TRAFFIC_BYTES_PER_LAYER) or 0) // (n_launch // args.layers) or None,
                         "frac_of_spec_8000_gbs": round(achieved / 8000.0, 4)},
            "clocks": clocks,
            "checked": checked,
        }
        if sharded is not None:
            line["sharded"] = sharded
            line["sharded_parity"] = sharded.get("sharded_parity")
        if world == 1 and extras & {"prefill", "decode"}:
            line["extra"] = {}
            if "prefill" in extras:
                line["extra"]["prefill"] = prefill_extra(torch, capi, gen)
            if "decode" in extras:
                line["extra"]["decode"] = decode_extra(torch, capi, gen, barrier)
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(sample_seconds=args.cpu_seconds, layers=args.layers)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def device_weights_q6k(torch, n_out: int, n_in: int, gen):
    """Q6_K blocks made on the device: ql/qh bytes uniform (6-bit q uniform), int8 sub-scales uniform in
    [-64, 63], d in [1e-4, 2e-3] as f16."""
    nblk = n_in // 256
    w = torch.randint(0, 256, (n_out, nblk, 210), dtype=torch.uint8, device="cuda", generator=gen)
    w[..., 192:208] = ((w[..., 192:208] & 127).to(torch.int16) - 64).to(torch.int8).view(torch.uint8)
    d = (1e-4 + 1.9e-3 * torch.rand((n_out, nblk), device="cuda", generator=gen)).to(torch.float16)
    w[..., 208:210] = d.view(torch.uint8).view(n_out, nblk, 2)
    return w.view(n_out, nblk * 210)


def timed(torch, fn, reps, barrier, variants=0, chain=False):
    """Device time per call of fn(i), events on the launching stream, after warm-up calls. With
    `variants` > 0 the calls fn(0..variants-1) are captured once each into CUDA graphs (kernels and, on
    several GPUs, the NCCL collective) and the graphs are replayed in turn: a decode loop replays a fixed
    launch sequence, and a latency-bound collective should not pay a host launch per token. With `chain` the
    calls are captured into ONE graph, back to back as a decode loop issues them, so that consecutive launches
    overlap their boundaries (programmatic dependent launch) as they do in the main measurement."""
    for i in range(max(3, variants)):
        fn(i)
    barrier()
    stream = torch.cuda.current_stream()
    run = fn
    if variants > 0:
        cap = torch.cuda.Stream()
        cap.wait_stream(stream)
        graphs = []
        with torch.cuda.stream(cap):
            if chain:
                g = torch.cuda.CUDAGraph()
                g.capture_begin()
                for v in range(variants):
                    fn(v)
                g.capture_end()
                graphs.append(g)
            else:
                for v in range(variants):
                    g = torch.cuda.CUDAGraph()
                    g.capture_begin()
                    fn(v)
                    g.capture_end()
                    graphs.append(g)
            for g in graphs:
                g.replay()
        barrier()
        stream = cap
        if chain:
            reps = max(1, reps // variants)

        def run(i):
            graphs[i % len(graphs)].replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for i in range(reps):
            run(i)
        e1.record(stream)
    barrier()
    return e0.elapsed_time(e1) / (reps * (variants if chain and variants > 0 else 1))


def sharded_extra(torch, dist, capi, gen, rank, world, barrier, reduce_max):
    """Configs 4 and 5 over `world` GPUs (world = 1 gives the unsharded numbers the others scale from).

    Head: Q6_K 128256 x 4096, rows split over the ranks, logits all-gathered. Weights of a rank are
    replicated R times in HBM and rotated so that a call never finds them in L2.
    MoE: 128 experts, top-8, hidden 4096, expert width 1536 (gate/up Q4_K, down Q6_K), experts split
    over the ranks, partial sums all-gathered and added in rank order; batch 1 and batch 8, sixteen
    different tokens rotated so that successive calls hit different experts."""
    from kraken_b200 import shard
    out = {"n_gpus": world}
    parity = {}
    # ---- head ----
    n_out, n_in = 128256, 4096
    begin, count = shard.row_range(n_out, world, rank, 8)
    slice_bytes = count * synth.row_bytes(synth.Q6_K, n_in)
    n_rep = max(2, int(4 * 126e6 / slice_bytes) + 1)
    ws = [device_weights_q6k(torch, count, n_in, gen) for _ in range(n_rep)]
    x = torch.randn((1, n_in), device="cuda", generator=torch.Generator(device="cuda").manual_seed(11))
    state = {"w": ws[0]}
    head = shard.ShardedHead(n_out, lambda v: capi.gemv(v, state["w"], synth.Q6_K, count, n_in), align=8)

    def head_call(i):
        state["w"] = ws[i % n_rep]
        return head.forward(x)

    def head_local(i):
        return capi.gemv(x, ws[i % n_rep], synth.Q6_K, count, n_in)
    ms_full = reduce_max(timed(torch, head_call, 60, barrier, variants=n_rep))
    ms_local = reduce_max(timed(torch, head_local, 60, barrier, variants=n_rep))
    ms_full_host = reduce_max(timed(torch, head_call, 60, barrier))
    ms_peer = ms_peer_host = ms_peer_chain = ms_c_nccl = ms_c_gather = None
    if world > 1 and count * world == n_out:
        # the same through the C ABI: GEMV into its slot of a persistent row + in-place ncclAllGather
        # (krk_cuda_shard_allgather), and the collective alone, so that the limiter is a number
        c_head = shard.NcclHead(n_out, n_in, synth.Q6_K, ws[0], align=8)

        def c_head_call(i):
            c_head.w_local = ws[i % n_rep]
            return c_head.forward(x)
        ms_c_nccl = reduce_max(timed(torch, c_head_call, 60, barrier, variants=n_rep))
        ms_c_gather = reduce_max(timed(torch, lambda i: c_head.gather_only(), 60, barrier, variants=1))
        c_head.w_local = state["w"] = ws[0]
        row_c = c_head.forward(x).clone()
        row_t = head.forward(x).clone()
        torch.cuda.synchronize()
        parity["head_c_nccl"] = bool(torch.equal(row_c, row_t))
        c_head.close()
    if world > 1:
        # the fused form: the GEMV's epilogue stores into every GPU's logits row and its last CTA waits
        # (bounded) for the peers' slices. An even number of captured steps keeps the two output buffers
        # alternating across replays.
        peer = shard.PeerHead(n_out, n_in, synth.Q6_K, ws[0], rows=1, align=8)

        def peer_call(i):
            peer.w_local = ws[i % n_rep]
            return peer.forward(x)
        ms_peer = reduce_max(timed(torch, peer_call, 60, barrier, variants=n_rep if n_rep % 2 == 0 else 2 * n_rep))
        ms_peer_host = reduce_max(timed(torch, peer_call, 60, barrier))
        # the same steps captured back to back into ONE graph: consecutive launches then overlap their boundaries
        # (programmatic dependent launch), which separate one-kernel graphs cannot do across graph launches
        nv = n_rep if n_rep % 2 == 0 else 2 * n_rep
        ms_peer_chain = reduce_max(timed(torch, peer_call, 6 * nv, barrier, variants=nv, chain=True))
        torch.cuda.synchronize()
        if capi.device_status() != 0:
            raise RuntimeError("a bounded wait of the fused all-gather gave up")
        # What was timed, checked: on every rank the fused kernel's gathered row and the NCCL form's row must be
        # the same bits, and this rank's slice of it must be what the unsharded kernel gives for these rows.
        state["w"] = peer.w_local = ws[0]
        row_nccl = head.forward(x).clone()
        row_peer = peer.forward(x).clone()
        own = capi.gemv(x, ws[0], synth.Q6_K, count, n_in)
        torch.cuda.synchronize()
        parity["head"] = bool(torch.equal(row_nccl, row_peer) and torch.equal(row_peer[:, begin:begin + count], own))
        peer.close()
    wbytes = n_out * synth.row_bytes(synth.Q6_K, n_in)
    out["head_q6_k_128256x4096"] = {
        "ms_per_token": round(ms_full, 5), "ms_gemv_only": round(ms_local, 5), "ms_per_token_host_launched": round(ms_full_host, 5),
        "launch": "CUDA graph replay (GEMV + NCCL all-gather)",
        "ms_per_token_c_abi_nccl_in_place": None if ms_c_nccl is None else round(ms_c_nccl, 5),
        "ms_nccl_all_gather_alone": None if ms_c_gather is None else round(ms_c_gather, 5),
        "ms_per_token_peer_store_fused": None if ms_peer is None else round(ms_peer, 5),
        "ms_per_token_peer_store_fused_host_launched": None if ms_peer_host is None else round(ms_peer_host, 5),
        "ms_per_token_peer_store_fused_one_graph": None if ms_peer_chain is None else round(ms_peer_chain, 5),
        "weight_gbps_peer_store_fused": None if ms_peer is None else round(n_out * synth.row_bytes(synth.Q6_K, n_in) / (ms_peer * 1e-3) / 1e9, 1),
        "weight_gbps_all_gpus": round(wbytes / (ms_full * 1e-3) / 1e9, 1),
        "weight_gbps_gemv_only": round(wbytes / (ms_local * 1e-3) / 1e9, 1),
        "rows_per_gpu": count, "gathered_bytes": n_out * 4, "replicas_rotated": n_rep}
    del ws
    # ---- MoE ----
    n_embd, n_ff, n_exp, k = 4096, 1536, 128, 8
    base, n_local = shard.expert_range(n_exp, world, rank)
    gate = device_weights(torch, n_local * n_ff, n_embd, gen)
    up = device_weights(torch, n_local * n_ff, n_embd, gen)
    down = device_weights_q6k(torch, n_local * n_embd, n_ff, gen)
    bank = capi.make_bank(gate, up, down, synth.Q4_K, synth.Q6_K, n_local, base, n_embd, n_ff)
    rgen = torch.Generator(device="cuda").manual_seed(12)          # the same tokens and logits on every rank
    toks = torch.randn((16, 8, n_embd), device="cuda", generator=rgen)
    logits = torch.randn((16, 8, n_exp), device="cuda", generator=rgen)
    route_fn, local_fn, combine_fn = shard.cuda_moe_fns(bank, k)
    routed_fn = shard.cuda_moe_routed_fn(bank, k)          # routing folded into the FFN's first kernel
    moe = shard.ShardedMoE(n_exp, route_fn, local_fn, combine_fn, routed_fn=routed_fn)
    peer_sum = shard.PeerSum(8 * n_embd) if world > 1 else None
    moe_peer = shard.ShardedMoE(n_exp, route_fn, local_fn, combine_fn, exchange=peer_sum, routed_fn=routed_fn) if world > 1 else None
    per_expert = 2 * n_ff * synth.row_bytes(synth.Q4_K, n_embd) + n_embd * synth.row_bytes(synth.Q6_K, n_ff)
    for batch in (1, 8):
        def moe_call(i):
            return moe.forward(toks[i % 16, :batch], logits[i % 16, :batch])
        ms = reduce_max(timed(torch, moe_call, 32, barrier, variants=16))
        ms_peer = None
        if moe_peer is not None:
            def moe_peer_call(i):
                return moe_peer.forward(toks[i % 16, :batch], logits[i % 16, :batch])
            ms_peer = reduce_max(timed(torch, moe_peer_call, 32, barrier, variants=16))
            torch.cuda.synchronize()
            if capi.device_status() != 0:
                raise RuntimeError("a bounded wait of the fused exchange gave up")
            # the two exchanges (NCCL all-gather + rank-ordered sum, fused peer-store kernel) must agree bit for bit
            y_nccl = moe.forward(toks[3, :batch], logits[3, :batch]).clone()
            y_peer = moe_peer.forward(toks[3, :batch], logits[3, :batch]).clone()
            torch.cuda.synchronize()
            parity[f"moe_batch{batch}"] = bool(torch.equal(y_nccl, y_peer) and torch.isfinite(y_peer).all())
        distinct = []
        for i in range(16):
            ids, _ = capi.route(logits[i, :batch], k)
            distinct.append(len(set(ids.cpu().reshape(-1).tolist())))
        mean_distinct = sum(distinct) / len(distinct)
        out[f"moe_qwen3_top8_batch{batch}"] = {
            "ms_per_step": round(ms, 5), "exchange": "NCCL all-gather + rank-ordered sum" if world > 1 else "none",
            "ms_per_step_peer_store_exchange": None if ms_peer is None else round(ms_peer, 5),
            "distinct_experts_mean": round(mean_distinct, 2),
            "expert_weight_gbps_all_gpus": round(mean_distinct * per_expert / (ms * 1e-3) / 1e9, 1),
            "experts_per_gpu": n_local}
    if peer_sum is not None:
        peer_sum.close()
    if world > 1:
        # every rank must have seen every check pass; a failed check fails the run
        ok = torch.tensor([1.0 if parity and all(parity.values()) else 0.0], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) != 1.0:
            raise RuntimeError(f"sharded results differ between the fused and the NCCL forms on rank {rank}: {parity}")
        out["sharded_parity"] = "ok"
        out["sharded_parity_checks"] = sorted(parity)
    else:
        out["sharded_parity"] = "single GPU: nothing to compare"
    return out


def device_weights_q8_0(torch, n_out: int, n_in: int, gen):
    """Q8_0 blocks made on the device: int8 quants uniform in [-127, 127], d in [1e-3, 2e-2] as f16."""
    nblk = n_in // 32
    w = torch.empty((n_out, nblk, 34), dtype=torch.uint8, device="cuda")
    q = torch.randint(-127, 128, (n_out, nblk, 32), dtype=torch.int8, device="cuda", generator=gen)
    w[..., 2:34] = q.view(torch.uint8)
    d = (1e-3 + 1.9e-2 * torch.rand((n_out, nblk), device="cuda", generator=gen)).to(torch.float16)
    w[..., 0:2] = d.view(torch.uint8).view(n_out, nblk, 2)
    return w.view(n_out, nblk * 34)


def device_weights_q4_0(torch, n_out: int, n_in: int, gen):
    """Q4_0 blocks made on the device: nibbles uniform, d in [1e-3, 2e-2] as f16."""
    nblk = n_in // 32
    w = torch.randint(0, 256, (n_out, nblk, 18), dtype=torch.uint8, device="cuda", generator=gen)
    d = (1e-3 + 1.9e-2 * torch.rand((n_out, nblk), device="cuda", generator=gen)).to(torch.float16)
    w[..., 0:2] = d.view(torch.uint8).view(n_out, nblk, 2)
    return w.view(n_out, nblk * 18)


def device_weights_q5_0(torch, n_out: int, n_in: int, gen):
    """Q5_0 blocks made on the device: nibbles and fifth bits uniform, d in [1e-3, 2e-2] as f16."""
    nblk = n_in // 32
    w = torch.randint(0, 256, (n_out, nblk, 22), dtype=torch.uint8, device="cuda", generator=gen)
    d = (1e-3 + 1.9e-2 * torch.rand((n_out, nblk), device="cuda", generator=gen)).to(torch.float16)
    w[..., 0:2] = d.view(torch.uint8).view(n_out, nblk, 2)
    return w.view(n_out, nblk * 22)


def device_weights_q5_1(torch, n_out: int, n_in: int, gen):
    """Q5_1 blocks made on the device: nibbles and fifth bits uniform, d in [1e-3, 2e-2], m in [-0.1, 0.1] as f16."""
    nblk = n_in // 32
    w = torch.randint(0, 256, (n_out, nblk, 24), dtype=torch.uint8, device="cuda", generator=gen)
    d = (1e-3 + 1.9e-2 * torch.rand((n_out, nblk), device="cuda", generator=gen)).to(torch.float16)
    m = (0.2 * torch.rand((n_out, nblk), device="cuda", generator=gen) - 0.1).to(torch.float16)
    w[..., 0:2] = d.view(torch.uint8).view(n_out, nblk, 2)
    w[..., 2:4] = m.view(torch.uint8).view(n_out, nblk, 2)
    return w.view(n_out, nblk * 24)


def device_weights_q2_k(torch, n_out: int, n_in: int, gen):
    """Q2_K blocks made on the device: 16 scale/min bytes and 64 quant bytes uniform, d and dmin in [1e-3, 1e-2] as
    f16 at the end of the 84-byte block."""
    nblk = n_in // 256
    w = torch.randint(0, 256, (n_out, nblk, 84), dtype=torch.uint8, device="cuda", generator=gen)
    d = (1e-3 + 9e-3 * torch.rand((n_out, nblk, 2), device="cuda", generator=gen)).to(torch.float16)
    w[..., 80:84] = d.view(torch.uint8).view(n_out, nblk, 4)
    return w.view(n_out, nblk * 84)


def device_weights_q3_k(torch, n_out: int, n_in: int, gen):
    """Q3_K blocks made on the device: mask, quant and packed scale bytes uniform, d in [1e-3, 1e-2] as f16 at the
    end of the 110-byte block."""
    nblk = n_in // 256
    w = torch.randint(0, 256, (n_out, nblk, 110), dtype=torch.uint8, device="cuda", generator=gen)
    d = (1e-3 + 9e-3 * torch.rand((n_out, nblk), device="cuda", generator=gen)).to(torch.float16)
    w[..., 108:110] = d.view(torch.uint8).view(n_out, nblk, 2)
    return w.view(n_out, nblk * 110)


def device_weights_q5_k(torch, n_out: int, n_in: int, gen):
    """Q5_K blocks made on the device: payload bytes uniform (5-bit quants and packed 6-bit scale/min uniform),
    d in [5e-4, 5e-3], dmin in [0, 5e-3] as f16."""
    nblk = n_in // 256
    w = torch.randint(0, 256, (n_out, nblk, 176), dtype=torch.uint8, device="cuda", generator=gen)
    d = (5e-4 + 4.5e-3 * torch.rand((n_out, nblk), device="cuda", generator=gen)).to(torch.float16)
    dm = (5e-3 * torch.rand((n_out, nblk), device="cuda", generator=gen)).to(torch.float16)
    w[..., 0:2] = d.view(torch.uint8).view(n_out, nblk, 2)
    w[..., 2:4] = dm.view(torch.uint8).view(n_out, nblk, 2)
    return w.view(n_out, nblk * 176)


def decode_extra(torch, capi, gen, barrier):
    """The decode GEMV on the other shapes the spec names, batch 1, weights rotated through replicas that
    together exceed 4x the L2, each replay a CUDA graph: config 1 (Q8_0 4096 x 4096) and one large matrix
    per format, where the per-launch fixed cost no longer matters and the number is the kernel's
    steady-state bandwidth."""
    peak, _ = measured_peaks()
    cases = [("config1_q8_0_4096x4096", synth.Q8_0, 4096, 4096, device_weights_q8_0),
             ("steady_q8_0_65536x4096", synth.Q8_0, 65536, 4096, device_weights_q8_0),
             ("steady_q4_k_131072x4096", synth.Q4_K, 131072, 4096, device_weights),
             ("steady_q6_k_128256x4096", synth.Q6_K, 128256, 4096, device_weights_q6k),
             ("steady_q4_0_131072x4096", synth.Q4_0, 131072, 4096, device_weights_q4_0),
             ("steady_q5_k_65536x4096", synth.Q5_K, 65536, 4096, device_weights_q5_k),
             ("steady_q5_0_65536x4096", synth.Q5_0, 65536, 4096, device_weights_q5_0),
             ("steady_q5_1_65536x4096", synth.Q5_1, 65536, 4096, device_weights_q5_1),
             # (IQ4_NL blocks have the layout of Q4_0 blocks)
             ("steady_iq4_nl_131072x4096", synth.IQ4_NL, 131072, 4096, device_weights_q4_0),
             ("steady_q2_k_131072x4096", synth.Q2_K, 131072, 4096, device_weights_q2_k),
             ("steady_q3_k_131072x4096", synth.Q3_K, 131072, 4096, device_weights_q3_k),
             # K not a multiple of 256: the warp-per-row kernel, so that its gap is on record
             ("warp_per_row_q8_0_65536x4064", synth.Q8_0, 65536, 4064, device_weights_q8_0)]
    out = {}
    for name, wt, n_out, n_in, make in cases:
        wbytes = n_out * synth.row_bytes(wt, n_in)
        n_rep = max(2, int(4 * 126e6 / wbytes) + 1)
        ws = [make(torch, n_out, n_in, gen) for _ in range(n_rep)]
        x = torch.randn((1, n_in), device="cuda", generator=gen)
        y = torch.empty((1, n_out), device="cuda")

        def call(i):
            capi.gemv(x, ws[i % n_rep], wt, n_out, n_in, out=y)
        ms = timed(torch, call, 20 * n_rep, barrier, variants=n_rep, chain=True)
        abytes = wbytes + 4 * n_in + 4 * n_out
        out[name] = {"us_per_launch": round(ms * 1e3, 3), "algorithmic_gbps": round(abytes / (ms * 1e-3) / 1e9, 1),
                     "frac_of_measured_hbm": round(abytes / (ms * 1e-3) / 1e9 / peak, 4),
                     "frac_of_spec_8000_gbs": round(abytes / (ms * 1e-3) / 1e9 / 8000.0, 4), "replicas_rotated": n_rep}
        if name.startswith("config1"):
            # the same launch over ONE replica: the weights stay in the 126 MB L2 (not an HBM number)
            def warm(i):
                capi.gemv(x, ws[0], wt, n_out, n_in, out=y)
            ms_warm = timed(torch, warm, 200, barrier, variants=1)
            out[name]["us_per_launch_l2_resident"] = round(ms_warm * 1e3, 3)
        del ws
    # the steps either side of the head, on the device: top-k of config 4's logits row and an embedding gather
    n_vocab = 128256
    logits = torch.randn(n_vocab, device="cuda", generator=gen) * 3.0
    for k in (1, 40):
        ws_k = torch.empty(capi.lib.krk_cuda_logits_topk_workspace_bytes(n_vocab, k), dtype=torch.uint8, device="cuda")

        def topk_call(i):
            capi.logits_topk(logits, k, workspace=ws_k)
        ms = timed(torch, topk_call, 100, barrier, variants=1)
        out[f"logits_topk_128256_k{k}"] = {"us_per_call": round(ms * 1e3, 3), "kernels": 2,
                                            "replaces": "513,024-byte logits download + host ranking per token"}
    table = device_weights_q6k(torch, 32768, 4096, gen)
    toks = torch.randint(0, 32768, (8,), dtype=torch.int32, device="cuda", generator=gen)

    def embed_call(i):
        capi.embed(table, synth.Q6_K, 32768, 4096, toks)
    ms = timed(torch, embed_call, 100, barrier, variants=1)
    out["embed_q6_k_8_tokens_x4096"] = {"us_per_call": round(ms * 1e3, 3)}
    return out


def prefill_extra(torch, capi, gen):
    """Config 3: Q4_K prefill GEMM, N=14336, K=4096, M in {128, 512, 2048}: f16 X, f32 Y, tensor cores.
    Four weight replicas (132 MB) are rotated so that no launch finds its weights in L2."""
    n_out, n_in = 14336, 4096
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    peak = float(peaks.get("bf16_tflops", 1590.0))
    ws = [device_weights(torch, n_out, n_in, gen) for _ in range(4)]
    out = []
    for rows in (128, 512, 2048):
        x = torch.randn((rows, n_in), device="cuda", generator=gen).to(torch.float16)
        y = torch.empty((rows, n_out), device="cuda")
        scratch = torch.empty(max(capi.gemm_workspace_bytes(capi.X_F16, n_out, n_in, rows), 256), dtype=torch.uint8, device="cuda")
        for i in range(4):
            capi.gemm(x, ws[i], WT, n_out, n_in, out=y, workspace=scratch)
        torch.cuda.synchronize()
        reps = 20
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            capi.gemm(x, ws[i % 4], WT, n_out, n_in, out=y, workspace=scratch)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        tf = 2.0 * rows * n_out * n_in / (ms * 1e-3) / 1e12
        # the same launches timed one by one: the measured peak is the best of ten cuBLAS launches, so the best single
        # launch is the like-for-like figure; the fractions above stay on the average of the back-to-back loop
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        for i, (a, b) in enumerate(evs):
            a.record()
            capi.gemm(x, ws[i % 4], WT, n_out, n_in, out=y, workspace=scratch)
            b.record()
        torch.cuda.synchronize()
        each = sorted(a.elapsed_time(b) for a, b in evs)
        tf_best = 2.0 * rows * n_out * n_in / (each[0] * 1e-3) / 1e12
        out.append({"M": rows, "ms": round(ms, 4), "tflops": round(tf, 1), "frac_of_measured_bf16_peak": round(tf / peak, 4),
                    "frac_of_spec_2250_tflops": round(tf / 2250.0, 4), "ms_best_single_launch": round(each[0], 4),
                    "ms_median_single_launch": round(each[reps // 2], 4), "tflops_best_single_launch": round(tf_best, 1)})
    # the same GEMM at M = 512 for the other formats
    other = {}
    del ws
    for name, wt, make in (("q6_k", synth.Q6_K, device_weights_q6k), ("q8_0", synth.Q8_0, device_weights_q8_0),
                           ("q4_0", synth.Q4_0, device_weights_q4_0), ("q5_k", synth.Q5_K, device_weights_q5_k),
                           ("q5_0", synth.Q5_0, device_weights_q5_0)):
        wf = [make(torch, n_out, n_in, gen) for _ in range(3)]
        rows = 512
        x = torch.randn((rows, n_in), device="cuda", generator=gen).to(torch.float16)
        y = torch.empty((rows, n_out), device="cuda")
        scratch = torch.empty(max(capi.gemm_workspace_bytes(capi.X_F16, n_out, n_in, rows), 256), dtype=torch.uint8, device="cuda")
        for i in range(3):
            capi.gemm(x, wf[i], wt, n_out, n_in, out=y, workspace=scratch)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(9):
            capi.gemm(x, wf[i % 3], wt, n_out, n_in, out=y, workspace=scratch)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 9
        tf = 2.0 * rows * n_out * n_in / (ms * 1e-3) / 1e12
        other[name] = {"M": rows, "ms": round(ms, 4), "tflops": round(tf, 1), "frac_of_measured_bf16_peak": round(tf / peak, 4)}
        del wf
    return {"workload": "q4_k_prefill_gemm_N14336_K4096", "kernel": "gemm_tc_kernel<Q4_K> (tcgen05)", "peak_tflops": peak,
            "results": out, "other_formats_M512": other}


# ncu dram__bytes_read.sum + dram__bytes_write.sum of the streaming kernel over the launches of one layer (a one-layer
# run of this file under ncu); the bench line divides it by the launches per layer. Re-measure when the kernel changes.
TRAFFIC_BYTES_PER_LAYER = None                # four launches: not captured for the current kernel
TRAFFIC_BYTES_PER_LAYER_GROUPED = 91480064    # three launches, read + write: 11,609,344 + 53,361,664 (gate and up) + 26,509,056


# ---- CPU arms ---------------------------------------------------------------------------------------

def cpu_engine(threads: int):
    """Kraken's CPU backend: the compiled reference when oracle/_ref travelled with the tree,
    else the in-repo restatement of its scalar path."""
    from oracle.krk_oracle import Oracle, Reference
    if Reference.available():
        try:
            return Reference(threads=threads)
        except OSError:
            pass
    return Oracle()


def cpu_layer(seed_off: int = 0):
    seed = synth.BASE_SEED + 2
    mats = []
    for i, (n_out, n_in) in enumerate(LAYER_SHAPES):
        w = synth.weights(WT, n_out, n_in, seed, stream=100 + i + 10 * seed_off)
        x = synth.activations(1, n_in, seed, stream=200 + i)
        mats.append((w, x, n_out, n_in))
    return mats


def cpu_step_fn(eng, layers: int, threads: int):
    """one_step(tier): one token's pass over `layers` layers on the CPU engine. Eight copies of the seeded layer
    (rows rotated, as on the GPU) are cycled so that a step streams its weights from memory rather than from the
    last-level cache."""
    base = cpu_layer()
    copies = []
    for c in range(8):
        copies.append([(w if c == 0 else np.ascontiguousarray(np.roll(w, -layer_shift(c, n_out), axis=0)), x, n_out, n_in)
                       for w, x, n_out, n_in in base])

    def one_step(tier):
        for li in range(layers):
            for w, x, n_out, n_in in copies[li % len(copies)]:
                if eng.kind == "reference":
                    eng.gemm(x, w, WT, n_out, n_in, rows=1, tier=tier)
                else:
                    eng.gemm(x, w, WT, n_out, n_in, rows=1, threads=threads)
    return one_step


def time_cpu_steps(one_step, tier: int, layers: int, budget_s: float, warm_s: float = 1.0):
    """GB/s of whole steps for about budget_s seconds after warm_s seconds of warm-up."""
    t_w = time.perf_counter()
    one_step(tier)
    while time.perf_counter() - t_w < warm_s:
        one_step(tier)
    t0 = time.perf_counter()
    n = 0
    while True:
        one_step(tier)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s or n >= 2000:
            break
    return layer_weight_bytes() * layers * n / dt / 1e9, n, dt


def cpu_baseline(sample_seconds: float = 10.0, layers: int = N_LAYERS):
    threads = os.cpu_count() or 1
    eng = cpu_engine(threads)
    one_step = cpu_step_fn(eng, layers, threads)
    out = {"unit": UNIT, "cores": threads, "kind": eng.kind}
    what = f"steps of {layers} layers x 4 matmuls ({layer_weight_bytes() * layers} weight bytes per step, 8 rotated copies of the seeded layer cycled)"
    if eng.kind == "reference":
        v1, n1, t1 = time_cpu_steps(one_step, 1, layers, sample_seconds * 0.5)
        v0, n0, t0 = time_cpu_steps(one_step, 0, layers, sample_seconds * 0.5, warm_s=0.0)
        out.update(value=round(v1, 3), tier="reference default (int8-activation AVX2 tier, lossy)",
                   exact_scalar_value=round(v0, 3),
                   sample=f"{n1} {what} on the default tier in {t1:.1f}s after 1s of warm-up, {n0} on the exact scalar tier "
                          f"in {t0:.1f}s, KRK_THREADS={threads}")
    else:
        v0, n0, t0 = time_cpu_steps(one_step, 0, layers, sample_seconds)
        out.update(value=round(v0, 3), tier="exact scalar f32 chain (restatement)",
                   sample=f"{n0} {what} in {t0:.1f}s, {threads} threads")
    return out


def run_reference(args):
    """The reference's own CPU implementation of the path on this box's host cores, same workload and config as
    the GPU arm: a step is one token's pass over all the layers' four matmuls. Eight copies of the seeded layer
    (rows rotated, as on the GPU) are cycled so that a step streams its weights from memory rather than from
    the last-level cache. The run is warmed up for at least a second before it is timed."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    eng = cpu_engine(threads)
    one_step = cpu_step_fn(eng, args.layers, threads)
    tier = 1 if eng.kind == "reference" else 0

    def timed_steps(t, steps, warm_s):
        t_w = time.perf_counter()
        n_w = 0
        while n_w < max(args.warmup, 1) or time.perf_counter() - t_w < warm_s:
            one_step(t)
            n_w += 1
        t0 = time.perf_counter()
        for _ in range(steps):
            one_step(t)
        return time.perf_counter() - t0, n_w

    dt, n_warm = timed_steps(tier, args.steps, 1.0)
    value = layer_weight_bytes() * args.layers * args.steps / dt / 1e9
    exact = None
    if eng.kind == "reference":     # the exact scalar tier beside it, on fewer steps (it is several times slower)
        es = max(1, args.steps // 10)
        dte, _ = timed_steps(0, es, 0.0)
        exact = layer_weight_bytes() * args.layers * es / dte / 1e9
    sample = (f"{args.steps} steps of {args.layers} layers x 4 matmuls ({layer_weight_bytes() * args.layers} weight bytes per step) "
              f"in {dt:.2f}s after {n_warm} warm-up steps, 8 rotated copies of the seeded layer cycled, "
              f"{'KRK_THREADS' if eng.kind == 'reference' else 'threads'}={threads}")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": n_warm,
        "ms_per_step": round(dt / args.steps * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (int8-activation tier)" if tier == 1 else "f32", "data": "synthetic",
        "config": workload_config(args.layers, world),
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": threads, "kind": eng.kind, "sample": sample,
                         "tier": "reference default (int8-activation AVX2 tier, lossy)" if tier == 1 else "exact scalar",
                         "exact_scalar_value": None if exact is None else round(exact, 3)},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_issue_rates():
    """Cycles per instruction and sub-partition for the instruction kinds the decode GEMV could be built from."""
    from kraken_b200 import capi
    rows = []
    for kind, name in enumerate(capi.PROBE_KINDS):
        thr = [round(capi.probe_issue(kind, w, 2048), 2) for w in (4, 8, 16)]
        lat = round(capi.probe_issue(kind, 1, 2048, chained=True), 1)
        rows.append({"instruction": name, "cycles_per_instr_per_smsp_at_1_2_4_warps": thr, "dependent_issue_latency": lat})
        print(f"{name:28s} {thr}  latency {lat}", file=sys.stderr)
    print(json.dumps({"issue_rates": rows}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-check", action="store_true", help="skip the check of the step against the CPU checker (profiling runs)")
    ap.add_argument("--issue-rates", action="store_true", help="print the instruction issue-rate table and exit")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-extras", action="store_true", help="skip every side measurement")
    ap.add_argument("--extras", default="prefill,decode,sharded",
                    help="side measurements to run: any of prefill,decode,sharded (profiling runs pick one)")
    ap.add_argument("--ungrouped", action="store_true", help="launch gate and up apart (four launches per layer instead of three)")
    ap.add_argument("--no-graph", action="store_true", help="launch from the host instead of replaying a CUDA graph")
    ap.add_argument("--layers", type=int, default=N_LAYERS,
                    help="layers per step; fewer than 32 is for profiler captures only, not a bench value")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    args = ap.parse_args()
    if args.issue_rates:
        run_issue_rates()
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
