"""Benchmark of the tensor-parallel row-parallel hot path (fused projection + reduction) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Workload of the bench line (BASELINE config 2, the Qwen3-style decoder layer): hidden 2560, o_proj K = 4096, down_proj
K = 9728, one 256-token block, BF16, TP = N. One STEP is the row-parallel hot path of a 36-layer round: for each layer the
two fused kernels `o_proj -> reduce + residual + RMSNorm` and `down_proj -> reduce + residual + RMSNorm`
(dlmrt/models/sdar/model.py:237-243), 72 launches, each layer with its own weights (2.56 GB at TP = 1, far above the
126 MB L2, so weights stream from HBM every step). Steps are captured once in a CUDA graph and replayed, as the
reference measures a round (dlmrt/entrypoints/bench/common.py:68-80).

  value      microseconds per decoder layer (o_proj + down_proj with their reductions) = total time of the K timed
             replays / K / 36, inputs resident in HBM; `replay_us` gives the median and spread of the single replays
  e2e        the same through host buffers: pinned-host -> device copy of the step's activations, the graph replay, and
             the device -> host copy of the last reduced block, all inside the timed region
  roofline   dominant kernel rowpar_kernel: algorithmic bytes = the weight shard N * K/w * 2 per launch (HBM) or, when
             larger in time, the reduction's per-GPU NVLink ingress 2 * (w-1)/w * M * N * 2, over the average launch
             duration (the chain is serial, so that is step time / launches). The NVLink peak is measured in the same
             run (a 256 MB copy out of a peer's memory, all ranks at once, CUDA events)
  parity     (N > 1) values checked on the real interconnect, outside the timed regions: identical bits on every rank,
             the CPU oracle, and the reference's own reduction kernel on the same partials; a mismatch exits non-zero
  moe        the NVFP4 expert path of BASELINE configs 4 (uniform and Zipf(1.2) routing) and 5, timed the same way:
             `value` the down-projection + combine + reduction launch, `whole_call` the three launches of a whole routed
             expert call (bookkeeping + input quantisation, GEMM1 + activation + re-quantisation, then that launch)
  round      a whole synthetic denoise round of the config-3 shape (36 layers: qkv / gate_up on cuBLAS, attention, the
             two fused projections, LM head + row statistics all-gather), median of the replays
  cpu_baseline / --impl reference   the CPU restatement of the same path (torch CPU matmul per K shard, rank-order FP32
             sum, residual, RMSNorm) on the host cores. The reference has no CPU implementation of this path, so this
             port is what is timed (kind "port").

Synthetic data: weights ~ N(0, 0.02), activations ~ N(0, 1), seeded; no dataset or checkpoint is read.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HIDDEN, K_O, K_DOWN, ROWS, LAYERS, EPS = 2560, 4096, 9728, 256, 36, 1e-6
NVLINK_NOMINAL_GBS = 900.0  # per direction per GPU: the figure BASELINE's roofline formula is written with
FALLBACK_HBM_GBS = 6650.0
METRIC = "fused row-parallel projection+reduction latency per decoder layer (o_proj + down_proj), denoise round"


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class Clocks:
    """Samples nvidia-smi during a timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        self.file.seek(0)
        rows = [[c.strip() for c in line.split(",")] for line in self.file.read().splitlines() if line.count(",") >= 5]
        self.file.close()
        os.unlink(self.file.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = sorted(int(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in rows)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def weight_bytes(world):
    return HIDDEN * (K_O // world) * 2, HIDDEN * (K_DOWN // world) * 2


def reduction_bytes(world, rows=None, hidden=None):
    rows, hidden = rows or ROWS, hidden or HIDDEN
    return 2 * (world - 1) * rows * hidden * 2 // world


# ---------------------------------------------------------------------------------------------------------------------
# CPU restatement (the reference arm and the cpu_baseline leg)
# ---------------------------------------------------------------------------------------------------------------------
def cpu_layer_seconds(world, repeats):
    """One decoder layer's hot path on the host: per K shard a BF16 torch.mm (dlmrt/layers/linear.py:47-48 on CPU
    tensors), the rank-ordered FP32 sum, BF16 rounding, residual add and RMSNorm (oracle.reduce order of operations),
    for o_proj and down_proj. Returns the median seconds per layer over `repeats`."""
    import torch

    # All the host's cores, also under torchrun (which starts every rank with OMP_NUM_THREADS=1).
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    if torch.get_num_threads() < cores:
        torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    h = torch.randn(ROWS, HIDDEN, generator=g).to(torch.bfloat16)
    norm = (torch.randn(HIDDEN, generator=g) * 0.1 + 1).to(torch.bfloat16)
    ops = []
    for k in (K_O, K_DOWN):
        x = torch.randn(ROWS, k, generator=g).to(torch.bfloat16)
        w = (torch.randn(HIDDEN, k, generator=g) * 0.02).to(torch.bfloat16)
        ops.append(([s.contiguous() for s in x.chunk(world, 1)], [s.contiguous() for s in w.chunk(world, 1)]))

    def layer(h):
        for xs, ws in ops:
            acc = torch.zeros(ROWS, HIDDEN)
            for x, w in zip(xs, ws):  # rank order
                acc = acc + torch.mm(x, w.t()).float()
            v = acc.to(torch.bfloat16).float() + h.float()
            h = v.to(torch.bfloat16)
            out = (v * torch.rsqrt((v * v).mean(-1, keepdim=True) + EPS) * norm.float()).to(torch.bfloat16)
        return h, out

    layer(h)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        layer(h)
        times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2], torch.get_num_threads()


def run_reference(args, rank):
    if rank != 0:
        return
    world = args.gpus
    for _ in range(max(args.warmup, 1) - 1):
        cpu_layer_seconds(world, 1)
    sec, cores = cpu_layer_seconds(world, max(args.steps, 3))
    us = sec * 1e6
    sample = f"one decoder layer (o_proj + down_proj, {ROWS} rows) per step on the host, median of {max(args.steps, 3)}"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(us, 1), "unit": "us", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3 * LAYERS, 3),
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config(world),
        "cpu_baseline": {"value": round(us, 1), "unit": "us", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(us, 1), "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def config(world, workload="c2"):
    if workload in ("k1", "k3"):
        what = "plain sums (K1)" if workload == "k1" else "reduce+residual+RMSNorm (K3)"
        return {"workload": f"reduction of given BF16 partials [{ROWS}, {HIDDEN}], {what}, TP={world}; a step = {LAYERS} x 2 "
                            "reductions on alternating call sites", "tp": world, "rows": ROWS, "hidden": HIDDEN,
                "layers": LAYERS, "l2": "L2 flushed by a 256 MB write between steps"}
    return {"workload": f"BASELINE config 2: Qwen3-style layer, hidden {HIDDEN}, o_proj K {K_O}, down_proj K {K_DOWN}, "
                        f"{ROWS}-token block, BF16, TP={world}; a step = {LAYERS} layers x 2 fused "
                        "projection+reduce+residual+RMSNorm launches with per-layer weights",
            "tp": world, "rows": ROWS, "hidden": HIDDEN, "layers": LAYERS,
            "l2": f"weights of a step ({sum(weight_bytes(world)) * LAYERS / 1e6:.0f} MB per GPU) exceed the 126 MB L2"
                  if sum(weight_bytes(world)) * LAYERS > 130e6 else "L2 flushed by a 256 MB write between steps"}


# ---------------------------------------------------------------------------------------------------------------------
# Shared GPU plumbing
# ---------------------------------------------------------------------------------------------------------------------
class Rig:
    """One rank's group, stream and timing helpers."""

    def __init__(self, world):
        import torch

        from dlmrt_b200 import _lib
        from dlmrt_b200.distributed import parallel

        self.torch, self.world = torch, world
        if world > 1:
            import torch.distributed as dist

            self.dist = dist
            self.group = parallel.init()
            self.device = self.group.device
        else:
            self.dist = None
            self.device = torch.device("cuda", 0)
            torch.cuda.set_device(self.device)
            self.group = parallel.Group.local(self.device)
        self.rank = self.group.rank
        self.lib = _lib.lib()
        if self.lib.dlm_device_arch() != 100:
            raise RuntimeError("bench.py needs an sm_100 GPU: there is no fallback path")
        self.stream = torch.cuda.Stream(self.device)

    def barrier(self):
        self.torch.cuda.synchronize(self.device)
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize(self.device)

    def max_over_ranks(self, value):
        t = self.torch.tensor([float(value)], device=self.device)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, steps, before=None):
        """`steps` calls of fn on the rig's stream, bracketed by barriers: (total ms, [ms of each call]), CUDA events on
        the launching stream, each the max over ranks. `before` runs ahead of every call outside the per-call events
        (an L2 flush) but inside the total."""
        torch = self.torch
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(2 * steps)]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        with torch.cuda.stream(self.stream):
            start.record(self.stream)
            for i in range(steps):
                if before is not None:
                    before()
                marks[2 * i].record(self.stream)
                fn()
                marks[2 * i + 1].record(self.stream)
            stop.record(self.stream)
        self.barrier()
        total = self.max_over_ranks(start.elapsed_time(stop))
        each = [self.max_over_ranks(marks[2 * i].elapsed_time(marks[2 * i + 1])) for i in range(steps)]
        return total, each

    def capture(self, step, eager=2):
        """Two eager passes (they allocate every symmetric buffer, in the same order on every rank), then one capture.
        Returns (graph, what step() returned during capture, launches of this library per replay)."""
        torch = self.torch
        with torch.cuda.stream(self.stream):
            for _ in range(eager):
                out = step()
            self.stream.synchronize()
            self.group.check()
            before = self.lib.dlm_launch_count()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.stream):
                out = step()
            launches = self.lib.dlm_launch_count() - before
        return graph, out, launches


def spread(each_ms, per):
    """Median, minimum and maximum of single replays, in microseconds per `per` units."""
    us = sorted(v * 1e3 / per for v in each_ms)
    return {"median": round(statistics.median(us), 2), "min": round(us[0], 2), "max": round(us[-1], 2), "replays": len(us)}


def nvlink_peak(rig, nbytes=256 << 20, reps=5):
    """Per-direction bandwidth of this run's interconnect: every rank copies `nbytes` out of its right neighbour's
    memory into its own at the same time (each GPU sends and receives one stream), CUDA events, best of `reps`, the
    slowest rank's figure. Returns GB/s, or None on one GPU."""
    if rig.world == 1:
        return None
    torch, g = rig.torch, rig.group
    buf = g.symmetric("bench.peer", (nbytes,), torch.uint8)
    handle = g._handles["bench.peer"].torch_handle
    if handle is None:
        return None
    peer = handle.get_buffer((g.rank + 1) % g.world, (nbytes,), torch.uint8)
    local = torch.empty(nbytes, dtype=torch.uint8, device=rig.device)
    best = float("inf")
    for _ in range(reps + 1):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        rig.barrier()
        with torch.cuda.stream(rig.stream):
            a.record(rig.stream)
            local.copy_(peer)
            b.record(rig.stream)
        rig.barrier()
        best = min(best, rig.max_over_ranks(a.elapsed_time(b)))
    del buf
    return nbytes / (best * 1e-3) / 1e9


def roofline(kernel, hbm_bytes, link_bytes, launch_s, link_gbs, extra=None):
    """The slower of (weight bytes / measured HBM copy peak) and (reduction ingress / measured peer-copy peak) bounds
    the launch; achieved = that bound's algorithmic bytes / the launch's duration."""
    hbm, which = peaks()
    t_hbm = hbm_bytes / (hbm * 1e9)
    t_link = link_bytes / (link_gbs * 1e9) if link_gbs else 0.0
    if t_hbm >= t_link:
        roof = {"bound": "hbm", "achieved": round(hbm_bytes / launch_s / 1e9, 1), "peak": hbm, "unit": "GB/s",
                "peak_source": f"of {which} (MEASURED_PEAKS.json copy bandwidth)" if which == "measured" else "of fallback",
                "algorithmic_bytes_per_launch": int(hbm_bytes)}
    else:
        roof = {"bound": "nvlink", "achieved": round(link_bytes / launch_s / 1e9, 1), "peak": round(link_gbs, 1),
                "unit": "GB/s", "peak_source": "of measured (peer copy of 256 MB per direction, this run)",
                "algorithmic_bytes_per_launch": int(link_bytes),
                "frac_of_nominal_900": round(link_bytes / launch_s / 1e9 / NVLINK_NOMINAL_GBS, 4)}
    roof["frac"] = round(roof["achieved"] / roof["peak"], 4)
    roof["kernel"] = kernel
    roof["avg_launch_us"] = round(launch_s * 1e6, 2)
    roof["avg_launch_how"] = "step time / launches per step (the launches of a step run back to back on one stream)"
    roof["roofline_us"] = round(max(t_hbm, t_link) * 1e6, 2)
    if extra:
        roof.update(extra)
    return roof


# ---------------------------------------------------------------------------------------------------------------------
# The bench line: BASELINE config 2 (and the reduction-only workloads k1 / k3)
# ---------------------------------------------------------------------------------------------------------------------
def run_dense(args, rig, link_gbs):
    torch, group, device, world, rank = rig.torch, rig.group, rig.device, rig.world, rig.rank
    from dlmrt_b200.layers.linear import Linear

    g = torch.Generator().manual_seed(1 + rank)
    ko, kd = K_O // world, K_DOWN // world
    only_reduce = args.workload in ("k1", "k3")  # the reduction of GIVEN partials alone (dlm_reduce_bf16), no GEMM
    plain_sum = args.workload == "k1"           # K1 (no residual, no norm) on a 32-row block: LLaDA2's call pattern
    weights = 0 if only_reduce else LAYERS
    lin_o = [Linear((torch.randn(HIDDEN, ko, generator=g) * 0.02).to(torch.bfloat16).to(device), group=group)
             for _ in range(weights)]
    lin_d = [Linear((torch.randn(HIDDEN, kd, generator=g) * 0.02).to(torch.bfloat16).to(device), group=group)
             for _ in range(weights)]
    gs = torch.Generator().manual_seed(7)  # identical on every rank
    norms = [(torch.randn(HIDDEN, generator=gs) * 0.1 + 1).to(torch.bfloat16).to(device) for _ in range(2 * LAYERS)]
    h0 = torch.randn(ROWS, HIDDEN, generator=gs).to(torch.bfloat16)
    h = h0.to(device)
    host_xo = torch.randn(ROWS, ko, generator=g).to(torch.bfloat16).pin_memory()
    host_xd = torch.randn(ROWS, kd, generator=g).to(torch.bfloat16).pin_memory()
    x_o, x_d = host_xo.to(device), host_xd.to(device)
    host_out = torch.empty(ROWS, HIDDEN, dtype=torch.bfloat16).pin_memory()
    flush = None
    if sum(weight_bytes(world)) * LAYERS <= 130e6 or only_reduce:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    given = group.symmetric("given", (ROWS, HIDDEN))
    given.copy_(torch.randn(ROWS, HIDDEN, generator=g).to(torch.bfloat16))

    def step():
        out = None
        for i in range(LAYERS):
            if plain_sum:
                group.reduce(given, site=f"{i}.post")
                out = group.reduce(given, site=f"{i + 1}.input")
                continue
            p = given if only_reduce else lin_o[i](x_o, out=group.partial(f"{i}.o", (ROWS, HIDDEN)))
            group.reduce_norm(p, h, norms[2 * i], EPS, site=f"{i}.post")
            p = given if only_reduce else lin_d[i](x_d, out=group.partial(f"{i}.down", (ROWS, HIDDEN)))
            out = group.reduce_norm(p, h, norms[2 * i + 1], EPS, site=f"{i + 1}.input")
        return out

    graph, out, launches_per_step = rig.capture(step)
    before = (lambda: flush.fill_(1)) if flush is not None else None

    def e2e_step():
        x_o.copy_(host_xo, non_blocking=True)
        x_d.copy_(host_xd, non_blocking=True)
        graph.replay()
        host_out.copy_(out, non_blocking=True)

    steps, warmup = args.steps, max(args.warmup, 3)
    with torch.cuda.stream(rig.stream):
        for _ in range(warmup):
            if before:
                before()
            graph.replay()
    flush_ms = rig.timed(lambda: flush.fill_(1), steps)[0] / steps if flush is not None else 0.0
    clocks = Clocks(device.index) if rank == 0 else None
    total, each = rig.timed(graph.replay, steps, before)
    ms = total / steps - flush_ms
    with torch.cuda.stream(rig.stream):
        for _ in range(3):
            e2e_step()
    e2e_total, _ = rig.timed(e2e_step, steps, before)
    e2e_ms = e2e_total / steps - flush_ms
    clock_report = clocks.stop() if clocks else None
    group.check()

    # The reference's own GPU building blocks on the same box: cuBLAS torch.mm into the partial, then the reference's
    # reduce_norm_residual kernel built from its sources (oracle/_ref). Informational; absent when it was not built.
    ref_gpu = reference_gpu_path(rig, lin_o, lin_d, norms, x_o, x_d, h0.to(device), args)

    wo, wd = weight_bytes(world)
    launches = 2 * LAYERS
    launch_s = ms * 1e-3 / launches
    if only_reduce:  # no weights: the bytes are the partial read, the slot write+read and the output write
        moved = 4 * ROWS * HIDDEN * 2
        roof = roofline("reduce_kernel", moved, reduction_bytes(world), launch_s, link_gbs)
    else:
        roof = roofline("rowpar_kernel", (wo + wd) / 2, reduction_bytes(world), launch_s, link_gbs)
    traffic = ROOT / "profiles" / "rowpar_kernel_traffic.json"
    roof["traffic"] = json.loads(traffic.read_text()).get(f"tp{world}") if traffic.exists() and not only_reduce else None
    line = {
        "metric": METRIC if args.workload == "c2" else "reduction of given partials (plain sum of a 32-row block), latency "
        "per pair of reductions" if plain_sum else "reduction of given partials (reduce + residual + RMSNorm), latency per "
        "pair of reductions", "value": round(ms * 1e3 / LAYERS, 2), "unit": "us", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config(world, args.workload),
        "e2e": {"value": round(e2e_ms * 1e3 / LAYERS, 2), "unit": "us",
                "h2d_bytes_per_step": host_xo.numel() * 2 + host_xd.numel() * 2, "d2h_bytes_per_step": host_out.numel() * 2},
        "gpu_launches": int(launches_per_step * steps), "replay_us": spread(each, LAYERS), "roofline": roof,
        "clocks": clock_report,
        "timing": "CUDA events on the launching stream around K graph replays, max over ranks; replay_us: each replay "
                  "between its own pair of events",
    }
    if ref_gpu is not None:
        line["reference_gpu_path"] = ref_gpu
    if args.timeline and not only_reduce:
        line["timeline"] = timeline(rig, step, group)
    return line


STAMP_NAMES = {7: "kernel entry", 5: "dependency released", 4: "accumulator ready", 0: "mainloop drained, comm begins",
               6: "tile summed and pushed", 2: "owned rows broadcast", 3: "collected"}


def timeline(rig, step, group, layers=(3, 4)):
    """Phase stamps (%globaltimer, written by thread 0 of every CTA when the caller passes a stamp buffer) of the two
    fused launches of a few layers inside a graph replay: per phase the median and maximum over CTAs, in microseconds
    after the median CTA of the launch entered; `next_entry` is when the following launch's median CTA entered. Plain
    run, no profiler."""
    import numpy as np

    torch = rig.torch
    sms = rig.lib.dlm_device_sms()
    # The stamp buffers exist before the capture: a tensor created while capturing would put a fill kernel into the
    # graph in front of the stamped launch, and that launch would then not be a programmatic dependent of its neighbour.
    sites = {}
    for layer in layers:
        sites[f"{layer}.post"] = (layer, "o_proj")
        sites[f"{layer + 1}.input"] = (layer, "down_proj")
    bufs = {key: torch.zeros(sms * 8, dtype=torch.int64, device=rig.device) for key in sites.values()}
    order = []
    original = group._comm

    def comm(rows, n, site, *a, **kw):
        c, out = original(rows, n, site, *a, **kw)
        if site in sites:
            if sites[site] not in order:
                order.append(sites[site])
            c.stamps = bufs[sites[site]].data_ptr()
        return c, out

    group._comm = comm
    try:
        with torch.cuda.stream(rig.stream):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=rig.stream):
                step()
    finally:
        group._comm = original
    rig.barrier()
    with torch.cuda.stream(rig.stream):
        for _ in range(5):
            graph.replay()
    rig.barrier()
    group.check()
    report, entries = {}, {}
    for key in order:
        s = bufs[key].cpu().numpy().reshape(sms, 8)
        # Blocks that found an idle SM enter as soon as the previous launch has triggered its dependents, long before
        # the rest; the launch's clock starts when the bulk of its blocks is in (the median entry).
        enter = s[:, 7][s[:, 7] > 0]
        t0 = int(np.median(enter))
        entries[key] = t0
        phases = {"ctas": int((s[:, 7] > 0).sum()), "first block entered": round(float(enter.min() - t0) / 1e3, 2)}
        for slot, name in STAMP_NAMES.items():
            v = s[:, slot]
            v = v[v > 0] - t0
            if len(v):
                phases[name] = {"median": round(float(np.median(v)) / 1e3, 2), "max": round(float(v.max()) / 1e3, 2)}
        report[f"layer {key[0]} {key[1]}"] = phases
    for i, key in enumerate(order[:-1]):
        report[f"layer {key[0]} {key[1]}"]["next_entry"] = round((entries[order[i + 1]] - entries[key]) / 1e3, 2)
    return report


def reference_gpu_path(rig, lin_o, lin_d, norms, x_o, x_d, h, args):
    """torch.mm (cuBLAS) into the symmetric partial followed by the reference's own reduce_norm_residual kernel, the
    same 72 operations, captured in a graph and timed the same way. Returns None when oracle/_ref is not present.
    At TP = 1 the reference never launches that kernel (dlmrt/models/sdar/model.py:160-163: a plain RMSNorm kernel
    follows the GEMM), so there the figure is an upper bound on what the reference would take, not its path."""
    torch, group, world = rig.torch, rig.group, rig.world
    ref = load_reference_kernel()
    if ref is None:
        return None
    device = group.device
    R = ROWS // world
    recv = group.symmetric("ref.recv", (3, world, R, HIDDEN), armed=True)
    recv_ptrs = torch.tensor(group.peer_addresses(recv), dtype=torch.int64, device=device)
    epochs = torch.zeros(R + 96, dtype=torch.int32, device=device)
    partial = group.symmetric("ref.partial", (ROWS, HIDDEN))
    outs = [group.symmetric(f"ref.out{i}", (ROWS, HIDDEN), armed=True) for i in range(2 * LAYERS)]
    peers = [group.peers(o) for o in outs]
    mcs = [group.multicast(o) for o in outs]
    state = {"last": None}

    def step():
        for i in range(2 * LAYERS):
            if args.workload == "c2":
                lin, x = (lin_o[i // 2], x_o) if i % 2 == 0 else (lin_d[i // 2], x_d)
                torch.mm(x, lin.weight.t(), out=partial)
            last = state["last"]
            rearm, numel = (last.data_ptr(), last.numel()) if last is not None else (0, 0)
            fn = ref.reduce if args.workload == "k1" else ref.reduce_norm_residual
            fn(partial, recv_ptrs, h, norms[i], outs[i], mcs[i], peers[i], rearm, numel, epochs, group.rank, world, EPS, 1.0,
               96, 0, True)
            state["last"] = outs[i]

    with torch.cuda.stream(rig.stream):
        for _ in range(2):
            step()
        rig.stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=rig.stream):
            step()
        for _ in range(3):
            graph.replay()
    total, each = rig.timed(graph.replay, args.steps)
    return {"value": round(total / args.steps * 1e3 / LAYERS, 2), "unit": "us", "replay_us": spread(each, LAYERS),
            "what": "the reference's tp_comm reduce kernel, same 72 reductions in a CUDA graph" if args.workload == "k1" else
            "torch.mm (cuBLAS) + the reference's tp_comm reduce_norm_residual kernel, same 72 ops in a CUDA graph"
            + ("; at TP = 1 the reference runs a plain RMSNorm kernel instead, so this is an upper bound" if world == 1 else "")}


def load_reference_kernel():
    try:
        from oracle.build_ref import load_built

        return load_built()
    except Exception:  # noqa: BLE001
        return None


# ---------------------------------------------------------------------------------------------------------------------
# Values on the real interconnect (outside every timed region)
# ---------------------------------------------------------------------------------------------------------------------
def parity_block(rig):
    """Runs, eagerly, the calls a round is made of and checks their VALUES: (a) every rank holds identical bits,
    (b) they equal the CPU oracle (exact-integer GEMM operands make the fused projections bit-comparable; normalised
    rows within one BF16 code point, the GPU's approximate rsqrt), (c) this library's reduction equals the reference's
    own kernel (oracle/_ref) bit for bit in all three modes on the same partials at the same world. Also the one-hop
    plain sum of a 32-row block and the all-gather of row statistics. The oracle and the reference kernel are used here
    as checkers only. Returns the `parity` dictionary; all ranks must call it."""
    import numpy as np

    from dlmrt_b200.layers.linear import Linear
    from oracle import reduce as red
    from oracle.bf16 import from_torch

    torch, group, device, world, rank = rig.torch, rig.group, rig.device, rig.world, rig.rank
    result = {"ranks_identical": True, "vs_oracle": True, "vs_reference_kernel": None,
              "multicast": bool(group.multicast(group.symmetric("parity.probe", (8, 256), armed=True))), "checked": []}

    def gather(t):
        t = t.contiguous()
        if world == 1:
            return [t]
        out = [torch.empty_like(t) for _ in range(world)]
        rig.dist.all_gather(out, t)
        return out

    def bits(t):
        return from_torch(t.detach().cpu())

    def distance(a, b):
        def key(x):
            x = np.asarray(x).astype(np.int32)
            return np.where(x & 0x8000, -(x & 0x7FFF), x & 0x7FFF)
        return np.abs(key(a) - key(b))

    def record(name, out, want, exact=True):
        torch.cuda.synchronize(device)
        group.check()
        mine = bits(out)
        same = all(np.array_equal(bits(o), mine) for o in gather(out))
        if exact:
            ok = np.array_equal(mine, want)
        else:
            d = distance(mine, want)
            ok = d.max() <= 1 and (d > 0).mean() <= 5e-3
        result["ranks_identical"] &= bool(same)
        result["vs_oracle"] &= bool(ok)
        result["checked"].append(name if same and ok else f"{name}: FAILED (identical={same}, oracle={bool(ok)})")

    with torch.cuda.stream(rig.stream):
        # -- two layers' worth of fused projections on exact-integer operands ------------------------------------------
        norm = (torch.randn(HIDDEN, generator=torch.Generator().manual_seed(21)) * 0.1 + 1).to(torch.bfloat16).to(device)
        h = torch.randn(ROWS, HIDDEN, generator=torch.Generator().manual_seed(22)).to(torch.bfloat16).to(device)
        for layer in range(2):
            for name, k_total in (("o_proj", K_O), ("down_proj", K_DOWN)):
                g = torch.Generator().manual_seed(1000 * layer + k_total)  # the same full matrices on every rank
                x = torch.randint(-3, 4, (ROWS, k_total), generator=g).to(torch.bfloat16)
                w = torch.randint(-2, 3, (HIDDEN, k_total), generator=g).to(torch.bfloat16)
                xs, ws = group.shard(x, 1).to(device), group.shard(w, 1).to(device)
                parts = np.stack([from_torch((a.float() @ b.float().t()).to(torch.bfloat16))
                                  for a, b in zip(x.chunk(world, 1), w.chunk(world, 1))])
                lin = Linear(ws, group=group)
                h_all = np.stack([bits(t) for t in gather(h)])
                p = lin(xs, out=group.partial("parity", (ROWS, HIDDEN)))
                if name == "o_proj":
                    out = group.reduce(p, site=f"parity.{layer}.o")
                    record(f"fused {name} K1 layer {layer}", out, red.reduce(parts))
                else:
                    out = group.reduce_norm(p, h, norm, EPS, site=f"parity.{layer}.d")
                    want, h_after = red.reduce_norm(parts, bits(norm), EPS, 1.0, h_all)
                    record(f"fused {name} K3 layer {layer}", out, want, exact=False)
                    ok = np.array_equal(bits(h), h_after[rank])
                    result["vs_oracle"] &= bool(ok)
                    result["checked"].append(f"residual stream after layer {layer}" + ("" if ok else ": FAILED"))
        # -- Gaussian partials through all three modes, against the oracle and against the reference's kernel -----------
        ref = load_reference_kernel()
        weight = norm
        given = [(torch.randn(ROWS, HIDDEN, generator=torch.Generator().manual_seed(31 + 10 * i + rank))).to(torch.bfloat16)
                 .to(device) for i in range(3)]
        if ref is not None:
            R = ROWS // world
            recv = group.symmetric("parity.ref.recv", (3, world, R, HIDDEN), armed=True)
            recv_ptrs = torch.tensor(group.peer_addresses(recv), dtype=torch.int64, device=device)
            epochs = torch.zeros(R + 96, dtype=torch.int32, device=device)
            ref_partial = group.symmetric("parity.ref.partial", (ROWS, HIDDEN))
            ref_outs = [group.symmetric(f"parity.ref.out{i}", (ROWS, HIDDEN), armed=True) for i in range(3)]
            result["vs_reference_kernel"] = True
        last = None
        for mode, p in enumerate(given):
            all_p = np.stack([bits(t) for t in gather(p)])
            h_all = np.stack([bits(t) for t in gather(h)])
            h_ref = h.clone()
            if mode == 0:
                out = group.reduce(p, site=f"parity.g{mode}")
                record("given partials K1", out, red.reduce(all_p))
            elif mode == 1:
                out = group.reduce_norm(p, None, weight, EPS, 0.75, site=f"parity.g{mode}")
                record("given partials K2", out, red.reduce_norm(all_p, bits(weight), EPS, 0.75)[0], exact=False)
            else:
                out = group.reduce_norm(p, h, weight, EPS, site=f"parity.g{mode}")
                want, h_after = red.reduce_norm(all_p, bits(weight), EPS, 1.0, h_all)
                record("given partials K3", out, want, exact=False)
                result["vs_oracle"] &= bool(np.array_equal(bits(h), h_after[rank]))
            if ref is not None:
                ref_partial.copy_(p)
                fn = (ref.reduce, ref.reduce_norm, ref.reduce_norm_residual)[mode]
                rearm, numel = (last.data_ptr(), last.numel()) if last is not None else (0, 0)
                ro = ref_outs[mode]
                fn(ref_partial, recv_ptrs, h_ref, weight, ro, group.multicast(ro), group.peers(ro), rearm, numel, epochs,
                   group.rank, world, EPS, 0.75 if mode == 1 else 1.0, 96, 0, False)
                last = ro
                torch.cuda.synchronize(device)
                same = bool(torch.equal(ro.view(torch.int16), out.view(torch.int16)))
                if mode == 2:
                    same &= bool(torch.equal(h_ref.view(torch.int16), h.view(torch.int16)))
                same = all(bool(v.item()) for v in gather(torch.tensor([same], device=device)))
                result["vs_reference_kernel"] &= same
                result["checked"].append(f"reference kernel mode {mode}" + ("" if same else ": FAILED"))
        # -- the one-hop plain sum of a 32-row block, and the all-gather of row statistics ---------------------------
        small = torch.randn(32, 2048, generator=torch.Generator().manual_seed(77 + rank)).to(torch.bfloat16).to(device)
        for rep in range(2):
            out = group.reduce(small, site=f"parity.small{rep}", chain=32)
            record(f"32-row plain sum #{rep}" + (" (one hop)" if group.one_shot(32, 2048, 0) else ""), out,
                    red.reduce(np.stack([bits(t) for t in gather(small)])))
        stats = torch.randn(32, 4, generator=torch.Generator().manual_seed(88 + rank)).to(device)
        for rep in range(2):
            got = group.all_gather(stats, "parity.stats")
            torch.cuda.synchronize(device)
            group.check()
            ok = bool(torch.equal(got.view(torch.int32), torch.stack(gather(stats)).view(torch.int32)))
            result["vs_oracle"] &= ok
            result["checked"].append(f"all_gather #{rep}" + ("" if ok else ": FAILED"))
    result["ok"] = bool(result["ranks_identical"] and result["vs_oracle"] and result["vs_reference_kernel"] is not False)
    return result


# ---------------------------------------------------------------------------------------------------------------------
# NVFP4 expert workloads (BASELINE configs 4 and 5)
# ---------------------------------------------------------------------------------------------------------------------
MOE_SHAPES = {"c4": dict(hidden=2048, f=512, experts=256, top_k=8, rows=32, layers=20,
                         name="BASELINE config 4: LLaDA2.1-mini-shape MoE, 256 experts top-8, F=512, 32-token block"),
              "c5": dict(hidden=2816, f=704, experts=128, top_k=8, rows=256, layers=30,
                         name="BASELINE config 5: DiffusionGemma-shape MoE, 128 experts top-8, F=704, 256-token canvas")}


def run_moe(args, rig, link_gbs, workload, routing, steps):
    """A step = `layers` fused launches of the NVFP4 expert down-projection + combine + reduction (one per layer, each
    layer with its own expert weights; random codes and scales, seeded routing, uniform or Zipf(1.2))."""
    import numpy as np

    from dlmrt_b200.quantization import nvfp4

    torch, group, device, world, rank = rig.torch, rig.group, rig.device, rig.world, rig.rank
    shape = MOE_SHAPES[workload]
    hidden, f, experts, top_k, rows = (shape[k] for k in ("hidden", "f", "experts", "top_k", "rows"))
    layers = min(args.layers, shape["layers"])
    e_local, lo = experts // world, rank * (experts // world)
    rng = np.random.default_rng(5)  # routing identical on every rank
    if routing == "zipf":
        p = 1.0 / np.arange(1, experts + 1) ** 1.2
        p = (p / p.sum())[rng.permutation(experts)]
        ids = np.stack([np.sort(rng.choice(experts, top_k, replace=False, p=p)) for _ in range(rows)])
    else:
        ids = np.stack([np.sort(rng.permutation(experts)[:top_k]) for _ in range(rows)])
    ids = ids.astype(np.int32)
    amap = np.zeros((experts, rows), dtype=np.int32)
    counts = np.zeros(experts, dtype=np.int32)
    for pair, e in enumerate(ids.reshape(-1).tolist()):
        amap[e, counts[e]] = pair
        counts[e] += 1
    active_local = int((counts[lo:lo + e_local] > 0).sum())
    active_max = int(rig.max_over_ranks(active_local))
    g = torch.Generator(device=device).manual_seed(1 + rank)
    u8 = dict(device=device, dtype=torch.uint8, generator=g)
    layer_experts = []
    for _ in range(layers):
        s2 = torch.randint(0x28, 0x48, (e_local, hidden, f // 16), **u8)  # E4M3 scales between 0.25 and 4
        layer_experts.append({"lo": lo, "w2": nvfp4.tile_codes(torch.randint(0, 256, (e_local, hidden, f // 2), **u8)),
                              "tiled": True, "n": hidden, "f": f,
                              "s2": nvfp4.interleave_scales(s2), "g2": torch.full((e_local,), 1e-4, device=device)})
    act_codes = torch.randint(0, 256, (e_local * rows, f // 2), **u8)
    act_scales = torch.randint(0x28, 0x48, (e_local * rows, f // 16), **u8)
    t = lambda a: torch.from_numpy(a).to(device)  # noqa: E731
    common = dict(act_codes=act_codes, act_scales=act_scales, amap=t(amap), counts=t(counts), ids=t(ids),
                  weights=torch.full((rows, top_k), 2.5 / top_k, device=device), num_experts=experts,
                  buffers=nvfp4.Buffers(rows, hidden, top_k, device))
    tag = f"{workload}.{routing}"

    def step():
        out = None
        for i in range(layers):
            out = nvfp4.moe_down(experts=layer_experts[i], out=None, group=group, site=f"{tag}.{i}.moe", chain=tag,
                                 **common)
        return out

    graph, _, launches_per_step = rig.capture(step)
    with torch.cuda.stream(rig.stream):
        for _ in range(max(args.warmup, 3)):
            graph.replay()
    clocks = Clocks(device.index) if rank == 0 else None
    total, each = rig.timed(graph.replay, steps)
    clock_report = clocks.stop() if clocks else None
    group.check()
    del graph

    # The whole routed-expert call as a model makes it (trtllm_moe): per-token bookkeeping + input quantisation, GEMM1 +
    # activation + re-quantisation, then the down-projection + combine deferred into the reduction: three launches per
    # layer. Gate / up weights are random codes as well; the routing is the one above.
    activation = "swiglu" if workload == "c4" else "geglu"
    for ex in layer_experts:
        s13 = torch.randint(0x28, 0x48, (e_local, 2 * f, hidden // 16), **u8)
        ex.update(w13=nvfp4.tile_codes(torch.randint(0, 256, (e_local, 2 * f, hidden // 2), **u8)),
                  s13=nvfp4.interleave_scales(s13), hidden=hidden, g1=torch.full((e_local,), 1e-4, device=device),
                  a1_inv=torch.full((1,), 8.0, device=device), a2_inv=torch.full((e_local,), 8.0, device=device),
                  group=group)
    x = (torch.randn(rows, hidden, generator=torch.Generator().manual_seed(9)) * 0.5).to(torch.bfloat16).to(device)
    packed = nvfp4.pack(t(ids), common["weights"]).contiguous()

    def whole():
        out = None
        for i in range(layers):
            p = nvfp4.trtllm_moe(x, packed, layer_experts[i], group.symmetric(f"{tag}.whole", (rows, hidden)), experts, lo,
                                 f, activation=activation)
            out = group.reduce(p, site=f"{tag}.{i}.whole", chain=tag + ".whole")
        return out

    graph, _, whole_launches = rig.capture(whole)
    with torch.cuda.stream(rig.stream):
        for _ in range(max(args.warmup, 3)):
            graph.replay()
    whole_total, whole_each = rig.timed(graph.replay, steps)
    group.check()
    gate_up = active_max * 2 * f * hidden * 9 // 16
    weight = active_max * hidden * f * 9 // 16  # codes + E4M3 scales of the busiest rank's active experts
    per_launch = total / steps * 1e-3 / layers
    roof = roofline("moe_kernel", weight, reduction_bytes(world, rows, hidden), per_launch, link_gbs)
    traffic = ROOT / "profiles" / "rowpar_kernel_traffic.json"  # ncu DRAM read + write per launch, where captured
    roof["traffic"] = json.loads(traffic.read_text()).get(f"moe_{workload}_{routing}_tp{world}") if traffic.exists() else None
    return {
        "metric": "fused NVFP4 expert down-projection+combine+reduction latency per MoE layer",
        "value": round(per_launch * 1e6, 2), "unit": "us", "n_gpus": world, "steps": steps,
        "ms_per_step": round(total / steps, 4), "replay_us": spread(each, layers),
        "dtype": "nvfp4 (e2m1 x ue4m3 per 16), fp32 accumulate",
        "config": {"workload": shape["name"] + f", {routing} routing, TP={world}, {layers} layers per step; the weights of a "
                   f"step ({weight * layers / 1e6:.0f} MB on the busiest rank) " +
                   ("exceed the 126 MB L2" if weight * layers > 130e6 else "fit the L2: an L2-resident figure"),
                   "active_local_experts": active_max, "tp": world},
        "gpu_launches": int(launches_per_step * steps), "roofline": roof, "clocks": clock_report,
        "whole_call": {"what": "trtllm_moe (routing bookkeeping + input quantisation, GEMM1 + activation + re-quantisation) "
                               "followed by the reduction that runs the down-projection + combine: three launches per layer",
                       "value": round(whole_total / steps * 1e3 / layers, 2), "unit": "us",
                       "replay_us": spread(whole_each, layers), "launches_per_layer": whole_launches / layers,
                       "weight_bytes_per_layer": int(gate_up + weight),
                       "frac_of_hbm_peak": round((gate_up + weight) / (whole_total / steps * 1e-3 / layers) / 1e9 /
                                                 peaks()[0], 4)}}


# ---------------------------------------------------------------------------------------------------------------------
# A whole synthetic denoise round of the config-3 shape
# ---------------------------------------------------------------------------------------------------------------------
ROUND = dict(layers=36, hidden=2560, heads=32, kv_heads=8, head_dim=128, ffn=9728, vocab=151936, rows=256)


def run_round(args, rig, steps):
    """One denoise round over a 256-token block of the QwenDLM-4B shape at empty context, captured once and replayed
    (median of the replays, dlmrt/entrypoints/bench/common.py:68-80). Per layer: qkv projection (cuBLAS torch.mm,
    column-parallel), attention over the block (torch SDPA, grouped KV heads), o_proj fused with reduce + residual +
    RMSNorm (this library), gate_up (cuBLAS) + SwiGLU, down_proj fused the same way; then the vocabulary-parallel LM head
    (cuBLAS), per-row statistics and their all-gather (this library). Only the two fused launches per layer and the
    all-gather are this repository's kernels: the rest stands in for the reference's neighbours with library calls so
    that the round has the right dependencies and memory traffic. The same round with the fused launches replaced by
    cuBLAS + the reference's reduce kernel is timed beside it where that kernel is present and N > 1."""
    torch, group, device, world, rank = rig.torch, rig.group, rig.device, rig.world, rig.rank
    from dlmrt_b200.layers.linear import Linear

    c = ROUND
    layers = min(args.layers, c["layers"])
    rows, hidden, d = c["rows"], c["hidden"], c["head_dim"]
    hq, hk, ffn, vocab = c["heads"] // world, c["kv_heads"] // world, c["ffn"] // world, c["vocab"] // world
    g = torch.Generator(device=device).manual_seed(11 + rank)

    def w(*shape):
        return (torch.randn(*shape, device=device, generator=g) * 0.02).to(torch.bfloat16)

    qkv = [w((hq + 2 * hk) * d, hidden) for _ in range(layers)]
    gate_up = [w(2 * ffn, hidden) for _ in range(layers)]
    lin_o = [Linear(w(hidden, hq * d), group=group) for _ in range(layers)]
    lin_d = [Linear(w(hidden, ffn), group=group) for _ in range(layers)]
    embed = w(vocab, hidden)
    gs = torch.Generator().manual_seed(7)
    norms = [(torch.randn(hidden, generator=gs) * 0.1 + 1).to(torch.bfloat16).to(device) for _ in range(2 * layers)]
    h = torch.randn(rows, hidden, generator=gs).to(torch.bfloat16).to(device)
    x0 = torch.randn(rows, hidden, generator=gs).to(torch.bfloat16).to(device)
    sdpa = torch.nn.functional.scaled_dot_product_attention
    ref = load_reference_kernel() if world > 1 else None

    def body(fused):
        x = x0
        for i in range(layers):
            q, k, v = torch.mm(x, qkv[i].t()).split((hq * d, hk * d, hk * d), 1)
            attn = sdpa(q.view(1, rows, hq, d).transpose(1, 2), k.view(1, rows, hk, d).transpose(1, 2),
                        v.view(1, rows, hk, d).transpose(1, 2), enable_gqa=True).transpose(1, 2).reshape(rows, hq * d)
            x = fused(lin_o[i], attn, norms[2 * i], f"r{i}.post")
            gu = torch.mm(x, gate_up[i].t())
            act = torch.nn.functional.silu(gu[:, :ffn]) * gu[:, ffn:]
            x = fused(lin_d[i], act, norms[2 * i + 1], f"r{i + 1}.input")
        logits = torch.mm(x, embed.t()).float()
        top = logits.max(-1)
        stats = torch.stack((top.values, top.indices.float() + rank * vocab, torch.logsumexp(logits, -1),
                             torch.zeros_like(top.values)), -1)
        return group.all_gather(stats, "round.stats")

    def ours(lin, x, norm, site):
        return group.reduce_norm(lin(x, out=group.partial(site, (rows, hidden))), h, norm, EPS, site=site, chain="round")

    graph, _, launches = rig.capture(lambda: body(ours))
    with torch.cuda.stream(rig.stream):
        for _ in range(3):
            graph.replay()
    total, each = rig.timed(graph.replay, steps)
    group.check()
    result = {"what": f"one denoise round, QwenDLM-4B shape ({layers} layers, hidden {hidden}, {c['heads']}q/{c['kv_heads']}kv x "
                      f"{d}, FFN {c['ffn']}, vocab {c['vocab']}), {rows}-token block, empty context, BF16 (KV kept in BF16), "
                      f"TP={world}; this library: {launches} launches per round, the rest cuBLAS / SDPA / elementwise torch",
              "value": round(statistics.median(each) * 1e3, 1), "unit": "us", "replay_us": spread(each, 1),
              "mean_us": round(total / steps * 1e3, 1)}
    if ref is not None:
        R = rows // world
        recv = group.symmetric("round.ref.recv", (3, world, R, hidden), armed=True)
        recv_ptrs = torch.tensor(group.peer_addresses(recv), dtype=torch.int64, device=device)
        epochs = torch.zeros(R + 96, dtype=torch.int32, device=device)
        partial = group.symmetric("round.ref.partial", (rows, hidden))
        state = {"last": None}

        def theirs(lin, x, norm, site):
            out = group.symmetric(f"round.ref.{site}", (rows, hidden), armed=True)
            torch.mm(x, lin.weight.t(), out=partial)
            last = state["last"]
            rearm, numel = (last.data_ptr(), last.numel()) if last is not None else (0, 0)
            ref.reduce_norm_residual(partial, recv_ptrs, h, norm, out, group.multicast(out), group.peers(out), rearm, numel,
                                     epochs, group.rank, world, EPS, 1.0, 96, 0, True)
            state["last"] = out
            return out

        graph_ref, _, _ = rig.capture(lambda: body(theirs))
        with torch.cuda.stream(rig.stream):
            for _ in range(3):
                graph_ref.replay()
        _, each_ref = rig.timed(graph_ref.replay, steps)
        result["reference_blocks"] = {"value": round(statistics.median(each_ref) * 1e3, 1), "unit": "us",
                                      "replay_us": spread(each_ref, 1),
                                      "what": "the same round with cuBLAS torch.mm + the reference's tp_comm "
                                              "reduce_norm_residual kernel in place of each fused launch"}
    return result


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=36, help="layers per step; fewer only for profiler captures")
    ap.add_argument("--workload", default="c2", choices=["c2", "k1", "k3", "c4", "c5", "round"], help="c2 is the bench line "
                    "(it also carries the parity, moe and round blocks); k1 / k3 time the reduction of given partials "
                    "alone; c4 / c5 / round run that block alone")
    ap.add_argument("--routing", default="uniform", choices=["uniform", "zipf"])
    ap.add_argument("--shard-of", type=int, default=1, help="profiling aid: run the K shard of a TP=<n> rank on the GPUs "
                    "given (the GEMM of a higher TP degree without its peers)")
    ap.add_argument("--timeline", action="store_true", help="c2: also record the kernels' phase stamps of two layers")
    ap.add_argument("--only", action="store_true", help="c2 / k1 / k3: leave out the parity, moe and round blocks "
                    "(profiler captures)")
    args = ap.parse_args()
    global LAYERS, K_O, K_DOWN
    LAYERS = args.layers
    K_O, K_DOWN = K_O // args.shard_of, K_DOWN // args.shard_of
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torchrun --nproc-per-node {args.gpus}); "
                         f"WORLD_SIZE is {world}")
    if args.workload == "k1":  # LLaDA2's block: 32 rows of hidden 2048
        global ROWS, HIDDEN
        ROWS, HIDDEN = 32, 2048
    rig = Rig(world)
    link_gbs = nvlink_peak(rig)
    failed = False
    if args.workload in ("c4", "c5"):
        line = run_moe(args, rig, link_gbs, args.workload, args.routing, args.steps)
        line.update(warmup=max(args.warmup, 3), higher_is_better=False, scaling="strong", vs_baseline=None, data="synthetic")
    elif args.workload == "round":
        line = run_round(args, rig, args.steps)
    else:
        line = run_dense(args, rig, link_gbs)
        full = args.workload == "c2" and not args.only and args.shard_of == 1
        if full:
            line["parity"] = parity_block(rig)
            failed = not line["parity"]["ok"]
            moe_steps = min(args.steps, 10)
            line["moe"] = {"c4_uniform": run_moe(args, rig, link_gbs, "c4", "uniform", moe_steps),
                           "c4_zipf": run_moe(args, rig, link_gbs, "c4", "zipf", moe_steps),
                           "c5": run_moe(args, rig, link_gbs, "c5", "uniform", moe_steps)}
            line["round"] = run_round(args, rig, min(args.steps, 20))
        if world == 1 and args.workload == "c2":
            cpu_sec, cores = cpu_layer_seconds(world, 5)
            line["cpu_baseline"] = {"value": round(cpu_sec * 1e6, 1), "unit": "us", "cores": cores, "kind": "port",
                                    "sample": "one decoder layer (o_proj + down_proj) on the host, median of 5"}
    if link_gbs:
        line["nvlink_peer_copy_gbs"] = round(link_gbs, 1)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        rig.dist.barrier()
        rig.dist.destroy_process_group()
    if failed:
        raise SystemExit("parity check failed: see the `parity` block of the line above")


if __name__ == "__main__":
    main()
