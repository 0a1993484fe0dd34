"""Benchmark of the tensor-parallel row-parallel hot path (fused projection + reduction) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Workload (BASELINE config 2, the Qwen3-style decoder layer): hidden 2560, o_proj K = 4096, down_proj K = 9728,
one 256-token block, BF16, TP = N. One STEP is the row-parallel hot path of a 36-layer round: for each layer the two
fused kernels `o_proj -> reduce + residual + RMSNorm` and `down_proj -> reduce + residual + RMSNorm`
(dlmrt/models/sdar/model.py:237-243), 72 launches, each layer with its own weights (2.56 GB at TP = 1, far above the
126 MB L2, so weights stream from HBM every step). Steps are captured once in a CUDA graph and replayed, as the
reference measures a round (dlmrt/entrypoints/bench/common.py:68-80).

  value      microseconds per decoder layer (o_proj + down_proj with their reductions), inputs resident in HBM
  e2e        the same through host buffers: pinned-host -> device copy of the step's activations, the graph replay, and
             the device -> host copy of the last reduced block, all inside the timed region
  roofline   dominant kernel rowpar_kernel: algorithmic bytes = the weight shard N * K/w * 2 per launch (HBM) or, when
             larger in time, the reduction's per-GPU NVLink ingress 2 * (w-1)/w * M * N * 2, over the average launch
             duration measured here with CUDA events
  cpu_baseline / --impl reference   the CPU restatement of the same path (torch CPU matmul per K shard, rank-order FP32
             sum, residual, RMSNorm) on the host cores. The reference has no CPU implementation of this path, so this
             port is what is timed (kind "port").

Synthetic data: weights ~ N(0, 0.02), activations ~ N(0, 1), seeded; no dataset or checkpoint is read.
"""

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HIDDEN, K_O, K_DOWN, ROWS, LAYERS, EPS = 2560, 4096, 9728, 256, 36, 1e-6
NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction on this pool (nominal 900)
FALLBACK_HBM_GBS = 6650.0


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class Clocks:
    """Samples nvidia-smi during the timed region."""

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


def reduction_bytes(world):
    return 2 * (world - 1) * ROWS * HIDDEN * 2 // world


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


METRIC = "fused row-parallel projection+reduction latency per decoder layer (o_proj + down_proj), denoise round"


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
# GPU arm
# ---------------------------------------------------------------------------------------------------------------------
def run_gpu(args, rank, world):
    import torch

    from dlmrt_b200 import _lib
    from dlmrt_b200.distributed import parallel
    from dlmrt_b200.layers.linear import Linear

    if world > 1:
        import torch.distributed as dist

        group = parallel.init()
        device = group.device
    else:
        device = torch.device("cuda", 0)
        torch.cuda.set_device(device)
        group = parallel.Group.local(device)
    lib = _lib.lib()
    if lib.dlm_device_arch() != 100:
        raise RuntimeError("bench.py needs an sm_100 GPU: there is no fallback path")

    g = torch.Generator().manual_seed(1 + rank)
    ko, kd = K_O // world, K_DOWN // world
    weights = 0 if args.workload in ("k1", "k3") else LAYERS  # the reduction-only workloads have no GEMM
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
    if sum(weight_bytes(world)) * LAYERS <= 130e6 or args.workload in ("k1", "k3"):
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    only_reduce = args.workload in ("k1", "k3")  # the reduction of GIVEN partials alone (dlm_reduce_bf16), no GEMM
    plain_sum = args.workload == "k1"           # K1 (no residual, no norm) on a 32-row block: LLaDA2's call pattern
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

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for _ in range(2):  # eager: allocates every symmetric buffer, in the same order on every rank
            out = step()
        stream.synchronize()
        group.check()
        before = lib.dlm_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = step()
        launches_per_step = lib.dlm_launch_count() - before

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    def timed(fn, steps):
        """Total milliseconds of `steps` calls on `stream`, CUDA events, max over ranks."""
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with torch.cuda.stream(stream):
            start.record(stream)
            for _ in range(steps):
                fn()
            stop.record(stream)
        barrier()
        ms = torch.tensor([start.elapsed_time(stop)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def device_step():
        if flush is not None:
            flush.fill_(1)
        graph.replay()

    def e2e_step():
        x_o.copy_(host_xo, non_blocking=True)
        x_d.copy_(host_xd, non_blocking=True)
        if flush is not None:
            flush.fill_(1)
        graph.replay()
        host_out.copy_(out, non_blocking=True)

    flush_ms = 0.0
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            device_step()
    if flush is not None:
        flush_ms = timed(lambda: flush.fill_(1), args.steps) / args.steps
    clocks = Clocks(device.index) if rank == 0 else None
    ms = timed(device_step, args.steps) / args.steps - flush_ms
    with torch.cuda.stream(stream):
        for _ in range(3):
            e2e_step()
    e2e_ms = timed(e2e_step, args.steps) / args.steps - flush_ms
    clock_report = clocks.stop() if clocks else None
    group.check()

    # The reference's own GPU building blocks on the same box: cuBLAS torch.mm into the partial, then the reference's
    # reduce_norm_residual kernel built from its sources (oracle/_ref). Informational; absent when it was not built.
    ref_gpu = reference_gpu_path(torch, group, lin_o, lin_d, norms, x_o, x_d, h0.to(device), stream, timed, args, world)

    if rank != 0:
        return
    hbm, which = peaks()
    wo, wd = weight_bytes(world)
    launches = 2 * LAYERS
    avg_launch_s = ms * 1e-3 / launches
    t_hbm = (wo + wd) / 2 / (hbm * 1e9)
    t_link = reduction_bytes(world) / (NVLINK_GBS * 1e9)
    if t_hbm >= t_link:
        roof = {"bound": "hbm", "achieved": round((wo + wd) / 2 / avg_launch_s / 1e9, 1), "peak": hbm, "unit": "GB/s"}
    else:
        roof = {"bound": "nvlink", "achieved": round(reduction_bytes(world) / avg_launch_s / 1e9, 1), "peak": NVLINK_GBS,
                "unit": "GB/s"}
    roof["frac"] = round(roof["achieved"] / roof["peak"], 4)
    roof["peak_source"] = f"of {which}"
    roof["kernel"] = "reduce_kernel" if only_reduce else "rowpar_kernel"
    if only_reduce:  # no weights: the bytes are the partial read, the slot write+read and the output write
        moved = 4 * ROWS * HIDDEN * 2
        roof.update(bound="latency", achieved=round(moved / avg_launch_s / 1e9, 1), peak=hbm, unit="GB/s",
                    algorithmic_bytes_per_launch=moved)
        roof["frac"] = round(roof["achieved"] / roof["peak"], 4)
    roof["algorithmic_bytes_per_launch"] = (wo + wd) // 2 if roof["bound"] == "hbm" else reduction_bytes(world)
    roof["avg_launch_us"] = round(avg_launch_s * 1e6, 2)
    traffic = ROOT / "profiles" / "rowpar_kernel_traffic.json"
    roof["traffic"] = json.loads(traffic.read_text()).get(f"tp{world}") if traffic.exists() else None

    cpu_sec, cores = cpu_layer_seconds(world, 5) if world == 1 else (None, None)
    line = {
        "metric": METRIC if args.workload == "c2" else "reduction of given partials (plain sum of a 32-row block), latency "
        "per pair of reductions" if plain_sum else "reduction of given partials (reduce + residual + RMSNorm), latency per "
        "pair of reductions", "value": round(ms * 1e3 / LAYERS, 2), "unit": "us", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config(world, args.workload),
        "e2e": {"value": round(e2e_ms * 1e3 / LAYERS, 2), "unit": "us",
                "h2d_bytes_per_step": host_xo.numel() * 2 + host_xd.numel() * 2, "d2h_bytes_per_step": host_out.numel() * 2},
        "gpu_launches": int(launches_per_step * args.steps), "roofline": roof, "clocks": clock_report,
        "timing": "CUDA events on the launching stream around K graph replays, max over ranks",
    }
    if cpu_sec is not None:
        line["cpu_baseline"] = {"value": round(cpu_sec * 1e6, 1), "unit": "us", "cores": cores, "kind": "port",
                                "sample": "one decoder layer (o_proj + down_proj) on the host, median of 5"}
    if ref_gpu is not None:
        line["reference_gpu_path"] = ref_gpu
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------------------------
# NVFP4 expert workloads (BASELINE configs 4 and 5): not the default bench line, run with --workload c4 | c5
# ---------------------------------------------------------------------------------------------------------------------
MOE_SHAPES = {"c4": dict(hidden=2048, f=512, experts=256, top_k=8, rows=32, layers=20,
                         name="BASELINE config 4: LLaDA2.1-mini-shape MoE, 256 experts top-8, F=512, 32-token block"),
              "c5": dict(hidden=2816, f=704, experts=128, top_k=8, rows=256, layers=30,
                         name="BASELINE config 5: DiffusionGemma-shape MoE, 128 experts top-8, F=704, 256-token canvas")}


def run_gpu_moe(args, rank, world):
    """A step = `layers` fused launches of the NVFP4 expert down-projection + combine + reduction (one per layer, each
    layer with its own expert weights; random codes and scales, seeded routing, uniform or Zipf(1.2))."""
    import numpy as np
    import torch

    from dlmrt_b200 import _lib
    from dlmrt_b200.distributed import parallel
    from dlmrt_b200.quantization import nvfp4

    shape = MOE_SHAPES[args.workload]
    hidden, f, experts, top_k, rows = (shape[k] for k in ("hidden", "f", "experts", "top_k", "rows"))
    layers = min(args.layers, shape["layers"])
    if world > 1:
        import torch.distributed as dist

        group = parallel.init()
        device = group.device
    else:
        device = torch.device("cuda", 0)
        torch.cuda.set_device(device)
        group = parallel.Group.local(device)
    e_local, lo = experts // world, rank * (experts // world)
    rng = np.random.default_rng(5)  # routing identical on every rank
    if args.routing == "zipf":
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
    g = torch.Generator(device=device).manual_seed(1 + rank)
    u8 = dict(device=device, dtype=torch.uint8, generator=g)
    layer_experts = []
    for _ in range(layers):
        s2 = torch.randint(0x28, 0x48, (e_local, hidden, f // 16), **u8)  # E4M3 scales between 0.25 and 4
        layer_experts.append({"lo": lo, "w2": torch.randint(0, 256, (e_local, hidden, f // 2), **u8),
                              "s2": nvfp4.interleave_scales(s2), "g2": torch.full((e_local,), 1e-4, device=device)})
    act_codes = torch.randint(0, 256, (e_local * rows, f // 2), **u8)
    act_scales = torch.randint(0x28, 0x48, (e_local * rows, f // 16), **u8)
    t = lambda a: torch.from_numpy(a).to(device)  # noqa: E731
    common = dict(act_codes=act_codes, act_scales=act_scales, amap=t(amap), counts=t(counts), ids=t(ids),
                  weights=torch.full((rows, top_k), 2.5 / top_k, device=device), num_experts=experts,
                  buffers=nvfp4.Buffers(rows, hidden, top_k, device))

    def step():
        out = None
        for i in range(layers):
            out = nvfp4.moe_down(experts=layer_experts[i], out=None, group=group, site=f"{i}.moe", chain=rows, **common)
        return out

    stream = torch.cuda.Stream(device)
    lib = _lib.lib()
    with torch.cuda.stream(stream):
        for _ in range(2):
            step()
        stream.synchronize()
        group.check()
        before = lib.dlm_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        launches_per_step = lib.dlm_launch_count() - before
        for _ in range(max(args.warmup, 3)):
            graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    clocks = Clocks(device.index) if rank == 0 else None
    with torch.cuda.stream(stream):
        start.record(stream)
        for _ in range(args.steps):
            graph.replay()
        stop.record(stream)
    torch.cuda.synchronize(device)
    ms = torch.tensor([start.elapsed_time(stop) / args.steps], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clock_report = clocks.stop() if clocks else None
    group.check()
    if rank != 0:
        return
    hbm, which = peaks()
    weight = active_local * hidden * f * 9 // 16  # codes + E4M3 scales of the active local experts
    per_launch = float(ms.item()) * 1e-3 / layers
    t_hbm, t_link = weight / (hbm * 1e9), 2 * (world - 1) * rows * hidden * 2 / world / (NVLINK_GBS * 1e9)
    if t_hbm >= t_link:
        roof = {"bound": "hbm", "achieved": round(weight / per_launch / 1e9, 1), "peak": hbm, "unit": "GB/s"}
    else:
        roof = {"bound": "nvlink", "achieved": round(t_link * NVLINK_GBS / per_launch, 1), "peak": NVLINK_GBS, "unit": "GB/s"}
    roof.update(frac=round(roof["achieved"] / roof["peak"], 4), peak_source=f"of {which}", kernel="moe_kernel",
                algorithmic_bytes_per_launch=weight, avg_launch_us=round(per_launch * 1e6, 2), traffic=None)
    print(json.dumps({
        "metric": "fused NVFP4 expert down-projection+combine+reduction latency per MoE layer", "value":
        round(per_launch * 1e6, 2), "unit": "us", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(float(ms.item()), 4), "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "nvfp4 (e2m1 x ue4m3 per 16), fp32 accumulate", "data": "synthetic",
        "config": {"workload": shape["name"] + f", {args.routing} routing, TP={world}, {layers} layers per step",
                   "active_local_experts": active_local, "tp": world},
        "gpu_launches": int(launches_per_step * args.steps), "roofline": roof, "clocks": clock_report}))



def reference_gpu_path(torch, group, lin_o, lin_d, norms, x_o, x_d, h, stream, timed, args, world):
    """torch.mm (cuBLAS) into the symmetric partial followed by the reference's own reduce_norm_residual kernel, the
    same 72 operations, captured in a graph and timed the same way. Returns None when oracle/_ref is not present."""
    try:
        from oracle.build_ref import load_built

        ref = load_built()
    except Exception:  # noqa: BLE001
        ref = None
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

    with torch.cuda.stream(stream):
        for _ in range(2):
            step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        for _ in range(3):
            graph.replay()
    ms = timed(graph.replay, args.steps) / args.steps
    return {"value": round(ms * 1e3 / LAYERS, 2), "unit": "us",
            "what": "the reference's tp_comm reduce kernel, same 72 reductions in a CUDA graph" if args.workload == "k1" else
            "torch.mm (cuBLAS) + the reference's tp_comm reduce_norm_residual kernel, same 72 ops in a CUDA graph"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=36, help="layers per step; fewer only for profiler captures")
    ap.add_argument("--workload", default="c2", choices=["c2", "k1", "k3", "c4", "c5"], help="c2 is the bench line; k3 times "
                    "the reduction of given partials alone; c4/c5 time the NVFP4 expert path of BASELINE configs 4 and 5")
    ap.add_argument("--routing", default="uniform", choices=["uniform", "zipf"])
    ap.add_argument("--shard-of", type=int, default=1, help="profiling aid: run the K shard of a TP=<n> rank on the GPUs "
                    "given (the GEMM of a higher TP degree without its peers)")
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
    (run_gpu if args.workload in ("c2", "k1", "k3") else run_gpu_moe)(args, rank, world)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
