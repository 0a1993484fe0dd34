"""One rank of the real multi-GPU parity run (launched by tests/test_multigpu.py through torch.distributed.run):
stand-alone reductions and fused projections over symmetric memory, checked bit for bit against the CPU oracle fed
with the all-gathered inputs, and for identity across ranks; first call by call with a host synchronisation after
each, then as a CUDA graph of back-to-back calls replayed without any (graph_section)."""

import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from gpu_util import assert_norm_close, assert_same_bits, bits, randn_bf16  # noqa: E402
from oracle import reduce as red  # noqa: E402


def gather(t):
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return out


def graph_section(group):
    """What the design is for, value-checked on real NVLink: back-to-back calls with NO host synchronisation and no
    NCCL in between, captured once in a CUDA graph and replayed. Twenty calls per pass: plain sums and residual +
    RMSNorm on alternating call sites, the fused GEMM in both modes, a one-hop chain of 32-row blocks and the
    all-gather of row statistics, so that triple-buffered slots, cross-call re-arming, programmatic dependent launch and
    the multicast stores all run the way a denoise round runs them. After several replays the final outputs and the
    residual stream must equal the oracle fed with the same sequence, and be identical on every rank."""
    from dlmrt_b200.layers.linear import Linear

    rank, world, dev = group.rank, group.world, group.device
    rows, n, k = 64, 2048, 512
    weight = randn_bf16(n, seed=41, std=0.1, device=dev) + 1
    h = randn_bf16(rows, n, seed=42, device=dev)
    given = [randn_bf16(rows, n, seed=300 + 10 * i + rank, device=dev) for i in range(4)]
    small = [randn_bf16(32, n, seed=400 + 10 * i + rank, device=dev) for i in range(2)]
    stats = torch.randn(32, 4, generator=torch.Generator().manual_seed(500 + rank)).to(dev)
    g = torch.Generator().manual_seed(600 + rank)
    x = torch.randint(-3, 4, (rows, k), generator=g).to(torch.bfloat16).to(dev)
    w = torch.randint(-2, 3, (n, k), generator=g).to(torch.bfloat16).to(dev)
    lin = Linear(w, group=group)
    own = (x.float() @ w.float().t()).to(torch.bfloat16)  # exact integers, one BF16 rounding: this rank's partial
    partial = group.symmetric("graph.partial", (rows, n))
    assert group.one_shot(32, n, 0) and not group.one_shot(rows, n, 2)

    def one_pass():
        o = {}
        group.reduce_norm(given[0], h, weight, 1e-6, site="g.a")
        group.reduce(lin(x, out=partial), site="g.b")
        group.reduce_norm(given[1], h, weight, 1e-6, site="g.a")
        group.reduce(small[0], site="g.s0", chain=32)
        group.reduce_norm(lin(x, out=partial), h, weight, 1e-6, site="g.b")
        o["stats"] = group.all_gather(stats, "g.stats")
        group.reduce(given[2], site="g.a")
        o["small"] = group.reduce(small[1], site="g.s1", chain=32)
        group.reduce_norm(given[3], None, weight, 1e-6, 0.5, site="g.b")
        group.reduce(lin(x, out=partial), site="g.a")
        o["last"] = group.reduce_norm(given[0], h, weight, 1e-6, site="g.b")
        return o

    h_start = np.stack([bits(t) for t in gather(h)])
    parts = {name: np.stack([bits(t) for t in gather(t_)]) for name, t_ in
             [("g0", given[0]), ("g1", given[1]), ("g2", given[2]), ("g3", given[3]), ("s1", small[1]), ("own", own)]}
    stats_all = torch.stack(gather(stats)).cpu()
    replays = 5
    stream = torch.cuda.Stream(dev)
    with torch.cuda.stream(stream):
        for _ in range(2):
            out = one_pass()
        stream.synchronize()
        group.check()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = one_pass()
        for _ in range(replays):
            graph.replay()
        stream.synchronize()
    group.check()
    # the oracle, fed with the same sequence: only the residual-stream calls carry state from pass to pass
    hs, want_last = h_start, None
    for _ in range(2 + replays):  # two eager passes and the replays (capturing launches nothing)
        for name in ("g0", "g1", "own", "g0"):
            want_last, hs = red.reduce_norm(parts[name], bits(weight), 1e-6, 1.0, hs)
    assert_same_bits(bits(h), hs[rank], "graph: residual stream after the replays")
    assert_norm_close(bits(out["last"]), want_last, "graph: last residual + RMSNorm output")
    assert_same_bits(bits(out["small"]), red.reduce(parts["s1"]), "graph: one-hop sum")
    assert torch.equal(out["stats"].cpu().view(torch.int32), stats_all.view(torch.int32)), "graph: all_gather"
    for name in ("last", "small"):
        for r, other in enumerate(gather(out[name])):
            assert_same_bits(bits(other), bits(out[name]), f"graph: {name} of rank {r} vs rank {rank}")


def main():
    from dlmrt_b200.distributed import parallel
    from dlmrt_b200.layers.linear import Linear

    parallel.TIMEOUT_NS = 2_000_000_000
    group = parallel.init()
    rank, world, dev = group.rank, group.world, group.device
    report = {"multicast": bool(group.multicast(group.symmetric("probe", (8, 256), armed=True)))}
    rows, n = 256, 2560
    weight = randn_bf16(n, seed=5, std=0.1, device=dev) + 1
    h = randn_bf16(rows, n, seed=6, device=dev)  # same start on every rank; each rank updates its own rows
    for i in range(9):
        mode = i % 3
        p = randn_bf16(rows, n, seed=100 * i + rank, device=dev)
        all_p = np.stack([bits(t) for t in gather(p)])
        h_all = np.stack([bits(t) for t in gather(h)])
        site = f"s{i % 2}.{mode}"
        if mode == 0:
            out = group.reduce(p, site=site)
            want = red.reduce(all_p)
        elif mode == 1:
            out = group.reduce_norm(p, None, weight, 1e-6, 0.75, site=site)
            want, _ = red.reduce_norm(all_p, bits(weight), 1e-6, 0.75)
        else:
            out = group.reduce_norm(p, h, weight, 1e-6, site=site)
            want, h_after = red.reduce_norm(all_p, bits(weight), 1e-6, 1.0, h_all)
        torch.cuda.synchronize()
        group.check()
        got = bits(out)
        for r, other in enumerate(gather(out)):
            assert_same_bits(bits(other), got, f"reduce {i}: rank {r} vs rank {rank}")
        (assert_same_bits if mode == 0 else assert_norm_close)(got, want, f"reduce {i} mode {mode}")
        if mode == 2:
            assert_same_bits(bits(h), h_after[rank], f"reduce {i}: residual")
    # fused projection + reduction, integer operands: exact end to end
    for i, (m, k_total) in enumerate([(256, 4096), (256, 9728 // 8 * 8), (32, 2048)]):
        g = torch.Generator().manual_seed(7 + i)
        x = torch.randint(-3, 4, (m, k_total), generator=g).to(torch.bfloat16)
        w = torch.randint(-2, 3, (n, k_total), generator=g).to(torch.bfloat16)
        if k_total % (64 * world):
            continue
        xs, ws = group.shard(x, 1).to(dev), group.shard(w, 1).to(dev)
        lin = Linear(ws, group=group)
        for rep in range(3):
            p = lin(xs, out=group.symmetric(f"partial{m}", (m, n)))
            out = group.reduce(p, site=f"f{i}.{rep % 2}", chain=m)
            torch.cuda.synchronize()
            group.check()
            want = (x.float() @ w.float().t())
            parts = [x.chunk(world, 1)[r].float() @ w.chunk(world, 1)[r].float().t() for r in range(world)]
            want = red.reduce(np.stack([bits(t.to(torch.bfloat16)) for t in parts]))
            assert_same_bits(bits(out), want, f"fused {i}.{rep}")
            for r, other in enumerate(gather(out)):
                assert_same_bits(bits(other), bits(out), f"fused {i}.{rep}: rank {r} vs rank {rank}")
    # NVFP4 experts split whole across the ranks (expert parallel), exact operands: bit-exact end to end
    from test_moe_gpu import device_args, make_case, oracle_out
    from dlmrt_b200.quantization import nvfp4

    case = make_case(32, 2048, 512, 64, 8, seed=11, exact=True)
    e_local = 64 // world
    args = device_args(case, rank * e_local, e_local, dev)
    want = red.reduce(np.stack([oracle_out(case, r * e_local, e_local)[0] for r in range(world)]))
    one_hop, default_limit = 0, group.one_shot_bytes
    for limit in (default_limit, 0):  # 32 rows: one NVLink hop by default; then forced onto the two-hop protocol
        group.one_shot_bytes = limit
        one_hop += int(group.one_shot(32, 2048, 0))
        for rep in range(3):
            out = nvfp4.moe_down(out=None, group=group, site=f"moe.{limit}.{rep % 2}", chain=32, **args)
            torch.cuda.synchronize()
            group.check()
            assert_same_bits(bits(out), want, f"moe {rep} (one-shot limit {limit})")
            for r, other in enumerate(gather(out)):
                assert_same_bits(bits(other), bits(out), f"moe {rep}: rank {r} vs rank {rank}")
        # the reduction of given small partials, same two ways
        for rep in range(3):
            p = randn_bf16(32, 2048, seed=900 + 10 * rep + rank, device=dev)
            all_p = np.stack([bits(t) for t in gather(p)])
            out = group.reduce(p, site=f"small.{limit}.{rep % 2}", chain=33)
            torch.cuda.synchronize()
            group.check()
            assert_same_bits(bits(out), red.reduce(all_p), f"small reduce {rep} (one-shot limit {limit})")
    assert one_hop == 1
    group.one_shot_bytes = default_limit
    # the round's other collective: all-gather of row statistics, several invocations per key
    for key, shape in (("row_stats", (32, 4)), ("logit_stats", (256, 2))):
        for call in range(4):
            stats = torch.randn(*shape, generator=torch.Generator().manual_seed(50 * call + rank)).to(dev)
            got = group.all_gather(stats, key)
            torch.cuda.synchronize()
            group.check()
            want = torch.stack([t.to(dev) for t in gather(stats)])
            assert torch.equal(got.view(torch.int32), want.view(torch.int32)), f"all_gather {key} call {call}"
    graph_section(group)
    dist.barrier()
    if rank == 0:
        print(f"MULTIGPU_OK world={world} multicast={report['multicast']}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
