"""The fused kernels inside the device-side loop of a block: begin -> WHILE(remaining and step < limit){round} -> commit
(dlmrt/ops/csrc/block_graph.cu:29-77, built as in dlmrt/models/sdar/engine.py:92-120). A round of fused projections is
captured once and re-executed by a conditional WHILE node; since the kernels keep their state (invocation counters,
split-K generations, armed buffers) in device memory, the loop must give bit for bit what the same rounds give when
launched one by one from the host."""

import numpy as np
import pytest
import torch

from gpu_util import assert_same_bits, bits, randn_bf16

pytestmark = pytest.mark.gpu


class Block:
    """A synthetic block: two fused projection + residual + RMSNorm launches per round, output fed back as input."""

    def __init__(self, m=32, n=2048):
        from dlmrt_b200.distributed.parallel import Group
        from dlmrt_b200.layers.linear import Linear

        self.m, self.n = m, n
        self.g = Group.local("cuda:0")
        self.lin = [Linear(randn_bf16(n, n, seed=60 + i, std=0.02), fp8=False, group=self.g) for i in range(2)]
        self.norm = [randn_bf16(n, seed=70 + i, std=0.1) + 1 for i in range(2)]
        self.x0, self.h0 = randn_bf16(m, n, seed=80), randn_bf16(m, n, seed=81)
        self.x, self.h = self.x0.clone(), self.h0.clone()
        self.final = torch.zeros_like(self.x)
        self.rounds = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.remaining = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.step = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.extra = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.flag = torch.zeros(1, dtype=torch.int32, device="cuda")

    def reset(self, rounds):
        self.x.copy_(self.x0)
        self.h.copy_(self.h0)
        self.final.zero_()
        self.extra.zero_()
        self.rounds.fill_(rounds)

    def begin(self):
        self.step.zero_()
        self.remaining.copy_(self.rounds)

    def round(self):
        g, (m, n) = self.g, (self.m, self.n)
        o = g.reduce_norm(self.lin[0](self.x, out=g.partial("a", (m, n))), self.h, self.norm[0], 1e-6, site="a")
        o = g.reduce_norm(self.lin[1](o, out=g.partial("b", (m, n))), self.h, self.norm[1], 1e-6, site="b")
        self.x.copy_(o)
        self.remaining.sub_(1)
        self.step.add_(1)

    def commit(self):
        self.final.copy_(self.x)

    def mark(self):
        self.extra.add_(1)

    def capture(self, names):
        """Each stage runs twice eagerly, then is captured with its graph kept (sdar/engine.py:103-111)."""
        graphs = {}
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for name in names:
                fn = getattr(self, name)
                fn()
                fn()
                graph = torch.cuda.CUDAGraph(keep_graph=True)
                with torch.cuda.graph(graph, stream=stream):
                    fn()
                graphs[name] = graph
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        return graphs

    def eager(self, rounds, limit):
        self.reset(rounds)
        self.begin()
        for _ in range(min(rounds, limit)):
            self.round()
        self.commit()
        torch.cuda.synchronize()
        self.g.check()
        return bits(self.final), bits(self.h)


@pytest.mark.parametrize("rounds, limit", [(5, 32), (100, 3), (0, 32), (1, 1)])
def test_block_graph_runs_fused_rounds_on_the_device(rounds, limit):
    from dlmrt_b200 import _lib
    from dlmrt_b200.ops.block_graph import BlockGraph

    b = Block()
    graphs = b.capture(["begin", "round", "commit"])
    want_final, want_h = b.eager(rounds, limit)
    block = BlockGraph(graphs["begin"].raw_cuda_graph(), graphs["round"].raw_cuda_graph(),
                       graphs["commit"].raw_cuda_graph(), b.remaining.data_ptr(), b.step.data_ptr(), limit)
    for _ in range(2):  # a block graph is replayed once per block
        b.reset(rounds)
        before = _lib.lib().dlm_launch_count()
        block.replay(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert _lib.lib().dlm_launch_count() == before  # every fused launch was issued by the device loop
        b.g.check()
        assert int(b.step.item()) == min(rounds, limit)
        assert int(b.remaining.item()) == rounds - min(rounds, limit)
        assert_same_bits(bits(b.final), want_final, "final activations")
        assert_same_bits(bits(b.h), want_h, "residual stream")
    assert not np.array_equal(want_final, bits(b.x0)) or min(rounds, limit) == 0


def test_loop_graph_and_staged_parts():
    """Two loops in sequence over the same round, then a body with a flagged part that runs only while its flag is
    positive (block_graph.cu:80-129, :137-207)."""
    from dlmrt_b200.ops.block_graph import LoopGraph, StagedLoopGraph

    b = Block()
    graphs = b.capture(["begin", "round", "commit", "mark"])
    raw = {k: v.raw_cuda_graph() for k, v in graphs.items()}
    stream = torch.cuda.current_stream().cuda_stream
    want_final, want_h = b.eager(4, 32)

    # begin -> loop A (limit 3 stops it) -> loop B (remaining stops it) -> commit: 3 + 1 rounds of 4.
    loops = LoopGraph(raw["begin"], [(raw["round"], b.remaining.data_ptr(), b.step.data_ptr(), 3),
                                     (raw["round"], b.remaining.data_ptr(), b.step.data_ptr(), 32)], raw["commit"])
    b.reset(4)
    loops.replay(stream)
    torch.cuda.synchronize()
    b.g.check()
    assert int(b.step.item()) == 4 and int(b.remaining.item()) == 0
    assert_same_bits(bits(b.final), want_final, "two loops")
    assert_same_bits(bits(b.h), want_h, "two loops: residual stream")

    staged = StagedLoopGraph(raw["begin"], [(raw["round"], 0), (raw["mark"], b.flag.data_ptr())],
                             b.remaining.data_ptr(), b.step.data_ptr(), 32)
    for flag, marks in ((0, 0), (1, 4)):
        b.reset(4)
        b.flag.fill_(flag)
        staged.replay(stream)
        b.commit()
        torch.cuda.synchronize()
        b.g.check()
        assert int(b.extra.item()) == marks
        assert_same_bits(bits(b.final), want_final, f"staged, flag {flag}")


def test_a_body_that_never_advances_cannot_spin():
    """`limit` also caps the passes of one execution: a body that forgets to advance *step ends after `limit` passes."""
    from dlmrt_b200.ops.block_graph import LoopGraph

    b = Block()
    graphs = b.capture(["mark"])
    b.extra.zero_()
    b.remaining.fill_(1)
    b.step.zero_()
    loop = LoopGraph(0, [(graphs["mark"].raw_cuda_graph(), b.remaining.data_ptr(), b.step.data_ptr(), 7)], 0)
    loop.replay(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert int(b.extra.item()) == 7
