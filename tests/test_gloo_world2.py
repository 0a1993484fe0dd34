"""The N > 1 host logic on CPU: two `gloo` ranks build their Groups over an address-exchanging allocator, shard the
operands, and run the exchange of the reduction (push to the owner, rank-ordered sum, all-gather) as messages, checked
against the single-process oracle. No GPU and no kernel launch is involved."""

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import reduce as red
from oracle import rowpar
from oracle.bf16 import from_torch, to_torch


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class GlooAllocator:
    """CPU stand-in for symmetric memory: every rank allocates its copy and the addresses are all-gathered."""

    def alloc(self, shape, dtype, armed):
        from dlmrt_b200.distributed.parallel import Handle

        t = torch.empty(*shape, dtype=dtype)
        if armed:
            t.view(torch.int16).fill_(-1)
        ptrs = [None] * dist.get_world_size()
        dist.all_gather_object(ptrs, t.data_ptr())
        return t, Handle(ptrs)


def worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from dlmrt_b200 import _lib
        from dlmrt_b200.distributed.parallel import Group

        g = Group(torch.device("cpu"), rank=rank, world=world, allocator=GlooAllocator())
        rows, n, k = 32, 256, 512
        x_bits, w_bits, _ = rowpar.config1(seed=3, m=rows, k=k, n=n, world=world)
        x, w = to_torch(x_bits), to_torch(w_bits)
        xs, ws = g.shard(x, 1), g.shard(w, 1)
        assert xs.shape == (rows, k // world) and torch.equal(xs, x[:, rank * k // world:(rank + 1) * k // world])
        try:
            g.shard(torch.zeros(3, 5), 1)
            raise AssertionError("uneven shard accepted")
        except ValueError:
            pass
        # bookkeeping of two consecutive call sites on one chain
        c1, out1 = g._comm(rows, n, "a", 0, _lib.REDUCE, None, None, 0.0, 1.0)
        g._last[0] = out1
        c2, out2 = g._comm(rows, n, "b", 0, _lib.REDUCE, None, None, 0.0, 1.0)
        assert c1.rank == rank and c1.world == world and c1.rearm is None and c2.rearm == out1.data_ptr()
        assert c2.rearm_bytes == rows * n * 2 and c1.out_peers[rank] == out1.data_ptr()
        everyone = [None] * world
        dist.all_gather_object(everyone, (c1.recv[rank], c1.out_peers[rank]))
        for s in range(world):  # every rank holds every rank's addresses, in rank order
            assert (c1.recv[s], c1.out_peers[s]) == everyone[s]
        try:
            g._last[0] = out2
            g._comm(rows, n, "b", 0, _lib.REDUCE, None, None, 0.0, 1.0)
            raise AssertionError("repeated call site accepted")
        except ValueError:
            pass
        # the exchange itself, as messages: push rows to their owner, sum in rank order, gather
        R = rows // world
        partial = to_torch(rowpar.f32_to_bf16(rowpar.gemm_f32(from_torch(xs), from_torch(ws))))
        pushed = [torch.empty(rows, n // 2, dtype=torch.int32) for _ in range(world)]  # gloo has no all-to-all: every rank
        dist.all_gather(pushed, partial.view(torch.int32))                         # sees all pushes, keeps its rows
        recv = [t[rank * R:(rank + 1) * R].view(torch.bfloat16) for t in pushed]
        mine = to_torch(red.reduce(np.stack([from_torch(t) for t in recv])))
        gathered = [torch.empty(R, n // 2, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, mine.view(torch.int32))
        results[rank] = from_torch(torch.cat(gathered).view(torch.bfloat16))
        # Small plain sums go over one hop: every rank keeps every pushed partial whole and sums all rows itself, in the
        # same rank order, so it must reach the same bits without the gather. Its slots hold whole partials.
        assert c1.one_shot == 1 and g.one_shot(rows, n, _lib.REDUCE) and not g.one_shot(rows, n, _lib.REDUCE_NORM)
        assert g._buffers[f"recv{rows}x{n}.0.all"].shape == (3, world, rows, n)
        one_hop = red.reduce(np.stack([from_torch(t.view(torch.bfloat16)) for t in pushed]))
        assert np.array_equal(one_hop, results[rank])
        g.one_shot_bytes = 0  # and none do when the threshold says so: slots of a row share per sender
        g._last[0] = out1
        c3, _ = g._comm(rows, n, "c", 0, _lib.REDUCE, None, None, 0.0, 1.0)
        assert c3.one_shot == 0 and c3.recv_mc is None and c3.recv[rank] != c1.recv[rank]
        assert g._buffers[f"recv{rows}x{n}.0"].shape == (3, world, R, n)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_oracle():
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(worker, args=(world, free_port(), results), nprocs=world, join=True)
        x_bits, w_bits, _ = rowpar.config1(seed=3, m=32, k=512, n=256, world=world)
        want, _ = rowpar.rowpar(x_bits, w_bits, world)
        assert np.array_equal(results[0], want)
        assert np.array_equal(results[1], results[0])
