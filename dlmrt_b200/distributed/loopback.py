"""Several tensor-parallel ranks on ONE GPU, for testing the multi-rank protocol where only one GPU is at hand.

Kernels that wait on one another must never run as separate launches on one GPU (nothing guarantees they run at the
same time), so a `LoopbackWorld` runs all ranks of a collective in a single cooperative launch
(dlm_reduce_bf16_loopback / dlm_rowpar_bf16_loopback): the grid's y index selects the rank, every rank has its own
buffers on the same device, "peer" addresses are simply the other ranks' buffers, and there is no multicast, so the
all-gather uses one store per rank. Each rank is an ordinary `Group`, with the same bookkeeping as on real GPUs.
"""

import ctypes as C

import torch

from .. import _lib
from .._lib import DlmComm, DlmGemm, DlmMoe
from .parallel import Group, Handle


class _SharedAllocator:
    """Allocates every rank's copy of a buffer on one device; rank i's view of a key is copy i."""

    def __init__(self, nranks, device):
        self.nranks, self.device = nranks, device
        self._cursor = [0] * nranks
        self._made = []

    def view(self, rank):
        return _RankView(self, rank)

    def alloc(self, rank, shape, dtype, armed):
        i = self._cursor[rank]
        self._cursor[rank] += 1
        if i == len(self._made):  # first rank to ask creates all copies (ranks allocate in the same order)
            copies = [torch.empty(*shape, device=self.device, dtype=dtype) for _ in range(self.nranks)]
            if armed:
                for t in copies:
                    t.view(torch.int16).fill_(-1)
            self._made.append((tuple(shape), dtype, copies))
        made_shape, made_dtype, copies = self._made[i]
        if made_shape != tuple(shape) or made_dtype != dtype:
            raise ValueError("ranks must allocate symmetric buffers in the same order with the same shapes")
        return copies[rank], Handle([t.data_ptr() for t in copies])


class _RankView:
    def __init__(self, shared, rank):
        self.shared, self.rank = shared, rank

    def alloc(self, shape, dtype, armed):
        return self.shared.alloc(self.rank, shape, dtype, armed)


class LoopbackWorld:
    def __init__(self, nranks, device="cuda:0", max_ctas=0, one_shot_bytes=None):
        self.device = torch.device(device)
        self.world = nranks
        shared = _SharedAllocator(nranks, self.device)
        self.groups = [Group(self.device, rank=r, world=nranks, allocator=shared.view(r), max_ctas=max_ctas)
                       for r in range(nranks)]
        if one_shot_bytes is not None:  # 0: always reduce-scatter + all-gather; large: one hop wherever allowed
            for g in self.groups:
                g.one_shot_bytes = one_shot_bytes

    def _mode(self, hs, weight):
        if weight is None:
            return _lib.REDUCE
        return _lib.REDUCE_NORM_RESIDUAL if hs is not None else _lib.REDUCE_NORM

    def _comms(self, rows, n, site, chain, hs, weight, eps, scale, replicated=False):
        comms = (DlmComm * self.world)()
        outs = []
        mode = self._mode(hs, weight)
        for r, g in enumerate(self.groups):
            c, out = g._comm(rows, n, site, chain, mode, hs[r] if hs is not None else None, weight, eps, scale,
                             replicated and hs is not None)
            c.pdl = 0
            comms[r] = c
            outs.append(out)
        return comms, outs

    def _done(self, chain, outs):
        for g, out in zip(self.groups, outs):
            g._last[chain] = out

    def reduce(self, partials, *, site, chain=0, hs=None, weight=None, eps=0.0, scale=1.0, replicated=False):
        """All ranks of Group.reduce / reduce_norm in one launch; partials[r] is rank r's [rows, n] partial.
        Returns every rank's output buffer."""
        rows, n = partials[0].shape
        comms, outs = self._comms(rows, n, site, chain, hs, weight, eps, scale, replicated)
        ptrs = (C.c_void_p * self.world)(*[p.data_ptr() for p in partials])
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(_lib.lib().dlm_reduce_bf16_loopback(ptrs, comms, self.world, stream), f"loopback reduce {site}")
        self._done(chain, outs)
        return outs

    def rowpar(self, xs, ws, *, site, chain=0, hs=None, weight=None, eps=0.0, scale=1.0, splits=0, token_tiles=0,
               replicated=False):
        """All ranks of the fused projection + reduction in one launch: xs[r] [m, k_r], ws[r] [n, k_r]."""
        m, n = xs[0].shape[0], ws[0].shape[0]
        comms, outs = self._comms(m, n, site, chain, hs, weight, eps, scale, replicated)
        gemms = (DlmGemm * self.world)()
        for r, g in enumerate(self.groups):
            x, w = xs[r], ws[r]
            nbytes = _lib.lib().dlm_workspace_bytes(m, n, x.shape[1])
            scratch = g.workspace(chain, nbytes)
            gm = DlmGemm()
            gm.x, gm.w, gm.m, gm.n, gm.k = x.data_ptr(), w.data_ptr(), m, n, x.shape[1]
            gm.ldx, gm.ldw = x.stride(0), w.stride(0)
            gm.workspace, gm.workspace_bytes, gm.splits = scratch.data_ptr(), scratch.numel(), splits
            gm.token_tiles = token_tiles
            gemms[r] = gm
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(_lib.lib().dlm_rowpar_bf16_loopback(gemms, comms, self.world, stream), f"loopback rowpar {site}")
        self._done(chain, outs)
        return outs

    def all_gather(self, xs, key):
        """All ranks of Group.all_gather in one launch; xs[r] is rank r's block. Returns every rank's [world, ...]."""
        nbytes = xs[0].numel() * xs[0].element_size()
        comms = (DlmComm * self.world)()
        outs = []
        for r, g in enumerate(self.groups):
            out = g.symmetric(key, (self.world, *xs[r].shape), xs[r].dtype)
            if key not in g._gather:
                g.symmetric(key + ".slots", (3, self.world, nbytes // 2), armed=True)
                epochs = torch.zeros(_lib.EPOCH_SLOTS, device=self.device, dtype=torch.int32)
                g._gather[key] = list(g._handles[key + ".slots"].buffer_ptrs), epochs, 0
            ptrs, epochs, _ = g._gather[key]
            c = DlmComm()
            c.rank, c.world = r, self.world
            for s in range(self.world):
                c.recv[s] = ptrs[s]
            c.out, c.epochs, c.status = out.data_ptr(), epochs.data_ptr(), g.status.data_ptr()
            c.timeout_ns, c.max_ctas = 500_000_000, g.max_ctas
            comms[r] = c
            outs.append(out)
        ptrs = (C.c_void_p * self.world)(*[x.data_ptr() for x in xs])
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(_lib.lib().dlm_all_gather_loopback(ptrs, nbytes, comms, self.world, stream), f"loopback all_gather {key}")
        return outs

    def moe(self, descriptors, *, site, chain=0, hs=None, weight=None, eps=0.0, scale=1.0, replicated=False):
        """All ranks of the fused NVFP4 expert down-projection + reduction in one launch; descriptors[r] is rank r's
        DlmMoe (dlmrt_b200.quantization.nvfp4.descriptor)."""
        comms, outs = self._comms(descriptors[0].m, descriptors[0].n, site, chain, hs, weight, eps, scale, replicated)
        moes = (DlmMoe * self.world)(*descriptors)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(_lib.lib().dlm_rowpar_nvfp4_moe_loopback(moes, comms, self.world, stream), f"loopback moe {site}")
        self._done(chain, outs)
        return outs

    def check(self):
        for g in self.groups:
            g.check()
