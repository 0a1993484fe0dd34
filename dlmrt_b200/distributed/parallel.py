"""Tensor parallelism over the GPUs of one NVSwitch node: the reduction entry point of the row-parallel hot path.

Mirror of the reference's `dlmrt/distributed/parallel.py` (init :34-44, Group :47-180): same names, arguments, buffer
discipline and error behaviour, so model code written against it runs unchanged. What differs is underneath:

  * `Group.reduce` / `Group.reduce_norm` call libdlmrt_b200.so through its C ABI (dlm_reduce_bf16, or dlm_rowpar_bf16
    when the partial's GEMM was deferred, see below) instead of the JIT-built tp_comm extension;
  * the row-parallel GEMM that produces a partial is FUSED into the reduction: `Linear.__call__(x, out=partial)` on a
    buffer obtained from `Group.partial` records the GEMM instead of running it, and the next `Group.reduce*` on that
    buffer launches one kernel that streams the weight shard through tcgen05, pushes finished tiles into the owner
    ranks' receive slots and reduces them (`Group.flush(partial)` materialises the partial if something else wants
    to read it);
  * NCCL is used only to create the process group torch symmetric memory rendezvouses over, as in the reference
    (parallel.py:42-43,73); on a single GPU a `Group.local` (world 1) runs the same kernels over ordinary buffers.

One process per GPU runs the same program; every reduction returns bitwise-identical values on all ranks.
"""

import ctypes as C
import os

import torch

from .. import _lib
from .._lib import DlmComm, DlmGemm, DlmStatus

# Budget of every wait on the device. The reference's kernel gives up after about 30 s and traps (tp_comm.cu:67-70);
# here the kernel records DLM_ERR_TIMEOUT in the group's status words and returns, and the failure is sticky (below).
# Ranks replay their graphs independently, so the budget has to cover the largest host-side skew between ranks.
TIMEOUT_NS = int(os.environ.get("DLMRT_TP_TIMEOUT_NS", 30_000_000_000))
PDL = os.environ.get("DLMRT_PDL", "1") != "0"


def init():
    """The group of this torchrun job (one process per GPU, NCCL only as the bootstrap of symmetric memory), or None
    when WORLD_SIZE is 1. Same contract as the reference's `init` (parallel.py:34-44)."""
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", 1))
    if world == 1:
        return None
    rank = int(os.environ["RANK"])
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(device)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=device)
    return Group(device)


class Handle:
    """What a rendezvous yields: every rank's address of the buffer and its NVLS multicast address (0 if none)."""

    def __init__(self, buffer_ptrs, multicast_ptr=0, torch_handle=None):
        self.buffer_ptrs = list(buffer_ptrs)
        self.multicast_ptr = multicast_ptr
        self.torch_handle = torch_handle  # torch's own symmetric-memory handle (views of peers' copies), if any


class SymmetricAllocator:
    """torch symmetric memory (CUDA VMM handles exchanged over the NCCL-bootstrapped group), parallel.py:61-79."""

    def __init__(self, device, name):
        self.device, self.name = device, name

    def alloc(self, shape, dtype, armed):
        import torch.distributed._symmetric_memory as symm

        with torch.inference_mode(False):  # shared by graphs captured in and out of inference mode
            t = symm.empty(*shape, device=self.device, dtype=dtype)
        if armed:  # every rank finishes arming before the rendezvous lets any rank write into it
            t.view(torch.int16).fill_(-1)
            torch.cuda.synchronize(self.device)
        h = symm.rendezvous(t, self.name)
        return t, Handle(h.buffer_ptrs, h.multicast_ptr if h.multicast_ptr else 0, h)


class LocalAllocator:
    """World 1: the 'symmetric' buffer is an ordinary tensor and its only peer is itself."""

    def __init__(self, device):
        self.device = device

    def alloc(self, shape, dtype, armed):
        with torch.inference_mode(False):
            t = torch.empty(*shape, device=self.device, dtype=dtype)
        if armed:
            t.view(torch.int16).fill_(-1)
        return t, Handle([t.data_ptr()])


class Group:
    def __init__(self, device, rank=None, world=None, allocator=None, max_ctas=0):
        if allocator is None:
            import torch.distributed as dist

            rank, world = dist.get_rank(), dist.get_world_size()
            self.name = dist.group.WORLD.group_name
            allocator = SymmetricAllocator(device, self.name)
        else:
            self.name = "local"
        self.rank, self.world = rank, world
        self.device = device
        self.max_ctas = max_ctas  # cap on every launch's grid (calls on concurrent chains must fit together)
        # Plain sums whose incoming partials total at most this many bytes per rank run as one NVLink hop.
        self.one_shot_bytes = int(os.environ.get("DLMRT_ONE_SHOT_BYTES", 1 << 20))
        self._alloc = allocator
        self._buffers = {}
        self._handles = {}
        self._recv = {}
        self._out_peers = {}
        self._last = {}      # per chain: the previous call's output buffer
        self._pending = {}   # partial data_ptr -> (linear, x): GEMMs deferred into the next reduction
        self._workspaces = {}
        self._gather = {}    # per key: slot addresses, invocation counters, multicast address of the slots
        self.stamps = 0      # device address of a [grid, 8] int64 buffer to record kernel phase times
        self._failed = False  # set by check() on a device time-out; the group must then be rebuilt
        self.status = torch.zeros(_lib.STATUS_WORDS, device=device, dtype=torch.int32)
        _lib.lib()  # fail now, not at the first reduction, when the library is missing

    @classmethod
    def local(cls, device):
        """A world-1 group on one GPU: same kernels, receive slots and output buffers in local memory."""
        return cls(torch.device(device), rank=0, world=1, allocator=LocalAllocator(torch.device(device)))

    def symmetric(self, key, shape, dtype=torch.bfloat16, armed=False):
        """The buffer named `key`, which exists at the same offset on every rank. The first request creates it, which
        is a collective: all ranks must make their first requests in the same order. Later requests return the same
        tensor and must repeat shape and dtype exactly (ValueError otherwise, as parallel.py:76-78).

        `armed` buffers start out as "nothing has arrived": all 16-bit lanes 0xFFFF, written before any peer can
        reach the buffer.
        """
        if key not in self._buffers:
            self._buffers[key], self._handles[key] = self._alloc.alloc(tuple(shape), dtype, armed)
        t = self._buffers[key]
        if tuple(t.shape) != tuple(shape) or t.dtype != dtype:  # never hand out a view the caller may overrun
            raise ValueError(f"symmetric buffer {key}: {tuple(t.shape)} {t.dtype} allocated, {tuple(shape)} {dtype} "
                             "requested")
        return t

    def _handle(self, t):
        for key, buf in self._buffers.items():
            base = buf.data_ptr()
            if base <= t.data_ptr() < base + buf.numel() * buf.element_size():
                return key, self._handles[key]
        raise ValueError("not a symmetric tensor of this group")

    def multicast(self, t):
        """The NVSwitch multicast address that aliases `t` on all ranks at once (one store lands in every copy);
        0 when the node has no multicast support. `t` may be a view into a symmetric buffer (parallel.py:88-93)."""
        handle = self._handle(t)[1]
        if not handle.multicast_ptr:
            return 0
        return handle.multicast_ptr + (t.data_ptr() - handle.buffer_ptrs[self.rank])

    def peer_addresses(self, t):
        """The address of `t` in every rank's copy, as Python ints (what the C ABI takes by value)."""
        handle = self._handle(t)[1]
        offset = t.data_ptr() - handle.buffer_ptrs[self.rank]
        return [p + offset for p in handle.buffer_ptrs]

    def peers(self, t):
        """peer_addresses(t) as an int64 device tensor of `world` entries, the form the reference's extension takes
        (parallel.py:95-102); cached per tensor."""
        key = self._handle(t)[0]
        if (key, t.data_ptr()) not in self._out_peers:
            self._out_peers[key, t.data_ptr()] = torch.tensor(self.peer_addresses(t), device=self.device,
                                                              dtype=torch.int64)
        return self._out_peers[key, t.data_ptr()]

    def _receive(self, rows, n, chain, one_shot=False):
        """Triple-buffered receive slots (symmetric, armed), every rank's slot address, invocation counters and the
        buffer's multicast address. One-shot calls have slots of their own, a whole partial per sender."""
        if (rows, n, chain, one_shot) not in self._recv:
            key = f"recv{rows}x{n}.{chain}" + (".all" if one_shot else "")
            t = self.symmetric(key, (3, self.world, rows if one_shot else rows // self.world, n), armed=True)
            epochs = torch.zeros(_lib.EPOCH_SLOTS, device=self.device, dtype=torch.int32)
            self._recv[rows, n, chain, one_shot] = list(self._handles[key].buffer_ptrs), epochs, self.multicast(t)
        return self._recv[rows, n, chain, one_shot]

    def one_shot(self, rows, n, mode):
        """Whether a reduction runs as one NVLink hop (every rank receives every partial whole and sums all rows
        itself) instead of reduce-scatter + all-gather: plain sums whose incoming partials stay under
        `one_shot_bytes` per rank (32-row blocks). The residual modes keep their residual stream per owner and take
        two hops, unless the caller says the stream is replicated (reduce_norm(..., replicated=True))."""
        return (self.world > 1 and mode == _lib.REDUCE
                and (self.world - 1) * rows * n * 2 <= self.one_shot_bytes)

    def partial(self, site, shape):
        """The destination of row-parallel GEMMs. All call sites get the SAME buffer (the argument `site` only
        documents the caller), hence one shape per group (parallel.py:114-117). A `Linear` that is handed this buffer
        defers its GEMM into the reduction that follows."""
        return self.symmetric("partial", shape)

    # -- deferred GEMMs ---------------------------------------------------------------------------------------------
    def is_partial(self, t):
        """True when `t` is (a leading-rows view of) this group's symmetric memory, i.e. a GEMM into it may be fused
        into the reduction that follows."""
        try:
            self._handle(t)
        except ValueError:
            return False
        return True

    def defer(self, linear, x, out):
        """Record `out = x @ linear.weight^T` instead of running it; the next reduce* of `out` runs it fused."""
        self._pending[out.data_ptr()] = ("linear", linear, x, out)
        return out

    def defer_experts(self, out, down):
        """Record the NVFP4 expert down-projection + combine into `out` (keyword arguments of
        dlmrt_b200.quantization.nvfp4.moe_down) instead of running it; the next reduce* of `out` runs it fused."""
        self._pending[out.data_ptr()] = ("experts", down, None, out)
        return out

    def _run_alone(self, pending):
        kind, what, x, out = pending
        if kind == "linear":
            what.gemm(x, out)
        else:
            from ..quantization import nvfp4

            nvfp4.moe_down(out=out, **what)

    def flush(self, partial):
        """Run a deferred producer on its own, for callers that read the partial before reducing it."""
        pending = self._pending.pop(partial.data_ptr(), None)
        if pending is not None:
            self._run_alone(pending)
        return partial

    def workspace(self, chain, nbytes):
        """Split-K scratch of the fused GEMMs of one chain (FP32 partial tiles + tile counters), grown on demand."""
        ws = self._workspaces.get(chain)
        if ws is None or ws.numel() < nbytes:
            with torch.inference_mode(False):
                ws = torch.zeros(nbytes, device=self.device, dtype=torch.uint8)
            self._workspaces[chain] = ws
        return ws

    # -- launches ---------------------------------------------------------------------------------------------------
    def _comm(self, rows, n, site, chain, mode, h, weight, eps, scale, replicated=False):
        """The DlmComm of one call and its output buffer (the bookkeeping of parallel.py:119-132)."""
        out = self.symmetric(f"out:{site}", (rows, n), armed=True)
        # A replicated residual stream needs every row on every rank: always one hop, whatever the size.
        one_shot = self.one_shot(rows, n, mode) or (replicated and self.world > 1)
        ptrs, epochs, recv_mc = self._receive(rows, n, chain, one_shot)
        last = self._last.get(chain)
        if last is out:  # same wording as parallel.py:124-125: callers may match on it
            raise ValueError(f"call site {site} ran twice in a row; its buffer would never be re-armed")
        c = DlmComm()
        c.rank, c.world, c.rows, c.n, c.mode = self.rank, self.world, rows, n, mode
        c.eps, c.scale = eps, scale
        peers = self.peer_addresses(out)
        for s in range(self.world):
            c.recv[s] = ptrs[s]
            c.out_peers[s] = peers[s]
        c.out = out.data_ptr()
        c.out_mc = self.multicast(out) or None
        # Whatever this chain produced last has been consumed by now: this launch resets it to "not arrived".
        if last is not None:
            c.rearm, c.rearm_bytes = last.data_ptr(), last.numel() * last.element_size()
        c.epochs = epochs.data_ptr()
        c.h = h.data_ptr() if h is not None else None
        c.weight = weight.data_ptr() if weight is not None else None
        c.status = self.status.data_ptr()
        c.stamps = self.stamps or None
        c.timeout_ns = TIMEOUT_NS
        c.pdl = int(PDL)
        c.max_ctas = self.max_ctas
        c.one_shot, c.recv_mc = int(one_shot), (recv_mc or None) if one_shot else None
        return c, out

    def _gemm(self, linear, x, chain):
        g = DlmGemm()
        m, k = x.shape
        if x.stride(1) != 1 or x.dtype != torch.bfloat16:
            raise ValueError("row-parallel input must be BF16 with contiguous K")
        nbytes = _lib.lib().dlm_workspace_bytes(m, linear.n, k)
        ws = self.workspace(chain, nbytes)
        linear.describe(g)
        g.x, g.m, g.n, g.k, g.ldx = x.data_ptr(), m, linear.n, k, x.stride(0)
        g.workspace, g.workspace_bytes = ws.data_ptr(), ws.numel()
        g.splits, g.token_tiles = linear.splits, linear.token_tiles
        return g

    @staticmethod
    def _overlap(a, b):
        """Whether tensors a and b share any byte (by address range)."""
        if a is None or b is None:
            return False
        a0, b0 = a.data_ptr(), b.data_ptr()
        a1 = a0 + ((a.shape[0] - 1) * a.stride(0) + a.shape[1]) * a.element_size() if a.dim() == 2 else \
            a0 + a.numel() * a.element_size()
        b1 = b0 + b.numel() * b.element_size()
        return a0 < b1 and b0 < a1

    def _launch(self, mode, partial, h, weight, site, eps=0.0, scale=1.0, chain=0, replicated=False):
        if self._failed:
            raise RuntimeError("this group reported a device time-out: its buffers may hold stale arrivals; build a new "
                               "Group before reducing again")
        rows, n = partial.shape
        last = self._last.get(chain)
        comm, out = self._comm(rows, n, site, chain, mode, h, weight, eps, scale, replicated)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        pending = self._pending.pop(partial.data_ptr(), None)
        # The fused kernel re-arms `last` and fills `out` while other CTAs still load the GEMM's input; an input that
        # IS one of those (a projection fed straight from the previous reduction) therefore runs as two kernels, the
        # order the reference has anyway.
        fusable = pending is not None and n <= _lib.FUSED_MAX_N and not self._overlap(pending[2], last) \
            and not self._overlap(pending[2], out)
        if fusable and pending[0] == "linear":
            gemm = self._gemm(pending[1], pending[2], chain)
            _lib.check(_lib.lib().dlm_rowpar_bf16(C.byref(gemm), C.byref(comm), stream), f"rowpar {site}")
        elif fusable:  # the experts' down-projection + combine (+ shared) in front of the same reduction
            from ..quantization import nvfp4

            down = dict(pending[1])
            shared = down.pop("shared", None)
            m = nvfp4.descriptor(shared=shared, **down)
            _lib.check(_lib.lib().dlm_rowpar_nvfp4_moe(C.byref(m), C.byref(comm), stream), f"experts {site}")
        else:
            if pending is not None:
                self._run_alone(pending)
            _lib.check(_lib.lib().dlm_reduce_bf16(partial.data_ptr(), C.byref(comm), stream), f"reduce {site}")
        self._last[chain] = out
        return out

    def reduce_norm(self, partial, h, weight, eps, scale=1.0, *, site, chain=0, replicated=False):
        """All-reduce `partial`, then RMSNorm, in one launch; every rank gets the same [rows, n] result
        (same arguments as parallel.py:134-143, plus `replicated`).

        h given:  v = bf16(sum) + h; this rank's rows of `h` become bf16(v) (each rank keeps only its own rows of
                  the residual stream current); returns rmsnorm(v) * weight * scale.
        h None:   returns rmsnorm(bf16(sum)) * weight * scale.
        replicated (with h): every rank holds the WHOLE residual stream and all its rows are updated on every rank:
                  the pair `reduce` -> `rmsnorm(h, weight, delta=reduced)` of LLaDA2's layers
                  (dlmrt/models/llada2/model.py:435-439, dlmrt/ops/triton/core.py:29-56) as one launch. Every rank then
                  receives every partial whole and sums all rows itself (one NVLink hop).

        The returned tensor is the buffer of call site `site`; it stays valid until the NEXT call on `chain`, whose
        launch resets it. Calls on one chain must be stream-ordered; calls that can overlap in time (two streams)
        must use different chains.
        """
        mode = _lib.REDUCE_NORM_RESIDUAL if h is not None else _lib.REDUCE_NORM
        return self._launch(mode, partial, h, weight, site, eps, scale, chain, replicated and h is not None)

    def reduce(self, partial, *, site, chain=0):
        """All-reduce (sum) of `partial` into the buffer of call site `site`, identical bits on every rank
        (parallel.py:145-147). Buffer lifetime and chain rules as for reduce_norm."""
        return self._launch(_lib.REDUCE, partial, None, None, site, chain=chain)

    def shard(self, t, dim=0):
        if t.shape[dim] % self.world:
            raise ValueError(f"Dimension {dim} of {tuple(t.shape)} does not split over {self.world} ranks")
        return t.chunk(self.world, dim)[self.rank].contiguous()

    def check(self):
        """Read the device status words (synchronises the current stream); raises TimeoutError when a wait ran out.
        The kernels make such a failure sticky (later calls exchange nothing), and so does the host: after the error
        the group refuses further reductions, because slots may hold late arrivals of the failed call. Call this
        wherever the host synchronises anyway (end of a block, end of a request)."""
        st = DlmStatus()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(_lib.lib().dlm_status_read(self.status.data_ptr(), C.byref(st), stream), "status")
        if st.code:
            self._failed = True
            where = f"rank slot {st.slot}, phase {st.phase}, invocation {st.epoch}"
            if st.phase == 3 and st.epoch >> 24:  # the dense kernel's own pipeline: who gave up, and at which k-block
                who = ("producer", "MMA issuer", "epilogue", "split-K rendezvous")[(st.epoch >> 24) & 3]
                where = f"pipeline stage or split {st.slot}: {who} gave up at k-block {st.epoch & 0xFFFF}"
            raise TimeoutError(f"rank {self.rank}: {_lib.lib().dlm_strerror(st.code).decode()} (block {st.block}, {where})")

    def all_reduce_(self, x):
        """The reference's UNFUSED switch (DLMRT_TP_FUSED=0, parallel.py:154-162), kept so model code that still calls
        it runs: in-place sum of a symmetric tensor through the same torch symmetric-memory operators the reference
        uses. Nothing on the fused path calls it."""
        if self.world == 1:
            return x
        if self.multicast(x):
            torch.ops.symm_mem.multimem_all_reduce_(x, "sum", self.name)
        else:
            torch.ops.symm_mem.two_shot_all_reduce_(x, "sum", self.name)
        return x

    # Payloads the gather kernel can tell from "not arrived": arithmetic never produces an all-ones 32-bit word in these.
    GATHER_DTYPES = (torch.float32, torch.float16, torch.bfloat16)

    def all_gather(self, x, key):
        """[world, *x.shape]: every rank's `x` in rank order (parallel.py:164-180). This is the other collective of a
        round (row statistics of the decoders) and runs on this library's barrier-free kernel only (`dlm_all_gather`:
        multicast stores into triple-buffered slots, arrival detected in band). The kernel needs a contiguous FP32 /
        FP16 / BF16 block of 16..1 MiB bytes, a multiple of 16; anything else is a ValueError rather than a silent
        detour through another backend."""
        nbytes = x.numel() * x.element_size()
        if x.dtype not in self.GATHER_DTYPES or not x.is_contiguous() or nbytes % 16 or not 0 < nbytes <= _lib.GATHER_MAX_BYTES:
            raise ValueError(f"all_gather {key}: needs a contiguous float32/float16/bfloat16 block whose size is a multiple "
                             f"of 16 bytes, at most {_lib.GATHER_MAX_BYTES}; got {tuple(x.shape)} {x.dtype}")
        if self._failed:
            raise RuntimeError("this group reported a device time-out; build a new Group")
        out = self.symmetric(key, (self.world, *x.shape), x.dtype)
        if key not in self._gather:
            slots = self.symmetric(key + ".slots", (3, self.world, nbytes // 2), armed=True)
            epochs = torch.zeros(_lib.EPOCH_SLOTS, device=self.device, dtype=torch.int32)
            self._gather[key] = list(self._handles[key + ".slots"].buffer_ptrs), epochs, self.multicast(slots)
        ptrs, epochs, recv_mc = self._gather[key]
        c = DlmComm()
        c.rank, c.world = self.rank, self.world
        for s in range(self.world):
            c.recv[s] = ptrs[s]
        c.recv_mc = recv_mc or None
        c.out, c.epochs, c.status = out.data_ptr(), epochs.data_ptr(), self.status.data_ptr()
        c.timeout_ns, c.pdl, c.max_ctas = TIMEOUT_NS, int(PDL), self.max_ctas
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(_lib.lib().dlm_all_gather(x.data_ptr(), nbytes, C.byref(c), stream), f"all_gather {key}")
        return out
