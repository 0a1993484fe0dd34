"""The per-block device loop: begin -> WHILE(remaining and step < limit){round} -> commit, one launch per block.

Mirror of the classes of the reference's block-graph extension (`dlmrt/ops/csrc/block_graph.cu`, obtained there through
`dlmrt.ops.extensions.block_graph()`): same constructor arguments (raw `cudaGraph_t` values from
`torch.cuda.CUDAGraph(keep_graph=True).raw_cuda_graph()`, device pointers of the int32 loop words) and the same
`replay(stream)` call, so `Engine._capture` (`dlmrt/models/sdar/engine.py:92-120`) can build its blocks from this
module unchanged. All three are one C-ABI program (`dlm_device_loop_create`): a head graph, a list of loops whose
bodies are lists of parts, and a tail graph.
"""

import ctypes as C

from .. import _lib
from .._lib import DlmLoop, DlmLoopPart


class _DeviceLoop:
    """Owns one DlmDeviceLoop. `loops`: [(parts, remaining_ptr, step_ptr, limit)], parts: [(graph, flag_ptr or 0)]."""

    def __init__(self, head, loops, tail):
        if len(loops) > _lib.MAX_LOOPS:
            raise ValueError(f"at most {_lib.MAX_LOOPS} loops, got {len(loops)}")
        array = (DlmLoop * max(len(loops), 1))()
        keep = []
        for slot, (parts, remaining, step, limit) in zip(array, loops):
            if not 1 <= len(parts) <= _lib.MAX_LOOP_PARTS:
                raise ValueError(f"a loop body has 1..{_lib.MAX_LOOP_PARTS} parts, got {len(parts)}")
            body = (DlmLoopPart * len(parts))()
            for p, (graph, flag) in zip(body, parts):
                p.graph, p.flag = graph or None, flag or None
            keep.append(body)
            slot.parts, slot.n_parts, slot.limit = body, len(parts), int(limit)
            slot.remaining, slot.step = remaining or None, step or None
        self._handle = C.c_void_p()
        _lib.check(_lib.lib().dlm_device_loop_create(head or None, array, len(loops), tail or None,
                                                     C.byref(self._handle)), type(self).__name__)

    def replay(self, stream):
        """Launches the whole program on `stream` (a raw cudaStream_t, as `torch.cuda.Stream.cuda_stream`)."""
        _lib.check(_lib.lib().dlm_device_loop_launch(self._handle, stream), f"{type(self).__name__}.replay")

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            try:
                _lib.lib().dlm_device_loop_destroy(handle)
            except Exception:  # interpreter shutdown
                pass


class BlockGraph(_DeviceLoop):
    """begin -> WHILE(*remaining > 0 and *step < limit){round} -> commit (block_graph.cu:29-77)."""

    def __init__(self, begin, round, commit, remaining_ptr, step_ptr, limit):
        super().__init__(begin, [([(round, 0)], remaining_ptr, step_ptr, limit)], commit)


class LoopGraph(_DeviceLoop):
    """begin -> WHILE(..){body_0} -> WHILE(..){body_1} -> ... -> tail; `loops` = [(body graph, remaining pointer, step
    pointer, limit)], `tail` may be 0 (block_graph.cu:80-129)."""

    def __init__(self, begin, loops, tail):
        super().__init__(begin, [([(body, 0)], remaining, step, limit) for body, remaining, step, limit in loops], tail)


class StagedLoopGraph(_DeviceLoop):
    """head -> WHILE(*run > 0 and *step < limit){part_0 -> part_1 -> ...}; `parts` = [(graph, flag pointer or 0)], a
    part with a flag runs only in passes where *flag > 0 (block_graph.cu:137-207)."""

    def __init__(self, head, parts, run_ptr, step_ptr, limit):
        super().__init__(head, [(list(parts), run_ptr, step_ptr, limit)], 0)
