"""The C-ABI library loads, exports every symbol include/dlmrt_b200.h declares, and rejects bad arguments with the
documented codes before touching a GPU (host-side checks of tp_comm.cu:282-287 as return codes)."""

import ctypes as C
import re
from pathlib import Path

import pytest

from dlmrt_b200 import _lib
from dlmrt_b200._lib import DlmComm, DlmGemm

HEADER = Path(__file__).resolve().parent.parent / "include" / "dlmrt_b200.h"


def declared():
    return re.findall(r"^DLM_API\s+[\w\s\*]+?\b(dlm_\w+)\(", HEADER.read_text(), flags=re.M)


def test_every_declared_symbol_is_exported_and_bound():
    names = declared()
    assert len(names) >= 14
    handle = C.CDLL(str(_lib.LIB_PATH))
    for name in names:
        assert hasattr(handle, name), name
        assert name in _lib.SIGNATURES, f"{name} is not bound in dlmrt_b200._lib"
    assert set(_lib.SIGNATURES) == set(names)


def test_struct_layouts_match():
    lib = _lib.lib()
    assert lib.dlm_abi_check(C.sizeof(DlmComm), C.sizeof(DlmGemm), C.sizeof(_lib.DlmStatus)) == _lib.OK
    assert lib.dlm_abi_check(C.sizeof(DlmComm) + 8, C.sizeof(DlmGemm), C.sizeof(_lib.DlmStatus)) == _lib.ERR_SHAPE


def test_header_constants_match_binding():
    text = HEADER.read_text()
    for name, value in [("DLM_MAX_WORLD", _lib.MAX_WORLD), ("DLM_EPOCH_SLOTS", _lib.EPOCH_SLOTS),
                        ("DLM_STATUS_WORDS", _lib.STATUS_WORDS), ("DLM_FUSED_MAX_N", _lib.FUSED_MAX_N)]:
        assert int(re.search(rf"#define {name} (\d+)", text).group(1)) == value
    for name, value in [("DLM_ERR_TIMEOUT", _lib.ERR_TIMEOUT), ("DLM_ERR_ARCH", _lib.ERR_ARCH),
                        ("DLM_ERR_WORKSPACE", _lib.ERR_WORKSPACE)]:
        assert int(re.search(rf"{name} = (-?\d+)", text).group(1)) == value


def test_strerror_and_sizes():
    lib = _lib.lib()
    for code in range(0, -12, -1):
        assert lib.dlm_strerror(code)
    assert lib.dlm_strerror(-99) == b"unknown error"
    assert lib.dlm_workspace_bytes(256, 2560, 9728) == 2048 + 8 * 256 * 2560 * 4
    assert lib.dlm_workspace_bytes(0, 2560, 64) == 0


def comm(**kw):
    c = DlmComm()
    c.rank, c.world, c.rows, c.n, c.mode = 0, 1, 32, 256, _lib.REDUCE
    c.recv[0], c.out, c.out_peers[0], c.epochs = 0x1000, 0x2000, 0x2000, 0x3000
    for k, v in kw.items():
        setattr(c, k, v)
    return c


@pytest.mark.parametrize("kw, code", [
    (dict(n=100), _lib.ERR_SHAPE), (dict(n=8448), _lib.ERR_SHAPE), (dict(rows=33, world=2, rank=0), _lib.ERR_WORLD),
    (dict(world=9), _lib.ERR_WORLD), (dict(rank=1), _lib.ERR_WORLD), (dict(out=None), _lib.ERR_NULL),
    (dict(out=0x2008), _lib.ERR_ALIGN), (dict(mode=_lib.REDUCE_NORM), _lib.ERR_NULL),
    (dict(mode=_lib.REDUCE_NORM_RESIDUAL, weight=0x4000), _lib.ERR_NULL), (dict(rearm_bytes=24, rearm=0x5000), _lib.ERR_ALIGN),
    (dict(rearm_bytes=32), _lib.ERR_ALIGN), (dict(epochs=None), _lib.ERR_NULL), (dict(mode=7), _lib.ERR_SHAPE),
])
def test_reduce_rejects_bad_arguments(kw, code):
    """No launch happens: the checks run before any CUDA call, as the reference's TORCH_CHECKs do."""
    assert _lib.lib().dlm_reduce_bf16(0x8000, C.byref(comm(**kw)), None) == code


def test_reduce_rejects_null_partial_and_missing_peer():
    assert _lib.lib().dlm_reduce_bf16(None, C.byref(comm()), None) == _lib.ERR_NULL
    c = comm(world=2, rows=32)
    c.recv[1] = 0x1100
    assert _lib.lib().dlm_reduce_bf16(0x8000, C.byref(c), None) == _lib.ERR_NULL  # out_peers[1] missing, no multicast


def gemm(**kw):
    g = DlmGemm()
    g.x, g.w, g.m, g.n, g.k, g.ldx, g.ldw = 0x1000, 0x2000, 32, 256, 128, 128, 128
    g.workspace, g.workspace_bytes = 0x10000, 1 << 24
    for k, v in kw.items():
        setattr(g, k, v)
    return g


@pytest.mark.parametrize("kw, code", [
    (dict(m=8), _lib.ERR_SHAPE), (dict(m=272), _lib.ERR_SHAPE), (dict(m=40), _lib.ERR_SHAPE), (dict(n=192), _lib.ERR_SHAPE),
    (dict(k=100), _lib.ERR_SHAPE), (dict(k=56), _lib.ERR_SHAPE), (dict(ldx=64), _lib.ERR_ALIGN), (dict(ldw=132), _lib.ERR_ALIGN),
    (dict(x=0x1004), _lib.ERR_ALIGN), (dict(workspace=0x10010), _lib.ERR_ALIGN), (dict(w=None), _lib.ERR_NULL),
    (dict(splits=9), _lib.ERR_SHAPE), (dict(token_tiles=3), _lib.ERR_SHAPE), (dict(m=48, token_tiles=2), _lib.ERR_SHAPE),
])
def test_gemm_rejects_bad_arguments(kw, code):
    assert _lib.lib().dlm_gemm_bf16(C.byref(gemm(**kw)), 0x9000, 256, 0, None) == code


def test_fused_requires_matching_shapes():
    c = comm(rows=32, n=256)
    assert _lib.lib().dlm_rowpar_bf16(C.byref(gemm(m=64)), C.byref(c), None) == _lib.ERR_SHAPE
    assert _lib.lib().dlm_rowpar_bf16(C.byref(gemm(n=512)), C.byref(c), None) == _lib.ERR_SHAPE


def test_fused_rejects_an_input_that_the_same_launch_rearms_or_writes():
    """CTAs of the fused kernel re-arm `rearm` and fill `out` while others still load x, so x may be neither."""
    lib = _lib.lib()
    g = gemm()  # x at 0x1000, 32 x 128 BF16 = 8 KiB
    assert lib.dlm_rowpar_bf16(C.byref(g), C.byref(comm(rearm=0x2000, rearm_bytes=4096)), None) == _lib.ERR_OVERLAP
    assert lib.dlm_rowpar_bf16(C.byref(g), C.byref(comm(out=0x1800, out_peers=(C.c_void_p * 8)(0x1800))), None) \
        == _lib.ERR_OVERLAP
    assert b"overlaps" in lib.dlm_strerror(_lib.ERR_OVERLAP)
    # disjoint buffers pass the pair check (and then fail later, on the missing GPU or nothing at all)
    assert lib.dlm_rowpar_bf16(C.byref(g), C.byref(comm(rearm=0x40000, rearm_bytes=4096, out=0x50000,
                                                       out_peers=(C.c_void_p * 8)(0x50000))), None) != _lib.ERR_OVERLAP


def test_noalloc_counts_the_splits_that_would_run():
    """More splits than K has 64-wide blocks run as that many blocks, and only those must fit the built-in scratch."""
    f = _lib.lib().dlm_gemm_bf16_noalloc
    # k = 64: one k-block, so "8 splits" is one split and needs no partial tiles; the call gets past the scratch check
    assert f(0x1000, 0x2000, 0x3000, 256, 2560, 64, 64, 64, 2560, 8, 1, 0, None) != _lib.ERR_SCRATCH
    assert f(0x1000, 0x2000, 0x3000, 256, 2560, 9728, 9728, 9728, 2560, 8, 1, 0, None) == _lib.ERR_SCRATCH


def test_all_gather_rejects_bad_arguments():
    lib = _lib.lib()
    c = DlmComm()
    c.rank, c.world = 0, 2
    assert lib.dlm_all_gather(None, 64, C.byref(c), None) == _lib.ERR_NULL
    assert lib.dlm_all_gather(4096, 60, C.byref(c), None) == _lib.ERR_SHAPE          # not a multiple of 16 bytes
    assert lib.dlm_all_gather(4096, _lib.GATHER_MAX_BYTES + 16, C.byref(c), None) == _lib.ERR_SHAPE
    assert lib.dlm_all_gather(4096, 64, C.byref(c), None) == _lib.ERR_NULL           # no out, epochs, slots
    c.out, c.epochs = 8192, 12288
    c.recv[0] = 16384
    assert lib.dlm_all_gather(4096, 64, C.byref(c), None) == _lib.ERR_NULL           # rank 1's slots missing
    c.recv[1] = 16392
    assert lib.dlm_all_gather(4096, 64, C.byref(c), None) == _lib.ERR_ALIGN
    c.world = 9
    assert lib.dlm_all_gather(4096, 64, C.byref(c), None) == _lib.ERR_WORLD


def test_device_loop_rejects_bad_programs_before_touching_cuda():
    from dlmrt_b200._lib import DlmLoop, DlmLoopPart
    from dlmrt_b200.ops.block_graph import BlockGraph, StagedLoopGraph

    lib, out = _lib.lib(), C.c_void_p()
    assert lib.dlm_device_loop_create(None, None, 1, None, C.byref(out)) == _lib.ERR_SHAPE
    assert lib.dlm_device_loop_create(None, None, _lib.MAX_LOOPS + 1, None, C.byref(out)) == _lib.ERR_SHAPE
    assert lib.dlm_device_loop_create(None, None, 0, None, None) == _lib.ERR_NULL
    parts = (DlmLoopPart * 1)()
    loop = (DlmLoop * 1)()
    loop[0].parts, loop[0].n_parts, loop[0].limit = parts, 1, 4
    assert lib.dlm_device_loop_create(None, loop, 1, None, C.byref(out)) == _lib.ERR_NULL  # no counters, no graph
    loop[0].remaining = loop[0].step = 8
    assert lib.dlm_device_loop_create(None, loop, 1, None, C.byref(out)) == _lib.ERR_NULL  # part without a graph
    loop[0].limit = -1
    assert lib.dlm_device_loop_create(None, loop, 1, None, C.byref(out)) == _lib.ERR_SHAPE
    assert lib.dlm_device_loop_launch(None, None) == _lib.ERR_NULL
    lib.dlm_device_loop_destroy(None)
    with pytest.raises(_lib.DlmError):
        BlockGraph(1, 0, 3, 8, 16, 4)  # no round graph
    with pytest.raises(ValueError):
        StagedLoopGraph(0, [], 8, 16, 4)


def test_missing_library_is_an_import_error(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libdlmrt_b200.so")
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_tiling_choice_follows_the_shape():
    """Long K (TP = 1) is split along K over all SMs; short K (TP = 8) is tiled along the tokens with no split."""
    lib = _lib.lib()
    t, sp = C.c_int(), C.c_int()
    assert lib.dlm_choose_tiling(256, 2560, 9728, 148, C.byref(t), C.byref(sp)) == _lib.OK
    assert (t.value, sp.value) == (1, 7)
    assert lib.dlm_choose_tiling(256, 2560, 1216, 148, C.byref(t), C.byref(sp)) == _lib.OK
    assert sp.value == 1 and t.value >= 2
    assert lib.dlm_choose_tiling(256, 2560, 9728, 20, C.byref(t), C.byref(sp)) == _lib.OK
    assert (t.value, sp.value) == (1, 1)
    assert lib.dlm_choose_tiling(250, 2560, 9728, 148, C.byref(t), C.byref(sp)) == _lib.ERR_SHAPE
