"""The tcgen05 row-parallel GEMM (dlm_gemm_bf16) and the fused projection + reduction (dlm_rowpar_bf16 / _loopback)
against the CPU oracle."""

import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import assert_norm_close, assert_same_bits, bits, randn_bf16
from oracle import reduce as red
from oracle import rowpar
from oracle.bf16 import f32_to_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def short_timeouts(monkeypatch):
    from dlmrt_b200.distributed import parallel

    monkeypatch.setattr(parallel, "TIMEOUT_NS", 500_000_000)


def gemm(x, w, splits=0, token_tiles=0):
    from dlmrt_b200 import _lib
    from dlmrt_b200._lib import DlmGemm

    m, k = x.shape
    n = w.shape[0]
    out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    ws = torch.zeros(_lib.lib().dlm_workspace_bytes(m, n, k), dtype=torch.uint8, device=x.device)
    g = DlmGemm()
    g.x, g.w, g.m, g.n, g.k, g.ldx, g.ldw = x.data_ptr(), w.data_ptr(), m, n, k, x.stride(0), w.stride(0)
    g.workspace, g.workspace_bytes, g.splits, g.token_tiles = ws.data_ptr(), ws.numel(), splits, token_tiles
    _lib.check(_lib.lib().dlm_gemm_bf16(C.byref(g), out.data_ptr(), n, 0, None), "gemm")
    torch.cuda.synchronize()
    return out


def integer_case(m, n, k, seed):
    """Small-integer operands: every product and partial sum is exact in FP32, so the BF16 result is the same whatever
    the summation order, and the comparison with the oracle is bit for bit at any size."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(-3, 4, (m, k), generator=g).to(torch.bfloat16).cuda()
    w = torch.randint(-2, 3, (n, k), generator=g).to(torch.bfloat16).cuda()
    return x, w


SHAPES = [(16, 128, 64), (32, 2048, 2048), (64, 2816, 512), (256, 2560, 4096), (256, 2560, 9728), (48, 256, 1216),
          (256, 2816, 2176), (32, 2048, 64)]


@pytest.mark.parametrize("m, n, k", SHAPES)
def test_gemm_exact_on_integer_operands(m, n, k):
    x, w = integer_case(m, n, k, seed=m + n + k)
    want = f32_to_bf16(rowpar.gemm_f32(bits(x), bits(w)))
    assert_same_bits(bits(gemm(x, w)), want, f"gemm {m}x{n}x{k}")


@pytest.mark.parametrize("m, n, k", SHAPES)
def test_gemm_within_tolerance_on_gaussian_operands(m, n, k):
    """Tolerance of the GEMM partial: per row max-abs <= 2 BF16 ulp of the row's largest magnitude and relative L2
    <= 4e-3 against float64 (bounds of the reference's tests/test_sdar_kernels.py:30, test_llada_nvfp4.py:166)."""
    x, w = randn_bf16(m, k, seed=1), randn_bf16(n, k, seed=2, std=0.02)
    out = gemm(x, w)
    truth = rowpar.gemm_f64(bits(x), bits(w))
    max_abs, rel = rowpar.row_errors(bits(out), truth)
    assert max_abs.max() <= rowpar.ULPS and rel.max() <= rowpar.REL_L2, (max_abs.max(), rel.max())
    # and no further from the truth than cuBLAS on the same GPU
    _, rel_cublas = rowpar.row_errors(bits(torch.mm(x, w.t())), truth)
    assert rel.max() <= 2 * rel_cublas.max() + 1e-6


@pytest.mark.parametrize("m, n, k, token_tiles, splits", [(256, 2560, 4864, 2, 3), (96, 512, 2048, 1, 1), (80, 2560, 2048, 1, 2),
                                                          (160, 2560, 2048, 2, 3)])
def test_two_issuers_on_a_ring_with_an_odd_number_of_stages(m, n, k, token_tiles, splits):
    """Tiles of up to 128 tokens have two MMA-issuing threads that take alternate k-blocks. On a ring with an odd number
    of stages (7 for 96- and 80-token tiles) they alternate on every stage, and each may only wait for a stage's barrier
    once the other has seen that stage's previous phase complete; a kernel without that guard, on a 3-stage ring, raised
    a launch failure on back-to-back launches of the first shape. Exact on integer operands."""
    from dlmrt_b200.layers.linear import Linear

    x, w = integer_case(m, n, k, seed=21)
    want = f32_to_bf16(rowpar.gemm_f32(bits(x), bits(w)))
    lins = [Linear(w, token_tiles=token_tiles, splits=splits) for _ in range(3)]
    outs = [torch.empty(m, n, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    for _ in range(10):
        for lin, out in zip(lins, outs):
            lin.gemm(x, out)
    torch.cuda.synchronize()
    for i, out in enumerate(outs):
        assert_same_bits(bits(out), want, f"launch chain {i}")


@pytest.mark.parametrize("splits", [1, 2, 3, 8])
def test_gemm_split_k_is_deterministic_and_ordered(splits):
    m, n, k = 64, 256, 2048
    x, w = randn_bf16(m, k, seed=5), randn_bf16(n, k, seed=6)
    a, b = gemm(x, w, splits), gemm(x, w, splits)
    assert_same_bits(bits(a), bits(b), "two runs")
    # the split result is the in-order FP32 sum of the per-range products (dlmrt/ops/triton/gemm.py:3-7)
    nkb = k // 64
    edges = [s * nkb // splits * 64 for s in range(splits + 1)]
    parts = [x[:, lo:hi].float() @ w[:, lo:hi].float().t() for lo, hi in zip(edges[:-1], edges[1:])]
    acc = parts[0]
    for p in parts[1:]:
        acc = acc + p
    from oracle.bf16 import bf16_to_f32

    want = acc.cpu().numpy()
    diff = np.abs(bf16_to_f32(bits(a)) - want)
    # inside a range the tensor core's own summation tree applies, so equality is up to FP32 rounding of the
    # accumulation plus the final BF16 rounding: half a BF16 ulp of the value plus a little of the row's scale
    assert (diff <= np.abs(want) * 2.0 ** -8 + np.abs(want).max(axis=1, keepdims=True) * 2.0 ** -16).all()


@pytest.mark.parametrize("token_tiles, splits", [(1, 1), (2, 1), (4, 1), (2, 3), (4, 2), (8, 1), (1, 0), (0, 1)])
def test_gemm_token_tiles_and_splits_agree(token_tiles, splits):
    """Any tiling gives the exact result on integer operands, and repeated launches on one workspace stay exact
    (the split-K arrival counters alternate banks by launch generation)."""
    m, n, k = 256, 512, 1024
    x, w = integer_case(m, n, k, seed=3)
    want = f32_to_bf16(rowpar.gemm_f32(bits(x), bits(w)))
    from dlmrt_b200.layers.linear import Linear
    for attempt in range(2):
        assert_same_bits(bits(gemm(x, w, splits, token_tiles)), want, f"tiles {token_tiles} splits {splits} #{attempt}")
    lin = Linear(w)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    for _ in range(5):  # same workspace, back to back, no host synchronisation in between
        lin.gemm(x, out)
    torch.cuda.synchronize()
    assert_same_bits(bits(out), want, "five launches on one workspace")


@pytest.mark.parametrize("m, n, k, tiled", [(32, 256, 200, True), (32, 256, 200, False), (256, 2560, 18992, True)])
def test_ragged_k_and_nn_layout(m, n, k, tiled):
    """K that is not a multiple of 64 (the vocabulary shard of the self-conditioning soft-embedding GEMM: 151936 / 8 =
    18992) and a [K, N] weight (`nn`), exact on integer operands."""
    from dlmrt_b200.layers.linear import Linear

    x, w = integer_case(m, n, k, seed=k)
    want = f32_to_bf16(rowpar.gemm_f32(bits(x), bits(w)))
    lin = Linear(w.t().contiguous(), nn=True, tiled=tiled)  # handed over as [K, N]
    assert (lin.n, lin.k) == (n, k)
    out = lin(x)
    torch.cuda.synchronize()
    assert_same_bits(bits(out), want, f"nn gemm {m}x{n}x{k}")


def test_gemm_strided_operands():
    m, n, k = 32, 256, 256
    xs, ws = randn_bf16(m, 2 * k, seed=7), randn_bf16(n, 3 * k, seed=8)
    x, w = xs[:, k:], ws[:, k:2 * k]
    from dlmrt_b200.layers.linear import Linear

    lin = Linear(w.contiguous())
    out = lin(x)
    torch.cuda.synchronize()
    assert rowpar.within_tolerance(bits(out), rowpar.gemm_f64(bits(x.contiguous()), bits(w.contiguous())))


@pytest.mark.parametrize("world, m, n, k, splits", [(1, 32, 2048, 2048, 0), (1, 256, 2560, 4096, 0), (2, 256, 2560, 9728, 3),
                                                     (2, 32, 2048, 2048, 2), (4, 256, 2816, 4096, 1), (8, 32, 2048, 2048, 1),
                                                     (8, 256, 2048, 9728, 1), (4, 64, 2560, 1024, 0),
                                                     (1, 256, 2560, 9728, 7), (1, 64, 2048, 2048, 3), (1, 32, 2816, 4096, 4)])
def test_fused_rowpar_loopback_matches_oracle(world, m, n, k, splits):
    """Fused projection + reduction over `world` emulated ranks: with exact (integer) operands the whole pipeline is
    bit-exact against the oracle; with Gaussian operands the reduction of this kernel's own GEMM partials is."""
    from dlmrt_b200.distributed.loopback import LoopbackWorld

    lw = LoopbackWorld(world)
    weight = randn_bf16(n, seed=9, std=0.1) + 1
    hs = [randn_bf16(m, n, seed=20 + r) for r in range(world)]
    for i, mode in enumerate([0, 2, 1, 0]):
        if i % 2:
            x, w = randn_bf16(m, k, seed=30 + i), randn_bf16(n, k, seed=40 + i, std=0.02)
        else:
            x, w = integer_case(m, n, k, seed=i)
        xs = [t.contiguous() for t in x.chunk(world, 1)]
        ws = [t.contiguous() for t in w.chunk(world, 1)]
        sp = splits or 1
        tt = 2 if (i == 3 and m >= 64 and 2 * (n // 128) * sp <= 148 // world) else 1
        partial_bits = np.stack([bits(gemm(xs[r], ws[r], sp, tt)) for r in range(world)])
        if i % 2 == 0:
            _, exact = rowpar.rowpar(bits(x), bits(w), world)
            assert_same_bits(partial_bits, exact, "integer partials")
        site = f"site{i}"
        if mode == 0:
            outs = lw.rowpar(xs, ws, site=site, splits=sp, token_tiles=tt)
            want = red.reduce(partial_bits)
        elif mode == 1:
            outs = lw.rowpar(xs, ws, site=site, weight=weight, eps=1e-6, scale=0.5, splits=sp, token_tiles=tt)
            want, _ = red.reduce_norm(partial_bits, bits(weight), 1e-6, 0.5)
        else:
            h_before = np.stack([bits(h) for h in hs])
            outs = lw.rowpar(xs, ws, site=site, hs=hs, weight=weight, eps=1e-6, splits=sp, token_tiles=tt)
            want, h_after = red.reduce_norm(partial_bits, bits(weight), 1e-6, 1.0, h_before)
        torch.cuda.synchronize()
        lw.check()
        got = [bits(o) for o in outs]
        for r in range(1, world):
            assert_same_bits(got[r], got[0], f"call {i}: rank {r} vs rank 0")
        if mode == 0:
            assert_same_bits(got[0], want, f"call {i}")
        else:
            assert_norm_close(got[0], want, f"call {i} mode {mode}")
        if mode == 2:
            for r in range(world):
                assert_same_bits(bits(hs[r]), h_after[r], f"call {i}: residual of rank {r}")


@pytest.mark.parametrize("world", [1, 2])
def test_alternating_tilings_share_one_workspace(world):
    """Calls of one chain share the split-K workspace whatever their tiling: the arrival counters a launch finds must
    be at zero even when the launches before it used more (or other) tiles."""
    from dlmrt_b200.distributed.loopback import LoopbackWorld

    lw = LoopbackWorld(world)
    m, n, k = 64, 1024, 2048 * world
    for i, (tt, sp) in enumerate([(2, 3), (1, 3), (2, 3), (1, 2), (2, 2), (1, 7 if world == 1 else 3), (2, 3), (1, 1), (2, 3)]):
        x, w = integer_case(m, n, k, seed=50 + i)
        xs = [t.contiguous() for t in x.chunk(world, 1)]
        ws = [t.contiguous() for t in w.chunk(world, 1)]
        outs = lw.rowpar(xs, ws, site=f"s{i}", splits=sp, token_tiles=tt)
        torch.cuda.synchronize()
        lw.check()
        _, exact = rowpar.rowpar(bits(x), bits(w), world)
        want = red.reduce(exact)
        for r in range(world):
            assert_same_bits(bits(outs[r]), want, f"call {i} (token tiles {tt}, splits {sp}) rank {r}")


def test_linear_defers_into_group_reduce():
    """The drop-in pair of the reference's call sites: Linear(x, out=group.partial(...)) then group.reduce_norm(...)
    (dlmrt/models/sdar/model.py:237-243) runs as one fused launch and matches GEMM-then-reduce."""
    from dlmrt_b200 import _lib
    from dlmrt_b200.distributed.parallel import Group
    from dlmrt_b200.layers.linear import Linear

    g = Group.local("cuda:0")
    m, n, k = 256, 2560, 4096
    x, w = randn_bf16(m, k, seed=1), randn_bf16(n, k, seed=2, std=0.02)
    weight, h = randn_bf16(n, seed=3, std=0.1) + 1, randn_bf16(m, n, seed=4)
    lin = Linear(w, fp8=False, group=g)
    before = _lib.lib().dlm_launch_count()
    p = lin(x, out=g.partial("0.post", (m, n)))
    assert _lib.lib().dlm_launch_count() == before  # deferred: nothing ran yet
    h_before = bits(h)[None]
    out = g.reduce_norm(p, h, weight, 1e-6, site="0.post")
    assert _lib.lib().dlm_launch_count() == before + 1  # one fused kernel
    torch.cuda.synchronize()
    g.check()
    partial_bits = bits(Linear(w).gemm(x, torch.empty(m, n, dtype=torch.bfloat16, device="cuda")))[None]
    want, h_after = red.reduce_norm(partial_bits, bits(weight), 1e-6, 1.0, h_before)
    assert_norm_close(bits(out), want, "fused reduce_norm")
    assert_same_bits(bits(h), h_after[0], "residual stream")
    # flush materialises a deferred partial instead
    p2 = lin(x, out=g.partial("1.post", (m, n)))
    g.flush(p2)
    torch.cuda.synchronize()
    assert_same_bits(bits(p2), partial_bits[0], "flushed partial")


def test_projection_fed_by_the_previous_output_runs_unfused():
    """The fused kernel re-arms the chain's previous output while some of its CTAs may still be loading x, so a
    projection whose input IS that output must not be fused: the Group runs GEMM and reduction as two launches (the
    reference's order), and the C entry point refuses the aliasing outright."""
    from dlmrt_b200 import _lib
    from dlmrt_b200._lib import DlmGemm
    from dlmrt_b200.distributed.parallel import Group
    from dlmrt_b200.layers.linear import Linear

    g = Group.local("cuda:0")
    m, n = 32, 2048
    w = [randn_bf16(n, n, seed=90 + i, std=0.02) for i in range(2)]
    lin = [Linear(w[i], group=g) for i in range(2)]
    x = randn_bf16(m, n, seed=92)
    before = _lib.lib().dlm_launch_count()
    first = g.reduce(lin[0](x, out=g.partial("a", (m, n))), site="a")
    assert _lib.lib().dlm_launch_count() == before + 1           # fused
    second = g.reduce(lin[1](first, out=g.partial("b", (m, n))), site="b")
    assert _lib.lib().dlm_launch_count() == before + 3           # GEMM, then reduction
    torch.cuda.synchronize()
    g.check()
    want = Linear(w[1]).gemm(Linear(w[0]).gemm(x, torch.empty(m, n, dtype=torch.bfloat16, device="cuda")),
                             torch.empty(m, n, dtype=torch.bfloat16, device="cuda"))
    torch.cuda.synchronize()
    assert_same_bits(bits(second), bits(want), "chained projections")
    # through the C ABI the same aliasing is an error
    comm, _ = g._comm(m, n, "c", 0, _lib.REDUCE, None, None, 0.0, 1.0)
    gm = g._gemm(lin[0], second, 0)   # x = the chain's previous output = what this call would re-arm
    assert _lib.lib().dlm_rowpar_bf16(C.byref(gm), C.byref(comm), None) == _lib.ERR_OVERLAP
