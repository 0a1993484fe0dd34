"""The plain-C restatement (oracle/c) against the numpy restatement and the reference-made fixtures: two independent
statements of the same arithmetic must agree bit for bit."""

from pathlib import Path

import numpy as np
import pytest

from oracle import c as orc
from oracle import nvfp4
from oracle import reduce as red
from oracle import rowpar
from oracle.bf16 import bf16_to_f32, f32_to_bf16

G = np.load(Path(__file__).parent / "golden" / "nvfp4_golden.npz")


def rand_bits(rng, *shape, std=1.0):
    return f32_to_bf16((rng.standard_normal(shape) * std).astype(np.float32))


@pytest.mark.parametrize("world", [1, 2, 8])
def test_reduce_matches_numpy(world):
    rng = np.random.default_rng(world)
    p = rand_bits(rng, world, 16, 512)
    p[0, 0, :4] = 0x8000
    assert np.array_equal(orc.reduce(p), red.reduce(p))


@pytest.mark.parametrize("world, n", [(1, 256), (2, 2560), (8, 2048)])
@pytest.mark.parametrize("residual", [False, True])
def test_reduce_norm_matches_numpy(world, n, residual):
    rng = np.random.default_rng(n + world)
    p, w = rand_bits(rng, world, 16, n), rand_bits(rng, n, std=0.1)
    h = rand_bits(rng, world, 16, n) if residual else None
    out_c, h_c = orc.reduce_norm(p, w, 1e-6, 1.5, h)
    out_np, h_np = red.reduce_norm(p, w, 1e-6, 1.5, h)
    assert np.array_equal(out_c, out_np)
    if residual:
        assert np.array_equal(h_c, h_np)


def test_rounding_matches_numpy():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(1 << 16).astype(np.float32) * 1e3
    assert np.array_equal(orc.round_bf16(x), f32_to_bf16(x))


def test_gemm_increasing_k_against_blas_and_exact_integers():
    rng = np.random.default_rng(1)
    x, w = rand_bits(rng, 8, 256), rand_bits(rng, 16, 256, std=0.02)
    got = orc.gemm_bf16(x, w)
    assert np.allclose(got, rowpar.gemm_f32(x, w), rtol=1e-4, atol=1e-5)
    xi = f32_to_bf16(rng.integers(-3, 4, (8, 256)).astype(np.float32))
    wi = f32_to_bf16(rng.integers(-2, 3, (16, 256)).astype(np.float32))
    for splits in (1, 2, 4):
        assert np.array_equal(orc.gemm_bf16(xi, wi, splits), rowpar.gemm_f32(xi, wi))  # exact whatever the order


@pytest.mark.parametrize("name", ["w", "act"])
def test_nvfp4_dequant_matches_reference_fixture(name):
    got = orc.nvfp4_dequant(G[f"{name}_packed"], G[f"{name}_scale"], float(G[f"{name}_scale2"]))
    assert np.array_equal(got, G[f"{name}_deq"])


def test_nvfp4_down_and_combine_match_numpy():
    rng = np.random.default_rng(2)
    a = rng.standard_normal((6, 64)).astype(np.float32)
    w = rng.standard_normal((32, 64)).astype(np.float32) * 0.02
    aq, as_ = nvfp4.quantize(a, np.abs(a).max() / 2688)
    wq, ws = nvfp4.quantize(w, np.abs(w).max() / 2688)
    y_c = orc.nvfp4_down(aq, as_, wq, ws, 0.37)
    y_np = nvfp4.expert_down(aq, as_, wq, ws, 0.37, accumulate=np.float64)
    d = np.abs(bf16_to_f32(y_c) - bf16_to_f32(y_np))
    assert (d <= np.abs(bf16_to_f32(y_np)) * 2.0 ** -7 + 1e-30).all()  # FP32 vs FP64 accumulation: at most one ulp
    ids = np.array([[0, 3], [1, 2], [2, 3]], dtype=np.int32)
    weights = bf16_to_f32(f32_to_bf16(rng.random((3, 2)).astype(np.float32)))
    shared = rand_bits(rng, 3, 32)
    for lo, local in ((0, 4), (2, 2)):
        for sh in (None, shared):
            assert np.array_equal(orc.moe_combine(y_c, ids, weights, lo, local, sh),
                                  nvfp4.combine(y_c, ids, weights, lo, local, sh))
