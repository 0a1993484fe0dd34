"""Properties of the CPU restatement of the fused reduction (oracle.reduce)."""

import numpy as np
import pytest
import torch

from oracle import reduce as red
from oracle.bf16 import bf16_to_f32, f32_to_bf16, from_torch


def partials(world, rows, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return from_torch(torch.randn(world, rows, n, generator=g).to(torch.bfloat16))


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_sum_is_rank_ordered_fp32(world):
    p = partials(world, 16, 256)
    got = red.reduce(p)
    acc = torch.zeros(16, 256)
    for s in range(world):
        acc = acc + torch.from_numpy(bf16_to_f32(p[s]))
    assert np.array_equal(got, from_torch(acc.to(torch.bfloat16)))


def test_order_matters_and_is_fixed():
    """A case where FP32 addition is not associative: the restatement must give the rank-order answer."""
    big, small = np.float32(2.0 ** 24), np.float32(1.0)
    p = np.zeros((3, 1, 256), dtype=np.uint16)
    p[0], p[1], p[2] = f32_to_bf16(np.float32([big]))[0], f32_to_bf16(np.float32([small]))[0], \
        f32_to_bf16(np.float32([-big]))[0]
    p = np.repeat(p, 3, axis=1)  # rows % world == 0
    assert (bf16_to_f32(red.reduce(p)) == 0.0).all()  # (2^24 + 1) - 2^24 = 0 in FP32
    assert (bf16_to_f32(red.reduce(p[[0, 2, 1]])) == 1.0).all()


def test_negative_zero_becomes_positive_zero():
    p = np.full((2, 2, 256), 0x8000, dtype=np.uint16)
    assert (red.reduce(p) == 0).all()


def test_world_one_is_identity_except_negative_zero():
    p = partials(1, 4, 256, seed=3)
    assert np.array_equal(red.reduce(p), np.where(p[0] == 0x8000, 0, p[0]))


@pytest.mark.parametrize("rows,n,world", [(8, 100, 2), (9, 256, 2), (8, 256, 9), (8, 8448, 2)])
def test_argument_checks(rows, n, world):
    with pytest.raises(ValueError):
        red.check_shape(rows, n, world)


@pytest.mark.parametrize("world", [1, 2, 8])
def test_norm_against_float64(world):
    """tests/test_sdar_kernels.py:17-30 of the reference: rmsnorm within 4e-3 relative of torch; h update exact."""
    rows, n, eps = 16, 2560, 1e-6
    p = partials(world, rows, n, seed=1)
    g = torch.Generator().manual_seed(2)
    w = from_torch((torch.randn(n, generator=g) * 0.1 + 1).to(torch.bfloat16))
    h = from_torch(torch.randn(world, rows, n, generator=g).to(torch.bfloat16))
    out, h_after = red.reduce_norm(p, w, eps, 1.0, h)
    R = rows // world
    summed = bf16_to_f32(red.reduce(p))
    for r in range(world):
        own = slice(r * R, (r + 1) * R)
        want_h = f32_to_bf16(summed[own] + bf16_to_f32(h[r, own]))
        assert np.array_equal(h_after[r, own], want_h)
        other = np.ones(rows, bool)
        other[own] = False
        assert np.array_equal(h_after[r, other], h[r, other])  # rows it does not own are untouched
        x = bf16_to_f32(want_h).astype(np.float64)
        x = (summed[own].astype(np.float64) + bf16_to_f32(h[r, own]).astype(np.float64))
        want = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * bf16_to_f32(w).astype(np.float64)
        got = bf16_to_f32(out[own]).astype(np.float64)
        assert np.linalg.norm(got - want) / np.linalg.norm(want) < 4e-3


def test_norm_without_residual_normalises_the_rounded_sum():
    p = partials(2, 4, 256, seed=5)
    w = f32_to_bf16(np.ones(256, dtype=np.float32))
    out, h_after = red.reduce_norm(p, w, 1e-6, 2.0)
    assert h_after is None
    x = bf16_to_f32(red.reduce(p)).astype(np.float64)
    want = 2.0 * x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-6)
    assert np.abs(bf16_to_f32(out) - want).max() <= np.abs(want).max() * 2 ** -7


def test_block_sum_tree_is_close_to_exact_and_order_sensitive():
    rng = np.random.default_rng(0)
    v = rng.standard_normal((4, 2048)).astype(np.float32)
    got = red.block_sum_of_squares(v)
    want = (v.astype(np.float64) ** 2).sum(-1)
    assert np.abs(got - want).max() / want.max() < 1e-6
