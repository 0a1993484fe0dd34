"""BASELINE config 1 on the CPU restatement: simulated TP=2 row-parallel projection, identical on both 'ranks'."""

import numpy as np
import pytest

from oracle import reduce as red
from oracle import rowpar
from oracle.bf16 import bf16_to_f32


@pytest.fixture(scope="module")
def case():
    return rowpar.config1()


def test_config1_shapes_and_rank_identity(case):
    x, w, world = case
    assert x.shape == (256, 9728) and w.shape == (2560, 9728) and world == 2
    out, parts = rowpar.rowpar(x, w, world)
    assert out.shape == (256, 2560) and out.dtype == np.uint16 and parts.shape == (2, 256, 2560)
    # every simulated rank reduces the same pushed partials in the same order: bit-identical
    per_rank = [red.reduce(parts) for _ in range(world)]
    assert all(np.array_equal(p, out) for p in per_rank)
    assert rowpar.within_tolerance(out, rowpar.gemm_f64(x, w))


def test_config1_fp32_partial_reading_differs_by_one_rounding(case):
    x, w, world = case
    bf, _ = rowpar.rowpar(x, w, world)
    fp, parts = rowpar.rowpar(x, w, world, fp32_partials=True)
    assert parts.dtype == np.float32
    truth = rowpar.gemm_f64(x, w)
    assert rowpar.within_tolerance(fp, truth)
    diff = np.abs(bf16_to_f32(bf) - bf16_to_f32(fp))
    assert (diff <= np.abs(truth).max(axis=1, keepdims=True) * 2.0 ** -6).all()
    assert (diff > 0).any()  # the two readings are distinguishable, so the choice is pinned


@pytest.mark.parametrize("world", [1, 4, 8])
def test_other_tp_degrees_agree_within_tolerance(world):
    x, w, _ = rowpar.config1(seed=1, m=32, k=2048, n=512)
    out, _ = rowpar.rowpar(x, w, world)
    assert rowpar.within_tolerance(out, rowpar.gemm_f64(x, w))


def test_shard_rejects_uneven_split():
    with pytest.raises(ValueError):
        rowpar.shard(np.zeros((4, 10), dtype=np.uint16), 4, 0, 1)
