"""oracle.nvfp4 against vectors produced by the reference's own code (tests/golden/make_nvfp4_golden.py)."""

from pathlib import Path

import numpy as np
import pytest

from oracle import nvfp4
from oracle.bf16 import bf16_to_f32, f32_to_bf16

G = np.load(Path(__file__).parent / "golden" / "nvfp4_golden.npz")


def test_tables():
    assert np.array_equal(nvfp4.E2M1, G["e2m1"])
    got, want = nvfp4.e4m3_to_f32(np.arange(256, dtype=np.uint8)), G["e4m3_table"]
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(got)], want[~np.isnan(want)])


@pytest.mark.parametrize("name", ["w", "act"])
def test_dequantize_matches_reference(name):
    got = nvfp4.dequantize(G[f"{name}_packed"], G[f"{name}_scale"], G[f"{name}_scale2"])
    assert np.array_equal(got, G[f"{name}_deq"])


@pytest.mark.parametrize("name", ["w", "act"])
def test_quantize_matches_reference(name):
    packed, scale = nvfp4.quantize(G[f"{name}_x"], G[f"{name}_scale2"])
    assert np.array_equal(scale, G[f"{name}_scale"])
    assert np.array_equal(packed, G[f"{name}_packed"])


def test_quantize_error_bound():
    """tests/test_nvfp4.py:57: the round trip is within 12% relative L2 of the FP32 weights."""
    x = G["w_x"]
    deq = bf16_to_f32(nvfp4.dequantize(*nvfp4.quantize(x, G["w_scale2"]), G["w_scale2"]))
    assert np.linalg.norm(deq - x) / np.linalg.norm(x) < 0.12


def test_e4m3_encoder_is_inverse_of_decoder():
    bits = np.arange(0, 0x7F, dtype=np.uint8)
    assert np.array_equal(nvfp4.f32_to_e4m3(nvfp4.e4m3_to_f32(bits)), bits)


def test_pack_topk_matches_reference():
    assert np.array_equal(nvfp4.pack_topk(G["ids"], G["weights"]), G["topk_packed"])
    ids, w = nvfp4.unpack_topk(G["topk_packed"])
    assert np.array_equal(ids, G["ids"])
    assert np.array_equal(f32_to_bf16(w), f32_to_bf16(G["weights"]))


def test_code_packing_round_trip():
    rng = np.random.default_rng(1)
    codes = rng.integers(0, 16, size=(5, 64), dtype=np.uint8)
    assert np.array_equal(nvfp4.unpack_codes(nvfp4.pack_codes(codes)), codes)


def _case(rng, rows=8, e_total=8, k=2, n=64, f=64):
    ids = np.sort(np.stack([rng.permutation(e_total)[:k] for _ in range(rows)]), axis=1).astype(np.int32)
    weights = bf16_to_f32(f32_to_bf16(rng.random((rows, k), dtype=np.float32)))
    amap, counts = nvfp4.route_slots(ids, e_total)
    w = rng.standard_normal((e_total, n, f)).astype(np.float32) * 0.02
    s2 = np.abs(w).max() / 2688
    wq = [nvfp4.quantize(w[e], s2) for e in range(e_total)]
    act = rng.standard_normal((e_total * rows, f)).astype(np.float32)
    a2 = np.float32(np.abs(act).max() / 2688)
    aq, as_ = nvfp4.quantize(act, a2)
    g2 = np.full(e_total, a2 * s2, dtype=np.float32)
    return ids, weights, amap, counts, np.stack([q[0] for q in wq]), np.stack([q[1] for q in wq]), aq, as_, g2, act, w


def test_moe_down_and_combine_against_dense_math():
    """W4A4 down-projection + combine equals the dense float64 computation on the dequantised operands."""
    rng = np.random.default_rng(2)
    ids, weights, amap, counts, wc, ws, aq, as_, g2, act, w = _case(rng)
    rows, k = ids.shape
    y = nvfp4.moe_down(aq, as_, amap, counts, wc, ws, g2, 0, rows * k)
    out = nvfp4.combine(y, ids, weights, 0, wc.shape[0])
    want = np.zeros((rows, wc.shape[1]))
    seen = {e: 0 for e in range(wc.shape[0])}
    for t in range(rows):
        for j in range(k):
            e = int(ids[t, j])
            slot = e * rows + seen[e]
            seen[e] += 1
            a = nvfp4.block_values(aq[slot], as_[slot]).astype(np.float64)
            wd = nvfp4.block_values(wc[e], ws[e]).astype(np.float64)
            want[t] += weights[t, j] * (wd @ a) * g2[e]
    got = bf16_to_f32(out)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-2


def test_expert_parallel_partials_sum_to_the_whole():
    """Splitting the experts over ranks and summing the per-rank combines approximates the single-rank result."""
    rng = np.random.default_rng(3)
    ids, weights, amap, counts, wc, ws, aq, as_, g2, act, w = _case(rng)
    rows, k = ids.shape
    whole = bf16_to_f32(nvfp4.combine(nvfp4.moe_down(aq, as_, amap, counts, wc, ws, g2, 0, rows * k), ids, weights,
                                      0, 8))
    parts = np.zeros_like(whole)
    for r in range(2):
        lo = 4 * r
        y = nvfp4.moe_down(aq[lo * rows:(lo + 4) * rows], as_[lo * rows:(lo + 4) * rows], amap, counts,
                           wc[lo:lo + 4], ws[lo:lo + 4], g2[lo:lo + 4], lo, rows * k)
        parts += bf16_to_f32(nvfp4.combine(y, ids, weights, lo, 4))
    assert np.linalg.norm(parts - whole) / np.linalg.norm(whole) < 1e-2


def test_combine_with_shared_rounds_twice():
    rng = np.random.default_rng(4)
    y = f32_to_bf16(rng.standard_normal((4 * 2, 32)).astype(np.float32))
    ids = np.array([[0, 1]] * 4, dtype=np.int32)
    w = np.ones((4, 2), dtype=np.float32)
    shared = f32_to_bf16(rng.standard_normal((4, 32)).astype(np.float32))
    plain = nvfp4.combine(y, ids, w, 0, 2)
    both = nvfp4.combine(y, ids, w, 0, 2, shared)
    assert np.array_equal(both, f32_to_bf16(bf16_to_f32(plain) + bf16_to_f32(shared)))
