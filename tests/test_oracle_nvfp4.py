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


# ---- GEMM2 + combine against the reference's own W4A4 torch math (tests/golden/make_moe_golden.py) -----------------
M = np.load(Path(__file__).parent / "golden" / "moe_golden.npz")


def rel(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


def golden_down(prefix):
    """The oracle's GEMM2 + combine on a golden case: the reference's BF16 activation per (token, k) pair is quantised
    against a2 (oracle.quantize, itself pinned to the reference's quantiser above), laid out in expert-major slots
    and pushed through moe_down + combine. Returns BF16 bits [T, H]."""
    ids, weights = M[f"{prefix}_ids"], M[f"{prefix}_weights"]
    rows, k = ids.shape
    e_total = M[f"{prefix}_down_packed"].shape[0]
    a2, ws2 = M[f"{prefix}_down_input_scale"], M[f"{prefix}_down_scale2"]
    act = bf16_to_f32(M[f"{prefix}_act"])
    amap, counts = nvfp4.route_slots(ids, e_total)
    m_max = amap.shape[1]
    f = act.shape[1]
    codes = np.zeros((e_total * m_max, f // 2), dtype=np.uint8)
    scales = np.zeros((e_total * m_max, f // 16), dtype=np.uint8)
    for e in range(e_total):
        for j in range(counts[e]):
            c, s = nvfp4.quantize(act[amap[e, j]][None], a2[e])
            codes[e * m_max + j], scales[e * m_max + j] = c[0], s[0]
    y = nvfp4.moe_down(codes, scales, amap, counts, M[f"{prefix}_down_packed"], M[f"{prefix}_down_scale"],
                       (a2 * ws2).astype(np.float32), 0, rows * k)
    return nvfp4.combine(y, ids, weights, 0, e_total)


@pytest.mark.parametrize("prefix", ["swiglu", "geglu"])
def test_down_and_combine_match_the_reference_w4a4_math(prefix):
    """The bounds the reference holds its own B200 back-end to (tests/test_llada_nvfp4.py:107-114,
    tests/test_nvfp4.py:147-152): within 8 % of the W4A4 torch math and as far from unquantised math as it is, to 2 %.
    GEMM2 has no data-dependent rounding flips, so the oracle in fact sits within 1 % (BF16 roundings only)."""
    out = bf16_to_f32(golden_down(prefix))
    ref, truth = M[f"{prefix}_ref"], M[f"{prefix}_truth"]
    assert rel(out, ref) < 0.08
    assert abs(rel(out, truth) - rel(ref, truth)) < 0.02
    assert rel(out, ref) < 1e-2


def test_down_and_combine_are_exact_where_the_reference_math_is():
    """Power-of-two scales and small integers: every product, sum and rounding of the reference's statement is exact,
    so the oracle must give the BF16 rounding of the reference's FP32 result, bit for bit."""
    assert np.array_equal(golden_down("exact"), f32_to_bf16(M["exact_ref"]))


@pytest.mark.parametrize("prefix", ["swiglu", "geglu"])
def test_activation_quantiser_matches_the_reference_round_trip(prefix):
    """fake_quantize(act, a2) of the reference == dequantise(quantise(act)) of the oracle, bit for bit."""
    a2 = M[f"{prefix}_down_input_scale"][0]
    act = bf16_to_f32(M[f"{prefix}_act"])
    got = nvfp4.dequantize(*nvfp4.quantize(act, a2), a2)
    assert np.array_equal(got, M[f"{prefix}_actq"])


# ---- the front half (input quantiser, GEMM1 + activation + re-quantisation) and the whole expert pipeline ------------
def golden_front(prefix):
    ids = M[f"{prefix}_ids"]
    e_total = M[f"{prefix}_gate_packed"].shape[0]
    a13, a2 = M[f"{prefix}_gate_input_scale"], M[f"{prefix}_down_input_scale"]
    g1 = (a13 * M[f"{prefix}_gate_scale2"]).astype(np.float32)
    return nvfp4.moe_front(bf16_to_f32(M[f"{prefix}_x"]), np.float32(1) / a13[0], ids, e_total,
                           (M[f"{prefix}_gate_packed"], M[f"{prefix}_gate_scale"]),
                           (M[f"{prefix}_up_packed"], M[f"{prefix}_up_scale"]), g1, (np.float32(1) / a2).astype(np.float32),
                           0, prefix)


@pytest.mark.parametrize("prefix", ["swiglu", "geglu"])
def test_run_time_input_quantiser_agrees_with_the_export_quantiser(prefix):
    """The engines quantise activations with the fast recipe (scale = E4M3(g * amax / 6), reciprocal multiplies); the
    reference's W4A4 math uses the export recipe (amax / (6 s), divisions). They are the same up to the last bit of
    the scale arithmetic: a fraction of a percent of the values lands one code apart."""
    a13 = M[f"{prefix}_gate_input_scale"][0]
    codes, scales = nvfp4.quantize_fast(bf16_to_f32(M[f"{prefix}_x"]), np.float32(1) / a13)
    assert (nvfp4.dequantize(codes, scales, a13) != M[f"{prefix}_xq"]).mean() < 5e-3


@pytest.mark.parametrize("prefix", ["swiglu", "geglu"])
def test_whole_expert_pipeline_within_the_reference_bounds(prefix):
    """Front half + down-projection + combine against the reference's W4A4 torch math: the two bounds the reference
    sets for its own B200 back-end (tests/test_llada_nvfp4.py:107-114, tests/test_nvfp4.py:147-152). The activation's
    FP4 rounding flips on BF16-level differences (the reference rounds GEMM1's output and the activation to BF16, the
    engine's kernels keep FP32), hence percent-level and not bit-level agreement, as the reference's tests note."""
    ids, weights = M[f"{prefix}_ids"], M[f"{prefix}_weights"]
    rows, k = ids.shape
    amap, counts, act_codes, act_scales = golden_front(prefix)
    a2, ws2 = M[f"{prefix}_down_input_scale"], M[f"{prefix}_down_scale2"]
    # the activation alone, against fake_quantize(act, a2) of the reference
    got = np.zeros((rows * k, act_codes.shape[1] * 2), dtype=np.float32)
    for e in range(amap.shape[0]):
        for j in range(counts[e]):
            s = e * rows + j
            got[amap[e, j]] = bf16_to_f32(nvfp4.dequantize(act_codes[s][None], act_scales[s][None], a2[e]))[0]
    assert rel(got, bf16_to_f32(M[f"{prefix}_actq"])) < 0.08
    y = nvfp4.moe_down(act_codes, act_scales, amap, counts, M[f"{prefix}_down_packed"], M[f"{prefix}_down_scale"],
                       (a2 * ws2).astype(np.float32), 0, rows * k)
    out = bf16_to_f32(nvfp4.combine(y, ids, weights, 0, amap.shape[0]))
    ref, truth = M[f"{prefix}_ref"], M[f"{prefix}_truth"]
    assert rel(out, ref) < 0.08
    assert abs(rel(out, truth) - rel(ref, truth)) < 0.02


def test_route_packed_lists_the_top_k_in_expert_order():
    rng = np.random.default_rng(3)
    logits = f32_to_bf16(rng.standard_normal((16, 128)).astype(np.float32))
    scale = f32_to_bf16((rng.random(128, dtype=np.float32) + 0.5))
    ids, w, packed = nvfp4.route_packed(logits, scale, 8)
    assert (np.diff(ids, axis=1) > 0).all()
    x = bf16_to_f32(logits).astype(np.float64)
    p = np.exp(x - x.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    for t in range(16):
        assert set(ids[t]) == set(np.argsort(-p[t])[:8])
        want = p[t, ids[t]] / p[t, ids[t]].sum() * bf16_to_f32(scale)[ids[t]]
        assert np.abs(w[t] - want).max() <= np.abs(want).max() * 2.0 ** -8
    got_ids, got_w = nvfp4.unpack_topk(packed)
    assert np.array_equal(got_ids, ids) and np.array_equal(got_w, w)
