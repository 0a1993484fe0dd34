"""The NVFP4 expert down-projection kernel (dlm_moe_nvfp4, dlm_rowpar_nvfp4_moe[_loopback]) against the CPU oracle."""

import numpy as np
import pytest
import torch

from gpu_util import assert_norm_close, assert_same_bits, bits, randn_bf16
from oracle import nvfp4 as onv
from oracle import reduce as red
from oracle.bf16 import bf16_to_f32, f32_to_bf16, to_torch

pytestmark = pytest.mark.gpu


def make_case(rows, hidden, f, e_total, top_k, seed, exact=False, skew=False, hot=False, m_max=None):
    """Routed inputs of one MoE layer call as numpy arrays in the layouts the kernel takes.

    exact: codes and power-of-two scales chosen so that every product and partial sum is exact in FP32; the kernel must
    then match the oracle bit for bit whatever its summation order, which also pins the scale-factor layout."""
    rng = np.random.default_rng(seed)
    if hot:  # expert 0 is on every token's list: it alone holds `rows` rows
        ids = np.stack([np.concatenate([[0], 1 + np.sort(rng.permutation(e_total - 1)[:top_k - 1])]) for _ in range(rows)])
        ids = ids.astype(np.int32)
    elif skew:
        p = 1.0 / np.arange(1, e_total + 1) ** 1.2
        p /= p.sum()
        ids = np.stack([np.sort(rng.choice(e_total, top_k, replace=False, p=p)) for _ in range(rows)]).astype(np.int32)
    else:
        ids = np.stack([np.sort(rng.permutation(e_total)[:top_k]) for _ in range(rows)]).astype(np.int32)
    weights = rng.random((rows, top_k), dtype=np.float32)
    weights = bf16_to_f32(f32_to_bf16(weights / weights.sum(-1, keepdims=True) * 2.5))
    amap, counts = onv.route_slots(ids, e_total)
    if m_max is None:
        m_max = rows
    else:  # fewer slots per expert than tokens: the caller guarantees no expert is routed more (llada2/kernels route)
        assert counts.max() <= m_max < rows
        amap = np.ascontiguousarray(amap[:, :m_max])
    if exact:
        w_codes = rng.integers(0, 256, (e_total, hidden, f // 2), dtype=np.uint8)
        a_codes = rng.integers(0, 256, (e_total * m_max, f // 2), dtype=np.uint8)
        pow2 = np.array([0x30, 0x38, 0x40, 0x48], dtype=np.uint8)  # E4M3 0.5, 1, 2, 4
        w_scales = pow2[rng.integers(0, 4, (e_total, hidden, f // 16))]
        a_scales = pow2[rng.integers(0, 4, (e_total * m_max, f // 16))]
        g2 = np.full(e_total, 2.0 ** -6, dtype=np.float32)
        weights = np.ones_like(weights) * 0.5
    else:
        w = rng.standard_normal((e_total, hidden, f)).astype(np.float32) * 0.02
        s2 = np.float32(np.abs(w).max() / 2688)
        q = [onv.quantize(w[e], s2) for e in range(e_total)]
        w_codes, w_scales = np.stack([c for c, _ in q]), np.stack([s for _, s in q])
        act = rng.standard_normal((e_total * m_max, f)).astype(np.float32) * 0.3
        a2 = np.float32(np.abs(act).max() / 2688)
        a_codes, a_scales = onv.quantize(act, a2)
        g2 = np.full(e_total, a2 * s2, dtype=np.float32)
    return dict(ids=ids, weights=weights.astype(np.float32), amap=amap, counts=counts, m_max=m_max, w_codes=w_codes,
                w_scales=w_scales, a_codes=a_codes, a_scales=a_scales, g2=g2, rows=rows, hidden=hidden, f=f,
                e_total=e_total, top_k=top_k)


def oracle_out(case, lo, e_local, shared=None):
    m_max = case["m_max"]
    y = onv.moe_down(case["a_codes"][lo * m_max:(lo + e_local) * m_max], case["a_scales"][lo * m_max:(lo + e_local) * m_max],
                     case["amap"], case["counts"], case["w_codes"][lo:lo + e_local], case["w_scales"][lo:lo + e_local],
                     case["g2"][lo:lo + e_local], lo, case["rows"] * case["top_k"], accumulate=np.float64)
    return onv.combine(y, case["ids"], case["weights"], lo, e_local, shared), y


def device_args(case, lo, e_local, dev="cuda"):
    from dlmrt_b200.quantization import nvfp4

    m_max = case["m_max"]
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    experts = {"lo": lo, "w2": t(case["w_codes"][lo:lo + e_local]),
               "s2": nvfp4.interleave_scales(t(case["w_scales"][lo:lo + e_local])), "g2": t(case["g2"][lo:lo + e_local])}
    buffers = nvfp4.Buffers(case["rows"], case["hidden"], case["top_k"], dev)
    args = dict(act_codes=t(case["a_codes"][lo * m_max:(lo + e_local) * m_max]),
                act_scales=t(case["a_scales"][lo * m_max:(lo + e_local) * m_max]), amap=t(case["amap"]),
                counts=t(case["counts"]), experts=experts, ids=t(case["ids"]), weights=t(case["weights"]),
                buffers=buffers, num_experts=case["e_total"])
    return args


def run_single(case, shared=None):
    from dlmrt_b200.quantization import nvfp4

    args = device_args(case, 0, case["e_total"])
    out = torch.empty(case["rows"], case["hidden"], dtype=torch.bfloat16, device="cuda")
    sh = to_torch(shared).cuda() if shared is not None else None
    for _ in range(2):  # twice on one workspace: the rendezvous counters must re-arm themselves
        nvfp4.moe_down(out=out, shared=sh, **args)
    torch.cuda.synchronize()
    return bits(out)


@pytest.mark.parametrize("rows, hidden, f, e_total, top_k", [(32, 2048, 512, 16, 4), (32, 2048, 512, 256, 8),
                                                            (64, 256, 704, 8, 2), (256, 2816, 704, 32, 8),
                                                            (256, 256, 512, 8, 8), (160, 512, 704, 4, 3)])
def test_exact_operands_match_bit_for_bit(rows, hidden, f, e_total, top_k):
    case = make_case(rows, hidden, f, e_total, top_k, seed=rows + f, exact=True)
    want, _ = oracle_out(case, 0, e_total)
    assert_same_bits(run_single(case), want, "exact NVFP4 expert down-projection")


def test_shapes_the_configs_reach_at_their_edges():
    """BASELINE config 4's real expert count under Zipf(1.2) routing at 32 rows; fewer slots per expert than tokens
    (m_max < rows); one expert that holds more than 128 rows at hidden 2048 (two row blocks of one work item list)."""
    for kw in (dict(rows=32, hidden=2048, f=512, e_total=256, top_k=8, seed=31, skew=True),
               dict(rows=64, hidden=2048, f=512, e_total=32, top_k=2, seed=32, m_max=16),
               dict(rows=256, hidden=2048, f=512, e_total=8, top_k=2, seed=33, hot=True)):
        case = make_case(exact=True, **kw)
        if kw.get("hot"):
            assert case["counts"][0] == 256 > 128
        want, _ = oracle_out(case, 0, kw["e_total"])
        assert_same_bits(run_single(case), want, f"{kw}")


def test_kernel_reproduces_the_reference_math_where_it_is_exact():
    """The golden case on which the reference's W4A4 torch statement of GEMM2 + combine rounds nowhere
    (tests/golden/make_moe_golden.py `exact`): the kernel must give the BF16 rounding of the reference's FP32 result,
    bit for bit. Hidden 256, F 128, 8 experts, top-2, 16 tokens."""
    from pathlib import Path

    g = np.load(Path(__file__).parent / "golden" / "moe_golden.npz")
    ids, weights = g["exact_ids"], g["exact_weights"]
    rows, top_k = ids.shape
    e_total, hidden, half_f = g["exact_down_packed"].shape
    a2, ws2 = g["exact_down_input_scale"], g["exact_down_scale2"]
    act = bf16_to_f32(g["exact_act"])
    amap, counts = onv.route_slots(ids, e_total)
    m_max = rows
    a_codes = np.zeros((e_total * m_max, half_f), dtype=np.uint8)
    a_scales = np.zeros((e_total * m_max, half_f // 8), dtype=np.uint8)
    for e in range(e_total):
        for j in range(counts[e]):
            c, sc = onv.quantize(act[amap[e, j]][None], a2[e])
            a_codes[e * m_max + j], a_scales[e * m_max + j] = c[0], sc[0]
    case = dict(ids=ids, weights=weights.astype(np.float32), amap=amap, counts=counts, m_max=m_max,
                w_codes=g["exact_down_packed"], w_scales=g["exact_down_scale"], a_codes=a_codes, a_scales=a_scales,
                g2=(a2 * ws2).astype(np.float32), rows=rows, hidden=hidden, f=half_f * 2, e_total=e_total, top_k=top_k)
    assert_same_bits(run_single(case), f32_to_bf16(g["exact_ref"]), "golden exact case")


@pytest.mark.parametrize("rows, hidden, f, e_total, top_k, skew", [(32, 2048, 512, 64, 8, False), (32, 2048, 512, 64, 8, True),
                                                                  (32, 2048, 512, 256, 8, True),
                                                                  (256, 2816, 704, 16, 8, False)])
def test_gaussian_operands_within_tolerance(rows, hidden, f, e_total, top_k, skew):
    """Per output row relative L2 <= 1e-2 against the W4A4 oracle on identical quantised inputs; with a shared-expert
    addend as well."""
    case = make_case(rows, hidden, f, e_total, top_k, seed=7, skew=skew)
    rng = np.random.default_rng(1)
    shared = f32_to_bf16(rng.standard_normal((rows, hidden)).astype(np.float32) * 0.05)
    for sh in (None, shared):
        want, _ = oracle_out(case, 0, e_total, sh)
        got = bf16_to_f32(run_single(case, sh)).astype(np.float64)
        ref = bf16_to_f32(want).astype(np.float64)
        rel = np.linalg.norm(got - ref, axis=1) / np.maximum(np.linalg.norm(ref, axis=1), 1e-30)
        assert rel.max() <= onv.GEMM2_REL_L2, rel.max()


@pytest.mark.parametrize("world, one_shot_bytes", [(1, None), (2, 0), (2, None), (8, 0), (8, None)])
def test_expert_parallel_loopback_matches_oracle(world, one_shot_bytes):
    """Experts split whole across emulated ranks; each rank's partial is exact (integer-like operands), so the fused
    reduction must equal the oracle's rank-ordered sum of the per-rank combines bit for bit, on every rank."""
    from dlmrt_b200.distributed.loopback import LoopbackWorld
    from dlmrt_b200.quantization import nvfp4

    rows, hidden, f, e_total, top_k = 32, 2048, 512, 64, 8
    case = make_case(rows, hidden, f, e_total, top_k, seed=world, exact=True)
    e_local = e_total // world
    lw = LoopbackWorld(world, one_shot_bytes=one_shot_bytes)  # None: 32 rows go over one NVLink hop; 0: two hops
    keep = []
    for rep in range(2):
        descs, partials = [], []
        for r in range(world):
            args = device_args(case, r * e_local, e_local)
            keep.append(args)
            descs.append(nvfp4.descriptor(**args))
            partials.append(oracle_out(case, r * e_local, e_local)[0])
        outs = lw.moe(descs, site=f"moe{rep}")
        torch.cuda.synchronize()
        lw.check()
        want = red.reduce(np.stack(partials))
        for r, out in enumerate(outs):
            assert_same_bits(bits(out), want, f"rep {rep} rank {r}")


@pytest.mark.parametrize("world", [1, 2])
def test_fused_residual_norm_after_the_experts(world):
    """The reduction's residual + RMSNorm variants behind the expert kernel (the post-reduction row kernel folded into
    the launch): residual stream bit-exact, normalised rows within one BF16 code point of the oracle."""
    from dlmrt_b200.distributed.loopback import LoopbackWorld
    from dlmrt_b200.quantization import nvfp4

    rows, hidden, f, e_total, top_k = 32, 2048, 512, 16, 4
    case = make_case(rows, hidden, f, e_total, top_k, seed=21, exact=True)
    e_local = e_total // world
    lw = LoopbackWorld(world)
    weight = randn_bf16(hidden, seed=3, std=0.1) + 1
    hs = [randn_bf16(rows, hidden, seed=4 + r) for r in range(world)]
    h_before = np.stack([bits(h) for h in hs])
    keep = [device_args(case, r * e_local, e_local) for r in range(world)]
    outs = lw.moe([nvfp4.descriptor(**a) for a in keep], site="moe.norm", hs=hs, weight=weight, eps=1e-6)
    torch.cuda.synchronize()
    lw.check()
    partials = np.stack([oracle_out(case, r * e_local, e_local)[0] for r in range(world)])
    want, h_after = red.reduce_norm(partials, bits(weight), 1e-6, 1.0, h_before)
    for r in range(world):
        assert_norm_close(bits(outs[r]), want, f"rank {r}")
        assert_same_bits(bits(hs[r]), h_after[r], f"residual of rank {r}")
