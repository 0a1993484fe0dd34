"""The front half of the NVFP4 routed experts (router top-k, slot bookkeeping, input quantisation, GEMM1 + activation +
re-quantisation) and the whole `trtllm_moe` call with the reference's signature, against the CPU oracle and against the
reference's own W4A4 torch math (tests/golden/moe_golden.npz, made by tests/golden/make_moe_golden.py)."""

from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from gpu_util import assert_same_bits, bits
from oracle import nvfp4 as onv
from oracle import reduce as red
from oracle.bf16 import bf16_to_f32, f32_to_bf16, to_torch

pytestmark = pytest.mark.gpu
G = np.load(Path(__file__).parent / "golden" / "moe_golden.npz")


def rel(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


def golden_parts(prefix, dev="cuda"):
    """The golden case as the checkpoint dictionary the reference's loaders take: parts[(layer, expert, proj, field)]."""
    parts = {}
    e_total = G[f"{prefix}_gate_packed"].shape[0]
    for proj in ("gate", "up", "down"):
        for e in range(e_total):
            parts[(0, e, proj, "weight")] = torch.from_numpy(G[f"{prefix}_{proj}_packed"][e]).to(dev)
            parts[(0, e, proj, "weight_scale")] = torch.from_numpy(G[f"{prefix}_{proj}_scale"][e]).to(dev)
            parts[(0, e, proj, "weight_scale_2")] = torch.tensor(G[f"{prefix}_{proj}_scale2"][e]).to(dev)
            parts[(0, e, proj, "input_scale")] = torch.tensor(G[f"{prefix}_{proj}_input_scale"][e]).to(dev)
    return parts, e_total


def oracle_front(prefix, lo=0, count=None, quantized=None):
    e_total = G[f"{prefix}_gate_packed"].shape[0]
    count = count or e_total
    a13, a2 = G[f"{prefix}_gate_input_scale"], G[f"{prefix}_down_input_scale"]
    g1 = (a13 * G[f"{prefix}_gate_scale2"]).astype(np.float32)[lo:lo + count]
    sl = slice(lo, lo + count)
    return onv.moe_front(bf16_to_f32(G[f"{prefix}_x"]), np.float32(1) / a13[0], G[f"{prefix}_ids"], e_total,
                         (G[f"{prefix}_gate_packed"][sl], G[f"{prefix}_gate_scale"][sl]),
                         (G[f"{prefix}_up_packed"][sl], G[f"{prefix}_up_scale"][sl]), g1,
                         (np.float32(1) / a2).astype(np.float32)[sl], lo, prefix, quantized=quantized)


def codes_close(got_codes, got_scales, want_codes, want_scales, what, fraction=1e-2):
    """The GPU's approximate reciprocals and exponentials (and, behind GEMM1, the FP4 tensor cores' own summation of
    each 64-element group) against the oracle's exact float64 dots: a value near a rounding boundary may come out one
    code apart, and a block maximum near a boundary may move the block's scale by one E4M3 step. Never more than one
    step, and only on a small `fraction` of the blocks / codes."""
    scale_diff = (got_scales != want_scales).mean()
    assert scale_diff <= fraction, f"{what}: {scale_diff:.4%} of the block scales differ"
    step = np.abs(got_scales.astype(np.int32) - want_scales.astype(np.int32))
    assert step.max(initial=0) <= 1, f"{what}: a block scale is off by more than one E4M3 step"
    g, w = onv.unpack_codes(got_codes).astype(np.int32), onv.unpack_codes(want_codes).astype(np.int32)
    same_scale = np.repeat(got_scales == want_scales, 16, axis=-1)
    differ = (g != w) & same_scale
    assert differ.mean() <= fraction, f"{what}: {differ.mean():.4%} of the codes differ"
    mag = np.abs((g & 7) - (w & 7))
    assert mag[differ].max(initial=0) <= 1, f"{what}: a code is off by more than one step"


@pytest.mark.parametrize("prefix", ["swiglu", "geglu"])
def test_front_half_matches_the_oracle(prefix):
    """Slot map and unpacked top-k exact; quantised rows and re-quantised activations equal to the oracle's except
    where approximate reciprocals sit on a rounding boundary."""
    from dlmrt_b200.quantization import nvfp4

    parts, e_total = golden_parts(prefix)
    experts = nvfp4.b200_experts(parts, 0, 0, e_total, "cuda")
    x = to_torch(G[f"{prefix}_x"]).cuda()
    packed = torch.from_numpy(G[f"{prefix}_topk_packed"]).cuda()
    rows, k = packed.shape
    hidden, f = x.shape[1], G[f"{prefix}_gate_packed"].shape[1]
    out = torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda")
    for _ in range(2):  # twice on the same buffers
        nvfp4.trtllm_moe(x, packed, experts, out, e_total, 0, f, activation=prefix)
    torch.cuda.synchronize()
    b = experts["_buffers"][rows]
    amap, counts, act_codes, act_scales = oracle_front(prefix)
    assert np.array_equal(b.ids.cpu().numpy(), G[f"{prefix}_ids"])
    assert np.array_equal(b.weights.cpu().numpy(), G[f"{prefix}_weights"])
    assert np.array_equal(b.counts.cpu().numpy(), counts)
    got_amap = b.amap.cpu().numpy()
    for e in range(e_total):
        assert np.array_equal(got_amap[e, :counts[e]], amap[e, :counts[e]]), f"slot map of expert {e}"
    xq, xs = onv.quantize_fast(bf16_to_f32(G[f"{prefix}_x"]), np.float32(1) / G[f"{prefix}_gate_input_scale"][0])
    slot_codes, slot_scales = b.slot_codes.cpu().numpy(), b.slot_scales.cpu().numpy()
    used = np.concatenate([np.arange(e * rows, e * rows + counts[e]) for e in range(e_total)])
    tokens = np.concatenate([amap[e, :counts[e]] // k for e in range(e_total)])
    codes_close(slot_codes[used], slot_scales[used], xq[tokens], xs[tokens], "quantised input rows")
    # GEMM1 + activation + re-quantisation, fed with the very rows the GPU quantised (so that a flipped input code
    # does not count against it).
    a13, a2 = G[f"{prefix}_gate_input_scale"], G[f"{prefix}_down_input_scale"]
    g1 = (a13 * G[f"{prefix}_gate_scale2"]).astype(np.float32)
    got_codes, got_scales = b.act_codes.cpu().numpy(), b.act_scales.cpu().numpy()
    want_codes, want_scales = np.zeros_like(got_codes), np.zeros_like(got_scales)
    for e in range(e_total):
        if counts[e]:
            sl = slice(e * rows, e * rows + counts[e])
            want_codes[sl], want_scales[sl], _ = onv.expert_gate_up(
                slot_codes[sl], slot_scales[sl], G[f"{prefix}_gate_packed"][e], G[f"{prefix}_gate_scale"][e],
                G[f"{prefix}_up_packed"][e], G[f"{prefix}_up_scale"][e], g1[e], np.float32(1) / a2[e], prefix)
    codes_close(got_codes[used], got_scales[used], want_codes[used], want_scales[used], "re-quantised activations", 5e-2)


@pytest.mark.parametrize("prefix", ["swiglu", "geglu"])
def test_trtllm_moe_within_the_reference_bounds(prefix):
    """The whole call with the reference's signature against the reference's W4A4 torch math: rel(out, ref) < 0.08 and
    |rel(out, truth) - rel(ref, truth)| < 0.02, the bounds of tests/test_llada_nvfp4.py:107-114 and
    tests/test_nvfp4.py:147-152; and equal to the oracle's pipeline to BF16 level."""
    from dlmrt_b200.quantization import nvfp4

    parts, e_total = golden_parts(prefix)
    experts = nvfp4.b200_experts(parts, 0, 0, e_total, "cuda")
    x = to_torch(G[f"{prefix}_x"]).cuda()
    ids, weights = torch.from_numpy(G[f"{prefix}_ids"]).cuda(), torch.from_numpy(G[f"{prefix}_weights"]).cuda()
    packed = nvfp4.pack(ids, weights)
    assert np.array_equal(packed.cpu().numpy(), G[f"{prefix}_topk_packed"])
    f = G[f"{prefix}_gate_packed"].shape[1]
    out = torch.empty_like(x)
    nvfp4.trtllm_moe(x, packed, experts, out, e_total, 0, f, activation=prefix)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    ref, truth = G[f"{prefix}_ref"], G[f"{prefix}_truth"]
    assert rel(got, ref) < 0.08
    assert abs(rel(got, truth) - rel(ref, truth)) < 0.02
    amap, counts, act_codes, act_scales = oracle_front(prefix)
    a2, ws2 = G[f"{prefix}_down_input_scale"], G[f"{prefix}_down_scale2"]
    y = onv.moe_down(act_codes, act_scales, amap, counts, G[f"{prefix}_down_packed"], G[f"{prefix}_down_scale"],
                     (a2 * ws2).astype(np.float32), 0, ids.numel())
    want = bf16_to_f32(onv.combine(y, G[f"{prefix}_ids"], G[f"{prefix}_weights"], 0, e_total))
    assert rel(got, want) < 5e-2  # a fraction of a percent of the activation codes flip (approximate exp / reciprocal)


def test_prequantised_input_and_expert_parallel_ranks():
    """DiffusionGemma's call: x None, the input already quantised (dlmrt/models/diffusion_gemma/experts.py:108-114), through
    the `Experts` mirror with router logits; and the experts split over two ranks, whose partial sums add up to the
    one-rank result's inputs (checked through the oracle's rank-ordered reduction of the two GPU partials)."""
    from dlmrt_b200.quantization import nvfp4

    prefix = "geglu"
    parts, e_total = golden_parts(prefix)
    rows, hidden = G[f"{prefix}_x"].shape
    f = G[f"{prefix}_gate_packed"].shape[1]
    config = SimpleNamespace(top_k_experts=2, hidden_size=hidden, num_experts=e_total, moe_intermediate_size=f)
    rng = np.random.default_rng(9)
    logits = to_torch(f32_to_bf16(rng.standard_normal((rows, e_total)).astype(np.float32))).cuda()
    scale = to_torch(f32_to_bf16(rng.random(e_total, dtype=np.float32) + 0.5)).cuda()
    ids, w, packed = onv.route_packed(bits(logits), bits(scale), 2)
    xq, xs = onv.quantize_fast(bf16_to_f32(G[f"{prefix}_x"]), np.float32(1) / G[f"{prefix}_gate_input_scale"][0])
    partials = []
    for lo, count in ((0, e_total // 2), (e_total // 2, e_total // 2)):
        layer = {"fp4": nvfp4.b200_experts(parts, 0, lo, count, "cuda"), "expert_scale": scale}
        experts = nvfp4.Experts(config, lo, rows, "cuda")
        _, codes, scales = experts.quantized(layer)
        codes.copy_(torch.from_numpy(xq))
        scales.copy_(torch.from_numpy(xs))
        out = torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda")
        experts(None, logits, layer, out)
        torch.cuda.synchronize()
        got_ids, got_w = nvfp4.unpack(experts.packed[:rows])
        assert np.array_equal(got_ids.cpu().numpy(), ids)
        assert np.abs(got_w.cpu().numpy() - w).max() <= np.abs(w).max() * 2.0 ** -7  # fast exp: a BF16 step at most
        partials.append(bits(out))
        # this rank's oracle: same routing, same pre-quantised rows
        a13, a2 = G[f"{prefix}_gate_input_scale"], G[f"{prefix}_down_input_scale"]
        sl = slice(lo, lo + count)
        amap, counts, act_codes, act_scales = onv.moe_front(
            None, None, ids, e_total, (G[f"{prefix}_gate_packed"][sl], G[f"{prefix}_gate_scale"][sl]),
            (G[f"{prefix}_up_packed"][sl], G[f"{prefix}_up_scale"][sl]), (a13 * G[f"{prefix}_gate_scale2"]).astype(np.float32)[sl],
            (np.float32(1) / a2).astype(np.float32)[sl], lo, prefix, quantized=(xq, xs))
        y = onv.moe_down(act_codes, act_scales, amap, counts, G[f"{prefix}_down_packed"][sl], G[f"{prefix}_down_scale"][sl],
                         (a2 * G[f"{prefix}_down_scale2"]).astype(np.float32)[sl], lo, rows * 2)
        want = bf16_to_f32(onv.combine(y, ids, got_w.cpu().numpy(), lo, count))
        assert rel(bf16_to_f32(partials[-1]), want) < 5e-2, f"rank with experts [{lo}, {lo + count})"
    assert red.reduce(np.stack(partials)).shape == (rows, hidden)


def test_down_projection_is_deferred_into_the_reduction():
    """`out` a symmetric partial of the experts' group: trtllm_moe runs the front half and leaves the down-projection to
    the Group.reduce that follows, one fused launch; same bits as the unfused call."""
    from dlmrt_b200 import _lib
    from dlmrt_b200.distributed.parallel import Group
    from dlmrt_b200.quantization import nvfp4

    prefix = "swiglu"
    parts, e_total = golden_parts(prefix)
    g = Group.local("cuda:0")
    experts = nvfp4.b200_experts(parts, 0, 0, e_total, "cuda", group=g)
    x = to_torch(G[f"{prefix}_x"]).cuda()
    packed = torch.from_numpy(G[f"{prefix}_topk_packed"]).cuda()
    f = G[f"{prefix}_gate_packed"].shape[1]
    plain = torch.empty_like(x)
    nvfp4.trtllm_moe(x, packed, experts, plain, e_total, 0, f, activation=prefix)
    before = _lib.lib().dlm_launch_count()
    partial = g.symmetric("moe.partial", tuple(x.shape))
    p = nvfp4.trtllm_moe(x, packed, experts, partial, e_total, 0, f, activation=prefix)
    assert _lib.lib().dlm_launch_count() == before + 2   # bookkeeping + GEMM1; the down-projection waits
    out = g.reduce(p, site="0.moe", chain=1)
    assert _lib.lib().dlm_launch_count() == before + 3   # one fused launch
    torch.cuda.synchronize()
    g.check()
    assert_same_bits(bits(out), bits(plain), "fused vs unfused")
