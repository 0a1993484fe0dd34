"""Generates tests/golden/moe_golden.npz: the REFERENCE's own W4A4 expert math on seeded inputs, run on the CPU.

Run where the reference is checked out (it cannot travel to the GPU box, the vectors do):

    python tests/golden/make_moe_golden.py /path/to/reference

It imports, unmodified, from that tree
  dlmrt.quantization.nvfp4.expert_weights / dequantize / pack   (dlmrt/quantization/nvfp4.py:41-57,275-277)
  tests/test_nvfp4.py  modelopt_quantize / fake_quantize         (tests/test_nvfp4.py:21-46)
and evaluates, with them, exactly the torch statement of the expert pipeline that the reference's own tests hold its
B200 back-end to (tests/test_llada_nvfp4.py:62-94 `swiglu_case`, tests/test_nvfp4.py:102-134 `w4a4_case`):

    xq   = fake_quantize(x, a13)
    mid  = bf16(xq[rows] @ w13[e]^T);  act = bf16(silu | gelu_tanh (mid[:, :F]) * mid[:, F:])
    ref += (fake_quantize(act, a2) @ w2[e]^T) * weight            (FP32, the W4A4 reference)
    truth: the same without any quantisation of activations

Three cases at small sizes (hidden 256, F 128, 8 experts, top-2, 16 tokens; seeded Gaussians with the reference's
distributions: weights N(0, 0.02), x 0.5 N(0, 1), a13 = 3 / 2688, a2 = 0.4 / 2688):
  swiglu, geglu   the whole pipeline; stored with its intermediates so GEMM1 and GEMM2 can each be pinned alone
  exact           GEMM2 + combine only, on operands built so that every product, sum and BF16 rounding of the
                  reference's statement is exact (power-of-two scales, small integers); there the reference's FP32
                  result must be reproduced bit for bit
"""

import sys
from pathlib import Path

import numpy as np
import torch

H, F, E, K, T = 256, 128, 8, 2, 16


def bits(t):
    return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)


def experts(modelopt_quantize, down_only=None):
    a13, a2 = torch.tensor(3.0 / 2688), torch.tensor(0.4 / 2688)
    parts = {}
    for e in range(E):
        gate, up, down = (torch.randn(*s) * 0.02 for s in ((F, H), (F, H), (H, F)))
        s13 = torch.maximum(gate.abs().max(), up.abs().max()) / 2688
        for proj, w, s2, a in (("gate", gate, s13, a13), ("up", up, s13, a13), ("down", down, down.abs().max() / 2688, a2)):
            packed, scale = modelopt_quantize(w, s2)
            parts[(0, e, proj, "weight")], parts[(0, e, proj, "weight_scale")] = packed, scale
            parts[(0, e, proj, "weight_scale_2")], parts[(0, e, proj, "input_scale")] = s2.float(), a.float()
    return parts, a13, a2


def store(out, prefix, parts):
    for proj in ("gate", "up", "down"):
        out[f"{prefix}_{proj}_packed"] = torch.stack([parts[(0, e, proj, "weight")] for e in range(E)]).numpy()
        out[f"{prefix}_{proj}_scale"] = torch.stack([parts[(0, e, proj, "weight_scale")].view(torch.uint8)
                                                     for e in range(E)]).numpy()
        out[f"{prefix}_{proj}_scale2"] = torch.stack([parts[(0, e, proj, "weight_scale_2")].reshape(())
                                                      for e in range(E)]).numpy()
        out[f"{prefix}_{proj}_input_scale"] = torch.stack([parts[(0, e, proj, "input_scale")].reshape(())
                                                           for e in range(E)]).numpy()


def pipeline(nvfp4, fake_quantize, parts, a13, a2, x, ids, weights, activation):
    w13, w2 = nvfp4.expert_weights(parts, 0, 0, E, "cpu")
    ref, truth = torch.zeros(T, H), torch.zeros(T, H)
    act_pairs, actq_pairs = torch.zeros(T * K, F, dtype=torch.bfloat16), torch.zeros(T * K, F, dtype=torch.bfloat16)
    xq = fake_quantize(x, a13).float()
    fn = torch.nn.functional.silu if activation == "swiglu" else lambda t: torch.nn.functional.gelu(t, approximate="tanh")
    for e in range(E):
        rows, slot = torch.where(ids == e)
        if rows.numel():
            mid = (xq[rows] @ w13[e].float().t()).to(torch.bfloat16).float()
            act = (fn(mid[:, :F]) * mid[:, F:]).to(torch.bfloat16)
            actq = fake_quantize(act, a2)
            act_pairs[rows * K + slot], actq_pairs[rows * K + slot] = act, actq
            ref[rows] += (actq.float() @ w2[e].float().t()) * weights[rows, slot, None]
            mid = x[rows].float() @ w13[e].float().t()
            truth[rows] += ((fn(mid[:, :F]) * mid[:, F:]) @ w2[e].float().t()) * weights[rows, slot, None]
    return xq, act_pairs, actq_pairs, ref, truth


def exact_case(nvfp4, fake_quantize, modelopt_quantize):
    """GEMM2 + combine where nothing rounds. Every block of 16 holds one +-6 that pins its scale to a power of two
    (weights at position 0, activations at position 1, so the two never multiply); the other 14 positions hold small
    integers, so an expert's output is an integer of at most 7 bits times a power of two."""
    g = torch.Generator().manual_seed(3)
    ws2, a2 = torch.tensor(2.0 ** -9), torch.tensor(2.0 ** -7)

    def blocks(rows, cols, pin, choices):
        v = torch.tensor(choices)[torch.randint(0, len(choices), (rows, cols), generator=g)]
        v = v.view(rows, cols // 16, 16)
        v[:, :, 0], v[:, :, 1] = 0.0, 0.0
        v[:, :, pin] = 6.0 * (torch.randint(0, 2, (rows, cols // 16), generator=g) * 2 - 1)
        return v.view(rows, cols)

    parts = {}
    for e in range(E):
        down = blocks(H, F, 0, [0.0, 0.0, 1.0, -1.0]) * ws2 * 4          # block scale 4, codes as drawn
        packed, scale = modelopt_quantize(down, ws2)
        parts[(0, e, "down", "weight")], parts[(0, e, "down", "weight_scale")] = packed, scale
        parts[(0, e, "down", "weight_scale_2")], parts[(0, e, "down", "input_scale")] = ws2.float(), a2.float()
        assert torch.equal(nvfp4.dequantize(packed, scale, ws2).float(), down)
    act = (blocks(T * K, F, 1, [0.0, 1.0, -1.0, 2.0, -2.0]) * a2 * 2).to(torch.bfloat16)  # block scale 2
    assert torch.equal(fake_quantize(act, a2).float(), act.float())
    ids = torch.rand(T, E, generator=g).topk(K, -1).indices.sort(-1).values.int()
    weights = torch.tensor([1.0, 0.5, 0.25, 2.0])[torch.randint(0, 4, (T, K), generator=g)]
    w2 = torch.stack([nvfp4.dequantize(parts[(0, e, "down", "weight")], parts[(0, e, "down", "weight_scale")], ws2)
                      for e in range(E)])
    ref = torch.zeros(T, H)
    for e in range(E):
        rows, slot = torch.where(ids == e)
        if rows.numel():
            y = fake_quantize(act[rows * K + slot], a2).float() @ w2[e].float().t()
            assert torch.equal(y.to(torch.bfloat16).float(), y)  # the per-(token, expert) BF16 rounding is exact
            ref[rows] += y * weights[rows, slot, None]
    return parts, act, ids, weights, ref


def main(reference):
    sys.path.insert(0, str(reference))
    sys.path.insert(0, str(Path(reference) / "tests"))
    from dlmrt.quantization import nvfp4
    from test_nvfp4 import fake_quantize, modelopt_quantize

    out = {"dims": np.array([H, F, E, K, T], dtype=np.int32)}
    for seed, activation in ((0, "swiglu"), (1, "geglu")):
        torch.manual_seed(seed)
        parts, a13, a2 = experts(modelopt_quantize)
        x = (torch.randn(T, H) * 0.5).to(torch.bfloat16)
        ids = torch.rand(T, E).topk(K, -1).indices.sort(-1).values.int()
        weights = torch.rand(T, K)
        weights = (weights / weights.sum(-1, keepdim=True) * 2.5).to(torch.bfloat16).float()
        xq, act, actq, ref, truth = pipeline(nvfp4, fake_quantize, parts, a13, a2, x, ids, weights, activation)
        p = activation
        store(out, p, parts)
        out[f"{p}_x"], out[f"{p}_xq"] = bits(x), bits(xq)
        out[f"{p}_ids"], out[f"{p}_weights"] = ids.numpy(), weights.numpy()
        out[f"{p}_topk_packed"] = nvfp4.pack(ids, weights).numpy()
        out[f"{p}_act"], out[f"{p}_actq"] = bits(act), bits(actq)
        out[f"{p}_ref"], out[f"{p}_truth"] = ref.numpy(), truth.numpy()
    parts, act, ids, weights, ref = exact_case(nvfp4, fake_quantize, modelopt_quantize)
    for field, name in (("weight", "packed"), ("weight_scale", "scale"), ("weight_scale_2", "scale2"),
                        ("input_scale", "input_scale")):
        ts = [parts[(0, e, "down", field)] for e in range(E)]
        out[f"exact_down_{name}"] = torch.stack([t.view(torch.uint8) if name == "scale" else t.reshape(t.shape or ())
                                                 for t in ts]).numpy()
    out["exact_act"], out["exact_ids"], out["exact_weights"], out["exact_ref"] = bits(act), ids.numpy(), weights.numpy(), \
        ref.numpy()
    np.savez_compressed(Path(__file__).with_name("moe_golden.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(Path(sys.argv[1]))
