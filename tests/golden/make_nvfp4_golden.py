"""Generates tests/golden/nvfp4_golden.npz by running the REFERENCE's own code on seeded inputs.

Run in a container that has the reference checked out (it cannot travel to the GPU box, the vectors do):

    python tests/golden/make_nvfp4_golden.py /path/to/reference

It imports, unmodified, from that tree:
  dlmrt.quantization.nvfp4.dequantize / pack            (dlmrt/quantization/nvfp4.py:41-46, 275-277)
  tests/test_nvfp4.py modelopt_quantize / fake_quantize  (the reference's transcription of ModelOpt's quantiser,
                                                          tests/test_nvfp4.py:21-46)
and stores their inputs and outputs as small arrays. All inputs are seeded synthetic tensors with the shapes' value
distributions (weights ~ N(0, 0.02), one all-zero block as in tests/test_nvfp4.py:53).
"""

import sys
from pathlib import Path

import numpy as np
import torch


def main(reference):
    sys.path.insert(0, str(reference))
    sys.path.insert(0, str(Path(reference) / "tests"))
    from dlmrt.quantization import nvfp4
    from test_nvfp4 import fake_quantize, modelopt_quantize

    torch.manual_seed(0)
    out = {}
    for name, (n, k, std) in {"w": (64, 128, 0.02), "act": (24, 64, 0.5)}.items():
        w = torch.randn(n, k) * std
        w[:, :16] = 0
        w[1, 16:32] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5,
                                    -3.5, -5.0, -6.0]) * w[1, 16:32].abs().max() / 6  # values on rounding ties
        scale2 = w.abs().max() / (6 * 448)
        packed, scale = modelopt_quantize(w, scale2)
        deq = nvfp4.dequantize(packed, scale, scale2)
        fake = fake_quantize(w, scale2)
        assert torch.equal(deq, fake)
        out[f"{name}_x"] = w.numpy()
        out[f"{name}_scale2"] = scale2.numpy()
        out[f"{name}_packed"] = packed.numpy()
        out[f"{name}_scale"] = scale.view(torch.uint8).numpy()
        out[f"{name}_deq"] = deq.view(torch.int16).numpy().view(np.uint16)
    ids = torch.rand(16, 32).topk(8, -1).indices.sort(-1).values.int()
    weights = torch.rand(16, 8)
    weights = (weights / weights.sum(-1, keepdim=True) * 2.5)
    out["ids"] = ids.numpy()
    out["weights"] = weights.numpy()
    out["topk_packed"] = nvfp4.pack(ids, weights).numpy()
    out["e2m1"] = np.array(nvfp4.E2M1, dtype=np.float32)
    # every E4M3 byte through torch's decoder, the dtype the reference views scales as (nvfp4.py:119,179)
    out["e4m3_table"] = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    np.savez_compressed(Path(__file__).with_name("nvfp4_golden.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(Path(sys.argv[1]))
