"""NVFP4 routed experts on the row-parallel hot path: formats, expert layout and the expert down-projection entry.

Mirror of the parts of the reference's `dlmrt/quantization/nvfp4.py` that sit on the path: the format (:1-12,23), the
packed top-k (`pack`, :275-277), an expert layout for this library's kernel (`b200_experts`, the counterpart of
`trtllm_experts` :89-121 / `triton_experts` :159-181) and the call that replaces the GEMM2 + finalize half of
`trtllm_moe` (:280-306), optionally fused with the reduction over ranks. GEMM1 (gate/up + activation + requantisation)
is the step before this path and is not part of it: the entry point takes GEMM2's input already quantised, in the
expert-major slot layout of `dlmrt/ops/triton/nvfp4_moe.py:11-12` (what its `_gate_up` kernel writes).

Nothing numeric runs in Python here: tensors are only laid out and handed to libdlmrt_b200.so.
"""

import ctypes as C

import torch

from .. import _lib
from .._lib import DlmMoe

E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def pack(ids, weights):
    """FlashInfer's packed top-k: expert << 16 | BF16 weight bits (nvfp4.py:275-277)."""
    return (ids << 16) | (weights.to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF)


def unpack(packed):
    """(ids int32, weights FP32 holding the BF16 routing weights) of a packed top-k."""
    ids = packed >> 16
    weights = (packed & 0xFFFF).to(torch.int16).view(torch.bfloat16).float()
    return ids.int(), weights


def interleave_scales(scales):
    """[..., n, f / 16] E4M3 block scales (linear, as exported) -> [..., n / 128, f / 64, 512] uint8 in the 128-row x
    4-scale atoms the block-scaled MMA reads from tensor memory: byte (r % 32) * 16 + (r / 32) * 4 + j of an atom is
    scale j of row r. Done once when the experts are loaded."""
    s = scales.view(torch.uint8)
    *lead, n, groups = s.shape
    if n % 128 or groups % 4:
        raise ValueError(f"scales {tuple(s.shape)}: rows must be a multiple of 128 and f a multiple of 64")
    s = s.reshape(*lead, n // 128, 4, 32, groups // 4, 4)           # (.., tile, q = r / 32, l = r % 32, step, j)
    d = len(lead)
    s = s.permute(*range(d), d, d + 3, d + 2, d + 1, d + 4)           # (.., tile, step, l, q, j)
    return s.contiguous().reshape(*lead, n // 128, groups // 4, 512)


def b200_experts(parts, layer, lo, count, device):
    """Layer `layer`'s experts [lo, lo + count) for this library: down-projection codes as exported, their block
    scales in atoms, and per expert the GEMM2 alpha (input scale x weight scale) and the GEMM2 input quantisation
    scale. `parts[(layer, expert, proj, field)]` are the checkpoint's tensors, as in the reference's loaders."""
    def get(e, field):
        return parts[(layer, e, "down", field)].to(device)

    w2 = torch.stack([get(e, "weight") for e in range(lo, lo + count)]).contiguous()
    s2 = torch.stack([get(e, "weight_scale").view(torch.uint8) for e in range(lo, lo + count)])
    a2 = torch.stack([get(e, "input_scale").float().reshape(()) for e in range(lo, lo + count)])
    ws2 = torch.stack([get(e, "weight_scale_2").float().reshape(()) for e in range(lo, lo + count)])
    return {"backend": "b200", "lo": lo, "w2": w2, "s2": interleave_scales(s2), "g2": (a2 * ws2).contiguous(),
            "a2_inv": (1 / a2).contiguous()}


class Buffers:
    """Scratch of the expert down-projection for up to `rows` tokens: the per-(token, expert) BF16 outputs and the
    rendezvous words. One per chain; zero-initialised once."""

    def __init__(self, rows, hidden, top_k, device):
        nbytes = _lib.lib().dlm_moe_workspace_bytes(rows, hidden, top_k)
        self.rows, self.hidden, self.top_k = rows, hidden, top_k
        self.workspace = torch.zeros(nbytes, device=device, dtype=torch.uint8)


def descriptor(act_codes, act_scales, amap, counts, experts, ids, weights, buffers, num_experts, shared=None):
    """The DlmMoe of one call. Keeps nothing alive: the caller owns every tensor."""
    rows, top_k = ids.shape
    n, half_f = experts["w2"].shape[1], experts["w2"].shape[2]
    m = DlmMoe()
    m.act_codes, m.act_scales = act_codes.data_ptr(), act_scales.data_ptr()
    m.amap, m.counts = amap.data_ptr(), counts.data_ptr()
    m.w_codes, m.w_scales, m.g2 = experts["w2"].data_ptr(), experts["s2"].data_ptr(), experts["g2"].data_ptr()
    m.ids, m.weights = ids.data_ptr(), weights.data_ptr()
    m.shared = shared.data_ptr() if shared is not None else None
    m.m, m.n, m.f, m.top_k = rows, n, half_f * 2, top_k
    m.m_max = amap.shape[1]
    m.lo, m.e_local, m.e_total = experts["lo"], experts["w2"].shape[0], num_experts
    m.workspace, m.workspace_bytes = buffers.workspace.data_ptr(), buffers.workspace.numel()
    for t, dtype in ((amap, torch.int32), (counts, torch.int32), (ids, torch.int32), (weights, torch.float32)):
        if t.dtype != dtype or not t.is_contiguous():
            raise ValueError(f"expected a contiguous {dtype} tensor, got {t.dtype}")
    if act_codes.shape[0] != m.e_local * m.m_max or act_codes.shape[1] != half_f:
        raise ValueError(f"activation slots {tuple(act_codes.shape)}: expected [{m.e_local * m.m_max}, {half_f}]")
    return m


def moe_down(act_codes, act_scales, amap, counts, experts, ids, weights, buffers, out, num_experts, shared=None,
             group=None, site=None, chain=0, h=None, norm_weight=None, eps=0.0, scale=1.0):
    """out = sum over each token's experts in this rank's [lo, lo + count) of weight * expert_down(activation)
    [+ shared], BF16; with `group`, the sum over ranks of that, in the call site's buffer (one fused launch).

    `act_codes` [count * m_max, F / 2] uint8 and `act_scales` [count * m_max, F / 16] E4M3: GEMM2's quantised input in
    expert-major slots; `amap` [num_experts, m_max] / `counts` [num_experts] the slot map of the router; `ids` int32 /
    `weights` FP32 [rows, top_k] hold global expert ids and the BF16-rounded routing weights.

    With `group` and `norm_weight` the owner rows are also normalised before the all-gather, and with `h` added to the
    residual stream first, exactly as `Group.reduce_norm` does: the row kernel that follows the reduction in the
    reference (`rmsnorm(h, weight, delta=reduced)`, dlmrt/ops/triton/core.py:29-56) folded into the same launch."""
    m = descriptor(act_codes, act_scales, amap, counts, experts, ids, weights, buffers, num_experts, shared)
    stream = torch.cuda.current_stream(act_codes.device).cuda_stream
    if group is None:
        _lib.check(_lib.lib().dlm_moe_nvfp4(C.byref(m), out.data_ptr(), out.stride(0), 1, stream), "moe_down")
        return out
    mode = _lib.REDUCE if norm_weight is None else _lib.REDUCE_NORM_RESIDUAL if h is not None else _lib.REDUCE_NORM
    comm, reduced = group._comm(m.m, m.n, site, chain, mode, h, norm_weight, eps, scale)
    _lib.check(_lib.lib().dlm_rowpar_nvfp4_moe(C.byref(m), C.byref(comm), stream), f"moe_down {site}")
    group._last[chain] = reduced
    return reduced
