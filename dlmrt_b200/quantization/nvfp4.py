"""NVFP4 routed experts on the row-parallel hot path: formats, expert layout and the MoE entry points.

Mirror of the parts of the reference's `dlmrt/quantization/nvfp4.py` that sit on the path: the format (:1-12,23), the
packed top-k (`pack`, :275-277), an expert layout for this library's kernels (`b200_experts`, the counterpart of
`trtllm_experts` :89-121 / `triton_experts` :159-181) and `trtllm_moe` (:280-306) with the reference's signature: the
whole routed-expert call (input quantisation, GEMM1 + activation + re-quantisation, GEMM2, weighted combine), which the
reference hands to FlashInfer's TRT-LLM-gen kernels on a B200. `Experts` mirrors DiffusionGemma's `TrtllmExperts`
(dlmrt/models/diffusion_gemma/experts.py:47-114). When the output is a tensor-parallel group's symmetric partial, the
down-projection half is deferred into the `Group.reduce*` that follows, one fused launch. `moe_down` is that half
alone, for callers that hold GEMM2's input already quantised in the expert-major slot layout of
`dlmrt/ops/triton/nvfp4_moe.py:11-12`.

Nothing numeric runs in Python here: tensors are only laid out and handed to libdlmrt_b200.so.
"""

import ctypes as C

import torch

from .. import _lib
from .._lib import DlmMoe, DlmMoeFront

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


def tile_codes(codes):
    """[..., n, k / 2] uint8 codes -> the streaming layout of the expert kernels: [..., n / 128, ceil(k / 256)] tiles of
    128 rows x 128 bytes, each 16 KB tile contiguous and already in the 128-byte-swizzled order it has in shared memory
    (16-byte chunk c of tile row r at chunk position c ^ (r % 8)); a last tile that k does not fill is zero-padded. One
    bulk copy then brings a tile in, and an expert's slab is a contiguous run of HBM. Done once when the experts load."""
    *lead, n, row_bytes = codes.shape
    if n % 128 or row_bytes % 16:
        raise ValueError(f"codes {tuple(codes.shape)}: rows must be a multiple of 128 and row bytes of 16")
    if row_bytes % 128:
        codes = torch.nn.functional.pad(codes, (0, 128 - row_bytes % 128))
        row_bytes = codes.shape[-1]
    d = len(lead)
    t = codes.reshape(*lead, n // 128, 128, row_bytes // 128, 8, 16)
    t = t.permute(*range(d), d, d + 2, d + 1, d + 3, d + 4)          # (.., tile row, tile col, r, chunk, 16 bytes)
    r = torch.arange(128, device=codes.device).view(128, 1)
    c = torch.arange(8, device=codes.device).view(1, 8)
    src = (c ^ (r % 8)).view(*([1] * (d + 2)), 128, 8, 1).expand(*t.shape)   # position p holds chunk p ^ (r % 8)
    return torch.gather(t, d + 3, src).contiguous()


def interleave_gate_up(gate, up):
    """[..., F, X] gate and up rows -> [..., 2F, X] with row 2i = gate row i, row 2i + 1 = up row i: the order GEMM1's
    kernel wants, so that a gate value and its up value land in neighbouring lanes of the accumulator."""
    return torch.stack((gate, up), dim=-2).flatten(-3, -2).contiguous()


def b200_experts(parts, layer, lo, count, device, group=None):
    """Layer `layer`'s experts [lo, lo + count) for this library (counterpart of `trtllm_experts`, nvfp4.py:89-121):
    codes as exported (GEMM1 rows interleaved gate / up), block scales in 128 x 4 atoms, and per expert the GEMM
    alphas (input scale x weight scale) and the reciprocal input scales. Gate and up must share their per-tensor
    scale and all experts one GEMM1 input scale, as the reference requires (nvfp4.py:75-86,103-104).
    `parts[(layer, expert, proj, field)]` are the checkpoint's tensors, as in the reference's loaders. `group`: the
    tensor-parallel group whose reductions the down-projection may be fused into."""
    def get(e, proj, field):
        return parts[(layer, e, proj, field)].to(device)

    def scalars(proj, field):
        return torch.stack([get(e, proj, field).float().reshape(()) for e in range(lo, lo + count)])

    experts = range(lo, lo + count)
    w2 = torch.stack([get(e, "down", "weight") for e in experts]).contiguous()
    s2 = torch.stack([get(e, "down", "weight_scale").view(torch.uint8) for e in experts])
    a2, ws2 = scalars("down", "input_scale"), scalars("down", "weight_scale_2")
    out = {"backend": "b200", "lo": lo, "w2": tile_codes(w2), "s2": interleave_scales(s2), "g2": (a2 * ws2).contiguous(),
           "a2_inv": (1 / a2).contiguous(), "group": group, "tiled": True, "n": w2.shape[1], "f": w2.shape[2] * 2}
    if (layer, lo, "gate", "weight") in parts:
        for e in experts:
            if not torch.equal(get(e, "gate", "weight_scale_2"), get(e, "up", "weight_scale_2")):
                raise ValueError(f"layer {layer} expert {e}: gate and up have different per-tensor scales")
        a1 = scalars("gate", "input_scale")
        if not torch.equal(a1, scalars("up", "input_scale")) or not bool((a1 == a1[0]).all()):
            raise ValueError(f"layer {layer}: the experts' GEMM1 input scales differ")
        w13 = interleave_gate_up(torch.stack([get(e, "gate", "weight") for e in experts]),
                                 torch.stack([get(e, "up", "weight") for e in experts]))
        s13 = interleave_gate_up(torch.stack([get(e, "gate", "weight_scale").view(torch.uint8) for e in experts]),
                                 torch.stack([get(e, "up", "weight_scale").view(torch.uint8) for e in experts]))
        out.update(w13=tile_codes(w13), s13=interleave_scales(s13), hidden=w13.shape[2] * 2,
                   g1=(a1 * scalars("gate", "weight_scale_2")).contiguous(), a1_inv=(1 / a1[:1]).contiguous())
    return out


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
    if experts.get("tiled"):
        n, half_f = experts["n"], experts["f"] // 2
    else:
        n, half_f = experts["w2"].shape[1], experts["w2"].shape[2]
    m = DlmMoe()
    m.w_tiled = int(bool(experts.get("tiled")))
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
             group=None, site=None, chain=0, h=None, norm_weight=None, eps=0.0, scale=1.0, replicated=False):
    """out = sum over each token's experts in this rank's [lo, lo + count) of weight * expert_down(activation)
    [+ shared], BF16; with `group`, the sum over ranks of that, in the call site's buffer (one fused launch).

    `act_codes` [count * m_max, F / 2] uint8 and `act_scales` [count * m_max, F / 16] E4M3: GEMM2's quantised input in
    expert-major slots; `amap` [num_experts, m_max] / `counts` [num_experts] the slot map of the router; `ids` int32 /
    `weights` FP32 [rows, top_k] hold global expert ids and the BF16-rounded routing weights.

    With `group` and `norm_weight` the owner rows are also normalised before the all-gather, and with `h` added to the
    residual stream first, exactly as `Group.reduce_norm` does: the row kernel that follows the reduction in the
    reference (`rmsnorm(h, weight, delta=reduced)`, dlmrt/ops/triton/core.py:29-56) folded into the same launch.
    `replicated`: every rank holds and updates the whole residual stream (LLaDA2), see `Group.reduce_norm`."""
    m = descriptor(act_codes, act_scales, amap, counts, experts, ids, weights, buffers, num_experts, shared)
    stream = torch.cuda.current_stream(act_codes.device).cuda_stream
    if group is None:
        _lib.check(_lib.lib().dlm_moe_nvfp4(C.byref(m), out.data_ptr(), out.stride(0), 1, stream), "moe_down")
        return out
    mode = _lib.REDUCE if norm_weight is None else _lib.REDUCE_NORM_RESIDUAL if h is not None else _lib.REDUCE_NORM
    comm, reduced = group._comm(m.m, m.n, site, chain, mode, h, norm_weight, eps, scale, replicated and h is not None)
    _lib.check(_lib.lib().dlm_rowpar_nvfp4_moe(C.byref(m), C.byref(comm), stream), f"moe_down {site}")
    group._last[chain] = reduced
    return reduced


ACTIVATIONS = {"swiglu": 0, "geglu": 1}


class FrontBuffers:
    """Scratch of one routed-expert call for up to `rows` tokens on `count` local experts: what the front half writes
    for the down-projection (ids, weights, slot map, quantised rows and activations in expert-major slots) and the
    down-projection's own workspace. Every expert has room for all rows, as in the reference's layouts."""

    def __init__(self, rows, hidden, intermediate, count, num_experts, top_k, device):
        u8 = dict(device=device, dtype=torch.uint8)
        i32 = dict(device=device, dtype=torch.int32)
        self.rows = rows
        self.ids = torch.zeros(rows, top_k, **i32)
        self.weights = torch.zeros(rows, top_k, device=device, dtype=torch.float32)
        self.counts = torch.zeros(num_experts, **i32)
        self.amap = torch.zeros(num_experts, rows, **i32)
        self.slot_codes = torch.zeros(count * rows, hidden // 2, **u8)
        self.slot_scales = torch.zeros(count * rows, hidden // 16, **u8)
        self.act_codes = torch.zeros(count * rows, intermediate // 2, **u8)
        self.act_scales = torch.zeros(count * rows, intermediate // 16, **u8)
        self.down = Buffers(rows, hidden, top_k, device)


def trtllm_moe(x, packed, experts, out, num_experts, lo, intermediate, quantized=None, activation="geglu", shared=None):
    """out = sum over each row's experts in [lo, lo + count) of weight * expert(x) [+ shared], all NVFP4: same
    arguments and meaning as the reference's `trtllm_moe` (dlmrt/quantization/nvfp4.py:280-306), on this library's
    kernels. `packed` [rows, k] int32: see `pack`. `quantized`: x already quantised, (codes [rows, hidden / 2] uint8,
    scales [rows, hidden / 16] uint8), with x None. `experts`: see `b200_experts`.

    `shared` (not in the reference's signature): a BF16 [rows, hidden] addend folded into the combine, in place of the
    `torch.add(routed, shared, out=...)` that follows the call in dlmrt/models/llada2/model.py:360-362.

    Three launches: per-token bookkeeping + input quantisation, GEMM1 + activation + re-quantisation, and the
    down-projection + combine. When `out` is a symmetric partial of `experts["group"]`, the third is not run here but
    deferred into the `Group.reduce*` of `out` that follows (one fused launch with the reduction over ranks)."""
    if quantized is None:
        rows, hidden = x.shape
        if x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError("x must be a contiguous BF16 [rows, hidden] tensor")
        device = x.device
    else:
        xq, xs = quantized
        rows, hidden = xq.shape[0], xq.shape[1] * 2
        device = xq.device
    count, top_k = experts["w2"].shape[0], packed.shape[1]
    if experts["lo"] != lo or "w13" not in experts:
        raise ValueError("experts were laid out for another rank, or without their gate / up weights (b200_experts)")
    if experts["f"] != intermediate or experts["hidden"] != hidden:
        raise ValueError(f"experts are hidden {experts['hidden']}, intermediate {experts['f']}; the call says {hidden}, "
                         f"{intermediate}")
    cache = experts.setdefault("_buffers", {})
    if rows not in cache:  # first call with this row count: before any graph capture, as the reference tunes
        cache[rows] = FrontBuffers(rows, hidden, intermediate, count, num_experts, top_k, device)
    b = cache[rows]
    f = DlmMoeFront()
    if quantized is None:
        f.x, f.a1_inv = x.data_ptr(), experts["a1_inv"].data_ptr()
    else:
        f.xq, f.xs = xq.data_ptr(), xs.data_ptr()
    f.packed = packed.data_ptr()
    f.w13_codes, f.w13_scales = experts["w13"].data_ptr(), experts["s13"].data_ptr()
    f.g1, f.a2_inv = experts["g1"].data_ptr(), experts["a2_inv"].data_ptr()
    f.ids, f.weights, f.counts, f.amap = b.ids.data_ptr(), b.weights.data_ptr(), b.counts.data_ptr(), b.amap.data_ptr()
    f.slot_codes, f.slot_scales = b.slot_codes.data_ptr(), b.slot_scales.data_ptr()
    f.act_codes, f.act_scales = b.act_codes.data_ptr(), b.act_scales.data_ptr()
    f.m, f.hidden, f.f, f.top_k, f.m_max = rows, hidden, intermediate, top_k, rows
    f.lo, f.e_local, f.e_total, f.activation = lo, count, num_experts, ACTIVATIONS[activation]
    f.w13_tiled = 1
    if packed.dtype != torch.int32 or not packed.is_contiguous():
        raise ValueError("packed must be a contiguous int32 [rows, top_k] tensor")
    stream = torch.cuda.current_stream(device).cuda_stream
    _lib.check(_lib.lib().dlm_moe_front_nvfp4(C.byref(f), 1, stream), "trtllm_moe: front half")
    down = dict(act_codes=b.act_codes, act_scales=b.act_scales, amap=b.amap, counts=b.counts, experts=experts, ids=b.ids,
                weights=b.weights, buffers=b.down, num_experts=num_experts, shared=shared)
    group = experts.get("group")
    if group is not None and group.is_partial(out):
        return group.defer_experts(out, down)
    return moe_down(out=out, **down)


def route_packed(logits, per_expert_scale, packed, top_k):
    """The router's top-k for this path, packed (dlmrt/ops/triton/moe.py:70-73): logits [rows, experts] BF16,
    per_expert_scale [experts] BF16 -> packed [rows, top_k] int32 = expert << 16 | BF16 weight bits."""
    rows, e = logits.shape
    if logits.dtype != torch.bfloat16 or per_expert_scale.dtype != torch.bfloat16 or packed.dtype != torch.int32:
        raise ValueError("route_packed takes BF16 logits and scales and an int32 output")
    stream = torch.cuda.current_stream(logits.device).cuda_stream
    _lib.check(_lib.lib().dlm_route_packed(logits.contiguous().data_ptr(), per_expert_scale.data_ptr(), packed.data_ptr(),
                                           rows, e, top_k, 1, stream), "route_packed")
    return packed


class Experts:
    """DiffusionGemma's NVFP4 routed experts on this library (mirror of `TrtllmExperts`,
    dlmrt/models/diffusion_gemma/experts.py:47-114): takes a layer's router logits and writes this rank's part of the
    MoE output. `config` needs `top_k_experts`, `hidden_size`, `num_experts`, `moe_intermediate_size`. `sample` and
    `extra_rows` are accepted for signature compatibility (there are no tactics to tune here)."""

    def __init__(self, config, lo, rows, device, sample=None, extra_rows=()):
        c = self.config = config
        self.lo = lo
        most = max([rows, *extra_rows])
        self.packed = torch.zeros(most, c.top_k_experts, dtype=torch.int32, device=device)
        # The expert input as the post-attention kernel writes it: NVFP4 codes and E4M3 scales (see `quantized`).
        self.codes = torch.zeros(most, c.hidden_size // 2, dtype=torch.uint8, device=device)
        self.scales = torch.zeros(most, c.hidden_size // 16, dtype=torch.uint8, device=device)

    def quantized(self, layer):
        """(global scale, codes, scales): where the kernel in front writes this layer's quantised expert input, read by
        __call__ with x None."""
        return layer["fp4"]["a1_inv"], self.codes, self.scales

    def __call__(self, x, logits, layer, out):
        """`x` None: the input is already in `codes` / `scales` (see `quantized`)."""
        c, n = self.config, logits.shape[0]
        packed = self.packed[:n]
        route_packed(logits, layer["expert_scale"], packed, c.top_k_experts)
        return trtllm_moe(x, packed, layer["fp4"], out, c.num_experts, self.lo, c.moe_intermediate_size,
                          quantized=None if x is not None else (self.codes[:n], self.scales[:n]))
