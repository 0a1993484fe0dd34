"""Linear layers of the row-parallel hot path on hand-written sm_100a kernels.

Mirror of the reference's `dlmrt/layers/linear.py` (Linear :16-51): `Linear(weight, fp8, b200=False)`, `.n`, `.k`,
`.weight`, `.fp8`, `.input(rows, device)`, `__call__(x, scales=None, out=None) -> out`. The reference runs BF16 on
cuBLAS (`torch.mm`) on SM >= 10 (:28,47-48); here the GEMM is libdlmrt_b200's tcgen05 weight streamer, and when `out`
is a tensor-parallel group's symmetric partial the GEMM is not run at all but deferred into the fused
projection + reduction kernel launched by the following `Group.reduce*` (see dlmrt_b200.distributed.parallel).

FP8 activations are outside this path (the reference forces the fused reduction off with FP8 GEMM inputs,
dlmrt/models/sdar/model.py:62-64), so `fp8=True` is rejected.
"""

import ctypes as C

import torch

from .. import _lib
from .._lib import DlmGemm


def tile_weight(weight):
    """[N, K] BF16 row-major -> the streaming layout of the kernels: [N / 128, K / 64] tiles of 128 rows x 64 columns,
    each 16 KB tile contiguous and already in the 128-byte-swizzled order it has in shared memory (16-byte chunk c of
    tile row r sits at chunk position c ^ (r % 8)). One bulk copy then brings a tile in, and a CTA's weight slab is a
    contiguous run of HBM instead of 128-byte pieces a row pitch apart."""
    n, k = weight.shape
    if n % 128 or k % 8:
        raise ValueError(f"weight {tuple(weight.shape)}: N must be a multiple of 128 and K of 8")
    if k % 64:  # a ragged last k-block is padded with zeros to a whole tile
        weight = torch.nn.functional.pad(weight, (0, 64 - k % 64))
        k = weight.shape[1]
    t = weight.reshape(n // 128, 128, k // 64, 8, 8).permute(0, 2, 1, 3, 4)  # (tile row, tile col, r, chunk, 8 elems)
    r = torch.arange(128, device=weight.device).view(128, 1)
    c = torch.arange(8, device=weight.device).view(1, 8)
    src = (c ^ (r % 8)).view(1, 1, 128, 8, 1).expand(n // 128, k // 64, 128, 8, 8)  # position p holds chunk p ^ (r % 8)
    return torch.gather(t, 3, src).contiguous()


class Linear:
    """y = x @ W^T, BF16 in and out, FP32 accumulation in increasing K (K ranges summed in order when split)."""

    def __init__(self, weight, fp8=False, b200=False, group=None, tiled=True, nn=False, token_tiles=0, splits=0):
        if fp8:
            raise NotImplementedError("FP8 linears are not part of the row-parallel BF16 path")
        if weight.dtype != torch.bfloat16 or weight.dim() != 2:
            raise ValueError("weight must be a BF16 [N, K] matrix")
        # `nn`: the weight is [K, N] (y = x @ W), as the tied embedding is for the self-conditioning soft-embedding
        # GEMM of the reference (dlmrt/models/sdar/model.py:196-203, torch.mm(probs, E)); it is re-laid as [N, K] once.
        if nn:
            weight = weight.t()
        self.n, self.k = weight.shape
        self.fp8 = False
        self.b200 = False  # the SM 12.x emulation switch of the reference has no meaning on a B200
        self.weight = weight.contiguous()
        # `tiled`: stream a re-laid copy of the weight (see tile_weight) instead of the row-major matrix.
        self.tiles = tile_weight(self.weight) if tiled and self.n % 128 == 0 and self.k % 8 == 0 else None
        self.group = group
        # Tiling of this layer's GEMM (tiles along the tokens, K splits): 0 = chosen by the library for each call.
        self.token_tiles, self.splits = token_tiles, splits
        self._workspace = None
        _lib.lib()

    def input(self, rows, device):
        """Activation buffers this layer consumes: BF16 needs none (linear.py:34-39)."""
        return None, None

    def gemm(self, x, out, pdl=True):
        """Run the GEMM now: out[m, n] = x[m, k] @ W[n, k]^T."""
        m, k = x.shape
        if k != self.k or tuple(out.shape) != (m, self.n) or out.dtype != torch.bfloat16 or x.dtype != torch.bfloat16:
            raise ValueError(f"Linear [{self.n}, {self.k}]: x {tuple(x.shape)} {x.dtype}, out {tuple(out.shape)}")
        if x.stride(1) != 1 or out.stride(1) != 1:
            raise ValueError("x and out must have a contiguous last dimension")
        nbytes = _lib.lib().dlm_workspace_bytes(m, self.n, k)
        if self._workspace is None or self._workspace.numel() < nbytes:
            with torch.inference_mode(False):
                self._workspace = torch.zeros(nbytes, device=x.device, dtype=torch.uint8)
        g = DlmGemm()
        self.describe(g)
        g.x, g.m, g.n, g.k, g.ldx = x.data_ptr(), m, self.n, k, x.stride(0)
        g.workspace, g.workspace_bytes = self._workspace.data_ptr(), self._workspace.numel()
        g.splits, g.token_tiles = self.splits, self.token_tiles
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _lib.check(_lib.lib().dlm_gemm_bf16(C.byref(g), out.data_ptr(), out.stride(0), int(pdl), stream),
                   f"gemm [{m}, {self.n}, {k}]")
        return out

    def describe(self, g):
        """Fill the weight fields of a DlmGemm."""
        if self.tiles is not None:
            g.w, g.ldw, g.w_tiled = self.tiles.data_ptr(), self.k, 1
        else:
            g.w, g.ldw, g.w_tiled = self.weight.data_ptr(), self.weight.stride(0), 0

    def __call__(self, x, scales=None, out=None):
        if out is None:
            out = torch.empty(x.shape[0], self.n, device=x.device, dtype=torch.bfloat16)
        elif self.group is not None and self.group.is_partial(out):
            return self.group.defer(self, x, out)
        return self.gemm(x, out)
