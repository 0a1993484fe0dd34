"""CPU restatement of a row-parallel projection followed by the reduction (test infrastructure only).

  per-rank GEMM  dlmrt/layers/linear.py:41-51: out[M, N] = x[M, K/w] @ W[N, K/w]^T, BF16 in, FP32 accumulate
                 (increasing K, dlmrt/ops/triton/gemm.py:1-8), BF16 out into the symmetric `partial`
  sharding       dlmrt/distributed/parallel.py:149-152 (Group.shard(t, dim=1): contiguous K ranges)
  reduction      oracle.reduce (tp_comm.cu:216-267)

The reference rounds every rank's partial to BF16 before the sum (the wire format is BF16, tp_comm.cu:112).
BASELINE config 1 words it as "accumulated to an FP32 partial, summed in rank order, rounded to bf16"; both readings
are implemented (`fp32_partials`), they differ by one rounding per rank.

The FP32 accumulation order inside a GEMM is not observable from the reference (cuBLAS), so GEMM partials are
compared within a tolerance, not bit for bit: per output row max-abs <= 2 BF16 ulp of the row's largest magnitude
and relative L2 <= 4e-3 (dlmrt tests/test_sdar_kernels.py:30, tests/test_llada_nvfp4.py:166).
"""

import numpy as np

from . import reduce as red
from .bf16 import bf16_to_f32, f32_to_bf16

REL_L2 = 4e-3
ULPS = 2


def shard(a, world, rank, dim):
    if a.shape[dim] % world:
        raise ValueError(f"Dimension {dim} of {a.shape} does not split over {world} ranks")
    return np.ascontiguousarray(np.split(a, world, axis=dim)[rank])


def gemm_f32(x_bits, w_bits):
    """x [M, K], W [N, K] BF16 bits -> FP32 [M, N] (products exact, FP32 accumulation by the host BLAS)."""
    return bf16_to_f32(x_bits) @ bf16_to_f32(w_bits).T


def gemm_f64(x_bits, w_bits):
    """The same product accumulated in float64: the 'truth' tolerances are quoted against."""
    return bf16_to_f32(x_bits).astype(np.float64) @ bf16_to_f32(w_bits).astype(np.float64).T


def rowpar(x_bits, w_bits, world, fp32_partials=False):
    """Full row-parallel projection + K1: x [M, K], W [N, K] BF16 bits -> (out [M, N] bits, partials).

    partials is [world, M, N]: BF16 bits (reference wire format) or FP32 (`fp32_partials`, BASELINE config 1)."""
    parts = [gemm_f32(shard(x_bits, world, r, 1), shard(w_bits, world, r, 1)) for r in range(world)]
    if fp32_partials:
        v = np.zeros_like(parts[0])
        for p in parts:
            v = v + p
        return f32_to_bf16(v), np.stack(parts)
    bits = np.stack([f32_to_bf16(p) for p in parts])
    return red.reduce(bits), bits


def config1(seed=0, m=256, k=9728, n=2560, world=2):
    """BASELINE config 1 inputs: x ~ N(0, 1), W ~ N(0, 0.02), BF16, torch.manual_seed(seed)."""
    import torch

    from .bf16 import from_torch

    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    return from_torch(x), from_torch(w), world


def row_errors(got_bits, want_f64):
    """Per-row (max-abs error in units of one BF16 ulp of the row's largest magnitude, relative L2)."""
    got = bf16_to_f32(got_bits).astype(np.float64)
    peak = np.abs(want_f64).max(axis=1)
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(peak, 1e-30))) - 7)
    max_abs = np.abs(got - want_f64).max(axis=1) / ulp
    rel = np.linalg.norm(got - want_f64, axis=1) / np.maximum(np.linalg.norm(want_f64, axis=1), 1e-30)
    return max_abs, rel


def within_tolerance(got_bits, want_f64):
    max_abs, rel = row_errors(got_bits, want_f64)
    return bool((max_abs <= ULPS).all() and (rel <= REL_L2).all())
