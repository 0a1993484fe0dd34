"""CPU restatement of the fused tensor-parallel reduction (test infrastructure, never on the product path).

Follows dlmrt/ops/csrc/tp_comm.cu of the reference:
  K1  reduce                 tp_comm.cu:216-236, 259-267   sum over ranks, FP32, rank order 0..w-1 starting at +0.0f
  K2  reduce_norm            tp_comm.cu:237-258            K1, round to BF16, RMSNorm * weight * scale
  K3  reduce_norm_residual   tp_comm.cu:243-246            K2 with h[own rows] = bf16(bf16(sum) + h) before the norm
Call-site semantics (which rows of h a rank updates, what every rank's OUT holds): dlmrt/distributed/parallel.py:134-147.

Parity status: the reference has no CPU implementation, test or fixture for this path, so this restatement is
UNPINNED against golden vectors; it is pinned against the reference's own kernel run on the GPU (oracle/_ref, see
oracle/build_ref.py and tests/test_reduce_gpu.py). K1 is pure IEEE FP32 addition and BF16 rounding, so the CPU and
GPU agree bit for bit. K2/K3 use the GPU's approximate rsqrtf (MUFU), which no CPU can reproduce bit for bit: the
restatement uses a correctly rounded 1/sqrt, and tests allow a one-BF16-ulp difference on a small fraction of
elements for the normalised output only (the residual update stays bit-exact).

All BF16 tensors are numpy uint16 bit patterns.
"""

import numpy as np

from .bf16 import bf16_to_f32, f32_to_bf16

VEC = 8  # BF16 lanes per 16-byte vector (kVec, tp_comm.cu:30): thread t of the owner block holds columns [8t, 8t+8)


def check_shape(rows, n, world):
    """The argument checks of launch<> (tp_comm.cu:282-287)."""
    if n % (VEC * 32) or n // VEC > 1024:
        raise ValueError("hidden size must be a multiple of 256, at most 8192")
    if rows % world:
        raise ValueError("rows must split over ranks")
    if not 1 <= world <= 8:
        raise ValueError("at most 8 ranks")


def rank_order_sum(partials):
    """[world, rows, n] BF16 bits -> FP32 [rows, n]: v = +0.0f; v += partial[s] for s = 0..world-1
    (tp_comm.cu:233-236). Starting from +0.0f makes an all -0.0 column come out +0.0."""
    partials = np.asarray(partials, dtype=np.uint16)
    v = np.zeros(partials.shape[1:], dtype=np.float32)
    for s in range(partials.shape[0]):
        v = v + bf16_to_f32(partials[s])
    return v


def reduce(partials):
    """K1: OUT [rows, n] BF16 bits, the same on every rank."""
    world, rows, n = np.asarray(partials).shape
    check_shape(rows, n, world)
    return f32_to_bf16(rank_order_sum(partials))


def _fma(a, b, c):
    """fmaf on float32 arrays: one rounding of a * b + c. The product of two float32 is exact in float64; the sum is
    rounded to float64 and then to float32 (a double rounding only on exact float32 ties of a 53-bit sum)."""
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


def _butterfly(x):
    """x [..., 32] float32 -> [...]: the xor-shuffle sum of block_sum (tp_comm.cu:98-100): five rounds
    x += x[lane ^ o], o = 16, 8, 4, 2, 1. Addition commutes, so every lane ends with the same balanced tree."""
    lanes = np.arange(32)
    for o in (16, 8, 4, 2, 1):
        x = x + x[..., lanes ^ o]
    return x[..., 0]


def block_sum_of_squares(v):
    """v FP32 [rows, n] -> FP32 [rows]: sum of squares in the order of tp_comm.cu:247-250 and block_sum (:98-109):
    per thread eight sequential FMAs over its columns (nvcc contracts ss += v * v), a butterfly inside each warp,
    then a butterfly over the warp sums padded with zeros to 32 lanes."""
    rows, n = v.shape
    threads = n // VEC
    warps = threads // 32
    t = v.reshape(rows, threads, VEC)
    ss = np.zeros((rows, threads), dtype=np.float32)
    for i in range(VEC):
        ss = _fma(t[:, :, i], t[:, :, i], ss)
    per_warp = _butterfly(ss.reshape(rows, warps, 32))
    second = np.zeros((rows, 32), dtype=np.float32)
    second[:, :warps] = per_warp
    return _butterfly(second)


def rsqrt(x):
    """Correctly rounded float32 1/sqrt(x); the GPU's rsqrtf is within 2 ulp of this."""
    return (1.0 / np.sqrt(x.astype(np.float64))).astype(np.float32)


def reduce_norm(partials, weight, eps, scale=1.0, h=None):
    """K2 (h is None) / K3.

    partials [world, rows, n], weight [n], h [world, rows, n] (each rank's local residual stream) as BF16 bits.
    Returns (out [rows, n], h_after [world, rows, n] or None). Rank r owns rows [r*R, (r+1)*R): only those rows of
    its h are read and rewritten (the residual stream is sequence-parallel, tp_comm.cu:7-8,243-246)."""
    partials = np.asarray(partials, dtype=np.uint16)
    world, rows, n = partials.shape
    check_shape(rows, n, world)
    R = rows // world
    v = bf16_to_f32(f32_to_bf16(rank_order_sum(partials)))  # rounded to BF16 first (tp_comm.cu:238-242)
    h_after = None
    if h is not None:
        h = np.asarray(h, dtype=np.uint16)
        h_after = h.copy()
        own = np.empty((rows, n), dtype=np.uint16)
        for r in range(world):
            own[r * R:(r + 1) * R] = h[r, r * R:(r + 1) * R]
        v = v + bf16_to_f32(own)
        new = f32_to_bf16(v)
        for r in range(world):
            h_after[r, r * R:(r + 1) * R] = new[r * R:(r + 1) * R]
    total = block_sum_of_squares(v)
    r_ = rsqrt(total / np.float32(n) + np.float32(eps)) * np.float32(scale)
    w = bf16_to_f32(np.asarray(weight, dtype=np.uint16))
    out = (v * r_[:, None]) * w[None, :]
    return f32_to_bf16(out), h_after
