"""BF16 bit helpers for the CPU oracle (test infrastructure, never imported by the product path).

BF16 values are carried as numpy uint16 bit patterns so that comparisons are on raw bits, as the reduction's parity
bar demands (compare raw int16, dlmrt/ops/csrc/tp_comm.cu:12-14).
"""

import numpy as np

SENTINEL = np.uint16(0xFFFF)  # the arrival sentinel of tp_comm.cu:12-14: a negative NaN arithmetic never produces


def bf16_to_f32(bits):
    """uint16 BF16 bit patterns -> float32 (exact)."""
    bits = np.asarray(bits, dtype=np.uint16)
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16(x):
    """float32 -> BF16 bits, round to nearest even; every NaN becomes the canonical 0x7FFF.

    This is the rounding of __floats2bfloat162_rn (tp_comm.cu:90-96, cvt.rn.bf16x2.f32)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    rounded = ((u + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)
    return np.where(np.isnan(x), np.uint16(0x7FFF), rounded).astype(np.uint16)


def round_bf16(x):
    """float32 -> nearest BF16, returned as float32."""
    return bf16_to_f32(f32_to_bf16(x))


def from_torch(t):
    """torch bf16 tensor -> uint16 numpy bits."""
    import torch

    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def to_torch(bits):
    """uint16 numpy bits -> torch bf16 tensor."""
    import torch

    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)
