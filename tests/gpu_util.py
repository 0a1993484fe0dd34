"""Helpers shared by the GPU parity tests: seeded inputs and bit-level comparisons with the CPU oracle."""

import numpy as np
import torch

from oracle.bf16 import from_torch


def bits(t):
    return from_torch(t.detach().cpu())


def randn_bf16(*shape, seed, std=1.0, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16).to(device)


def assert_same_bits(got, want, what=""):
    got, want = np.asarray(got), np.asarray(want)
    bad = np.flatnonzero(got.reshape(-1) != want.reshape(-1))
    assert bad.size == 0, f"{what}: {bad.size} of {got.size} BF16 words differ, first at {bad[:5]}: " \
                          f"{got.reshape(-1)[bad[:5]]} vs {want.reshape(-1)[bad[:5]]}"


def bf16_ulp_distance(a, b):
    """Distance in BF16 code points between two bit arrays (sign-magnitude -> monotone integer)."""
    def key(x):
        x = np.asarray(x).astype(np.int32)
        return np.where(x & 0x8000, -(x & 0x7FFF), x & 0x7FFF)
    return np.abs(key(a) - key(b))


def assert_norm_close(got, want, what=""):
    """Normalised outputs go through the GPU's approximate rsqrtf, which a CPU cannot reproduce bit for bit: allow a
    one-code-point difference on at most 0.5% of the elements, nothing larger."""
    d = bf16_ulp_distance(got, want)
    assert d.max() <= 1, f"{what}: BF16 distance {d.max()}"
    assert (d > 0).mean() <= 5e-3, f"{what}: {(d > 0).mean():.4%} of elements differ by one code point"
