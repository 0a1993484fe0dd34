"""oracle.bf16 against torch's own BF16 casts (RNE, canonical NaN) on every interesting bit pattern."""

import numpy as np
import torch

from oracle import bf16


def test_round_trip_every_bf16_pattern():
    bits = np.arange(1 << 16, dtype=np.uint32).astype(np.uint16)
    f = bf16.bf16_to_f32(bits)
    assert np.array_equal(f.view(np.uint32), bits.astype(np.uint32) << 16)
    back = bf16.f32_to_bf16(f)
    nan = np.isnan(f)
    assert np.array_equal(back[~nan], bits[~nan])
    assert (back[nan] == 0x7FFF).all()


def test_rounding_matches_torch():
    rng = np.random.default_rng(0)
    u = rng.integers(0, 1 << 32, size=1 << 18, dtype=np.uint64).astype(np.uint32)
    ties = (rng.integers(0, 1 << 16, size=1 << 12, dtype=np.uint64).astype(np.uint32) << 16) | 0x8000
    u = np.concatenate([u, ties, ties - 1, ties + 1])
    x = u.view(np.float32)
    x = x[~np.isnan(x)]
    want = torch.from_numpy(x.copy()).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bf16.f32_to_bf16(x), want)


def test_sentinel_is_never_produced():
    x = np.array([np.nan, -np.nan, np.inf, -np.inf, -0.0, 3.4e38, -3.4e38], dtype=np.float32)
    assert not (bf16.f32_to_bf16(x) == bf16.SENTINEL).any()
    assert bf16.f32_to_bf16(np.array([-np.nan], dtype=np.float32))[0] == 0x7FFF


def test_torch_bridge():
    t = torch.randn(5, 7).to(torch.bfloat16)
    assert torch.equal(bf16.to_torch(bf16.from_torch(t)), t)
