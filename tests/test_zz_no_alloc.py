"""dlm_gemm_bf16_noalloc: the GEMM for callers that may not allocate device memory (a plugin running inside somebody
else's stream capture, a host that forbids allocation after start-up, a process whose memory pool another runtime
owns). Its split-K scratch is an 8 MiB array built into the library instead of a caller-provided workspace.

Called through the C ABI only, twice in a row, and compared bit for bit with dlm_gemm_bf16 on the same tiling (the
arithmetic is the same kernel, so the tolerance is zero), and once directly with the CPU oracle on exact operands. This file sorts last on purpose: a run that stops at the
first failure has then already run every other test. It must pass alone in a fresh process and after all the others.
"""

import ctypes as C

import pytest
import torch

from gpu_util import assert_same_bits, bits, randn_bf16


def call_noalloc(x, w, out, splits, token_tiles):
    from dlmrt_b200 import _lib

    m, k = x.shape
    return _lib.lib().dlm_gemm_bf16_noalloc(x.data_ptr(), w.data_ptr(), out.data_ptr(), m, w.shape[0], k, x.stride(0),
                                            w.stride(0), out.stride(0), splits, token_tiles, 0, None)


def call_workspace(x, w, out, splits, token_tiles):
    from dlmrt_b200 import _lib
    from dlmrt_b200._lib import DlmGemm

    m, k = x.shape
    n = w.shape[0]
    ws = torch.zeros(_lib.lib().dlm_workspace_bytes(m, n, k), dtype=torch.uint8, device=x.device)
    g = DlmGemm()
    g.x, g.w, g.m, g.n, g.k, g.ldx, g.ldw = x.data_ptr(), w.data_ptr(), m, n, k, x.stride(0), w.stride(0)
    g.workspace, g.workspace_bytes, g.splits, g.token_tiles = ws.data_ptr(), ws.numel(), splits, token_tiles
    rc = _lib.lib().dlm_gemm_bf16(C.byref(g), out.data_ptr(), out.stride(0), 0, None)
    torch.cuda.synchronize()
    return rc


@pytest.mark.gpu
@pytest.mark.parametrize("m, n, k, splits, token_tiles", [(64, 512, 2048, 4, 1), (256, 2560, 1024, 3, 1),
                                                           (32, 2048, 2048, 8, 1), (256, 1024, 512, 1, 4)])
def test_noalloc_matches_workspace_entry_point_twice_in_a_row(m, n, k, splits, token_tiles):
    x, w = randn_bf16(m, k, seed=1), randn_bf16(n, k, seed=2, std=0.02)
    want = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    assert call_workspace(x, w, want, splits, token_tiles) == 0
    before = torch.cuda.memory_allocated()
    first = torch.full((m, n), -1, dtype=torch.int16, device="cuda").view(torch.bfloat16)
    second = torch.full((m, n), -1, dtype=torch.int16, device="cuda").view(torch.bfloat16)
    x2 = randn_bf16(m, k, seed=3)
    want2 = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    assert call_workspace(x2, w, want2, splits, token_tiles) == 0
    held = torch.cuda.memory_allocated()
    # two calls back to back on one stream, no synchronisation in between: they share the built-in scratch
    assert call_noalloc(x, w, first, splits, token_tiles) == 0
    assert call_noalloc(x2, w, second, splits, token_tiles) == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == held >= before  # nothing was taken from torch's allocator by the calls
    assert_same_bits(bits(first), bits(want), "first call")
    assert_same_bits(bits(second), bits(want2), "second call")


@pytest.mark.gpu
def test_noalloc_rejects_what_does_not_fit_and_caps_what_it_picks_itself():
    from dlmrt_b200 import _lib

    m, n, k = 256, 2560, 9728
    x, w = randn_bf16(m, k, seed=4), randn_bf16(n, k, seed=5, std=0.02)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    assert 2048 + 7 * m * n * 4 > _lib.NOALLOC_SCRATCH_BYTES
    assert call_noalloc(x, w, out, 7, 1) == _lib.ERR_SCRATCH
    assert b"scratch" in _lib.lib().dlm_strerror(_lib.ERR_SCRATCH)
    assert call_noalloc(x, w, out, 0, 0) == 0  # the library lowers its own choice of splits until it fits
    torch.cuda.synchronize()
    want = torch.empty_like(out)
    assert call_workspace(x, w, want, 3, 1) == 0  # 2 KiB + 3 * m * n * 4 is the most that fits in 8 MiB
    assert_same_bits(bits(out), bits(want), "capped tiling")


@pytest.mark.gpu
@pytest.mark.parametrize("m, n, k, splits", [(64, 512, 2048, 4), (256, 2560, 4096, 0), (32, 2048, 64, 8)])
def test_noalloc_matches_the_cpu_oracle_on_exact_operands(m, n, k, splits):
    """Not only equal to its sibling: small-integer operands make every product and sum exact, so the result must
    equal the CPU restatement bit for bit, twice in a row on the shared scratch."""
    from oracle import rowpar
    from oracle.bf16 import f32_to_bf16

    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randint(-3, 4, (m, k), generator=g).to(torch.bfloat16).cuda()
    w = torch.randint(-2, 3, (n, k), generator=g).to(torch.bfloat16).cuda()
    want = f32_to_bf16(rowpar.gemm_f32(bits(x), bits(w)))
    for attempt in range(2):
        out = torch.full((m, n), -1, dtype=torch.int16, device="cuda").view(torch.bfloat16)
        assert call_noalloc(x, w, out, splits, 1 if splits else 0) == 0
        torch.cuda.synchronize()
        assert_same_bits(bits(out), want, f"call {attempt}")


def test_noalloc_argument_checks_need_no_gpu():
    from dlmrt_b200 import _lib

    f = _lib.lib().dlm_gemm_bf16_noalloc
    assert f(0x1000, 0x2000, 0x3000, 40, 256, 128, 128, 128, 256, 0, 0, 0, None) == _lib.ERR_SHAPE
    assert f(0x1000, 0x2000, None, 32, 256, 128, 128, 128, 256, 0, 0, 0, None) == _lib.ERR_NULL
    assert f(0x1000, 0x2000, 0x3000, 256, 2560, 9728, 9728, 9728, 2560, 8, 1, 0, None) == _lib.ERR_SCRATCH
