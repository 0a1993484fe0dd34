"""The stand-alone fused reduction (dlm_reduce_bf16 / _loopback through the Group mirror) against the CPU oracle and
against the reference's own kernel, bit for bit."""

import numpy as np
import pytest
import torch

from gpu_util import assert_norm_close, assert_same_bits, bits, randn_bf16
from oracle import reduce as red

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def short_timeouts(monkeypatch):
    from dlmrt_b200.distributed import parallel

    monkeypatch.setattr(parallel, "TIMEOUT_NS", 500_000_000)


def run_sequence(world, rows, n, calls, seed=0, one_shot_bytes=None):
    """`calls` reductions alternating over two call sites and all three modes; returns nothing, asserts parity.
    `one_shot_bytes`: 0 keeps every plain sum on the two-hop protocol, a large value sends them all over one hop."""
    from dlmrt_b200.distributed.loopback import LoopbackWorld

    lw = LoopbackWorld(world, one_shot_bytes=one_shot_bytes)
    weight = randn_bf16(n, seed=seed + 99, std=0.1) + 1
    hs = [randn_bf16(rows, n, seed=seed + 50 + r) for r in range(world)]
    for i in range(calls):
        mode = i % 3
        partials = [randn_bf16(rows, n, seed=seed + 1000 * i + r) for r in range(world)]
        site = f"s{i % 2}.{mode}"
        p_bits = np.stack([bits(p) for p in partials])
        if mode == 0:
            outs = lw.reduce(partials, site=site)
            want = red.reduce(p_bits)
        elif mode == 1:
            outs = lw.reduce(partials, site=site, weight=weight, eps=1e-6, scale=1.5)
            want, _ = red.reduce_norm(p_bits, bits(weight), 1e-6, 1.5)
        else:
            h_before = np.stack([bits(h) for h in hs])
            outs = lw.reduce(partials, site=site, hs=hs, weight=weight, eps=1e-6, scale=1.0)
            want, h_after = red.reduce_norm(p_bits, bits(weight), 1e-6, 1.0, h_before)
        torch.cuda.synchronize()
        lw.check()
        got = [bits(o) for o in outs]
        for r in range(1, world):
            assert_same_bits(got[r], got[0], f"call {i}: rank {r} vs rank 0")
        if mode == 0:
            assert_same_bits(got[0], want, f"call {i} K1")
        else:
            assert_norm_close(got[0], want, f"call {i} mode {mode}")
        if mode == 2:
            for r in range(world):
                assert_same_bits(bits(hs[r]), h_after[r], f"call {i}: residual of rank {r}")


@pytest.mark.parametrize("world, rows, n", [(1, 32, 256), (1, 256, 2560), (2, 32, 2048), (2, 256, 2560),
                                            (4, 64, 2816), (8, 32, 2048), (8, 256, 2560), (4, 16, 8192)])
@pytest.mark.parametrize("one_shot_bytes", [0, 1 << 30])
def test_loopback_sequences_match_oracle(world, rows, n, one_shot_bytes):
    run_sequence(world, rows, n, calls=7, one_shot_bytes=one_shot_bytes)


def test_special_values_survive():
    """-0.0 sums to +0.0, infinities and NaN propagate as canonical values, nothing is mistaken for the sentinel."""
    from dlmrt_b200.distributed.loopback import LoopbackWorld

    lw = LoopbackWorld(2)
    rows, n = 4, 256
    a = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    a[0], b[0] = -0.0, -0.0
    a[1, :8], b[1, :8] = float("inf"), float("-inf")
    a[2, 8:16] = float("nan")
    a[3], b[3] = 3.0e38, 3.0e38
    outs = lw.reduce([a, b], site="special")
    torch.cuda.synchronize()
    lw.check()
    want = red.reduce(np.stack([bits(a), bits(b)]))
    assert_same_bits(bits(outs[0]), want, "special values")
    assert_same_bits(bits(outs[1]), want, "special values, rank 1")


def test_group_local_world_one_matches_oracle_and_rejects_repeated_site():
    from dlmrt_b200.distributed.parallel import Group

    g = Group.local("cuda:0")
    p = randn_bf16(32, 2048, seed=3)
    out = g.reduce(p, site="a")
    torch.cuda.synchronize()
    g.check()
    assert_same_bits(bits(out), red.reduce(bits(p)[None]), "world 1")
    with pytest.raises(ValueError, match="twice in a row"):
        g.reduce(p, site="a")
    with pytest.raises(ValueError, match="allocated"):
        g.symmetric("out:a", (64, 2048))


@pytest.mark.parametrize("one_shot", [False, True])
def test_withheld_push_times_out_without_trapping(one_shot):
    """A rank whose pushes never reach their destination: the owners' bounded waits run out, the status words say
    so on every rank, the kernel returns normally and the GPU stays usable."""
    import ctypes as C

    from dlmrt_b200 import _lib
    from dlmrt_b200.distributed import parallel
    from dlmrt_b200.distributed.loopback import LoopbackWorld

    parallel.TIMEOUT_NS = 2_000_000  # 2 ms
    lw = LoopbackWorld(2, one_shot_bytes=(1 << 30) if one_shot else 0)
    rows, n = 8, 256
    partials = [randn_bf16(rows, n, seed=r) for r in range(2)]
    comms, outs = lw._comms(rows, n, "lost", 0, None, None, 0.0, 1.0)
    assert bool(comms[1].one_shot) == one_shot
    # a stand-in for rank 0's receive buffer, of the same size (one-shot slots hold a whole partial per sender)
    lost = torch.full((3, 2, rows if one_shot else rows // 2, n), -1, dtype=torch.int16, device="cuda")
    comms[1].recv[0] = lost.data_ptr()  # rank 1's pushes to rank 0 land in a buffer nobody reads
    ptrs = (C.c_void_p * 2)(*[p.data_ptr() for p in partials])
    _lib.check(_lib.lib().dlm_reduce_bf16_loopback(ptrs, comms, 2, None), "loopback")
    torch.cuda.synchronize()
    for r, g in enumerate(lw.groups):
        if one_shot and r == 1:
            # One hop has no broadcast to withhold: the rank that received everything finishes, with the right sum;
            # the rank that misses a partial reports it.
            g.check()
            assert_same_bits(bits(outs[1]), red.reduce(np.stack([bits(p) for p in partials])), "rank 1")
            continue
        with pytest.raises(TimeoutError, match="never arrived"):
            g.check()
    # the context is alive and a fresh world works
    run_sequence(2, 8, 256, calls=3, seed=7)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_all_gather_of_row_statistics(world):
    """The round's other collective (parallel.py:164-180): every rank's block of statistics in every rank's output,
    in rank order, over several invocations (the slots are triple-buffered and re-armed) and for several payloads."""
    from dlmrt_b200.distributed.loopback import LoopbackWorld

    lw = LoopbackWorld(world)
    for key, shape, dtype in (("row_stats32", (32, 4), torch.float32), ("logit_stats", (256, 2), torch.float32),
                              ("wide", (8, 4096), torch.bfloat16)):
        for call in range(5):
            g = torch.Generator().manual_seed(1000 * call + len(key))
            xs = [(torch.randn(*shape, generator=g) * (r + 1)).to(dtype).cuda() for r in range(world)]
            if call == 3:  # special values travel too: infinities, NaN, signed zeros
                for x in xs:
                    x.view(-1)[:4] = torch.tensor([float("inf"), float("-inf"), float("nan"), -0.0], dtype=dtype)
            outs = lw.all_gather(xs, key)
            torch.cuda.synchronize()
            lw.check()
            want = torch.stack(xs)
            view = torch.int32 if dtype == torch.float32 else torch.int16
            for r, out in enumerate(outs):
                assert out.shape == (world, *shape) and out.dtype == dtype
                assert torch.equal(out.view(view), want.view(view)), f"{key} call {call} rank {r}"


def test_group_all_gather_world_one_and_fallback():
    from dlmrt_b200 import _lib
    from dlmrt_b200.distributed.parallel import Group

    g = Group.local("cuda:0")
    x = torch.randn(32, 4, device="cuda")
    before = _lib.lib().dlm_launch_count()
    for _ in range(4):
        out = g.all_gather(x, "stats")
    torch.cuda.synchronize()
    g.check()
    assert _lib.lib().dlm_launch_count() == before + 4 and torch.equal(out[0], x)
    # Payloads the in-band arrival flag cannot carry are refused, not sent through another backend.
    for bad in (torch.randn(5, 3, device="cuda"),                                  # 60 bytes: not a multiple of 16
                torch.full((8, 4), -1, dtype=torch.int32, device="cuda"),          # integers may be all-ones words
                torch.randn(8, 4, dtype=torch.float64, device="cuda"),             # low mantissa words may be all ones
                torch.randn(8, 8, device="cuda")[:, :4]):                          # not contiguous
        with pytest.raises(ValueError, match="all_gather"):
            g.all_gather(bad, "bad")
    assert _lib.lib().dlm_launch_count() == before + 4


def test_a_timed_out_group_stays_failed():
    """After a wait ran out, slots may hold late arrivals of the failed call. Later calls must therefore report an
    error instead of data: on the device (status words non-zero at entry: push nothing, accept nothing, broadcast
    nothing) and on the host (the Group refuses to launch once check() has raised)."""
    import ctypes as C

    from dlmrt_b200 import _lib
    from dlmrt_b200.distributed import parallel
    from dlmrt_b200.distributed.loopback import LoopbackWorld

    parallel.TIMEOUT_NS = 2_000_000  # 2 ms
    lw = LoopbackWorld(2, one_shot_bytes=0)
    rows, n = 8, 256
    partials = [randn_bf16(rows, n, seed=r) for r in range(2)]
    comms, outs = lw._comms(rows, n, "lost", 0, None, None, 0.0, 1.0)
    lost = torch.full((3, 2, rows // 2, n), -1, dtype=torch.int16, device="cuda")
    comms[1].recv[0] = lost.data_ptr()  # rank 1's pushes to rank 0 never arrive
    ptrs = (C.c_void_p * 2)(*[p.data_ptr() for p in partials])
    _lib.check(_lib.lib().dlm_reduce_bf16_loopback(ptrs, comms, 2, None), "loopback")
    lw._done(0, outs)
    torch.cuda.synchronize()
    assert int(lw.groups[0].status[0]) == _lib.ERR_TIMEOUT
    # A second call with every address right, WITHOUT the host having looked at the status: the device words are
    # still set, so the kernel exchanges nothing and the outputs stay armed (no row is broadcast).
    comms2, outs2 = lw._comms(rows, n, "after", 0, None, None, 0.0, 1.0)
    _lib.check(_lib.lib().dlm_reduce_bf16_loopback(ptrs, comms2, 2, None), "loopback")
    lw._done(0, outs2)
    torch.cuda.synchronize()
    for r in range(2):
        assert int(lw.groups[r].status[0]) == _lib.ERR_TIMEOUT
        armed = outs2[r].view(torch.int16) == -1
        assert bool(armed.all()), f"rank {r}: {int((~armed).sum())} lanes of the output were written after a failure"
    # The host side: check() raises once and the group then refuses to reduce.
    for g in lw.groups:
        with pytest.raises(TimeoutError):
            g.check()
        with pytest.raises(RuntimeError, match="new Group"):
            g.reduce(partials[0], site="again")
    run_sequence(2, 8, 256, calls=3, seed=11)  # a fresh world works


def test_reference_kernel_agrees_bit_for_bit():
    """This library's kernel, the reference's own kernel (built from its sources into oracle/_ref) and the CPU
    oracle on the same seeded inputs, world 1 (one GPU): all three modes, several invocations."""
    from oracle.build_ref import load_built

    ref = load_built()
    if ref is None:
        pytest.skip("oracle/_ref was not built (python oracle/build_ref.py <reference>)")
    from dlmrt_b200.distributed.parallel import Group

    rows, n = 64, 2560
    g = Group.local("cuda:0")
    dev = "cuda"
    recv = torch.full((3, 1, rows, n), -1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    recv_ptrs = torch.tensor([recv.data_ptr()], dtype=torch.int64, device=dev)
    epochs = torch.zeros(rows + 96, dtype=torch.int32, device=dev)
    ref_outs = [torch.full((rows, n), -1, dtype=torch.int16, device=dev).view(torch.bfloat16) for _ in range(2)]
    weight = randn_bf16(n, seed=11, std=0.1) + 1
    h_mine, h_ref = randn_bf16(rows, n, seed=12), randn_bf16(rows, n, seed=12)
    last = None
    for i in range(6):
        mode = i % 3
        p = randn_bf16(rows, n, seed=100 + i)
        out = ref_outs[i % 2]
        peers = torch.tensor([out.data_ptr()], dtype=torch.int64, device=dev)
        rearm, rearm_numel = (last.data_ptr(), last.numel()) if last is not None else (0, 0)
        fn = [ref.reduce, ref.reduce_norm, ref.reduce_norm_residual][mode]
        fn(p, recv_ptrs, h_ref if mode == 2 else p, weight if mode else p, out, 0, peers, rearm, rearm_numel, epochs, 0,
           1, 1e-6, 1.25, 96, 0, False)
        last = out
        site = f"r{i % 2}"
        if mode == 0:
            mine = g.reduce(p, site=site)
        else:
            mine = g.reduce_norm(p, h_mine if mode == 2 else None, weight, 1e-6, 1.25, site=site)
        torch.cuda.synchronize()
        g.check()
        assert_same_bits(bits(mine), bits(out), f"call {i} mode {mode}: this kernel vs the reference kernel")
        if mode == 2:
            assert_same_bits(bits(h_mine), bits(h_ref), f"call {i}: residual stream")
        if mode == 0:
            assert_same_bits(bits(out), red.reduce(bits(p)[None]), f"call {i}: reference kernel vs CPU oracle")


def test_one_chain_sees_calls_of_different_row_counts():
    """LLaDA2's pair rounds (dlmrt/models/llada2/engine.py:139, llada2/model.py:291-297): the 32-row self-conditioning
    reduction is issued on the chain of the 64-row forward that follows it, so consecutive calls of ONE chain differ in
    rows. Receive slots are per (rows, n, chain), but the chain's previous output is shared bookkeeping: every call
    must re-arm it over ITS OWN size (tp_comm.cu:201-208), whatever this call's rows are."""
    from dlmrt_b200.distributed.loopback import LoopbackWorld

    world, n, chain = 2, 2048, 64
    lw = LoopbackWorld(world, one_shot_bytes=0)
    previous = None
    for i, rows in enumerate([32, 64, 64, 32, 64, 32, 32, 64, 64]):
        partials = [randn_bf16(rows, n, seed=700 + 10 * i + r) for r in range(world)]
        site = f"{rows}.{i % 2}.{'sc' if rows == 32 else 'attn'}"
        outs = lw.reduce(partials, site=site, chain=chain)
        torch.cuda.synchronize()
        lw.check()
        want = red.reduce(np.stack([bits(p) for p in partials]))
        for r in range(world):
            assert_same_bits(bits(outs[r]), want, f"call {i} ({rows} rows) rank {r}")
        if previous is not None:  # the output of the call before, of whatever size, is armed again in full
            for r, old in enumerate(previous):
                armed = old.view(torch.int16) == -1
                assert bool(armed.all()), f"call {i}: {int((~armed).sum())} lanes of rank {r}'s previous output not re-armed"
        previous = outs


def test_two_chains_resident_at_once_on_two_streams():
    """DiffusionGemma reduces the dense MLP (chain 2, side stream) while the experts' reduction (chain 1) runs
    (dlmrt/models/diffusion_gemma/model.py:281-288, dlmrt/distributed/parallel.py:139-140). Both kernels spin on peers,
    so both grids must fit on the GPU together: the caller caps each at half the SMs with `max_ctas`. Waits are bounded
    to milliseconds here, so a grid that did not fit would surface as DLM_ERR_TIMEOUT, not as a stall."""
    from dlmrt_b200 import _lib
    from dlmrt_b200.distributed import parallel
    from dlmrt_b200.distributed.loopback import LoopbackWorld

    parallel.TIMEOUT_NS = 50_000_000  # 50 ms
    world, rows, n, k = 2, 256, 2816, 2176
    sms = _lib.lib().dlm_device_sms()
    lw = LoopbackWorld(world, max_ctas=sms // world // 2)
    side, main = torch.cuda.Stream(), torch.cuda.Stream()
    x, w = randn_bf16(rows, k * world, seed=1), randn_bf16(n, k * world, seed=2, std=0.02)
    xs = [t.contiguous() for t in x.chunk(world, 1)]
    ws = [t.contiguous() for t in w.chunk(world, 1)]
    results = []
    torch.cuda.synchronize()
    for i in range(6):
        moe = [randn_bf16(rows, n, seed=800 + 10 * i + r) for r in range(world)]
        torch.cuda.synchronize()
        with torch.cuda.stream(side):   # dense down-projection fused with its reduction, chain 2
            dense = lw.rowpar(xs, ws, site=f"{i % 2}.mlp", chain=2)
        with torch.cuda.stream(main):   # the experts' partial, chain 1
            routed = lw.reduce(moe, site=f"{i % 2}.moe", chain=1)
        results.append((moe, dense, routed))
        torch.cuda.synchronize()
        lw.check()
        want_routed = red.reduce(np.stack([bits(p) for p in moe]))
        for r in range(world):
            assert_same_bits(bits(routed[r]), want_routed, f"round {i}: experts' sum, rank {r}")
            assert_same_bits(bits(dense[r]), bits(dense[0]), f"round {i}: dense sum, rank {r} vs 0")
    # the dense result equals the same call (same grid cap, hence the same K ranges) with nothing beside it
    alone = LoopbackWorld(world, max_ctas=sms // world // 2).rowpar(xs, ws, site="alone", chain=2)
    torch.cuda.synchronize()
    assert_same_bits(bits(results[-1][1][0]), bits(alone[0]), "dense sum: two streams vs alone")


@pytest.mark.parametrize("world, rows", [(1, 32), (2, 32), (8, 32), (4, 64), (2, 256)])
def test_replicated_residual_stream(world, rows):
    """LLaDA2 keeps the whole residual stream on every rank and follows each plain sum with
    `rmsnorm(h, weight, delta=reduced)` (dlmrt/models/llada2/model.py:435-439, dlmrt/ops/triton/core.py:29-56). Folded
    into the reduction (`replicated=True`): every rank receives every partial, sums all rows itself and updates ALL
    rows of its own copy of h. Stand-alone and behind the fused projection; h stays identical on every rank."""
    from dlmrt_b200.distributed.loopback import LoopbackWorld

    n, k = 2048, 512
    lw = LoopbackWorld(world)
    weight = randn_bf16(n, seed=5, std=0.1) + 1
    h0 = randn_bf16(rows, n, seed=6)
    hs = [h0.clone() for _ in range(world)]
    h_want = bits(h0)
    for i in range(4):
        if i % 2 == 0:
            partials = [randn_bf16(rows, n, seed=900 + 10 * i + r) for r in range(world)]
            p_bits = np.stack([bits(p) for p in partials])
            outs = lw.reduce(partials, site=f"rep{i % 2}", chain=rows, hs=hs, weight=weight, eps=1e-6, replicated=True)
        else:
            g = torch.Generator().manual_seed(i)
            xs = [torch.randint(-3, 4, (rows, k), generator=g).to(torch.bfloat16).cuda() for _ in range(world)]
            ws = [torch.randint(-2, 3, (n, k), generator=g).to(torch.bfloat16).cuda() for _ in range(world)]
            p_bits = np.stack([bits((x.float() @ w.float().t()).to(torch.bfloat16)) for x, w in zip(xs, ws)])
            outs = lw.rowpar(xs, ws, site=f"rep{i % 2}", chain=rows, hs=hs, weight=weight, eps=1e-6, replicated=True)
        torch.cuda.synchronize()
        lw.check()
        summed = red.reduce(p_bits)
        want, h_after = red.reduce_norm(summed[None], bits(weight), 1e-6, 1.0, h_want[None])
        h_want = h_after[0]
        for r in range(world):
            assert_same_bits(bits(hs[r]), h_want, f"call {i}: residual stream of rank {r}")
            assert_norm_close(bits(outs[r]), want, f"call {i}: rank {r}")
            assert_same_bits(bits(outs[r]), bits(outs[0]), f"call {i}: rank {r} vs rank 0")
