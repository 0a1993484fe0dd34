// Device side of the barrier-free tensor-parallel reduction, shared by the stand-alone reduction kernel and by the
// fused GEMM + reduction kernels.
//
// Protocol (the one dlmrt/ops/csrc/tp_comm.cu:1-22 describes; every rank runs the same code):
//   push      row s*R + c of this rank's BF16 partial goes into rank s's receive slot [e % 3][rank][c] with plain
//             16-byte stores over NVLink. The payload is its own flag: slots start filled with 0xFFFF lanes, which
//             BF16 arithmetic never produces, so a vector has arrived once no lane holds that value.
//   re-arm    the receive buffer peers write two invocations from now ((e + 2) % 3) and the previous output of this
//             chain are refilled with the sentinel.
//   own       the CTA that owns row c polls its `world` slots, sums them in FP32 in rank order from +0.0f, optionally
//             adds the residual and applies RMSNorm, rounds to BF16 and stores the row into OUT on every rank (one
//             multimem.st through the NVSwitch, or one store per rank).
//   collect   every CTA polls the rows of its own OUT copy that correspond to the rows it owned, so OUT is complete on
//             this rank when the kernel ends.
// One-shot variant (plain sums of small partials, c.one_shot): every rank stores its WHOLE partial into every rank's
// slots [e % 3][rank][row] (one multimem.st per vector, or one store per rank) and every rank then sums all rows itself,
// in the same rank order, into its own OUT: one NVLink hop instead of two, no broadcast, no collect; the result is
// the same on every rank, bit for bit, because every rank adds the same BF16 partials in the same order.
// Differences from the reference kernel, by design: there are no dedicated pusher CTAs (every CTA pushes, re-arms,
// then owns rows, so a fused GEMM's tiles can be pushed by the CTA that produced them); address tables live in
// kernel parameters; every wait is bounded and reports through status words instead of trapping; invocation
// counters are kept equal across all DLM_EPOCH_SLOTS entries so kernels of different grid sizes can share them.
#pragma once

#include "common.cuh"

namespace dlm {

constexpr int kMaxWorld = 8;
constexpr int kEpochSlots = 256;
constexpr int kStampSlots = 8; //  // %globaltimer stamps per CTA: 0 start, 1 pushed, 2 owned rows broadcast, 3 collected;
                                // fused kernels add 4 accumulator ready, 5 dependency wait returned, 6 tile summed and pushed

enum Mode { kReduce = 0, kReduceNorm = 1, kReduceNormResidual = 2 };

struct CommDev {
    __nv_bfloat16* recv[kMaxWorld];
    __nv_bfloat16* out_peers[kMaxWorld];
    __nv_bfloat16* out;
    __nv_bfloat16* out_mc;
    __nv_bfloat16* recv_mc;  // one-shot: multicast address of the receive buffer, or null (one store per rank)
    __nv_bfloat16* rearm;
    __nv_bfloat16* h;
    const __nv_bfloat16* weight;
    int* epochs;
    int* status;
    long long* stamps;
    long long timeout_ns;
    int rearm_vecs;
    int rank, world, rows, n, R;
    int one_shot;   // every rank receives every row and sums all rows itself
    int slot_rows;  // rows of one sender's slot, = rows summed by this rank: R, or rows when one_shot
    int mode;
    float eps, scale;
};

struct CommCtx {
    int block, blocks;  // this CTA's index among the CTAs of its rank, and their number
    int e, buf;         // invocation number and receive buffer e % 3
    int dead;           // an earlier call on this group failed: push nothing, accept nothing (see comm_begin)
    long long deadline;
    size_t slot_elems, buf_elems;
};

__device__ __forceinline__ void stamp(const CommDev& c, const CommCtx& x, int phase) {
    if (c.stamps && threadIdx.x == 0) c.stamps[x.block * kStampSlots + phase] = globaltimer();
}

// `previous` is epochs[block] and `failed` is status[0], both as read after the previous kernel completed (callers may
// have fetched them early). A failure is sticky: once a wait of this group ran out, receive slots may hold vectors of an
// older invocation that would pass for arrived data, so every later call pushes nothing, waits for nothing and
// broadcasts nothing (its peers' waits run out in turn and every rank learns of it) until the host has read the status
// and rebuilt the group.
__device__ __forceinline__ int comm_failed(const CommDev& c) {
    int v = 0;
    if (c.status) asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(c.status) : "memory");
    return v;
}

__device__ __forceinline__ CommCtx comm_begin(const CommDev& c, int block, int blocks, int previous, int failed) {
    CommCtx x;
    x.block = block;
    x.blocks = blocks;
    x.e = previous + 1;
    x.buf = x.e % 3;
    x.dead = failed != 0;
    x.deadline = globaltimer() + c.timeout_ns;
    x.slot_elems = static_cast<size_t>(c.slot_rows) * c.n;
    x.buf_elems = static_cast<size_t>(c.world) * x.slot_elems;
    return x;
}

// Where row `row` (0 <= row < rows), column `col` of this rank's partial lands: owner rank s = row / R.
__device__ __forceinline__ __nv_bfloat16* push_address(const CommDev& c, const CommCtx& x, int row, int col) {
    const int s = row / c.R, r = row - s * c.R;
    return c.recv[s] + x.buf * x.buf_elems + c.rank * x.slot_elems + static_cast<size_t>(r) * c.n + col;
}

// Stores one 16-byte vector of this rank's partial (row, col) where the protocol wants it: into the owner's slot, or
// (one-shot) into this rank's slot on every rank.
__device__ __forceinline__ void push_store(const CommDev& c, const CommCtx& x, int row, int col, uint4 v) {
    if (x.dead) return;
    if (!c.one_shot) {
        store_v4(push_address(c, x, row, col), v);
        return;
    }
    const size_t off = x.buf * x.buf_elems + c.rank * x.slot_elems + static_cast<size_t>(row) * c.n + col;
    if (c.recv_mc) {
        multicast_store(c.recv_mc + off, v);
    } else {
        for (int s = 0; s < c.world; ++s) store_v4(c.recv[(c.rank + s) % c.world] + off, v);
    }
}

// Push phase of the stand-alone reduction: the whole partial, spread over all threads of all CTAs of the rank.
// Consecutive logical rows go to consecutive destinations starting at this rank, so the first stores of all ranks
// spread over all destinations instead of all landing on rank 0 (tp_comm.cu:154-163).
__device__ __forceinline__ void push_partial(const CommDev& c, const CommCtx& x, const __nv_bfloat16* partial) {
    const int vpr = c.n / kVec;
    const int total = c.rows * vpr;
    const int stride = x.blocks * blockDim.x;
    for (int i = x.block * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int l = i / vpr, col = (i - l * vpr) * kVec;
        const int r = l / c.world, s = (c.rank + l % c.world) % c.world;
        const int row = c.one_shot ? l : s * c.R + r;
        const uint4 v = *reinterpret_cast<const uint4*>(partial + static_cast<size_t>(row) * c.n + col);
        push_store(c, x, row, col, v);
    }
}

// Re-arm the receive buffer peers write in invocation e + 2 and the previous call site's output (over that output's
// own size: calls on one chain may differ in rows, tp_comm.cu:201-208).
// The work is spread over `parts` CTAs of which this one is number `part`.
__device__ __forceinline__ void rearm(const CommDev& c, const CommCtx& x, int part, int parts) {
    const uint4 sentinel = make_uint4(kSentinel, kSentinel, kSentinel, kSentinel);
    const int stride = parts * blockDim.x;
    const int first = part * blockDim.x + threadIdx.x;
    __nv_bfloat16* stale = c.recv[c.rank] + ((x.e + 2) % 3) * x.buf_elems;
    const int total = static_cast<int>(x.buf_elems / kVec);
    for (int i = first; i < total; i += stride) store_v4(stale + static_cast<size_t>(i) * kVec, sentinel);
    for (int i = first; i < c.rearm_vecs; i += stride) store_v4(c.rearm + static_cast<size_t>(i) * kVec, sentinel);
}

// Waits until the 16-byte vectors at base + s * stride (s < world) have all arrived and returns them. Every round
// issues all pending loads before testing any (one L2 round trip per round, tp_comm.cu:52-54). Returns false when the
// deadline passed first; the words of slots that did not arrive are then meaningless.
// `pending` names the slots still to be waited for (the others already hold arrived data in v).
__device__ __forceinline__ bool poll_all(const __nv_bfloat16* base, size_t stride, int world, uint4 (&v)[kMaxWorld],
                                         const CommDev& c, const CommCtx& x, int phase, unsigned pending = ~0u) {
    pending &= (1u << world) - 1;
    if (x.dead) return false;
    if (!pending) return true;
    while (true) {
        const unsigned was = pending;
#pragma unroll
        for (int s = 0; s < kMaxWorld; ++s)
            if (was >> s & 1) v[s] = load_volatile(base + s * stride);
#pragma unroll
        for (int s = 0; s < kMaxWorld; ++s)
            if ((was >> s & 1) && arrived(v[s])) pending &= ~(1u << s);
        if (!pending) return true;
        if (globaltimer() > x.deadline) {
            report(c.status, kErrTimeout, __ffs(pending) - 1, phase, x.e);
            return false;
        }
    }
}

// Sum over a thread block of (blockDim >= threads) threads of which the first `threads` (a multiple of 32) carry
// values; the same tree as the reference's block_sum (tp_comm.cu:98-109): butterfly inside each warp, then a
// butterfly over the warp sums padded with zeros to 32 lanes. All threads of the block must call it.
__device__ __forceinline__ float block_sum(float x, float* scratch, int threads) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffff, x, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) scratch[warp] = x;
    __syncthreads();
    x = lane < (threads >> 5) ? scratch[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffff, x, o);
    __syncthreads();  // scratch is reused by the next row
    return x;
}

// block_sum of NROWS independent values at once (same tree for each, so each equals block_sum of it alone); `scratch`
// holds 32 floats per value.
template <int NROWS>
__device__ __forceinline__ void block_sum_n(float (&x)[NROWS], float* scratch, int threads) {
#pragma unroll
    for (int i = 0; i < NROWS; ++i) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) x[i] += __shfl_xor_sync(0xffffffff, x[i], o);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < NROWS; ++i) scratch[i * 32 + warp] = x[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NROWS; ++i) {
        x[i] = lane < (threads >> 5) ? scratch[i * 32 + lane] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) x[i] += __shfl_xor_sync(0xffffffff, x[i], o);
    }
    __syncthreads();  // scratch is reused by the next rows
}

// What an owner does with rows once it holds the rank-ordered FP32 sums `v[i]` of its thread's eight columns:
// optional residual add and RMSNorm (tp_comm.cu:237-258), BF16 rounding, and the store into OUT on every rank.
// NROWS rows go through the block-wide sums together. `off[i]` is the element offset of the thread's columns in row
// i; rows with store[i] false are computed but not written (their inputs never arrived, or there is no such row).
// All threads of the block must call it.
template <int MODE, int NROWS>
__device__ __forceinline__ void finish_rows(const CommDev& c, float (&v)[NROWS][kVec], const uint4 (&hraw)[NROWS],
                                            uint4 wraw, const size_t (&off)[NROWS], bool active,
                                            const bool (&store)[NROWS], float* scratch, int threads) {
    if (MODE != kReduce) {
        float ss[NROWS];
#pragma unroll
        for (int i = 0; i < NROWS; ++i) {
            // The reduced sum is rounded to BF16 before the residual add, as an unfused all-reduce would hand it over.
            const uint4 rounded = pack_bf16x8(v[i]);
#pragma unroll
            for (int j = 0; j < kVec; ++j) v[i][j] = 0.f;
            add_bf16x8(v[i], rounded);
            if (MODE == kReduceNormResidual) {
                add_bf16x8(v[i], hraw[i]);
                if (active && store[i]) *reinterpret_cast<uint4*>(c.h + off[i]) = pack_bf16x8(v[i]);
            }
            ss[i] = 0.f;
#pragma unroll
            for (int j = 0; j < kVec; ++j) ss[i] = fmaf(v[i][j], v[i][j], ss[i]);
            if (!active) ss[i] = 0.f;
        }
        block_sum_n<NROWS>(ss, scratch, threads);
        const __nv_bfloat162* w = reinterpret_cast<const __nv_bfloat162*>(&wraw);
#pragma unroll
        for (int i = 0; i < NROWS; ++i) {
            const float rs = rsqrtf(ss[i] / c.n + c.eps) * c.scale;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(w[j]);
                v[i][2 * j] = v[i][2 * j] * rs * f.x;
                v[i][2 * j + 1] = v[i][2 * j + 1] * rs * f.y;
            }
        }
    }
    // Broadcast the rows: one multicast store, or one store per rank. A row whose inputs never arrived is not
    // broadcast, so every rank's collect phase reports the failure too.
#pragma unroll
    for (int i = 0; i < NROWS; ++i) {
        if (active && store[i]) {
            const uint4 packed = pack_bf16x8(v[i]);
            if (c.one_shot) {
                store_v4(c.out + off[i], packed);  // every rank computes every row: nothing to broadcast
            } else if (c.out_mc) {
                multicast_store(c.out_mc + off[i], packed);
            } else {
                for (int s = 0; s < c.world; ++s) store_v4(c.out_peers[s] + off[i], packed);
            }
        }
    }
}

template <int MODE>
__device__ __forceinline__ void finish_row(const CommDev& c, float (&v)[kVec], uint4 hraw, uint4 wraw, size_t off,
                                           bool active, bool ok, float* scratch, int threads) {
    float vv[1][kVec];
#pragma unroll
    for (int j = 0; j < kVec; ++j) vv[0][j] = v[j];
    const uint4 hh[1] = {hraw};
    const size_t oo[1] = {off};
    const bool st[1] = {ok};
    finish_rows<MODE, 1>(c, vv, hh, wraw, oo, active, st, scratch, threads);
}

// Owner phase: CTA `block` owns slot rows block, block + blocks, ... and takes them NROWS at a time (the rows' waits,
// sums and block-wide reductions overlap; NROWS = 2 where CTAs own several rows, i.e. one or two ranks). Thread
// t < n / 8 holds columns [8t, 8t + 8) of the rows being reduced; threads beyond that only take part in the block-wide
// synchronisation. `scratch` is 32 * NROWS floats of shared memory.
template <int MODE, int NROWS>
__device__ __forceinline__ void own_rows(const CommDev& c, const CommCtx& x, float* scratch) {
    const int t = threadIdx.x;
    const int threads = c.n / kVec;
    const bool active = t < threads;
    const size_t col = static_cast<size_t>(active ? t : 0) * kVec;
    const __nv_bfloat16* mine = c.recv[c.rank] + x.buf * x.buf_elems;
    const int first_row = c.one_shot ? 0 : c.rank * c.R;  // row of OUT that slot row 0 holds
    uint4 wraw = make_uint4(0, 0, 0, 0);
    if (MODE != kReduce && active) wraw = *reinterpret_cast<const uint4*>(c.weight + col);
    for (int r0 = x.block; r0 < c.slot_rows; r0 += NROWS * x.blocks) {
        size_t off[NROWS];
        uint4 hraw[NROWS];
        bool store[NROWS];
        // Local operands first, so their latency overlaps the wait for the peers (tp_comm.cu:225-228).
#pragma unroll
        for (int i = 0; i < NROWS; ++i) {
            const int r = r0 + i * x.blocks;
            store[i] = r < c.slot_rows;
            off[i] = static_cast<size_t>(first_row + (store[i] ? r : 0)) * c.n + col;
            hraw[i] = make_uint4(0, 0, 0, 0);
            if (MODE == kReduceNormResidual && active && store[i]) hraw[i] = *reinterpret_cast<const uint4*>(c.h + off[i]);
        }
        // With one or two ranks the second row's slots are read before the first row is waited for, so that the rows
        // do not each pay a round trip to L2.
        uint4 early[2];
        const bool have_early = NROWS > 1 && c.world <= 2 && active && store[NROWS - 1];
        if (have_early) {
#pragma unroll
            for (int s = 0; s < 2; ++s)
                if (s < c.world)
                    early[s] = load_volatile(mine + static_cast<size_t>(r0 + (NROWS - 1) * x.blocks) * c.n + col + s * x.slot_elems);
        }
        float v[NROWS][kVec] = {};
#pragma unroll
        for (int i = 0; i < NROWS; ++i) {
            if (active && store[i]) {
                uint4 slots[kMaxWorld];
                unsigned pending = ~0u;
                if (have_early && i == NROWS - 1) {
                    pending = 0;
#pragma unroll
                    for (int s = 0; s < 2; ++s) {
                        if (s < c.world) {
                            slots[s] = early[s];
                            if (!arrived(early[s])) pending |= 1u << s;
                        }
                    }
                }
                const int r = r0 + i * x.blocks;
                store[i] = poll_all(mine + static_cast<size_t>(r) * c.n + col, x.slot_elems, c.world, slots, c, x, kPhaseReceive,
                                    pending);
#pragma unroll
                for (int s = 0; s < kMaxWorld; ++s)
                    if (s < c.world) add_bf16x8(v[i], slots[s]);
            }
        }
        finish_rows<MODE, NROWS>(c, v, hraw, wraw, off, active, store, scratch, threads);
    }
}

__device__ __forceinline__ void rearm_late(const CommDev& c, const CommCtx& x);

// Owner phase + late re-arm + collect phase. `scratch`: 64 floats.
// PAIRS: rows are taken two at a time where CTAs own several (off for the 1024-thread kernel, whose 64 registers per
// thread do not hold two rows).
template <int MODE, bool PAIRS>
__device__ __forceinline__ void own_and_collect(const CommDev& c, const CommCtx& x, float* scratch) {
    if (PAIRS && c.slot_rows > x.blocks) own_rows<MODE, PAIRS ? 2 : 1>(c, x, scratch);
    else own_rows<MODE, 1>(c, x, scratch);
    const bool active = static_cast<int>(threadIdx.x) < c.n / kVec;
    const size_t col = static_cast<size_t>(active ? threadIdx.x : 0) * kVec;
    uint4 slots[kMaxWorld];
    stamp(c, x, 2);
    // The late re-arm goes here, between the broadcast of the owned rows and the wait for everyone else's: its stores
    // fill the time the broadcasts are in flight instead of lengthening the kernel's tail.
    rearm_late(c, x);
    // Collect: rows s * R + r of this rank's OUT copy, from every owner s. With one rank, or one-shot, every row of
    // OUT was stored by this very grid, so it is complete when the kernel ends and there is nothing to wait for.
    if (active && c.world > 1 && !c.one_shot) {
        for (int r = x.block; r < c.R; r += x.blocks)
            if (!poll_all(c.out + static_cast<size_t>(r) * c.n + col, x.slot_elems, c.world, slots, c, x, kPhaseOut)) break;
    }
    stamp(c, x, 3);
}

template <bool PAIRS = true>
__device__ __forceinline__ void own_and_collect(const CommDev& c, const CommCtx& x, float* scratch) {
    if (c.mode == kReduce) own_and_collect<kReduce, PAIRS>(c, x, scratch);
    else if (c.mode == kReduceNorm) own_and_collect<kReduceNorm, PAIRS>(c, x, scratch);
    else own_and_collect<kReduceNormResidual, PAIRS>(c, x, scratch);
}

// Nothing waits for the re-arm inside this launch, but the owners' sums are on the critical path of every rank. So
// CTAs that own no row (block >= R) re-arm at once, on behalf of everyone; only when every CTA owns rows does each
// re-arm its share, and then after its own phase (own_and_collect calls rearm_late before it collects).
__device__ __forceinline__ void rearm_early(const CommDev& c, const CommCtx& x) {
    if (x.blocks > c.slot_rows && x.block >= c.slot_rows) rearm(c, x, x.block - c.slot_rows, x.blocks - c.slot_rows);
}
__device__ __forceinline__ void rearm_late(const CommDev& c, const CommCtx& x) {
    if (x.blocks <= c.slot_rows) rearm(c, x, x.block, x.blocks);
}

// Advance the invocation counters: every entry of the table ends equal to e, whatever the grid size.
__device__ __forceinline__ void comm_end(const CommDev& c, const CommCtx& x) {
    if (threadIdx.x == 0)
        for (int j = x.block; j < kEpochSlots; j += x.blocks) c.epochs[j] = x.e;
}

}  // namespace dlm
