// Row-parallel BF16 projection fused with the tensor-parallel reduction that follows it, for sm_100a.
//
//   out[m, n] = sum over ranks of  x_r[m, k] * W_r[n, k]^T          (k = this rank's K shard)
//
// The shape of a denoise round is small-M (32, 64 or 256 block tokens) against a wide weight shard, so the kernel is a
// weight streamer: weights sit on the 128-row M axis of the MMA and the tokens on its N axis (D[128 features, m
// tokens] in tensor memory), every CTA pulls a disjoint [128 x K/splits] slab of W through a TMA ring, and the x
// slab comes out of L2.
//
//   warp 0   TMA producer: W slab (evict-first) + x slab (evict-last) per 64-wide k-block into a ring of 128-byte
//            swizzled stages. The first ring-full of weight loads is issued BEFORE griddepcontrol.wait: weights never
//            depend on the previous kernel, only x does.
//   warp 1   MMA issuer: four tcgen05.mma kind::f16 (K = 16) per k-block, FP32 accumulator in TMEM; tcgen05.commit
//            frees the stage and finally signals the epilogue.
//   warp 2   TMEM allocation / release.
//   warps 4-11  epilogue: tcgen05.ld the accumulator.
//   The grid is (feature tiles) x (token tiles) x (K splits), at most one CTA per SM. With one split the BF16 tile is
//   staged in shared memory and goes straight out. With several, every CTA writes its FP32 partial tile to the
//   workspace, the CTAs of a tile meet on an arrival counter, and each then sums its share of the tile's tokens over
//   the splits in split order (the value never depends on timing). Either way each token row's 256 bytes are stored
//   (plain GEMM) or pushed straight into the owner rank's receive slot over NVLink, and every CTA goes on to the
//   re-arm / own / collect phases of the reduction (comm.cuh).
#include "kernels.cuh"

namespace dlm {

namespace {

struct SmemLayout {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full;
    uint32_t tmem_base;
    int epoch, gen, failed;  // epochs[block], gen[block] and status[0], fetched by a spare warp while the pipeline runs
    int seen[2];             // k-blocks each of two issuers has seen arrive (only kept on rings with an odd number of stages)
    float scratch[64];
};

constexpr int kTileBytesW = kBlockF * kBlockK * 2;  // 16 KB

__device__ __forceinline__ uint32_t tmem_cols(int m) {
    uint32_t c = 32;
    while (c < static_cast<uint32_t>(m)) c <<= 1;
    return c;
}

}  // namespace

// Owner phase of a single rank whose K was split: CTA `block` owns rows block, block + blocks, ... and takes them two
// at a time (their loads and block-wide sums overlap). For each it waits until every CTA of the row's token tile has
// announced its partial tile, sums the row's FP32 split partials in split order, rounds to BF16 (that is the rank's
// partial, as the push path would have stored it) and finishes the row as any owner does. Thread t < n / 8 holds
// columns [8t, 8t + 8): feature tile t / 16, 32 bytes of that tile's row. `scratch`: 64 floats.
template <int MODE>
__device__ __forceinline__ void own_rows_from_splits(const GemmDev& g, const CommDev& c, const CommCtx& x,
                                                     const int* counter, int mt, float* scratch) {
    constexpr int kRows = 2;
    constexpr int kGroup = 3;  // splits whose loads are in flight together (per row)
    const int t = threadIdx.x;
    const int threads = c.n / kVec;
    const bool active = t < threads;
    const int col = (active ? t : 0) * kVec;
    const int f = col / kBlockF, j = col % kBlockF;
    const int expected = (g.n / kBlockF) * g.splits;
    const size_t split_stride = static_cast<size_t>(mt) * kBlockF;
    uint4 wraw = make_uint4(0, 0, 0, 0);
    if (MODE != kReduce && active) wraw = *reinterpret_cast<const uint4*>(c.weight + col);
    int ready_tile = -1;  // rows are owned in increasing order, so token tiles are waited for in increasing order
    bool ok = true;
    for (int r0 = x.block; r0 < c.rows; r0 += kRows * x.blocks) {
        size_t off[kRows];
        uint4 hraw[kRows];
        bool store[kRows];
        const float* src[kRows];
        int last_tile = 0;
#pragma unroll
        for (int i = 0; i < kRows; ++i) {
            const int r = r0 + i * x.blocks;
            store[i] = r < c.rows;
            const int tt = store[i] ? r / mt : 0, token = store[i] ? r - tt * mt : 0;
            off[i] = static_cast<size_t>(store[i] ? r : 0) * c.n + col;
            hraw[i] = make_uint4(0, 0, 0, 0);
            if (MODE == kReduceNormResidual && active && store[i]) hraw[i] = *reinterpret_cast<const uint4*>(c.h + off[i]);
            src[i] = g.ws + (static_cast<size_t>(f) * g.token_tiles + tt) * g.splits * split_stride +
                     static_cast<size_t>(token) * kBlockF + j;
            if (store[i]) last_tile = tt;
        }
        if (ok && last_tile > ready_tile) {  // uniform over the block
            if (t == 0) {
                bool arrived_all = true;
                for (int tt = ready_tile + 1; tt <= last_tile && arrived_all; ++tt) {
                    int seen;
                    do {
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(counter + tt) : "memory");
                        if (seen >= expected) break;
                        if (globaltimer() > x.deadline) {
                            report(c.status, kErrTimeout, tt, kPhasePipeline, 3 << 24);
                            arrived_all = false;
                            break;
                        }
                    } while (true);
                }
                scratch[0] = arrived_all ? 1.f : 0.f;
            }
            __syncthreads();
            ok = scratch[0] != 0.f;
            __syncthreads();  // scratch is reused by the block-wide sums
            if (ok) ready_tile = last_tile;
        }
        float v[kRows][kVec] = {};
        if (active && ok) {
            float acc[kRows][kVec];
            for (int base_sp = 0; base_sp < g.splits; base_sp += kGroup) {
                float4 a[kRows][kGroup], b[kRows][kGroup];
#pragma unroll
                for (int i = 0; i < kRows; ++i) {
#pragma unroll
                    for (int u = 0; u < kGroup; ++u) {
                        if (base_sp + u < g.splits && store[i]) {
                            a[i][u] = __ldcg(reinterpret_cast<const float4*>(src[i] + (base_sp + u) * split_stride));
                            b[i][u] = __ldcg(reinterpret_cast<const float4*>(src[i] + (base_sp + u) * split_stride) + 1);
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < kRows; ++i) {
#pragma unroll
                    for (int u = 0; u < kGroup; ++u) {
                        if (base_sp + u < g.splits && store[i]) {
                            if (base_sp + u == 0) {
                                acc[i][0] = a[i][u].x, acc[i][1] = a[i][u].y, acc[i][2] = a[i][u].z, acc[i][3] = a[i][u].w;
                                acc[i][4] = b[i][u].x, acc[i][5] = b[i][u].y, acc[i][6] = b[i][u].z, acc[i][7] = b[i][u].w;
                            } else {
                                acc[i][0] += a[i][u].x, acc[i][1] += a[i][u].y, acc[i][2] += a[i][u].z, acc[i][3] += a[i][u].w;
                                acc[i][4] += b[i][u].x, acc[i][5] += b[i][u].y, acc[i][6] += b[i][u].z, acc[i][7] += b[i][u].w;
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < kRows; ++i)
                if (store[i]) add_bf16x8(v[i], pack_bf16x8(acc[i]));  // +0.0f + partial: the rank-ordered sum over one rank
        }
#pragma unroll
        for (int i = 0; i < kRows; ++i) store[i] = store[i] && ok;
        finish_rows<MODE, kRows>(c, v, hraw, wraw, off, active, store, scratch, threads);
    }
    stamp(c, x, 2);
    stamp(c, x, 3);
}

// The early L2 prefetch of the rest of the weight slab pays for narrow tiles only; with 256-token tiles the stream is
// already bandwidth-bound when the CTA starts.
__device__ __forceinline__ bool prefetch_rest_of_slab(int mt) { return mt <= 128; }

template <int NR>
__global__ void __launch_bounds__(kFusedThreads, 1) rowpar_kernel(const __grid_constant__ RowparParams<NR> p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const int slot = NR == 1 ? 0 : static_cast<int>(blockIdx.y);
    const GemmDev& g = p.g[slot];
    const CommDev& c = p.c[slot];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int block = static_cast<int>(blockIdx.x), blocks = static_cast<int>(gridDim.x);
    if (c.stamps && threadIdx.x == 0) c.stamps[block * kStampSlots + 7] = globaltimer();

    // This CTA's output tile (feature tile f, token tile t) and K range (split s).
    const int s = block % g.splits;
    const int tile = block / g.splits;  // f * token_tiles + t
    const int f = tile / g.token_tiles, t = tile - f * g.token_tiles;
    const int mt = g.m / g.token_tiles;  // tokens of this tile: the MMA's N
    const int token0 = t * mt;
    const int nkb = (g.k + kBlockK - 1) / kBlockK;  // a ragged last k-block is zero-filled (TMA out-of-bounds fill, padded tiles)
    const int kb0 = static_cast<int>(static_cast<long long>(s) * nkb / g.splits);
    const int kb1 = static_cast<int>(static_cast<long long>(s + 1) * nkb / g.splits);
    const int iters = kb1 - kb0;
    const int stage_bytes = kTileBytesW + mt * kBlockK * 2;

    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    SmemLayout* sm = reinterpret_cast<SmemLayout*>(tiles + g.stages * stage_bytes);
    const uint32_t cols = tmem_cols(mt);                 // columns of one accumulator
    const int issuers = cols <= 128 && iters >= 2 ? 2 : 1;  // MMA-issuing threads, each with its own accumulator
    // One rank, K split: the owner of a row sums the FP32 split partials itself (in split order), so the BF16 partial
    // never travels through the receive slots; the value is the same, bit for bit, as pushing and summing one rank.
    const bool local_rows = p.fused && c.world == 1 && g.splits > 1;

    const int pre = iters < g.stages ? iters : g.stages;
    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < g.stages; ++i) {
                mbar_init(&sm->full[i], 1);
                mbar_init(&sm->empty[i], 1);
            }
            mbar_init(&sm->acc_full, static_cast<uint32_t>(issuers));
            fence_barrier_init();
            if (!g.w_tiles) tma_prefetch_descriptor(&g.tm_w);
            tma_prefetch_descriptor(&g.tm_x);
            // The first ring-full of loads is requested at once, by the thread that has just set the barriers up, while
            // the rest of the block is still allocating tensor memory: weights depend on nothing, x only on the kernels
            // in front of this one.
            for (int it = 0; it < pre; ++it) {
                mbar_expect_tx(&sm->full[it], static_cast<uint32_t>(stage_bytes));
                if (g.w_tiles)
                    bulk_load(tiles + it * stage_bytes, g.w_tiles + (static_cast<size_t>(f) * nkb + kb0 + it) * kTileBytesW,
                              kTileBytesW, &sm->full[it], kEvictFirst);
                else
                    tma_load_2d(tiles + it * stage_bytes, &g.tm_w, &sm->full[it], (kb0 + it) * kBlockK, f * kBlockF,
                                kEvictFirst);
            }
            // The rest of this CTA's weight slab is pulled into L2 now: the ring then refills at L2 latency instead of
            // HBM latency.
            if (iters > pre && prefetch_rest_of_slab(mt)) {
                if (g.w_tiles) {
                    bulk_prefetch_l2(g.w_tiles + (static_cast<size_t>(f) * nkb + kb0 + pre) * kTileBytesW,
                                     static_cast<uint32_t>(iters - pre) * kTileBytesW);
                } else {
                    for (int it = pre; it < iters; ++it) tma_prefetch_l2_2d(&g.tm_w, (kb0 + it) * kBlockK, f * kBlockF);
                }
            }
            pdl_wait();
            if (c.stamps) c.stamps[block * kStampSlots + 5] = globaltimer();
            for (int it = 0; it < pre; ++it)
                tma_load_2d(tiles + it * stage_bytes + kTileBytesW, &g.tm_x, &sm->full[it], (kb0 + it) * kBlockK,
                            token0, kEvictLast);
            sm->seen[0] = sm->seen[1] = 0;
        }
        __syncwarp();  // the warp reaches the block-wide barrier together
    }
    if (warp == 2) tmem_alloc(&sm->tmem_base, cols * issuers);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = sm->tmem_base;
    // The next kernel of the stream may be set up from now on: its blocks move in as this kernel's blocks leave, and it
    // waits for this kernel to complete before it reads anything this kernel writes.
    pdl_launch_dependents();
    // Budget of the local pipeline and of the split-K rendezvous; the cross-rank waits take theirs in comm_begin.
    const long long pipeline_deadline = globaltimer() + (c.timeout_ns > 0 ? c.timeout_ns : kDefaultTimeoutNs);
    // What a pipeline wait that ran out puts in the status' last word: who gave up (0 producer, 1 issuer, 2 epilogue,
    // 3 split-K rendezvous) and the k-block it was at.
    auto stalled = [](int who, int it) { return who << 24 | (it & 0xFFFF); };
    if (warp == 0) {
        if (lane == 0) {
            int st = pre == g.stages ? 0 : pre;
            uint32_t parity = 0;  // second lap of the ring waits for the first release of each stage
            for (int it = pre; it < iters; ++it) {
                if (!mbar_wait(&sm->empty[st], parity, pipeline_deadline)) {
                    report(c.status, kErrTimeout, st, kPhasePipeline, stalled(0, it));
                    break;
                }
                uint8_t* stage = tiles + st * stage_bytes;
                mbar_expect_tx(&sm->full[st], static_cast<uint32_t>(stage_bytes));
                if (g.w_tiles)
                    bulk_load(stage, g.w_tiles + (static_cast<size_t>(f) * nkb + kb0 + it) * kTileBytesW, kTileBytesW,
                              &sm->full[st], kEvictFirst);
                else
                    tma_load_2d(stage, &g.tm_w, &sm->full[st], (kb0 + it) * kBlockK, f * kBlockF, kEvictFirst);
                tma_load_2d(stage + kTileBytesW, &g.tm_x, &sm->full[st], (kb0 + it) * kBlockK, token0, kEvictLast);
                if (++st == g.stages) st = 0, parity ^= 1;
            }
        }
        __syncwarp();  // lanes 1-31 must not run ahead to the block-wide barrier while lane 0 is still issuing
    } else if (warp == 1 || warp == 3) {
        // MMA issue. One thread feeds the tensor pipe; for narrow tiles its own instruction stream (barrier wait,
        // descriptors, four MMAs, commit per k-block) is slower than the MMAs it issues, so tiles of up to 128 tokens
        // get a second issuer with its own accumulator: warp 1 takes the even k-blocks, warp 3 the odd ones, and the
        // epilogue adds the two accumulators.
        // A parity wait tells a barrier's phases apart only if the waiter is never a whole phase behind. With an odd
        // number of stages the two issuers alternate on every stage, so before an issuer waits for k-block `it` it makes
        // sure the other one has seen k-block `it - stages` arrive (the same stage's previous phase): each publishes
        // the k-blocks it has seen in shared memory. The loads of `it` cannot have been requested before that anyway.
        const int who = warp == 1 ? 0 : 1;
        if (lane == 0) {
            if (who == 1) {
                pdl_wait();
                if (p.fused) sm->epoch = c.epochs[block], sm->failed = comm_failed(c);
                if (g.splits > 1) sm->gen = g.gen[block];
            }
            if (who < issuers) {
                const uint32_t idesc = umma_idesc_bf16(kBlockF, mt);
                const uint32_t acc = tmem + who * cols;
                volatile int* seen = sm->seen;
                const bool guarded = issuers == 2 && (g.stages & 1);  // see above; even rings need no hand-over
                const uint64_t desc_hi = umma_desc_k128(tiles) & 0xFFFFFFFF00000000ull;
                const uint32_t stage0 = smem_u32(tiles);
                int st = 0;
                uint32_t parity = 0;
                for (int it = 0; it < iters; ++it) {
                    if ((it & (issuers - 1)) == who) {
                        bool ok = true;
                        if (guarded && it >= g.stages) {  // k-block it - stages was the other issuer's
                            while (seen[1 - who] <= it - g.stages) {
                                if (globaltimer() > pipeline_deadline) {
                                    ok = false;
                                    break;
                                }
                            }
                        }
                        if (!ok || !mbar_wait(&sm->full[st], parity, pipeline_deadline)) {
                            report(c.status, kErrTimeout, st, kPhasePipeline, stalled(1, it));
                            break;
                        }
                        if (guarded) seen[who] = it + 1;
                        tcgen05_fence_after();
                        const uint32_t base = stage0 + st * stage_bytes;
                        const uint64_t dw = desc_hi | ((base & 0x3FFFF) >> 4);
                        const uint64_t dx = desc_hi | (((base + kTileBytesW) & 0x3FFFF) >> 4);
#pragma unroll
                        for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
                            // Advancing 16 BF16 = 32 bytes inside the swizzled row: +2 in the descriptor's 16-byte units.
                            umma_bf16(acc, dw + 2 * kk, dx + 2 * kk, idesc, (it >= issuers) | (kk != 0));
                        }
                        umma_commit(&sm->empty[st]);
                    }
                    if (++st == g.stages) st = 0, parity ^= 1;
                }
                umma_commit(&sm->acc_full);
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // Epilogue: thread `lane` of a warp holds feature 32 * quarter + lane; 16 token columns per tcgen05.ld.
        const int quarter = warp & 3, half = (warp - 4) >> 2;
        const int feature = quarter * 32 + lane;
        bool ok = true;
        if (iters > 0) {
            ok = mbar_wait(&sm->acc_full, 0, pipeline_deadline);
            if (!ok) report(c.status, kErrTimeout, 0, kPhasePipeline, stalled(2, iters));
            tcgen05_fence_after();
        }
        if (c.stamps && threadIdx.x == 128) c.stamps[block * kStampSlots + 4] = globaltimer();
        // One K split: the BF16 tile is staged in shared memory, token-major, over the drained pipeline stages.
        // Several: this CTA's FP32 partial tile goes to the workspace (which the previous kernel of the chain may
        // still be reading, hence the wait).
        float* part = g.ws + (static_cast<size_t>(tile) * g.splits + s) * mt * kBlockF;
        __nv_bfloat16* staged = reinterpret_cast<__nv_bfloat16*>(tiles);
        if (g.splits > 1) pdl_wait();
        for (int chunk = half; chunk < mt / 16; chunk += 2) {
            uint32_t r[16];
            if (iters > 0 && ok) {
                const uint32_t at = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + chunk * 16;
                tmem_load_16(at, r);
                tmem_load_wait();
                if (issuers == 2) {
                    uint32_t q[16];
                    tmem_load_16(at + cols, q);
                    tmem_load_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(q[j]));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0;
            }
            if (g.splits > 1) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    part[static_cast<size_t>(chunk * 16 + j) * kBlockF + feature] = __uint_as_float(r[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    staged[(chunk * 16 + j) * kBlockF + feature] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
        }
        tcgen05_fence_before();
    }
    pdl_wait();
    __syncthreads();
    if (warp == 2) {
        tcgen05_fence_after();
        tmem_dealloc(tmem, cols * issuers);
    }

    CommCtx x{};
    if (p.fused) {
        x = comm_begin(c, block, blocks, sm->epoch, sm->failed);
        stamp(c, x, 0);
    }
    if (local_rows) {
        // Announce this CTA's partial tile on the counter of its token tile; the rows' owners wait for it below.
        const int gen = sm->gen + 1;
        if (threadIdx.x == 0) {
            for (int j = block; j < kMaxTiles; j += blocks) g.counters[((gen + 1) & 1) * kMaxTiles + j] = 0;
            __threadfence();  // after the block barrier: orders every thread's partial-tile stores before the announce
            atomicAdd(g.counters + (gen & 1) * kMaxTiles + t, 1);
            for (int j = block; j < kEpochSlots; j += blocks) g.gen[j] = gen;
        }
    } else if (g.splits > 1) {
        // Split-K rendezvous: every CTA of the tile announces its partial, waits for the others, then sums ITS share of
        // the tile's tokens over the splits in split order (so the value never depends on timing) and pushes it.
        // Arrival counters alternate between two banks by launch generation; this launch clears the whole other bank
        // (whatever tiling the next launch on this workspace uses, it finds its counters at zero).
        const int gen = sm->gen + 1;
        int* counter = g.counters + (gen & 1) * kMaxTiles + tile;
        if (threadIdx.x == 0) {
            for (int j = block; j < kMaxTiles; j += blocks) g.counters[((gen + 1) & 1) * kMaxTiles + j] = 0;
            __threadfence();  // after the block barrier: orders every thread's partial-tile stores before the announce
            atomicAdd(counter, 1);
            int seen;
            do {
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
                if (seen >= g.splits) break;
                if (globaltimer() > pipeline_deadline) {
                    report(c.status, kErrTimeout, s, kPhasePipeline, 3 << 24);
                    break;
                }
            } while (true);
            for (int j = block; j < kEpochSlots; j += blocks) g.gen[j] = gen;
        }
        __syncthreads();
        const int tok_lo = static_cast<int>(static_cast<long long>(s) * mt / g.splits);
        const int tok_hi = static_cast<int>(static_cast<long long>(s + 1) * mt / g.splits);
        const float* base = g.ws + static_cast<size_t>(tile) * g.splits * mt * kBlockF;
        const size_t split_stride = static_cast<size_t>(mt) * kBlockF;
        for (int v = threadIdx.x; v < (tok_hi - tok_lo) * (kBlockF / kVec); v += kFusedThreads) {
            const int token = tok_lo + v / (kBlockF / kVec), j = v % (kBlockF / kVec);
            const float* src = base + static_cast<size_t>(token) * kBlockF + j * kVec;
            // Summed in split order, four splits' loads in flight at a time.
            float acc[kVec];
            for (int base_sp = 0; base_sp < g.splits; base_sp += 4) {
                float4 a[4], b[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (base_sp + u < g.splits) {
                        a[u] = __ldcg(reinterpret_cast<const float4*>(src + (base_sp + u) * split_stride));
                        b[u] = __ldcg(reinterpret_cast<const float4*>(src + (base_sp + u) * split_stride) + 1);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (base_sp + u < g.splits) {
                        if (base_sp + u == 0) {
                            acc[0] = a[u].x, acc[1] = a[u].y, acc[2] = a[u].z, acc[3] = a[u].w;
                            acc[4] = b[u].x, acc[5] = b[u].y, acc[6] = b[u].z, acc[7] = b[u].w;
                        } else {
                            acc[0] += a[u].x, acc[1] += a[u].y, acc[2] += a[u].z, acc[3] += a[u].w;
                            acc[4] += b[u].x, acc[5] += b[u].y, acc[6] += b[u].z, acc[7] += b[u].w;
                        }
                    }
                }
            }
            const uint4 packed = pack_bf16x8(acc);
            const int col = f * kBlockF + j * kVec;
            if (p.fused) {
                push_store(c, x, token0 + token, col, packed);
            } else {
                store_v4(g.out + static_cast<size_t>(token0 + token) * g.ldo + col, packed);
            }
        }
    } else {
        const uint4* staged = reinterpret_cast<const uint4*>(tiles);
        for (int v = threadIdx.x; v < mt * (kBlockF / kVec); v += kFusedThreads) {
            const int token = v / (kBlockF / kVec), j = v % (kBlockF / kVec);
            const uint4 packed = staged[v];
            const int col = f * kBlockF + j * kVec;
            if (p.fused) {
                push_store(c, x, token0 + token, col, packed);
            } else {
                store_v4(g.out + static_cast<size_t>(token0 + token) * g.ldo + col, packed);
            }
        }
    }
    if (p.fused) {
        if (c.stamps && threadIdx.x == 0) c.stamps[block * kStampSlots + 6] = globaltimer();
        stamp(c, x, 1);
        rearm_early(c, x);
        if (local_rows) {
            const int* counter = g.counters + ((sm->gen + 1) & 1) * kMaxTiles;
            if (c.mode == kReduce) own_rows_from_splits<kReduce>(g, c, x, counter, mt, sm->scratch);
            else if (c.mode == kReduceNorm) own_rows_from_splits<kReduceNorm>(g, c, x, counter, mt, sm->scratch);
            else own_rows_from_splits<kReduceNormResidual>(g, c, x, counter, mt, sm->scratch);
            rearm_late(c, x);
        } else {
            own_and_collect(c, x, sm->scratch);  // re-arms late shares between its own and collect phases
        }
        comm_end(c, x);
    }
}

int rowpar_stages(int m) {  // m: tokens per tile
    const int stage = kTileBytesW + m * kBlockK * 2;
    int stages = kSmemBudget / stage;  // the ring takes what an SM has
    if (stages > kMaxStages) stages = kMaxStages;
    return stages;
}

int rowpar_smem_bytes(int m, int stages) {
    return stages * (kTileBytesW + m * kBlockK * 2) + static_cast<int>(sizeof(SmemLayout)) + 1024;
}

template <int NR>
static int launch_impl(const RowparParams<NR>& p, dim3 grid, const LaunchOpts& o) {
    const int smem = rowpar_smem_bytes(p.g[0].m / p.g[0].token_tiles, p.g[0].stages);
    // Raised once per device to the largest configuration (not a stream operation, but kept out of graph captures).
    static bool raised[64] = {};
    cudaError_t err = cudaSuccess;
    int dev = 0;
    (void)cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !raised[dev]) {
        err = cudaFuncSetAttribute(rowpar_kernel<NR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   kSmemBudget + static_cast<int>(sizeof(SmemLayout)) + 1024);
        raised[dev] = err == cudaSuccess;
    }
    if (err == cudaSuccess) {
        cudaLaunchConfig_t config{};
        config.gridDim = grid;
        config.blockDim = dim3(kFusedThreads);
        config.dynamicSmemBytes = static_cast<size_t>(smem);
        config.stream = o.stream;
        cudaLaunchAttribute attrs[2];
        int n = 0;
        if (o.pdl) {
            attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attrs[n].val.programmaticStreamSerializationAllowed = 1;
            ++n;
        }
        if (o.cooperative) {
            attrs[n].id = cudaLaunchAttributeCooperative;
            attrs[n].val.cooperative = 1;
            ++n;
        }
        config.attrs = attrs;
        config.numAttrs = n;
        err = cudaLaunchKernelEx(&config, rowpar_kernel<NR>, p);
    }
    if (err != cudaSuccess) {
        g_last_cuda_error = static_cast<int>(err);
        (void)cudaGetLastError();
        return -6;
    }
    ++g_launches;
    return 0;
}

int launch_rowpar(const RowparParams<1>& p, int grid, const LaunchOpts& o) { return launch_impl<1>(p, dim3(grid), o); }

int launch_rowpar_loopback(const RowparParams<kMaxWorld>& p, int grid, int nranks, const LaunchOpts& o) {
    return launch_impl<kMaxWorld>(p, dim3(grid, nranks), o);
}

}  // namespace dlm
