// NVFP4 MoE expert down-projection (GEMM2 of the routed experts), the weighted top-k combine, and the tensor-parallel
// reduction that follows, in one kernel for sm_100a.
//
//   y[token, k]   = bf16( (sum over f of act[slot, f] * W2[e, :, f]) * g2[e] )        e = ids[token, k] local to the rank
//   out[token]    = bf16( sum over k in list order of weight[token, k] * y[token, k] )  (+ shared -> bf16)
//   then out is this rank's partial of the all-reduce (experts are split whole across ranks).
//
// Arithmetic follows the reference's statement of the TRT-LLM-gen MoE roundings, dlmrt/ops/triton/nvfp4_moe.py:107-150
// (FP32 dot of E2M1 x E4M3-per-16 operands, times g2, BF16 per (token, expert); FP32 combine in list order); the entry
// point replaces dlmrt/quantization/nvfp4.py:280-306 (`trtllm_moe`) plus the add and reduce of
// dlmrt/models/llada2/model.py:354-362,437-438.
//
// Work item = (active local expert, 128 output features): W2's [128 x F] slab sits on the MMA's M axis, the expert's
// rows (tokens routed to it, padded to 16) on its N axis. Persistent CTAs take items round-robin:
//   warp 0   TMA: per 256-element k-block the 16 KB code slab of W2 (one bulk copy of a pre-tiled slab, or one box)
//   warp 12  TMA: the expert's activation rows of the k-block (boxes of 8 rows)
//   warp 3   scale loader: W2's pre-interleaved 128 x 4 scale atoms and the activation rows' linear E4M3 scales,
//            rewritten into the same atom layout, into the stage
//   warp 1   per k-block: tcgen05.cp the scale atoms into tensor memory, then up to four
//            tcgen05.mma.kind::mxf4nvf4.block_scale (K = 64) into the FP32 accumulator
//   warps 4-11  per item: tcgen05.ld, times g2, BF16, scatter rows to Y[pair] through the expert's slot map
// When all CTAs are through their items (arrival counter), rows of the output are combined from Y in FP32 and pushed
// into the owner ranks' receive slots, and the reduction phases of comm.cuh follow.
//
// The same pipeline, instantiated with GATE_UP, is GEMM1 of the experts (the step in front of the down-projection,
// dlmrt/ops/triton/nvfp4_moe.py:69-104 `_gate_up`): W13 [2F x hidden] streams instead of W2, its rows interleaved
// (row 2i = gate feature i, row 2i + 1 = up feature i) so that a gate value and its up value sit in neighbouring lanes
// of the accumulator; the expert's rows are the NVFP4-quantised tokens routed to it. The epilogue scales by g1, applies
// SwiGLU or GeGLU in FP32, re-quantises to NVFP4 against 1 / a2 (per 16 features: E4M3 scale, E2M1 codes, the
// approximate-reciprocal recipe of nvfp4_moe.py:36-47) and writes codes and scales straight into the expert-major
// slots the down-projection reads. It ends there: no combine, no reduction.
#include "kernels.cuh"

namespace dlm {

namespace {

constexpr int kMoeThreads = kFusedThreads + 32;  // the dense kernel's twelve warps and a second producer
constexpr int kCodeTileW = 128 * 128;  // 128 rows x 128 bytes (256 FP4) of W2 codes
constexpr int kBoxRows = 8;            // activation rows per TMA box (one 1 KB swizzle atom)
constexpr int kAtom = 512;             // one 128-row x 4-scale atom
constexpr int kStepsPerBlock = 4;      // K = 64 instructions per 256-element k-block
constexpr int kItemRows = 128;         // rows of one work item: the MMA's N; experts with more rows take several items
constexpr int kTmemAcc = 0, kTmemSfa = 256, kTmemSfb = 384, kTmemCols = 512;  // two 128-column accumulators, then scales
// Scale columns rotate over four sets (two per issuer: (2 * who + set) below), so copying a k-block's scales in does
// not have to wait for the previous k-block's MMAs to finish reading theirs.
constexpr int kMaxLocalExperts = 256;
constexpr int kMaxEntries = 2 * kMaxLocalExperts;  // (expert, row block) pairs: m_max <= 256 gives at most two blocks

struct MoeSmem {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int n_active, epoch, gen, failed;
    int seen[2];  // k-blocks (counted over this CTA's items) each issuer has seen arrive
    int warp_count[8];
    float scratch[64];
    short active[kMaxEntries];  // expert | row block << 8
    short rows[kMaxEntries];    // rows of that block
};

}  // namespace

int moe_stage_bytes(int rows_cap) {  // rows_cap: rows of one item's activation tile (a multiple of 32, <= 128)
    return kCodeTileW + rows_cap * 128 + 2 * kStepsPerBlock * kAtom;
}

int moe_stages(int rows_cap) {
    int s = kSmemBudget / moe_stage_bytes(rows_cap);
    return s > kMaxStages ? kMaxStages : s;
}

// A token's expert list for the combine step, eight entries at a time: local expert index (or -1) and routing weight.
constexpr int kCombineBatch = 8;
struct CombineMeta {
    int e[kCombineBatch];
    float w[kCombineBatch];
};

// Entries [k0, k0 + 8) of row `row`: all loads are independent, so they cost one round trip, and they depend on
// nothing this launch computes (callers issue them before waiting for the expert outputs).
__device__ __forceinline__ CombineMeta combine_meta(const MoeDev& g, int row, int k0) {
    CombineMeta m;
#pragma unroll
    for (int j = 0; j < kCombineBatch; ++j) {
        const bool have = k0 + j < g.top_k;
        const int e = have ? g.ids[row * g.top_k + k0 + j] - g.lo : -1;
        m.e[j] = e >= 0 && e < g.e_local ? e : -1;
        m.w[j] = have ? g.weights[row * g.top_k + k0 + j] : 0.f;
    }
    return m;
}

// One output row of the combine step for thread t's eight columns: FP32 sum over the token's expert list, in list
// order, of weight * y (fused multiply-add; experts of other ranks contribute 0 * 0), rounded to BF16, then the
// shared expert's BF16 row added and rounded again (dlmrt/ops/triton/nvfp4_moe.py:134-150). `first` holds entries
// [0, 8) of the row, fetched early; the expert outputs of a batch are loaded together and added in list order.
__device__ __forceinline__ uint4 combine_row(const MoeDev& g, int row, int t, const CombineMeta& first) {
    float acc[kVec] = {};
    for (int k0 = 0; k0 < g.top_k; k0 += kCombineBatch) {
        const CombineMeta m = k0 == 0 ? first : combine_meta(g, row, k0);
        uint4 raw[kCombineBatch];
#pragma unroll
        for (int j = 0; j < kCombineBatch; ++j) {
            raw[j] = make_uint4(0, 0, 0, 0);
            if (m.e[j] >= 0)
                raw[j] = __ldcg(reinterpret_cast<const uint4*>(g.y + static_cast<size_t>(row * g.top_k + k0 + j) * g.n) + t);
        }
#pragma unroll
        for (int j = 0; j < kCombineBatch; ++j) {
            if (k0 + j < g.top_k) {
                const float w = m.e[j] >= 0 ? m.w[j] : 0.f;
                const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(b[i]);
                    acc[2 * i] = fmaf(w, f.x, acc[2 * i]);
                    acc[2 * i + 1] = fmaf(w, f.y, acc[2 * i + 1]);
                }
            }
        }
    }
    uint4 packed = pack_bf16x8(acc);
    if (g.shared) {
        float v[kVec] = {};
        add_bf16x8(v, packed);
        add_bf16x8(v, *(reinterpret_cast<const uint4*>(g.shared + static_cast<size_t>(row) * g.n) + t));
        packed = pack_bf16x8(v);
    }
    return packed;
}

// Single rank: combine each owned row and finish it (residual + RMSNorm by mode, store into OUT) in one go.
template <int MODE>
__device__ __forceinline__ void combine_and_finish(const MoeDev& g, const CommDev& c, int block, int blocks, float* scratch,
                                                   const CombineMeta& first) {
    const int t = threadIdx.x, threads = g.n / kVec;
    const bool active = t < threads;
    const int col = (active ? t : 0) * kVec;
    uint4 wraw = make_uint4(0, 0, 0, 0);
    if (MODE != kReduce && active) wraw = *reinterpret_cast<const uint4*>(c.weight + col);
    for (int row = block; row < g.m; row += blocks) {
        const size_t off = static_cast<size_t>(row) * c.n + col;
        uint4 hraw = make_uint4(0, 0, 0, 0);
        if (MODE == kReduceNormResidual && active) hraw = *reinterpret_cast<const uint4*>(c.h + off);
        float v[kVec] = {};
        if (active) {  // +0.0f + partial: the rank-ordered sum over one rank
            add_bf16x8(v, combine_row(g, row, t, row == block ? first : combine_meta(g, row, 0)));
        }
        finish_row<MODE>(c, v, hraw, wraw, off, active, true, scratch, threads);
    }
}

// ---- NVFP4 re-quantisation of the activation (nvfp4_moe.py:20-47) --------------------------------------------------
__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// FP32 -> FP8 E4M3 bits (round to nearest even, saturating) and back.
__device__ __forceinline__ uint32_t f32_to_e4m3(float x) {
    uint16_t pair;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(0.f), "f"(x));
    return pair & 0xFFu;
}
__device__ __forceinline__ float e4m3_to_f32(uint32_t bits) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(bits)));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xFFFFu)));
}

// One byte of two E2M1 codes (nearest, ties to the even code, saturating at 6): `lo` in the low nibble.
__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
    uint32_t out;
    asm("{\n.reg .b8 t;\ncvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\ncvt.u32.u8 %0, t;\n}" : "=r"(out) : "f"(hi), "f"(lo));
    return out;
}

__device__ __forceinline__ float gated_activation(float gate, float up, int kind) {
    if (kind == 0) return gate * (1.f / (1.f + __expf(-gate))) * up;  // SwiGLU: g * sigmoid(g) * u
    const float inner = 0.7978845608028654f * (gate + 0.044715f * gate * gate * gate);
    return 0.5f * gate * (1.f + tanhf(inner)) * up;                  // GeGLU with the tanh GELU
}

template <int NR, bool GATE_UP>
__global__ void __launch_bounds__(kMoeThreads, 1) moe_kernel(const __grid_constant__ MoeParams<NR> p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const int slot = NR == 1 ? 0 : static_cast<int>(blockIdx.y);
    const MoeDev& g = p.g[slot];
    const CommDev& c = p.c[slot];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int block = static_cast<int>(blockIdx.x), blocks = static_cast<int>(gridDim.x);
    if (c.stamps && threadIdx.x == 0) c.stamps[block * kStampSlots + 7] = globaltimer();

    const int stage_bytes = kCodeTileW + g.rows_cap * 128 + 2 * kStepsPerBlock * kAtom;
    const int off_a = kCodeTileW, off_sfa = off_a + g.rows_cap * 128, off_sfb = off_sfa + kStepsPerBlock * kAtom;
    const int feature_tiles = g.n / kBlockF;
    const int steps = g.f / 64;                  // K = 64 instructions per item
    const int nkb = (steps + kStepsPerBlock - 1) / kStepsPerBlock;
    const int scale_row = g.f / 16;              // bytes of scales per activation row

    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    MoeSmem* sm = reinterpret_cast<MoeSmem*>(tiles + g.stages * stage_bytes);

    if (threadIdx.x == 0) {
        for (int i = 0; i < g.stages; ++i) {
            mbar_init(&sm->full[i], 33);  // the TMA producer's expect_tx arrival and the scale loader's 32 lanes
            mbar_init(&sm->empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sm->acc_full[i], 1);
            mbar_init(&sm->acc_empty[i], 8);  // one arrival per epilogue warp
        }
        fence_barrier_init();
        tma_prefetch_descriptor(&g.tm_w);
        tma_prefetch_descriptor(&g.tm_a);
        sm->seen[0] = sm->seen[1] = 0;
    }
    if (warp == 2) tmem_alloc(&sm->tmem_base, kTmemCols);
    // The next kernel of the stream may be set up from now on (its blocks move in as this kernel's blocks leave).
    pdl_launch_dependents();
    // Routing (counts, slots, activations) comes from the previous kernels of the stream: nothing of it may be read
    // before they are complete.
    pdl_wait();
    // Compact list of (expert, block of 128 rows) pairs that have rows, in expert order.
    {
        const int e = threadIdx.x;
        const int total_rows = e < g.e_local ? min(g.counts[g.lo + e], g.m_max) : 0;
        int early = 0;  // the invocation counters, fetched in the same round trip as the counts
        if (!GATE_UP) {
            if (threadIdx.x == 352 && p.fused) early = c.epochs[block];
            if (threadIdx.x == 353) early = g.gen[block];
            if (threadIdx.x == 354 && p.fused) early = comm_failed(c);
        }
        const int nb = (total_rows + kItemRows - 1) / kItemRows;
        int incl = nb;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffff, incl, o);
            if (lane >= o) incl += up;
        }
        if (warp < 8 && lane == 31) sm->warp_count[warp] = incl;
        tcgen05_fence_before();
        __syncthreads();
        tcgen05_fence_after();
        if (warp < 8) {
            int base = 0;
            for (int wv = 0; wv < warp; ++wv) base += sm->warp_count[wv];
            for (int j = 0; j < nb; ++j) {
                sm->active[base + incl - nb + j] = static_cast<short>(e | (j << 8));
                sm->rows[base + incl - nb + j] = static_cast<short>(min(total_rows - j * kItemRows, kItemRows));
            }
            if (threadIdx.x == 0) {
                int total = 0;
                for (int wv = 0; wv < 8; ++wv) total += sm->warp_count[wv];
                sm->n_active = total;
            }
        }
        if (threadIdx.x == 352) sm->epoch = early;
        if (threadIdx.x == 353) sm->gen = early;
        if (threadIdx.x == 354) sm->failed = early;
        __syncthreads();
    }
    if (c.stamps && threadIdx.x == 0) c.stamps[block * kStampSlots + 0] = globaltimer();
    const uint32_t tmem = sm->tmem_base;
    const int n_items = sm->n_active * feature_tiles;
    const long long deadline = globaltimer() + (c.timeout_ns > 0 ? c.timeout_ns : kDefaultTimeoutNs);

    // An item: entry (expert e, row block rb) x feature tile ft; `cnt` rows of the expert starting at row0.
    struct Item {
        int e, ft, row0, cnt;
    };
    auto item_of = [&](int i) {
        const int entry = sm->active[i / feature_tiles];
        Item t;
        t.e = entry & 0xFF, t.ft = i % feature_tiles, t.row0 = (entry >> 8) * kItemRows;
        t.cnt = sm->rows[i / feature_tiles];
        return t;
    };

    if (warp == 0) {
        if (lane == 0) {
            int st = 0;
            uint32_t phase = 1;  // waiting for parity 1 on a fresh barrier returns at once: the first lap is free
            for (int i = block; i < n_items; i += blocks) {
                const Item t = item_of(i);
                const int boxes = (t.cnt + kBoxRows - 1) / kBoxRows;
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait(&sm->empty[st], phase, deadline)) {
                        report(c.status, kErrTimeout, st, kPhasePipeline, 0);
                        i = n_items;
                        break;
                    }
                    uint8_t* stage = tiles + st * stage_bytes;
                    mbar_expect_tx(&sm->full[st], static_cast<uint32_t>(kCodeTileW + boxes * kBoxRows * 128));
                    if (g.w_tiles)  // one contiguous 16 KB run of HBM, already in the swizzled shared-memory order
                        bulk_load(stage, g.w_tiles + (static_cast<size_t>(t.e * feature_tiles + t.ft) * nkb + kb) * kCodeTileW,
                                  kCodeTileW, &sm->full[st], kEvictFirst);
                    else
                        tma_load_2d(stage, &g.tm_w, &sm->full[st], kb * 128, t.e * g.n + t.ft * kBlockF, kEvictFirst);
                    if (++st == g.stages) st = 0, phase ^= 1;
                }
            }
        }
        __syncwarp();  // lanes 1-31 must not run ahead to the block-wide barrier while lane 0 is still issuing
    } else if (warp == 12) {
        // Second producer: the expert's activation rows (boxes of 8 rows), so that the thread that requests the weight
        // slabs has one copy per k-block to issue (config 5, several boxes per k-block: 47.9 instead of 49.5 us per
        // layer; config 4: no change). It only adds bytes to a phase the weight producer announces.
        if (lane == 0) {
            int st = 0;
            uint32_t phase = 1;
            for (int i = block; i < n_items; i += blocks) {
                const Item t = item_of(i);
                const int boxes = (t.cnt + kBoxRows - 1) / kBoxRows;
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait(&sm->empty[st], phase, deadline)) {
                        report(c.status, kErrTimeout, st, kPhasePipeline, 0);
                        i = n_items;
                        break;
                    }
                    uint8_t* stage = tiles + st * stage_bytes;
                    for (int b = 0; b < boxes; ++b)
                        tma_load_2d(stage + off_a + b * kBoxRows * 128, &g.tm_a, &sm->full[st], kb * 128,
                                    t.e * g.m_max + t.row0 + b * kBoxRows, kEvictLast);
                    if (++st == g.stages) st = 0, phase ^= 1;
                }
            }
        }
        __syncwarp();
    } else if (warp == 3) {
        // Scale loader: asynchronous copies straight into the atoms, so it never waits for data and runs as far ahead
        // as the ring allows. Atom byte (r % 32) * 16 + (r / 32) * 4 + j holds scale j of row r (< 128).
        const int last_slot = g.e_local * g.m_max - 1;
        int st = 0;
        uint32_t phase = 1;
        for (int i = block; i < n_items; i += blocks) {
            const Item t = item_of(i);
            const int rows = (t.cnt + 15) & ~15;  // the MMA reads scales of all its N rows
            bool alive = true;
            for (int kb = 0; kb < nkb; ++kb) {
                if (!mbar_wait(&sm->empty[st], phase, deadline)) {
                    alive = false;
                    break;
                }
                uint8_t* stage = tiles + st * stage_bytes;
                const int nsteps = min(kStepsPerBlock, steps - kb * kStepsPerBlock);
                const uint8_t* wsrc =
                    g.w_scales + (static_cast<size_t>(t.e * feature_tiles + t.ft) * steps + kb * kStepsPerBlock) * kAtom;
                for (int v = lane; v < nsteps * (kAtom / 16); v += 32) cp_async_16(stage + off_sfa + v * 16, wsrc + v * 16);
                for (int r = lane; r < rows; r += 32) {
                    // Rows past the expert's count are padding: any readable scale will do for them.
                    const int srow = min(t.e * g.m_max + t.row0 + r, last_slot);
                    const uint8_t* src = g.a_scales + static_cast<size_t>(srow) * scale_row + kb * kStepsPerBlock * 4;
                    uint8_t* dst = stage + off_sfb + (r % 32) * 16 + (r / 32) * 4;
                    for (int s2 = 0; s2 < nsteps; ++s2) cp_async_4(dst + s2 * kAtom, src + s2 * 4);
                }
                cp_async_arrive(&sm->full[st]);
                if (++st == g.stages) st = 0, phase ^= 1;
            }
            if (!alive) break;
        }
    } else if (warp == 1 || warp == 2) {
        // Two threads feed the tensor pipe: warp 1 takes this CTA's even work items, warp 2 the odd ones. Each item has
        // its own accumulator buffer anyway (item & 1), and each issuer its own two sets of scale columns, so the two
        // instruction streams never touch the same tensor memory. One thread alone is the bottleneck of the stream:
        // per 256-element k-block it waits on a barrier, issues eight scale copies and four MMAs and commits. Ring
        // position, phase and scale set advance by increments (no divisions); descriptors differ by constants.
        const int who = warp - 1;
        if (lane == 0) {
            const uint32_t stage0 = smem_u32(tiles);
            const uint64_t desc_hi = umma_desc_k128(tiles) & 0xFFFFFFFF00000000ull;     // swizzled operand tiles
            const uint64_t sf_hi = utccp_desc(tiles) & 0xFFFFFFFF00000000ull;           // scale atoms
            int st = 0, set = 0, item = 0, seq = 0;  // seq: this k-block's number in the CTA's sequence
            uint32_t phase = 0;
            bool alive = true;
            // A parity wait tells a barrier's phases apart only while the waiter is never a whole phase behind, and an
            // issuer skips the phases of the other's items. So before it waits for k-block `seq` it makes sure that
            // k-block `seq - stages` (the same stage's previous phase) has been seen to arrive by whoever owns it; the
            // two publish what they have seen in shared memory. That k-block belongs to the other issuer iff the
            // number of items between the two is odd: (stages / nkb), or one more for the first stages % nkb k-blocks
            // of an item.
            const int q_items = g.stages / nkb, r_blocks = g.stages % nkb;
            volatile int* seen = sm->seen;
            const bool guarded = (q_items & 1) || r_blocks != 0;  // otherwise a stage always belongs to the same issuer
            for (int i = block; i < n_items && alive; i += blocks, ++item) {
                if ((item & 1) != who) {  // the other issuer's item: only step over its k-blocks in the ring
                    st += nkb;
                    seq += nkb;
                    while (st >= g.stages) st -= g.stages, phase ^= 1;
                    continue;
                }
                const int cnt = sm->rows[i / feature_tiles];
                const uint32_t idesc = umma_idesc_nvfp4(kBlockF, max(16, (cnt + 15) & ~15));
                const uint32_t acc = tmem + kTmemAcc + who * kItemRows;
                // The accumulator buffer must have been read out by the epilogue of two items ago.
                if (item >= 2 && !mbar_wait(&sm->acc_empty[who], ((item >> 1) - 1) & 1, deadline)) {
                    report(c.status, kErrTimeout, 0, kPhasePipeline, 4);
                    break;
                }
                for (int kb = 0; kb < nkb; ++kb, ++seq) {
                    if (guarded && seq >= g.stages && ((kb >= r_blocks ? q_items : q_items + 1) & 1)) {
                        while (alive && seen[1 - who] <= seq - g.stages) alive = globaltimer() <= deadline;
                    }
                    if (!alive || !mbar_wait(&sm->full[st], phase, deadline)) {
                        report(c.status, kErrTimeout, st, kPhasePipeline, 1);
                        alive = false;
                        break;
                    }
                    if (guarded) seen[who] = seq + 1;
                    fence_proxy_async();  // the scale atoms were written through the generic proxy
                    tcgen05_fence_after();
                    const uint32_t base = stage0 + st * stage_bytes;
                    const uint64_t dw = desc_hi | ((base & 0x3FFFF) >> 4), da = desc_hi | (((base + off_a) & 0x3FFFF) >> 4);
                    const uint64_t fa = sf_hi | (((base + off_sfa) & 0x3FFFF) >> 4), fb = sf_hi | (((base + off_sfb) & 0x3FFFF) >> 4);
                    const uint32_t sfa = tmem + kTmemSfa + (2 * who + set) * 4 * kStepsPerBlock;
                    const uint32_t sfb = tmem + kTmemSfb + (2 * who + set) * 4 * kStepsPerBlock;
                    const int nsteps = min(kStepsPerBlock, steps - kb * kStepsPerBlock);
                    if (nsteps == kStepsPerBlock) {
#pragma unroll
                        for (int s2 = 0; s2 < kStepsPerBlock; ++s2) {
                            utccp_128x4(sfa + 4 * s2, fa + s2 * (kAtom >> 4));
                            utccp_128x4(sfb + 4 * s2, fb + s2 * (kAtom >> 4));
                        }
#pragma unroll
                        for (int s2 = 0; s2 < kStepsPerBlock; ++s2)
                            umma_nvfp4(acc, dw + 2 * s2, da + 2 * s2, idesc, sfa + 4 * s2, sfb + 4 * s2, (kb | s2) != 0);
                    } else {
                        for (int s2 = 0; s2 < nsteps; ++s2) {
                            utccp_128x4(sfa + 4 * s2, fa + s2 * (kAtom >> 4));
                            utccp_128x4(sfb + 4 * s2, fb + s2 * (kAtom >> 4));
                        }
                        for (int s2 = 0; s2 < nsteps; ++s2)
                            umma_nvfp4(acc, dw + 2 * s2, da + 2 * s2, idesc, sfa + 4 * s2, sfb + 4 * s2, (kb | s2) != 0);
                    }
                    umma_commit(&sm->empty[st]);
                    set ^= 1;
                    if (++st == g.stages) st = 0, phase ^= 1;
                }
                if (alive) umma_commit(&sm->acc_full[who]);
            }
        }
        __syncwarp();
    } else if (warp >= 4 && warp < 12) {
        // Epilogue: lane = output feature of the tile, registers = the expert's rows.
        const int quarter = warp & 3, half = (warp - 4) >> 2;
        int item = 0;
        // What an item's epilogue needs from global memory: the expert's scale(s) and, for the down-projection, for each
        // of this warp's 16-row chunks (at most four) the destination row of lane % 16's accumulator column. Fetched
        // one item AHEAD: the epilogue warps go from item to item without a pause when the stream runs well, and a
        // round trip to L2 per item would then set the pace of the whole CTA.
        struct Meta {
            float g2, a2i;
            int dest[4];
        };
        auto fetch = [&](int i) {
            Meta m{0.f, 0.f, {-1, -1, -1, -1}};
            if (i >= n_items) return m;
            const Item t = item_of(i);
            m.g2 = g.g2[t.e];
            if (GATE_UP) {
                m.a2i = g.a2_inv[t.e];
            } else {
                const int* slots = g.amap + static_cast<size_t>(g.lo + t.e) * g.m_max + t.row0;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int row = (half + 2 * q) * 16 + (lane & 15);
                    m.dest[q] = row < t.cnt ? slots[row] : -1;
                }
            }
            return m;
        };
        Meta next = fetch(block);
        for (int i = block; i < n_items; i += blocks, ++item) {
            const Item t = item_of(i);
            const int n_mma = max(16, (t.cnt + 15) & ~15);
            const int buf = item & 1;
            const Meta cur = next;
            next = fetch(i + blocks);
            const float g2 = cur.g2, a2i = cur.a2i;
            const int(&dest)[4] = cur.dest;
            const bool ok = mbar_wait(&sm->acc_full[buf], (item >> 1) & 1, deadline);
            if (!ok) report(c.status, kErrTimeout, 0, kPhasePipeline, 2);
            tcgen05_fence_after();
            const int col = t.ft * kBlockF + quarter * 32 + lane;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int chunk = half + 2 * q;
                if (chunk < n_mma / 16 && ok) {
                    uint32_t r[16];
                    tmem_load_16(tmem + kTmemAcc + buf * kItemRows + (static_cast<uint32_t>(quarter * 32) << 16) + chunk * 16, r);
                    tmem_load_wait();
                    if (GATE_UP) {
                        // Tile row 2i holds gate feature i, row 2i + 1 its up feature: neighbouring lanes. The warp's 32
                        // lanes are one block of 16 activation features (ft * 64 + quarter * 16 ..) of 16 token rows.
                        const size_t slot0 = static_cast<size_t>(t.e) * g.m_max + t.row0;
                        const int half_f = g.f_out / 2, groups = g.f_out / 16;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float mine = __uint_as_float(r[j]) * g2;
                            const float other = __shfl_xor_sync(0xffffffff, mine, 1);
                            const float act = gated_activation(lane & 1 ? other : mine, lane & 1 ? mine : other, g.act_kind);
                            float amax = fabsf(act);
#pragma unroll
                            for (int o = 2; o < 32; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffff, amax, o));
                            const uint32_t sf = f32_to_e4m3(a2i * (amax * rcp_approx(6.f)));
                            const float scale = amax != 0.f ? rcp_approx(e4m3_to_f32(sf) * rcp_approx(a2i)) : 0.f;
                            const float y = act * scale;
                            const float y_next = __shfl_down_sync(0xffffffff, y, 2);  // the next feature's value
                            const int row = chunk * 16 + j;
                            if (row < t.cnt) {
                                if ((lane & 3) == 0)
                                    g.aq_out[(slot0 + row) * half_f + t.ft * 32 + quarter * 8 + (lane >> 2)] =
                                        static_cast<uint8_t>(e2m1x2(y, y_next));
                                if (lane == 0) g.as_out[(slot0 + row) * groups + t.ft * 4 + quarter] = static_cast<uint8_t>(sf);
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int pair = __shfl_sync(0xffffffff, dest[q], j);
                            if (pair >= 0)
                                g.y[static_cast<size_t>(pair) * g.n + col] = __float2bfloat16_rn(__uint_as_float(r[j]) * g2);
                        }
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->acc_empty[buf]);
            if (!ok) break;
        }
    }
    // Every Y row this CTA produced is written; announce it and wait for the rest of the grid (the combine reads rows
    // written by other CTAs). Counters are banked by launch generation as in the BF16 kernel.
    tcgen05_fence_before();
    __syncthreads();
    if (c.stamps && threadIdx.x == 0) c.stamps[block * kStampSlots + 4] = globaltimer();
    if (warp == 2) {
        tcgen05_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
    if (GATE_UP) return;  // the activation slots are written; the down-projection launch that follows does the rest
    CommCtx x{};
    if (p.fused) x = comm_begin(c, block, blocks, sm->epoch, sm->failed);
    // The expert list of this CTA's first output row is fetched now, ahead of the wait for the experts' outputs.
    CombineMeta first;
    if (block < g.m) first = combine_meta(g, block, 0);
    {
        const int gen = sm->gen + 1;
        int* counter = g.counters + (gen & 1) * kMaxTiles;
        if (threadIdx.x == 0) {
            if (block == 0) g.counters[((gen + 1) & 1) * kMaxTiles] = 0;
            __threadfence();  // after the block barrier: orders every thread's Y stores before the announce
            atomicAdd(counter, 1);
            // Only CTAs that have output rows to combine need the others' Y rows; polling is paced so that the
            // arrivals of the rest of the grid are not queued behind a storm of loads on the same word.
            while (block < g.m) {
                int seen;
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
                if (seen >= blocks) break;
                if (globaltimer() > deadline) {
                    report(c.status, kErrTimeout, 0, kPhasePipeline, 3);
                    break;
                }
                __nanosleep(100);
            }
            for (int j = block; j < kEpochSlots; j += blocks) g.gen[j] = gen;
        }
        __syncthreads();
    }
    if (c.stamps && threadIdx.x == 0) c.stamps[block * kStampSlots + 5] = globaltimer();
    // Combine: out[row] = bf16(sum over k in list order of w_k * y_k), experts of other ranks contribute 0 * 0.
    // With one rank the sum over ranks is the identity and the CTA that combines a row is also its owner (rows block,
    // block + blocks, ... in both roles), so the row is finished here and never travels through the receive slots.
    const bool local_rows = p.fused && c.world == 1;
    if (local_rows) {
        if (c.mode == kReduce) combine_and_finish<kReduce>(g, c, block, blocks, sm->scratch, first);
        else if (c.mode == kReduceNorm) combine_and_finish<kReduceNorm>(g, c, block, blocks, sm->scratch, first);
        else combine_and_finish<kReduceNormResidual>(g, c, block, blocks, sm->scratch, first);
    } else {
        const int t = threadIdx.x, threads = g.n / kVec;
        for (int row = block; row < g.m; row += blocks) {
            if (t < threads) {
                const uint4 packed = combine_row(g, row, t, row == block ? first : combine_meta(g, row, 0));
                if (p.fused) {
                    push_store(c, x, row, t * kVec, packed);
                } else {
                    store_v4(g.out + static_cast<size_t>(row) * g.ldo + t * kVec, packed);
                }
            }
        }
    }
    if (p.fused) {
        stamp(c, x, 1);
        rearm_early(c, x);
        if (local_rows) {
            stamp(c, x, 2);
            stamp(c, x, 3);
            rearm_late(c, x);
        } else {
            own_and_collect(c, x, sm->scratch);  // re-arms late shares between its own and collect phases
        }
        comm_end(c, x);
    }
}

template <int NR, bool GATE_UP>
static int launch_impl(const MoeParams<NR>& p, dim3 grid, const LaunchOpts& o) {
    const int smem = p.g[0].stages * moe_stage_bytes(p.g[0].rows_cap) + static_cast<int>(sizeof(MoeSmem)) + 1024;
    static bool raised[64] = {};
    cudaError_t err = cudaSuccess;
    int dev = 0;
    (void)cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !raised[dev]) {
        err = cudaFuncSetAttribute(moe_kernel<NR, GATE_UP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   kSmemBudget + static_cast<int>(sizeof(MoeSmem)) + 1024);
        raised[dev] = err == cudaSuccess;
    }
    if (err == cudaSuccess) {
        cudaLaunchConfig_t config{};
        config.gridDim = grid;
        config.blockDim = dim3(kMoeThreads);
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
        err = cudaLaunchKernelEx(&config, moe_kernel<NR, GATE_UP>, p);
    }
    if (err != cudaSuccess) {
        g_last_cuda_error = static_cast<int>(err);
        (void)cudaGetLastError();
        return -6;
    }
    ++g_launches;
    return 0;
}

int launch_moe(const MoeParams<1>& p, int grid, const LaunchOpts& o) { return launch_impl<1, false>(p, dim3(grid), o); }

int launch_moe_gate_up(const MoeParams<1>& p, int grid, const LaunchOpts& o) { return launch_impl<1, true>(p, dim3(grid), o); }

int launch_moe_loopback(const MoeParams<kMaxWorld>& p, int grid, int nranks, const LaunchOpts& o) {
    return launch_impl<kMaxWorld, false>(p, dim3(grid, nranks), o);
}

}  // namespace dlm
