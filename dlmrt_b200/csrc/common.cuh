// PTX building blocks for sm_100a: mbarrier, TMA, tcgen05 / TMEM, NVLS multicast store, programmatic dependent
// launch, bounded waits. Everything here is inline device code shared by the kernels of this library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace dlm {

constexpr int kVec = 8;                     // BF16 lanes per 16-byte vector
constexpr uint32_t kSentinel = 0xFFFFFFFFu; // two armed BF16 lanes (0xFFFF: a negative NaN arithmetic never yields)

// ---------------------------------------------------------------------------------------------------------------
// Time and status
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ long long globaltimer() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");  // ordered with barriers and memory operations
    return t;
}

enum Phase { kPhaseReceive = 1, kPhaseOut = 2, kPhasePipeline = 3 };
constexpr int kErrTimeout = -8;  // DLM_ERR_TIMEOUT

// First error wins; the words are read and cleared by the host (dlm_status_read).
__device__ __forceinline__ void report(int* status, int code, int slot, int phase, int epoch) {
    if (status == nullptr) return;
    if (atomicCAS(status, 0, code) == 0) {
        status[1] = (static_cast<int>(blockIdx.x) << 8) | (slot & 0xFF);
        status[2] = phase;
        status[3] = epoch;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Programmatic dependent launch
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------------------------
// Global memory: volatile 16-byte loads for in-band arrival polling, multicast store
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 load_volatile(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__device__ __forceinline__ void store_v4(void* p, const uint4& v) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// One store that lands in every rank's copy through the NVSwitch multicast object.
__device__ __forceinline__ void multicast_store(void* mc, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}

// A 16-byte vector has arrived once none of its eight BF16 lanes holds the sentinel.
__device__ __forceinline__ bool arrived(const uint4& v) {
    auto ok = [](uint32_t w) { return (w & 0xFFFFu) != 0xFFFFu && (w >> 16) != 0xFFFFu; };
    return ok(v.x) && ok(v.y) && ok(v.z) && ok(v.w);
}

// ---------------------------------------------------------------------------------------------------------------
// BF16 <-> FP32 on 16-byte vectors
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void add_bf16x8(float (&acc)[kVec], const uint4& v) {
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(b[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
    }
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&v)[kVec]) {
    uint4 out;
    __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return out;
}

// ---------------------------------------------------------------------------------------------------------------
// Shared memory addresses, mbarrier
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait on an mbarrier phase: false when the deadline passed (the caller reports and unwinds). try_wait itself
// blocks for a hardware-defined slice, so the timer is read only between slices.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, long long deadline) {
    while (!mbar_try_wait(bar, parity)) {
        if (globaltimer() > deadline) return mbar_try_wait(bar, parity);
    }
    return true;
}

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Asynchronous 4- and 16-byte global -> shared copies (no register staging) and their completion on an mbarrier:
// the arrival fires once all of this thread's earlier cp.async copies have landed; .noinc means the barrier's
// expected count must already include it.
__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n"
        ".reg .b32 rx;\n"
        ".reg .pred px;\n"
        "elect.sync rx|px, %1;\n"
        "@px mov.s32 %0, 1;\n"
        "}\n"
        : "+r"(pred)
        : "r"(0xFFFFFFFFu));
    return pred != 0;
}

// ---------------------------------------------------------------------------------------------------------------
// TMA (tiled bulk tensor loads into this CTA's shared memory; no cluster multicast anywhere in this library)
// ---------------------------------------------------------------------------------------------------------------
constexpr uint64_t kEvictNormal = 0x1000000000000000ull;
constexpr uint64_t kEvictFirst = 0x12F0000000000000ull;
constexpr uint64_t kEvictLast = 0x14F0000000000000ull;

__device__ __forceinline__ void tma_prefetch_descriptor(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// x = innermost coordinate (elements; x * element size must be a multiple of 16 bytes), y = row.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int x, int y,
                                            uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(hint)
        : "memory");
}

// Untiled bulk copy of `bytes` (a multiple of 16, both addresses 16-byte aligned) of contiguous global memory.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar,
                                          uint64_t hint) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)), "l"(hint)
        : "memory");
}

// Prefetches into L2 only: a contiguous range, or one box of a tensor map. Nothing is written to shared memory and
// nothing signals completion; the loads that follow simply find the data closer.
__device__ __forceinline__ void bulk_prefetch_l2(const void* gmem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_prefetch_l2_2d(const void* tmap, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(tmap)),
                 "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, uint64_t* bar, int x, int y, int z,
                                            uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5}], [%2], %6;"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z),
        "l"(hint)
        : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// tcgen05: tensor memory and the 5th-generation MMA (one CTA, cta_group::1)
// ---------------------------------------------------------------------------------------------------------------
// Allocates `cols` (a power of two >= 32) TMEM columns; the base address is written to *smem_result. One full warp.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the 128-byte swizzle
// (what a TMA box of 64 BF16 x rows with CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups 1024 bytes apart.
// Bits: [0,14) start address >> 4; [16,30) leading byte offset >> 4 (unused for swizzled K-major, set to 1);
// [32,46) stride byte offset >> 4 (1024 >> 4); [46,48) descriptor version 1 (Blackwell); [61,64) layout 2 = 128B.
__device__ __forceinline__ uint64_t umma_desc_k128(const void* smem_tile) {
    const uint32_t addr = smem_u32(smem_tile);
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor of kind::f16 with BF16 A and B (both K-major), FP32 accumulate, D = [m x n].
// Bits: [4,6) D format 1 = F32; [7,10) A format 1 = BF16; [10,13) B format 1 = BF16; 15/16 A/B major 0 = K;
// [17,23) n >> 3; [24,29) m >> 4.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread. accumulate = 0 overwrites D.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// ---- block-scaled FP4 (NVFP4: E2M1 values, one UE4M3 scale per 16 elements along K) --------------------------------
// Instruction descriptor of kind::mxf4nvf4: bits [7,10) A format 1 = E2M1, [10,13) B format 1 = E2M1, 15/16 majors 0 = K,
// [17,23) n >> 3, bit 23 scale format 0 = UE4M3, [24,29) m >> 4, bit 31 = 0: K = 64 per instruction. The scale-factor
// ids at [4,6) and [29,31) stay 0: with four scales per row (scale_vec::4X) the whole 32-bit TMEM word is used.
__host__ __device__ constexpr uint32_t umma_idesc_nvfp4(int m, int n) {
    return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= (A * SFA)[smem] * (B * SFB)[smem]^T, K = 64 FP4 elements (32 bytes of each K-major row). The scale
// factors are read from tensor memory: row r of the operand finds its four bytes at lane r % 32, column r / 32 of the
// given address (each 32-lane quarter holds a copy), which is what utccp_128x4() below writes.
__device__ __forceinline__ void umma_nvfp4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

// Descriptor of one 512-byte scale-factor atom in shared memory: 32 rows of 16 bytes, unswizzled, 8-row groups 128
// bytes apart. Byte (r % 32) * 16 + (r / 32) * 4 + j of the atom is scale j (0..3) of operand row r (0..127).
__device__ __forceinline__ uint64_t utccp_desc(const void* smem_atom) {
    const uint32_t addr = smem_u32(smem_atom);
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(128 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}

// Copies one such atom into four TMEM columns starting at `taddr`, replicated into all four 32-lane quarters.
__device__ __forceinline__ void utccp_128x4(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

// Arrives on `bar` once every MMA issued so far by this thread has completed (implies fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 32 lanes x 16 consecutive FP32 columns: thread l of the warp receives row (lane base + l), columns [c, c + 16).
__device__ __forceinline__ void tmem_load_16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
        "[%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace dlm
