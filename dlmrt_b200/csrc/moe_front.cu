// What runs in front of the experts' GEMM1: the router's top-k (route_packed_kernel) and, per token, the slot
// bookkeeping plus the NVFP4 quantisation of the expert input (moe_prepare_kernel).
//
//   route_packed   dlmrt/ops/triton/moe.py:14-47,70-73: FP32 softmax of the router logits, top-k (ties to the lower
//                  expert), renormalised, times the per-expert scale, listed in ascending expert order and packed as
//                  expert << 16 | BF16 weight bits (dlmrt/quantization/nvfp4.py:275-277).
//   prepare        what FlashInfer's routed MoE does inside its one call (dlmrt/quantization/nvfp4.py:280-306) and the
//                  reference's own kernels do in pieces: unpack the top-k; number every expert's rows in token order
//                  (deterministic, no atomics on the result: dlmrt/ops/triton/moe.py:50-60 `_route_slots`, slot map as
//                  token * top_k + k, dlmrt/ops/triton/nvfp4_moe.py:11-12); quantise the token's row to NVFP4 against
//                  the GEMM1 input scale (dlmrt/ops/triton/nvfp4_moe.py:36-66, the approximate-reciprocal recipe of
//                  fp4_quantize) or take it pre-quantised (dlmrt/models/diffusion_gemma/experts.py:64-67); copy it into
//                  the expert-major slot of each of its local experts.
#include "kernels.cuh"

namespace dlm {

namespace {

constexpr int kPrepareThreads = 256;
constexpr int kMaxTopK = 16;
constexpr int kMaxHidden = 8192;
constexpr int kMaxPairs = 256 * kMaxTopK;  // rows <= 256

__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

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

__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
    uint32_t out;
    asm("{\n.reg .b8 t;\ncvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\ncvt.u32.u8 %0, t;\n}" : "=r"(out) : "f"(hi), "f"(lo));
    return out;
}

}  // namespace

__global__ void __launch_bounds__(kPrepareThreads) moe_prepare_kernel(const __grid_constant__ PrepareDev p) {
    __shared__ int my_e[kMaxTopK], my_slot[kMaxTopK];
    __shared__ int expert_of[kMaxPairs];  // the whole routing, read once: both counts below scan it
    __shared__ __align__(16) uint8_t row_codes[kMaxHidden / 2];
    __shared__ __align__(16) uint8_t row_scales[kMaxHidden / 16];
    const int t = static_cast<int>(blockIdx.x), tid = static_cast<int>(threadIdx.x);
    const int k = p.top_k, pairs = p.rows * k;
    pdl_wait();  // the packed top-k and the input row come from the kernels before
    // The experts' first GEMM may be set up from now on; it waits for this kernel before it reads the slots.
    pdl_launch_dependents();
    for (int i = tid; i < pairs; i += kPrepareThreads) expert_of[i] = p.packed[i] >> 16;
    if (tid < k) {
        const int word = p.packed[t * k + tid];
        my_e[tid] = word >> 16;
        my_slot[tid] = 0;
        p.ids[t * k + tid] = word >> 16;
        p.weights[t * k + tid] = __uint_as_float(static_cast<uint32_t>(word & 0xFFFF) << 16);
    }
    __syncthreads();
    // Slot of each of this token's pairs: how many earlier pairs (lower token; a token lists an expert once) go to the
    // same expert. The count is a pure function of the routing, whatever order the threads add in.
    for (int i = tid; i < t * k; i += kPrepareThreads) {
        const int e = expert_of[i];
        for (int j = 0; j < k; ++j)
            if (e == my_e[j]) atomicAdd(&my_slot[j], 1);
    }
    // This CTA also counts the rows of experts t, t + rows, ...: one warp per expert, no block-wide step.
    for (int e = t + (tid >> 5) * p.rows; e < p.e_total; e += (kPrepareThreads / 32) * p.rows) {
        int mine = 0;
        for (int i = tid & 31; i < pairs; i += 32) mine += expert_of[i] == e;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffff, mine, o);
        if ((tid & 31) == 0) p.counts[e] = mine;
    }
    // The token's row as NVFP4: quantised here, or copied from the caller's pre-quantised input.
    const int blocks16 = p.hidden / 16;
    if (p.x != nullptr) {
        const float gs = *p.a1_inv;
        for (int b = tid; b < blocks16; b += kPrepareThreads) {
            const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(t) * p.hidden + b * 16);
            const uint4 raw[2] = {src[0], src[1]};
            const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(raw);
            float v[16];
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 f = __bfloat1622float2(v2[i]);
                v[2 * i] = f.x, v[2 * i + 1] = f.y;
                amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
            const uint32_t sf = f32_to_e4m3(gs * (amax * rcp_approx(6.f)));
            const float scale = amax != 0.f ? rcp_approx(e4m3_to_f32(sf) * rcp_approx(gs)) : 0.f;
            uint32_t lo = 0, hi = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                lo |= e2m1x2(v[2 * i] * scale, v[2 * i + 1] * scale) << (8 * i);
                hi |= e2m1x2(v[8 + 2 * i] * scale, v[9 + 2 * i] * scale) << (8 * i);
            }
            *reinterpret_cast<uint2*>(row_codes + b * 8) = make_uint2(lo, hi);
            row_scales[b] = static_cast<uint8_t>(sf);
        }
    } else {
        for (int i = tid; i < p.hidden / 32; i += kPrepareThreads)
            reinterpret_cast<uint4*>(row_codes)[i] = reinterpret_cast<const uint4*>(p.xq + static_cast<size_t>(t) * (p.hidden / 2))[i];
        for (int i = tid; i < blocks16 / 16; i += kPrepareThreads)
            reinterpret_cast<uint4*>(row_scales)[i] = reinterpret_cast<const uint4*>(p.xs + static_cast<size_t>(t) * blocks16)[i];
    }
    __syncthreads();
    if (tid < k && my_slot[tid] < p.m_max)
        p.amap[static_cast<size_t>(my_e[tid]) * p.m_max + my_slot[tid]] = t * k + tid;
    for (int j = 0; j < k; ++j) {
        const int e = my_e[j] - p.lo, slot = my_slot[j];
        if (e < 0 || e >= p.e_local || slot >= p.m_max) continue;
        const size_t dst = static_cast<size_t>(e) * p.m_max + slot;
        for (int i = tid; i < p.hidden / 32; i += kPrepareThreads)
            reinterpret_cast<uint4*>(p.slot_codes + dst * (p.hidden / 2))[i] = reinterpret_cast<const uint4*>(row_codes)[i];
        for (int i = tid; i < blocks16 / 16; i += kPrepareThreads)
            reinterpret_cast<uint4*>(p.slot_scales + dst * blocks16)[i] = reinterpret_cast<const uint4*>(row_scales)[i];
    }
}

// One token per CTA of one warp; lane l holds experts l, l + 32, ... (at most 256 experts).
__global__ void __launch_bounds__(32) route_packed_kernel(const __grid_constant__ RouteDev p) {
    constexpr int kPerLane = 8;
    const int row = static_cast<int>(blockIdx.x), lane = static_cast<int>(threadIdx.x);
    pdl_wait();
    float prob[kPerLane];
    bool taken[kPerLane];
    float top = -INFINITY;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        const int e = lane + 32 * i;
        prob[i] = e < p.e ? __bfloat162float(p.logits[static_cast<size_t>(row) * p.e + e]) : -INFINITY;
        taken[i] = false;
        top = fmaxf(top, prob[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffff, top, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        prob[i] = lane + 32 * i < p.e ? expf(prob[i] - top) : 0.f;
        sum += prob[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffff, sum, o);
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) prob[i] = prob[i] / sum;
    float kept = 0.f;
    for (int pick = 0; pick < p.top_k; ++pick) {
        float best = -1.f;
        int where = 1 << 30;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const int e = lane + 32 * i;
            const float v = (e < p.e && !taken[i]) ? prob[i] : -1.f;
            if (v > best || (v == best && e < where)) best = v, where = e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffff, best, o);
            const int ow = __shfl_xor_sync(0xffffffff, where, o);
            if (ob > best || (ob == best && ow < where)) best = ob, where = ow;
        }
        kept += best;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i)
            if (lane + 32 * i == where) taken[i] = true;
    }
    // Ascending expert order: list position = number of taken experts below.
    int before = 0;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        const unsigned mask = __ballot_sync(0xffffffff, taken[i]);
        if (taken[i]) {
            const int e = lane + 32 * i;
            const int rank = before + __popc(mask & ((1u << lane) - 1));
            const float w = prob[i] / kept * __bfloat162float(p.scale[e]);
            const uint32_t bits = __bfloat16_as_ushort(__float2bfloat16_rn(w));
            p.packed[row * p.top_k + rank] = (e << 16) | static_cast<int>(bits);
        }
        before += __popc(mask);
    }
    pdl_launch_dependents();
}

static int launch_small(const void* kernel, dim3 grid, dim3 block, void** args, const LaunchOpts& o) {
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = block;
    config.stream = o.stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attr;
    config.numAttrs = o.pdl ? 1 : 0;
    const cudaError_t err = cudaLaunchKernelExC(&config, kernel, args);
    if (err != cudaSuccess) {
        g_last_cuda_error = static_cast<int>(err);
        (void)cudaGetLastError();
        return -6;
    }
    ++g_launches;
    return 0;
}

int launch_moe_prepare(const PrepareDev& p, const LaunchOpts& o) {
    void* args[] = {const_cast<PrepareDev*>(&p)};
    return launch_small(reinterpret_cast<const void*>(moe_prepare_kernel), dim3(p.rows), dim3(kPrepareThreads), args, o);
}

int launch_route_packed(const RouteDev& p, const LaunchOpts& o) {
    void* args[] = {const_cast<RouteDev*>(&p)};
    return launch_small(reinterpret_cast<const void*>(route_packed_kernel), dim3(p.rows), dim3(32), args, o);
}

}  // namespace dlm
