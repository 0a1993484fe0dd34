// Kernel parameter blocks and host launchers shared between the .cu files of the library.
#pragma once

#include <cuda.h>

#include "comm.cuh"

namespace dlm {

constexpr int kFusedThreads = 384;  // 12 warps: TMA producer, MMA issuer, TMEM allocator, spare, 8 epilogue warps
constexpr int kBlockF = 128;        // weight rows (output features) per tile: the MMA's M
constexpr int kBlockK = 64;         // BF16 per k-block: one 128-byte swizzled row
constexpr int kUmmaK = 16;          // K of one tcgen05.mma kind::f16
constexpr int kMaxSplits = 8;
constexpr int kMaxTiles = 128;      // (feature tiles) x (token tiles) of one GEMM
constexpr int kWorkspaceHeader = 2048;  // int32 gen[256] then int32 counters[2][128]
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 200 * 1024;
constexpr long long kDefaultTimeoutNs = 30000000000ll;  // budget of a device wait when the caller passes 0 (tp_comm.cu:67-70: ~30 s)

// The GEMM half of one rank. `out` is used by the plain GEMM (no communication) only.
struct alignas(64) GemmDev {
    CUtensorMap tm_w;  // W [n, k] BF16, box 64 x 128, 128-byte swizzle
    CUtensorMap tm_x;  // x [m, k] BF16, box 64 x (m / token_tiles), 128-byte swizzle
    const uint8_t* w_tiles;  // or: W pre-tiled [n / 128][k / 64][16 KB], each tile already in the swizzled smem layout
    float* ws;         // FP32 partial tiles [tile][split][tokens per tile][128]
    int* gen;          // [256] launch generation of this workspace, every entry kept equal (like the epochs)
    int* counters;     // [2][kMaxTiles] split-K arrivals per tile, banked by generation parity
    __nv_bfloat16* out;
    long long ldo;
    int m, n, k, splits, token_tiles, stages;
};

template <int NR>
struct ReduceParams {
    CommDev c[NR];
    const __nv_bfloat16* partial[NR];
};

template <int NR>
struct alignas(64) RowparParams {
    GemmDev g[NR];
    CommDev c[NR];
    int fused;  // 0: plain GEMM into g.out; 1: push + reduce
};

// The NVFP4 expert down-projection of one rank (GEMM2 of the routed experts + the weighted combine).
struct alignas(64) MoeDev {
    CUtensorMap tm_w;         // W2 codes as bytes [e_local * n, f / 2], box 128 B x 128 rows, 128-byte swizzle
    const uint8_t* w_tiles;   // or: the codes pre-tiled [e_local][n / 128][ceil(f / 256)][16 KB], each tile 128 rows x 128
                              // bytes already in the swizzled shared-memory order (zero-padded along f)
    CUtensorMap tm_a;         // activation codes [e_local * m_max, f / 2], box 128 B x 8 rows, 128-byte swizzle
    const uint8_t* a_scales;  // [e_local * m_max, f / 16] E4M3, linear
    const uint8_t* w_scales;  // [e_local][n / 128][f / 64][512] E4M3 in 128 x 4 atoms
    const int* amap;          // [e_total, m_max] pair index (token * top_k + k) of each expert's slots
    const int* counts;        // [e_total]
    const float* g2;          // [e_local]
    const int* ids;           // [m, top_k] global expert ids
    const float* weights;     // [m, top_k]
    const __nv_bfloat16* shared;  // [m, n] or null
    __nv_bfloat16* y;         // [m * top_k, n] per-(token, expert) outputs (workspace)
    int* gen;                 // workspace header: launch generation [256]
    int* counters;            //                   arrival counters [2][kMaxTiles]
    __nv_bfloat16* out;       // plain (unfused) output [m, n]
    long long ldo;
    int m, n, f, top_k, m_max, lo, e_local, e_total, stages, rows_cap;
    // GEMM1 (gate / up) only: n = 2F interleaved weight rows, f = hidden, g2 = the GEMM1 alpha g1
    const float* a2_inv;      // [e_local] 1 / (GEMM2 input scale): global scale of the activation's NVFP4 rounding
    uint8_t* aq_out;          // [e_local * m_max, f_out / 2] activation codes written into the expert-major slots
    uint8_t* as_out;          // [e_local * m_max, f_out / 16] their E4M3 scales (linear)
    int f_out, act_kind;      // F; 0 = SwiGLU, 1 = GeGLU (tanh GELU)
};

// Routing bookkeeping + input quantisation in front of the experts' GEMM1 (one CTA per token).
struct PrepareDev {
    const __nv_bfloat16* x;    // [rows, hidden] BF16, or null when the input comes quantised
    const uint8_t* xq;         // [rows, hidden / 2] codes and
    const uint8_t* xs;         // [rows, hidden / 16] E4M3 scales of a pre-quantised input (x null)
    const float* a1_inv;       // device scalar: global scale of the input's NVFP4 rounding (x given)
    const int* packed;         // [rows, top_k] expert << 16 | BF16 weight bits
    int* ids;                  // out [rows, top_k]
    float* weights;            // out [rows, top_k]
    int* counts;               // out [e_total]
    int* amap;                 // out [e_total, m_max]
    uint8_t* slot_codes;       // out [e_local * m_max, hidden / 2]
    uint8_t* slot_scales;      // out [e_local * m_max, hidden / 16]
    int rows, hidden, top_k, e_total, lo, e_local, m_max;
};

// Softmax top-k routing of one token per CTA (dlmrt/ops/triton/moe.py:14-47, PACK variant).
struct RouteDev {
    const __nv_bfloat16* logits;  // [rows, e] BF16
    const __nv_bfloat16* scale;   // [e] per-expert scale
    int* packed;                  // out [rows, top_k]
    int rows, e, top_k;
};

template <int NR>
struct alignas(64) MoeParams {
    MoeDev g[NR];
    CommDev c[NR];
    int fused;
};

struct LaunchOpts {
    cudaStream_t stream;
    bool pdl;
    bool cooperative;
};

int launch_reduce(const ReduceParams<1>& p, int grid, int threads, const LaunchOpts& o);
int launch_reduce_loopback(const ReduceParams<kMaxWorld>& p, int grid, int nranks, int threads, const LaunchOpts& o);
int launch_gather(const ReduceParams<1>& p, int grid, const LaunchOpts& o);
int launch_gather_loopback(const ReduceParams<kMaxWorld>& p, int grid, int nranks, const LaunchOpts& o);
int launch_rowpar(const RowparParams<1>& p, int grid, const LaunchOpts& o);
int launch_rowpar_loopback(const RowparParams<kMaxWorld>& p, int grid, int nranks, const LaunchOpts& o);
int launch_moe(const MoeParams<1>& p, int grid, const LaunchOpts& o);
int launch_moe_loopback(const MoeParams<kMaxWorld>& p, int grid, int nranks, const LaunchOpts& o);
int launch_moe_gate_up(const MoeParams<1>& p, int grid, const LaunchOpts& o);
int launch_moe_prepare(const PrepareDev& p, const LaunchOpts& o);
int launch_route_packed(const RouteDev& p, const LaunchOpts& o);
int moe_stage_bytes(int rows_cap);
int moe_stages(int rows_cap);
int rowpar_smem_bytes(int m, int stages);
int rowpar_stages(int m);

extern int g_last_cuda_error;
extern long long g_launches;

}  // namespace dlm
