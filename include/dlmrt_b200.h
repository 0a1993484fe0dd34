/* dlmrt_b200 -- C ABI of the B200-native tensor-parallel row-parallel hot path.
 *
 * One shared library (libdlmrt_b200.so, sm_100a only) replaces, for this path, what the reference engine binds
 * through two interfaces:
 *   - the pybind module of dlmrt/ops/csrc/tp_comm.cu:315-319 (`reduce`, `reduce_norm`, `reduce_norm_residual`,
 *     17 positional arguments each, tp_comm.cu:278-280), called from dlmrt/distributed/parallel.py:119-132;
 *   - the row-parallel GEMM that feeds it: `torch.mm(x, W.t(), out=partial)` in dlmrt/layers/linear.py:47-48
 *     (cuBLAS on SM >= 10) and FlashInfer's `trtllm_fp4_block_scale_routed_moe` behind
 *     dlmrt/quantization/nvfp4.py:280-306 for the NVFP4 expert down-projection.
 *
 * Conventions
 *   - plain C types only: device addresses are `void*` / `const void*`, sizes are integers, the stream is the
 *     CUstream / cudaStream_t handle passed as `void*` (NULL = the legacy default stream);
 *   - every entry point returns 0 (DLM_OK) or a negative DLM_ERR_* code and never throws; dlm_strerror() names it,
 *     dlm_last_cuda_error() gives the cudaError_t behind DLM_ERR_CUDA;
 *   - nothing is allocated after dlm_* returns and no host state is kept that a CUDA-graph replay would bypass:
 *     epochs, tile counters and the status words live in device memory owned by the caller (tp_comm.cu:178,211 keeps
 *     its epochs the same way);
 *   - device-side waits are bounded (timeout_ns, measured with %globaltimer). A wait that runs out records a code in
 *     the caller's status words, stops waiting, finishes its bookkeeping and returns normally; it never traps
 *     (the reference prints and traps after ~30 s, tp_comm.cu:67-70).
 *
 * All BF16 matrices are row-major with the hidden / K dimension contiguous, as in the reference.
 */
#ifndef DLMRT_B200_H
#define DLMRT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DLM_API __attribute__((visibility("default")))
#else
#define DLM_API
#endif

#define DLM_MAX_WORLD 8      /* tp_comm.cu:52 kMaxWorld */
#define DLM_EPOCH_SLOTS 256  /* int32 invocation counters per receive buffer; every kernel keeps all of them equal */
#define DLM_STAMP_SLOTS 8
#define DLM_STATUS_WORDS 4   /* int32: [0] first error code, [1] block << 8 | slot, [2] phase, [3] epoch */
#define DLM_MAX_N 8192       /* tp_comm.cu:282: hidden size a multiple of 256, at most 8192 */
#define DLM_FUSED_MAX_N 3072 /* the fused GEMM+reduce kernels run 384 threads: hidden / 8 <= 384 */
#define DLM_NOALLOC_SCRATCH_BYTES (8u << 20) /* built-in scratch of dlm_gemm_bf16_noalloc, held by every GPU in use */
#define DLM_MAX_M 256        /* rows of one block forward (32, 64 or 256 in the reference's rounds) */

enum {
    DLM_OK = 0,
    DLM_ERR_SHAPE = -1,     /* a size the kernels do not take (see each entry point) */
    DLM_ERR_ALIGN = -2,     /* an address or leading dimension that is not 16-byte aligned */
    DLM_ERR_WORLD = -3,     /* world outside 1..8, rank outside 0..world-1, rows % world != 0 */
    DLM_ERR_NULL = -4,      /* a required pointer is NULL */
    DLM_ERR_GRID = -5,      /* the grid cannot be co-resident on this GPU (ranks wait on each other) */
    DLM_ERR_CUDA = -6,      /* a CUDA call failed: see dlm_last_cuda_error() */
    DLM_ERR_WORKSPACE = -7, /* workspace smaller than dlm_workspace_bytes() */
    DLM_ERR_TIMEOUT = -8,   /* device status: a bounded wait ran out (data from a rank never arrived) */
    DLM_ERR_ARCH = -9,      /* not an sm_100 device */
    DLM_ERR_SCRATCH = -10,  /* dlm_gemm_bf16_noalloc: the requested K splits do not fit the built-in scratch */
    DLM_ERR_OVERLAP = -11   /* dlm_rowpar_bf16: the GEMM's input overlaps `rearm` or `out` of the same call */
};

/* What follows the rank-ordered sum (tp_comm.cu:138 template <NORM, RESIDUAL>). */
enum {
    DLM_REDUCE = 0,               /* K1  tp_comm.cu:318  out = sum                                            */
    DLM_REDUCE_NORM = 1,          /* K2  tp_comm.cu:317  out = rmsnorm(bf16(sum)) * weight * scale             */
    DLM_REDUCE_NORM_RESIDUAL = 2  /* K3  tp_comm.cu:316  h[own rows] = bf16(bf16(sum) + h); out = rmsnorm(..)  */
};

/* The reduction half of a call: where partial rows are pushed, where the result lands, what is re-armed.
 * Replaces arguments 2-17 of the reference's launch<> (tp_comm.cu:278-280); the address tables the reference
 * passes as int64 device tensors (`recv`, `out_peers`, parallel.py:95-112) are passed by value here and travel in
 * kernel parameter space. */
typedef struct DlmComm {
    int32_t rank, world;
    int32_t rows, n;               /* the partial is [rows, n] BF16; rows % world == 0; n % 256 == 0, n <= 8192 */
    int32_t mode;                  /* DLM_REDUCE* */
    float eps, scale;              /* RMSNorm epsilon and output scale (modes 1, 2) */
    void* recv[DLM_MAX_WORLD];     /* every rank's receive buffer [3][world][rows/world][n] BF16, armed (0xFFFF) */
    void* out;                     /* this rank's copy of the call site's output [rows, n] BF16, armed */
    void* out_mc;                  /* NVLS multicast address of `out`, or NULL: then one store per rank */
    void* out_peers[DLM_MAX_WORLD];/* every rank's copy of `out` (used when out_mc is NULL) */
    void* rearm;                   /* previous output on this chain (local) to re-arm, or NULL */
    int64_t rearm_bytes;           /* its size; a multiple of 16 */
    int32_t* epochs;               /* [DLM_EPOCH_SLOTS] int32, zero-initialised, one array per receive buffer */
    void* h;                       /* [rows, n] BF16 residual stream (mode 2): own rows read and rewritten */
    const void* weight;            /* [n] BF16 RMSNorm weight (modes 1, 2) */
    int32_t* status;               /* [DLM_STATUS_WORDS] int32 device words, zero-initialised, or NULL. A failure is
                                      sticky: while status[0] != 0 every call on these words pushes nothing, accepts
                                      nothing and broadcasts nothing (slots may hold an older invocation's vectors), so
                                      its peers' waits run out too. After DLM_ERR_TIMEOUT the receive slots, outputs and
                                      epochs of the group must be re-created before it is used again. */
    int64_t* stamps;               /* [grid, DLM_STAMP_SLOTS] int64 %globaltimer phase stamps per CTA, or NULL
                                      (tp_comm.cu:121): 0 start, 1 pushed, 2 owned rows broadcast, 3 collected; fused
                                      kernels also 4 accumulator ready, 5 dependency wait returned, 6 tile summed+pushed,
                                      7 kernel entry */
    int64_t timeout_ns;            /* budget of every device wait; 0 = 30 s (the reference's budget, tp_comm.cu:67-70) */
    int32_t pdl;                   /* launch as a programmatic dependent launch (tp_comm.cu:304-309) */
    int32_t max_ctas;              /* cap on the grid, 0 = one CTA per SM. Calls that may run concurrently (different
                                      chains on different streams) must together fit on the GPU. */
    int32_t one_shot;              /* 1: every rank stores its whole partial into every rank's slots and sums all rows
                                      itself, in rank order, into its own `out`: one NVLink hop, no broadcast; meant
                                      for small partials (32-row blocks). `recv` buffers are then [3][world][rows][n].
                                      Same bits as the two-hop protocol. In mode DLM_REDUCE_NORM_RESIDUAL the residual
                                      stream is then REPLICATED: every rank holds all rows of `h` and updates all of
                                      them, which is how LLaDA2 keeps it (`rmsnorm(h, w, delta=reduced)`,
                                      dlmrt/ops/triton/core.py:29-56, dlmrt/models/llada2/model.py:435-439); with
                                      one_shot 0 only the owner's rows of `h` are read and written. With world == 1
                                      the two are the same thing. */
    int32_t reserved;
    void* recv_mc;                 /* one_shot: NVLS multicast address of the receive buffer, or NULL (one store per rank) */
} DlmComm;

/* The GEMM half of a fused call: out[M, N] = x[M, K] * W[N, K]^T, this rank's K shard (linear.py:41-51). */
typedef struct DlmGemm {
    const void* x;   /* [m, k] BF16, leading dimension ldx elements */
    const void* w;   /* [n, k] BF16, leading dimension ldw elements */
    int32_t m, n, k; /* m % 16 == 0, 16 <= m <= 256; n % 128 == 0; k % 8 == 0, k >= 64 (a last k-block shorter than 64 is
                        zero-filled; pre-tiled weights are padded to whole tiles) */
    int64_t ldx, ldw;/* multiples of 8 */
    void* workspace; /* dlm_workspace_bytes(m, n, k) bytes, zero-initialised once, 256-byte aligned; one per chain
                        (split-K partial tiles, arrival counters and a launch generation live in it) */
    int64_t workspace_bytes;
    int32_t splits;  /* K splits across CTAs, 0 = chosen by the library; FP32 partial tiles are summed in split
                        order, so the result does not depend on scheduling */
    int32_t token_tiles; /* tiles along m (each m / token_tiles tokens, a multiple of 16), 0 = chosen by the library */
    int32_t w_tiled; /* 0: w is row-major [n, k] (ldw). 1: w is pre-tiled for streaming, [n / 128][ceil(k / 64)] tiles of
                        128 rows x 64 BF16 (16 KB, contiguous, K zero-padded), the 16-byte chunk c of tile row r stored at chunk
                        position c ^ (r % 8) (the 128-byte shared-memory swizzle); ldw is ignored. Weights are static,
                        so the layout is made once when they are loaded, as the reference re-lays its FP8 and NVFP4
                        weights (linear.py:30-31, nvfp4.py:104-112). */
    int32_t reserved;    /* must be 0 */
} DlmGemm;

/* The NVFP4 expert half of a fused call: GEMM2 (down-projection) of this rank's routed experts and the weighted top-k
 * combine. Formats follow the reference: E2M1 codes two per byte with the even element in the low nibble, one FP8
 * E4M3 scale per 16 input elements, FP32 per-expert output scale g2 = input scale x weight scale
 * (dlmrt/quantization/nvfp4.py:1-12,117-121); expert-major activation slots and slot map as in
 * dlmrt/ops/triton/nvfp4_moe.py:11-12,107-150. Weight scales are NOT linear: they are pre-arranged once, when the
 * experts are loaded, into 128-row x 4-scale atoms ([e_local][n / 128][f / 64][512] bytes, byte (r % 32) * 16 +
 * (r / 32) * 4 + j = scale j of row r), as the reference pre-arranges them for its own B200 back-end
 * (nvfp4.py:108-112). */
typedef struct DlmMoe {
    const void* act_codes;   /* [e_local * m_max, f / 2] uint8: GEMM2 input rows, slot e * m_max + j */
    const void* act_scales;  /* [e_local * m_max, f / 16] E4M3, linear */
    const int32_t* amap;     /* [e_total, m_max] int32: token * top_k + k of the j-th row routed to expert e */
    const int32_t* counts;   /* [e_total] int32 rows per expert */
    const void* w_codes;     /* [e_local, n, f / 2] uint8 */
    const void* w_scales;    /* [e_local, n / 128, f / 64, 512] E4M3 atoms */
    const float* g2;         /* [e_local] */
    const int32_t* ids;      /* [m, top_k] int32 global expert ids, in the order the combine sums them */
    const float* weights;    /* [m, top_k] FP32 routing weights (BF16-representable in the reference) */
    const void* shared;      /* [m, n] BF16 added after the combine (shared expert), or NULL */
    int32_t m, n, f, top_k;  /* m <= 256; n % 128 == 0, n <= 3072; f % 64 == 0; top_k <= 16 */
    int32_t m_max;           /* rows reserved per expert (<= 256) */
    int32_t lo, e_local, e_total; /* this rank's experts are [lo, lo + e_local), e_local <= 256 */
    void* workspace;         /* dlm_moe_workspace_bytes(m, n, top_k) bytes, zero-initialised once, 256-byte aligned */
    int64_t workspace_bytes;
    int32_t w_tiled;         /* 0: w_codes is [e_local, n, f / 2] as exported. 1: pre-tiled for streaming,
                                [e_local][n / 128][ceil(f / 256)] tiles of 128 rows x 128 bytes (16 KB, contiguous, zero-padded
                                along f), the 16-byte chunk c of tile row r stored at chunk position c ^ (r % 8) (the
                                128-byte shared-memory swizzle): one bulk copy brings a tile in */
    int32_t reserved;
} DlmMoe;

/* What runs in front of the expert down-projection inside the reference's one FlashInfer call
 * (dlmrt/quantization/nvfp4.py:280-306; arithmetic as stated in dlmrt/ops/triton/nvfp4_moe.py:36-104): the packed top-k
 * is unpacked and every expert's rows are numbered in token order, the input rows are quantised to NVFP4 against the
 * GEMM1 input scale (or taken pre-quantised, dlmrt/models/diffusion_gemma/experts.py:64-67) and copied into
 * expert-major slots, and GEMM1 (gate and up, FP4 tensor cores) + SwiGLU / GeGLU in FP32 + NVFP4 re-quantisation against
 * 1 / a2 writes GEMM2's input straight into the slots DlmMoe.act_codes / act_scales name. Everything the
 * down-projection needs (ids, weights, counts, amap, activation slots) is produced here on the device.
 * Weight layout, made once when the experts are loaded: W13 rows interleaved, row 2i = gate feature i, row 2i + 1 = up
 * feature i ([e_local, 2F, hidden / 2] codes), block scales of those rows in the same 128-row x 4-scale atoms as
 * DlmMoe.w_scales ([e_local, 2F / 128, hidden / 64, 512]). */
typedef struct DlmMoeFront {
    const void* x;            /* [m, hidden] BF16 expert input, or NULL: then xq / xs hold it already quantised */
    const void* xq;           /* [m, hidden / 2] uint8 codes (x NULL) */
    const void* xs;           /* [m, hidden / 16] E4M3 scales, linear (x NULL) */
    const float* a1_inv;      /* device scalar: 1 / (GEMM1 input scale), the global scale of the input's rounding */
    const int32_t* packed;    /* [m, top_k] expert << 16 | BF16 routing-weight bits, ascending experts per token */
    const void* w13_codes;    /* [e_local, 2F, hidden / 2] uint8, rows interleaved gate / up; or, with w13_tiled, the same
                                 pre-tiled like DlmMoe.w_codes: [e_local][2F / 128][ceil(hidden / 256)][16 KB] */
    const void* w13_scales;   /* [e_local, 2F / 128, hidden / 64, 512] E4M3 atoms */
    const float* g1;          /* [e_local] GEMM1 alpha = input scale x weight scale */
    const float* a2_inv;      /* [e_local] 1 / (GEMM2 input scale) */
    int32_t* ids;             /* out [m, top_k] */
    float* weights;           /* out [m, top_k] */
    int32_t* counts;          /* out [e_total] */
    int32_t* amap;            /* out [e_total, m_max] */
    void* slot_codes;         /* scratch [e_local * m_max, hidden / 2]: the quantised input rows, expert-major */
    void* slot_scales;        /* scratch [e_local * m_max, hidden / 16] */
    void* act_codes;          /* out [e_local * m_max, f / 2]: GEMM2's input */
    void* act_scales;         /* out [e_local * m_max, f / 16] */
    int32_t m, hidden, f, top_k; /* m <= 256; hidden % 256 == 0, <= 8192; f % 64 == 0; top_k <= 16 */
    int32_t m_max;            /* rows reserved per expert (<= 256); rows beyond it are dropped */
    int32_t lo, e_local, e_total;
    int32_t activation;       /* 0 SwiGLU (g * sigmoid(g) * u), 1 GeGLU (tanh GELU) */
    int32_t w13_tiled;        /* see w13_codes */
} DlmMoeFront;

/* Device status read back by dlm_status_read(). */
typedef struct DlmStatus {
    int32_t code;   /* DLM_OK or DLM_ERR_TIMEOUT */
    int32_t block;  /* CTA that gave up */
    int32_t slot;   /* rank slot it was waiting for */
    int32_t phase;  /* 1 = receive slots (reduce-scatter), 2 = own OUT copy (all-gather), 3 = GEMM pipeline */
    int32_t epoch;
} DlmStatus;

typedef void* dlm_stream_t;

/* Stand-alone fused reduction of a given BF16 partial [rows, n] (local memory): push reduce-scatter, rank-ordered
 * FP32 sum (+ residual + RMSNorm), multicast all-gather, in-band arrival detection. Bit-exact with
 * reduce_kernel<NORM, RESIDUAL> (tp_comm.cu:138-275), whose three pybind entry points it replaces. */
DLM_API int dlm_reduce_bf16(const void* partial, const DlmComm* comm, dlm_stream_t stream);

/* One launch that runs `nranks` ranks of the same reduction on ONE GPU (rank i = partial[i], comm[i]; every
 * comm[i].recv / out_peers names buffers on this GPU; out_mc must be NULL). For testing the multi-rank protocol
 * without several GPUs: kernels that wait on one another must not run as separate launches on one GPU.
 * No counterpart in the reference. */
DLM_API int dlm_reduce_bf16_loopback(const void* const* partial, const DlmComm* comm, int nranks, dlm_stream_t stream);

/* Plain row-parallel-shaped GEMM without communication: out[m, n] BF16 (ldo elements) = x * W^T.
 * Replaces Linear.__call__ on one GPU (linear.py:47-48, torch.mm on cuBLAS). */
DLM_API int dlm_gemm_bf16(const DlmGemm* gemm, void* out, int64_t ldo, int pdl, dlm_stream_t stream);

/* dlm_gemm_bf16 for callers that cannot allocate device memory. No counterpart in the reference.
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- inside a CUDA-graph capture of someone else's
 * stream, in a plugin whose host forbids allocations after start-up, or in a process whose memory pool is owned by
 * another runtime -- cannot provide the workspace dlm_gemm_bf16 asks for. Here the split-K scratch (FP32 partial
 * tiles, arrival counters) is a fixed array of DLM_NOALLOC_SCRATCH_BYTES (8 MiB) inside the library, which every GPU
 * that uses the library keeps until the process ends. The caller passes only inputs and the output; the call issues
 * no cudaMalloc / cudaFree and no allocating library routine.
 *
 * Limits and rules:
 *   - m, n, k, ld* as for dlm_gemm_bf16. `splits` > 1 needs 2 KiB + splits * m * n * 4 bytes of scratch; an explicit
 *     request beyond 8 MiB returns DLM_ERR_SCRATCH. With splits = 0 the library picks a tiling and lowers the number
 *     of splits until it fits (a single split needs no partial tiles), so every legal shape runs, if slower;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress with that device
 *     current); make that first call before any stream capture starts. The address is remembered per device for the
 *     life of the process and does not survive cudaDeviceReset or a re-created primary context;
 *   - `splits` larger than the number of 64-wide k-blocks runs as that number, and only that number has to fit;
 *   - all calls on a GPU share the one array. Each call clears the small header it depends on (stream-ordered
 *     memset) and rewrites the partial tiles before reading them, so calls that follow each other on one stream are
 *     safe; calls that overlap on the GPU (different streams, different host threads) race on it and give wrong
 *     results. */
DLM_API int dlm_gemm_bf16_noalloc(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx,
                                  int64_t ldw, int64_t ldo, int splits, int token_tiles, int pdl, dlm_stream_t stream);

/* Fused row-parallel projection + reduction: the GEMM above whose finished BF16 tiles are pushed straight into the
 * owner ranks' receive slots, followed in the same kernel by the reduction of dlm_reduce_bf16.
 * Replaces the pair Linear.__call__(x, out=partial) -> Group.reduce / reduce_norm
 * (dlmrt/models/sdar/model.py:237-243, llada2/model.py:435-439, diffusion_gemma/model.py:272-292).
 * gemm->m == comm->rows, gemm->n == comm->n <= DLM_FUSED_MAX_N.
 * gemm->x must not overlap comm->rearm or comm->out (DLM_ERR_OVERLAP): CTAs re-arm and fill those while others still
 * load x. A caller whose input IS the previous output of the chain runs dlm_gemm_bf16 + dlm_reduce_bf16 instead. */
DLM_API int dlm_rowpar_bf16(const DlmGemm* gemm, const DlmComm* comm, dlm_stream_t stream);

/* NVFP4 routed experts on one GPU: out[m, n] BF16 (ldo elements) = combine(GEMM2). Replaces the GEMM2 + finalize
 * half of nvfp4.trtllm_moe (dlmrt/quantization/nvfp4.py:280-306) and the `torch.add(routed, shared)` that follows it
 * (dlmrt/models/llada2/model.py:360-362). */
DLM_API int dlm_moe_nvfp4(const DlmMoe* moe, void* out, int64_t ldo, int pdl, dlm_stream_t stream);

/* The same fused with the reduction over ranks (experts are split whole across ranks): replaces
 * trtllm_moe -> [add shared] -> Group.reduce (llada2/model.py:354-362,437-438; diffusion_gemma/model.py:281-292).
 * moe->m == comm->rows, moe->n == comm->n. */
DLM_API int dlm_rowpar_nvfp4_moe(const DlmMoe* moe, const DlmComm* comm, dlm_stream_t stream);
DLM_API int dlm_rowpar_nvfp4_moe_loopback(const DlmMoe* moe, const DlmComm* comm, int nranks, dlm_stream_t stream);
DLM_API size_t dlm_moe_workspace_bytes(int m, int n, int top_k);

/* Two launches: the per-token bookkeeping + quantisation, then GEMM1 + activation + re-quantisation (see DlmMoeFront).
 * With dlm_moe_nvfp4 / dlm_rowpar_nvfp4_moe behind it this replaces the whole of nvfp4.trtllm_moe
 * (dlmrt/quantization/nvfp4.py:280-306). */
DLM_API int dlm_moe_front_nvfp4(const DlmMoeFront* front, int pdl, dlm_stream_t stream);

/* The router's top-k as the reference packs it for this path (dlmrt/ops/triton/moe.py:70-73 `route_packed`): FP32
 * softmax of `logits` [rows, e] BF16, the top_k largest (ties to the lower expert), renormalised, times `scale` [e]
 * BF16, in ascending expert order, packed[rows, top_k] = expert << 16 | BF16 weight bits. e <= 256, top_k <= 16. */
DLM_API int dlm_route_packed(const void* logits, const void* scale, int32_t* packed, int rows, int e, int top_k, int pdl,
                             dlm_stream_t stream);
DLM_API int dlm_abi_check_front(size_t sizeof_front);

/* Single-GPU loopback of `nranks` ranks of dlm_rowpar_bf16 in one launch (see dlm_reduce_bf16_loopback). */
DLM_API int dlm_rowpar_bf16_loopback(const DlmGemm* gemm, const DlmComm* comm, int nranks, dlm_stream_t stream);

/* ---- all-gather of a small block (row statistics) ---------------------------------------------------------------
 * Replaces Group.all_gather (dlmrt/distributed/parallel.py:164-180; callers ops/triton/decoding.py:126,
 * models/diffusion_gemma/kernels.py:436,590), the one other collective of a round: every rank's `x` (`bytes` bytes, a
 * multiple of 16, at most DLM_GATHER_MAX_BYTES) ends up in every rank's `comm->out` [world][bytes], in rank order,
 * without a barrier: one multimem.st (or one store per rank) per 16 bytes into triple-buffered slots, arrival detected
 * in band. Of `comm` only rank, world, recv (every rank's [3][world][bytes] buffer, armed with all-ones), recv_mc,
 * out, epochs, status, timeout_ns, pdl and max_ctas are read. The payload must not contain an all-ones 32-bit word
 * (FP32 / FP16 / BF16 values never do). */
#define DLM_GATHER_MAX_BYTES (1 << 20)
DLM_API int dlm_all_gather(const void* x, int64_t bytes, const DlmComm* comm, dlm_stream_t stream);
/* All ranks in one cooperative launch on one GPU (tests), as the other *_loopback entry points. */
DLM_API int dlm_all_gather_loopback(const void* const* x, int64_t bytes, const DlmComm* comm, int nranks,
                                    dlm_stream_t stream);

/* Bytes of workspace (FP32 split-K partial tiles + tile counters) a GEMM of this shape needs. */
DLM_API size_t dlm_workspace_bytes(int m, int n, int k);

/* The (token tiles, K splits) the library would pick for this shape with `max_ctas` CTAs available (0 = all SMs). */
DLM_API int dlm_choose_tiling(int m, int n, int k, int max_ctas, int* token_tiles, int* splits);

/* Copies the device status words to the host (synchronises `stream`) and clears them on the device. */
DLM_API int dlm_status_read(int32_t* device_status, DlmStatus* out, dlm_stream_t stream);

/* Returns DLM_OK when the caller's struct sizes (a binding in another language) match the library's. */
DLM_API int dlm_abi_check(size_t sizeof_comm, size_t sizeof_gemm, size_t sizeof_status);
DLM_API int dlm_abi_check_moe(size_t sizeof_moe);

DLM_API const char* dlm_strerror(int code);
DLM_API int dlm_last_cuda_error(void);
/* Number of SMs of the current device, and 100 when it is an sm_100 part (0 otherwise). */
DLM_API int dlm_device_sms(void);
DLM_API int dlm_device_arch(void);
/* Number of kernel launches this library has issued in this process (for the benchmark's gpu_launches). */
DLM_API int64_t dlm_launch_count(void);

/* ---- device-side loop around captured graphs ------------------------------------------------------------------
 * Replaces the reference's block-graph module (dlmrt/ops/csrc/block_graph.cu: BlockGraph :29-77, LoopGraph :80-129,
 * StagedLoopGraph :137-207, built by Engine._capture, dlmrt/models/sdar/engine.py:92-120): the captured stages of a
 * block (begin, round, commit) are tied into ONE graph whose rounds are decided on the device,
 *
 *     head -> WHILE(*remaining > 0 && *step < limit){ part_0 -> part_1 -> ... } -> ... next loop ... -> tail
 *
 * A part with a non-NULL `flag` runs only in passes where *flag > 0 (an IF evaluated when the part is reached). The
 * WHILE condition is evaluated before the first pass and after every pass, and one execution makes at most `limit`
 * passes of a loop even if its body fails to advance *step (the GPU is never left spinning). Graph
 * handles are cudaGraph_t values (torch: CUDAGraph(keep_graph=True).raw_cuda_graph()); they are cloned, so the
 * caller may destroy them afterwards. `head` and `tail` may be NULL. The fused kernels of this library are loop-safe:
 * all their state lives in device memory and advances with every execution, captured or not. */
#define DLM_MAX_LOOPS 8
#define DLM_MAX_LOOP_PARTS 16

typedef struct DlmLoopPart {
    void* graph;     /* cudaGraph_t of the part */
    const int* flag; /* device int32; NULL = the part always runs */
} DlmLoopPart;

typedef struct DlmLoop {
    const DlmLoopPart* parts;
    int32_t n_parts;
    int32_t limit;        /* upper bound on *step for the body to run */
    const int* remaining; /* device int32, written by the body (work left) */
    const int* step;      /* device int32, advanced by the body */
} DlmLoop;

typedef struct DlmDeviceLoop DlmDeviceLoop;

DLM_API int dlm_device_loop_create(void* head, const DlmLoop* loops, int n_loops, void* tail, DlmDeviceLoop** out);
/* One launch runs the whole program on `stream` (cudaStream_t). */
DLM_API int dlm_device_loop_launch(DlmDeviceLoop* loop, void* stream);
DLM_API void dlm_device_loop_destroy(DlmDeviceLoop* loop);

#ifdef __cplusplus
}
#endif
#endif /* DLMRT_B200_H */
