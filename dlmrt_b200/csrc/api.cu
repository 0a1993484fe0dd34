// extern "C" boundary of libdlmrt_b200.so (include/dlmrt_b200.h): argument checks, tensor-map construction, launch.
// Mirrors the host checks of the reference's launch<> (dlmrt/ops/csrc/tp_comm.cu:282-287) as return codes.
#include <cstring>

#include "../../include/dlmrt_b200.h"
#include "kernels.cuh"

using namespace dlm;

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int cuda_fail(cudaError_t err) {
    g_last_cuda_error = static_cast<int>(err);
    (void)cudaGetLastError();
    return DLM_ERR_CUDA;
}

struct DeviceInfo {
    int device = -1, sms = 0, major = 0;
};

int device_info(DeviceInfo* out) {
    static DeviceInfo cache[64];
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return cuda_fail(err);
    if (dev < 0 || dev >= 64) return DLM_ERR_ARCH;
    if (cache[dev].device != dev) {
        cudaDeviceProp prop;
        err = cudaGetDeviceProperties(&prop, dev);
        if (err != cudaSuccess) return cuda_fail(err);
        cache[dev].device = dev;
        cache[dev].sms = prop.multiProcessorCount;
        cache[dev].major = prop.major;
    }
    *out = cache[dev];
    return out->major == 10 ? DLM_OK : DLM_ERR_ARCH;
}

int check_comm(const DlmComm* c) {
    if (c == nullptr) return DLM_ERR_NULL;
    if (c->world < 1 || c->world > DLM_MAX_WORLD || c->rank < 0 || c->rank >= c->world) return DLM_ERR_WORLD;
    if (c->rows <= 0 || c->rows % c->world) return DLM_ERR_WORLD;
    if (c->n <= 0 || c->n % 256 || c->n > DLM_MAX_N) return DLM_ERR_SHAPE;
    if (c->mode < DLM_REDUCE || c->mode > DLM_REDUCE_NORM_RESIDUAL) return DLM_ERR_SHAPE;
    if (c->out == nullptr || c->epochs == nullptr) return DLM_ERR_NULL;
    for (int s = 0; s < c->world; ++s) {
        if (c->recv[s] == nullptr) return DLM_ERR_NULL;
        if (!aligned16(c->recv[s])) return DLM_ERR_ALIGN;
        if (c->out_mc == nullptr) {
            if (c->out_peers[s] == nullptr) return DLM_ERR_NULL;
            if (!aligned16(c->out_peers[s])) return DLM_ERR_ALIGN;
        }
    }
    // One-shot: every rank sums (and, in modes 1 and 2, normalises) all rows itself; with mode 2 the residual stream
    // is then REPLICATED: each rank updates all rows of its own copy of h.
    if (c->one_shot != 0 && c->one_shot != 1) return DLM_ERR_SHAPE;
    if (!aligned16(c->recv_mc)) return DLM_ERR_ALIGN;
    if (c->mode != DLM_REDUCE && c->weight == nullptr) return DLM_ERR_NULL;
    if (c->mode == DLM_REDUCE_NORM_RESIDUAL && c->h == nullptr) return DLM_ERR_NULL;
    if (!aligned16(c->out) || !aligned16(c->out_mc) || !aligned16(c->rearm) || !aligned16(c->h) || !aligned16(c->weight))
        return DLM_ERR_ALIGN;
    if (c->rearm_bytes < 0 || c->rearm_bytes % 16 || (c->rearm == nullptr && c->rearm_bytes != 0)) return DLM_ERR_ALIGN;
    if (c->rearm_bytes / 16 > 0x7FFFFFFF || c->timeout_ns < 0 || c->max_ctas < 0) return DLM_ERR_SHAPE;
    return DLM_OK;
}

void fill_comm(CommDev* d, const DlmComm* c) {
    std::memset(d, 0, sizeof(*d));
    for (int s = 0; s < c->world; ++s) {
        d->recv[s] = static_cast<__nv_bfloat16*>(c->recv[s]);
        d->out_peers[s] = static_cast<__nv_bfloat16*>(c->out_peers[s]);
    }
    d->out = static_cast<__nv_bfloat16*>(c->out);
    d->out_mc = static_cast<__nv_bfloat16*>(c->out_mc);
    d->rearm = static_cast<__nv_bfloat16*>(c->rearm);
    d->rearm_vecs = static_cast<int>(c->rearm_bytes / 16);
    d->h = static_cast<__nv_bfloat16*>(c->h);
    d->weight = static_cast<const __nv_bfloat16*>(c->weight);
    d->epochs = c->epochs;
    d->status = c->status;
    d->stamps = reinterpret_cast<long long*>(c->stamps);
    d->timeout_ns = c->timeout_ns > 0 ? c->timeout_ns : kDefaultTimeoutNs;
    d->rank = c->rank;
    d->world = c->world;
    d->rows = c->rows;
    d->n = c->n;
    d->R = c->rows / c->world;
    d->one_shot = c->one_shot != 0 && c->world > 1;
    d->slot_rows = d->one_shot ? c->rows : d->R;
    d->recv_mc = d->one_shot ? static_cast<__nv_bfloat16*>(c->recv_mc) : nullptr;
    d->mode = c->mode;
    d->eps = c->eps;
    d->scale = c->scale;
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(p);
        else
            (void)cudaGetLastError();
    }
    return fn;
}

// A [rows, cols] BF16 row-major matrix with leading dimension ld, read in boxes of 64 columns x box_rows rows with
// the 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int rows, int cols, long long ld, int box_rows) {
    EncodeTiled fn = encode_tiled();
    if (fn == nullptr) return DLM_ERR_CUDA;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockK), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = 100000 + static_cast<int>(r);
        return DLM_ERR_CUDA;
    }
    return DLM_OK;
}

// Picks (token tiles, K splits) for a [m, n, k] GEMM on `avail` CTAs with a cost model fitted to measurements on B200
// (256 x 2560 outputs, K from 512 to 9728, every tiling, and phase stamps of the fused kernel at one and two ranks;
// microseconds):
//   4.8                          launch, prologue, first loads, epilogue and push
//   + kb * (0.24 + 0.0009 * mt)  kb k-blocks per CTA; a k-block costs more the more tokens (mt) the tile holds
//   + 2.8 + 0.019 * mt           if K is split: FP32 partial tiles out to L2, the rendezvous, and the tiles read back
//                                (5.2 at 128 tokens, 7.7 at 256). Fused at ONE rank the rows'
//                                owners read the partials themselves, one rendezvous less: 0.3 + 0.0176 * mt
//   + 1.3 + 0.5 * (rows - 1)     owner phase of the reduction, rows = ceil(R / CTAs) per CTA (later rows overlap)
// and never less than the weight shard takes to stream from HBM. Long K (TP = 1) ends up split seven ways over 140 SMs,
// short K (TP = 8) tiled along the tokens, in between a mix of both.
void choose_tiling(int m, int n, int k, int avail, int* tiles_out, int* splits_out, int owner_rows = 0,
                   bool single_rank = false) {
    const double hbm_bytes_per_us = 6.0e6;
    const int feature_tiles = n / kBlockF, nkb = (k + kBlockK - 1) / kBlockK;
    double best = 1e30;
    *tiles_out = 1;
    *splits_out = 1;
    for (int t = 1; t <= 8; t *= 2) {
        if (m % (16 * t)) break;
        const int mt = m / t;
        if (feature_tiles * t > avail || feature_tiles * t > kMaxTiles) break;
        for (int sp = 1; sp <= kMaxSplits && sp <= nkb; ++sp) {
            const int ctas = feature_tiles * t * sp;
            if (ctas > avail) break;
            const int kb = (nkb + sp - 1) / sp;
            double us = kb * (0.24 + 0.0009 * mt);
            const double hbm = static_cast<double>(n) * k * 2 / hbm_bytes_per_us;
            if (us < hbm) us = hbm;
            us += 4.8;
            if (sp > 1) {
                if (single_rank && owner_rows > 0) us += 0.3 + 0.0176 * mt;
                else us += 2.8 + 0.019 * mt;
            }
            if (owner_rows > 0) us += 1.3 + 0.5 * ((owner_rows + ctas - 1) / ctas - 1);
            if (us < best - 1e-9) {
                best = us;
                *tiles_out = t;
                *splits_out = sp;
            }
        }
    }
}

int check_gemm(const DlmGemm* g) {
    if (g == nullptr) return DLM_ERR_NULL;
    if (g->x == nullptr || g->w == nullptr || g->workspace == nullptr) return DLM_ERR_NULL;
    if (g->m < 16 || g->m > DLM_MAX_M || g->m % 16) return DLM_ERR_SHAPE;
    if (g->n < kBlockF || g->n % kBlockF || g->k < kBlockK || g->k % 8) return DLM_ERR_SHAPE;
    if (g->n / kBlockF > 64) return DLM_ERR_SHAPE;
    if (g->ldx < g->k || g->ldx % 8 || (!g->w_tiled && (g->ldw < g->k || g->ldw % 8))) return DLM_ERR_ALIGN;
    if (g->w_tiled < 0 || g->w_tiled > 1) return DLM_ERR_SHAPE;
    if (!aligned16(g->x) || !aligned16(g->w) || (reinterpret_cast<uintptr_t>(g->workspace) & 255)) return DLM_ERR_ALIGN;
    if (g->splits < 0 || g->splits > kMaxSplits) return DLM_ERR_SHAPE;
    if (g->token_tiles < 0 || (g->token_tiles > 0 && (g->m % (16 * g->token_tiles) || g->token_tiles > 16)))
        return DLM_ERR_SHAPE;
    return DLM_OK;
}

// Fills the device-side GEMM block; returns the per-rank grid in *grid.
int fill_gemm(GemmDev* d, const DlmGemm* g, int max_ctas, int sms, int* grid, int owner_rows = 0,
              bool single_rank = false) {
    std::memset(d, 0, sizeof(*d));
    const int avail = max_ctas > 0 && max_ctas < sms ? max_ctas : sms;
    const int feature_tiles = g->n / kBlockF, nkb = (g->k + kBlockK - 1) / kBlockK;
    int token_tiles = g->token_tiles, splits = g->splits;
    if (token_tiles == 0 || splits == 0) {
        int t = 1, sp = 1;
        choose_tiling(g->m, g->n, g->k, avail, &t, &sp, owner_rows, single_rank);
        if (token_tiles == 0 && splits == 0) {
            token_tiles = t;
            splits = sp;
        } else if (token_tiles == 0) {
            token_tiles = 1;
        } else {
            splits = 1;
        }
    }
    if (splits > nkb) splits = nkb;
    const int tiles = feature_tiles * token_tiles;
    if (tiles > kMaxTiles || tiles * splits > avail) return DLM_ERR_GRID;
    const int mt = g->m / token_tiles;
    int rc = g->w_tiled ? DLM_OK : make_map(&d->tm_w, g->w, g->n, g->k, g->ldw, kBlockF);
    if (g->w_tiled) d->w_tiles = static_cast<const uint8_t*>(g->w);
    if (rc == DLM_OK) rc = make_map(&d->tm_x, g->x, g->m, g->k, g->ldx, mt);
    if (rc != DLM_OK) return rc;
    const size_t need = kWorkspaceHeader + (splits > 1 ? static_cast<size_t>(splits) * g->m * g->n * sizeof(float) : 0);
    if (g->workspace_bytes < static_cast<int64_t>(need)) return DLM_ERR_WORKSPACE;
    d->gen = static_cast<int*>(g->workspace);
    d->counters = d->gen + kEpochSlots;
    d->ws = reinterpret_cast<float*>(static_cast<char*>(g->workspace) + kWorkspaceHeader);
    d->m = g->m;
    d->n = g->n;
    d->k = g->k;
    d->splits = splits;
    d->token_tiles = token_tiles;
    d->stages = rowpar_stages(mt);
    *grid = tiles * splits;
    return DLM_OK;
}

}  // namespace

extern "C" {

int dlm_reduce_bf16(const void* partial, const DlmComm* comm, dlm_stream_t stream) {
    int rc = check_comm(comm);
    if (rc != DLM_OK) return rc;
    if (partial == nullptr) return DLM_ERR_NULL;
    if (!aligned16(partial)) return DLM_ERR_ALIGN;
    DeviceInfo info;
    rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    ReduceParams<1> p;
    fill_comm(&p.c[0], comm);
    p.partial[0] = static_cast<const __nv_bfloat16*>(partial);
    int grid = comm->max_ctas > 0 && comm->max_ctas < info.sms ? comm->max_ctas : info.sms;
    if (grid > DLM_EPOCH_SLOTS) grid = DLM_EPOCH_SLOTS;
    return launch_reduce(p, grid, comm->n / kVec, {static_cast<cudaStream_t>(stream), comm->pdl != 0, false});
}

int dlm_reduce_bf16_loopback(const void* const* partial, const DlmComm* comm, int nranks, dlm_stream_t stream) {
    DeviceInfo info;
    int rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    if (partial == nullptr || comm == nullptr) return DLM_ERR_NULL;
    if (nranks < 1 || nranks > DLM_MAX_WORLD) return DLM_ERR_WORLD;
    ReduceParams<kMaxWorld> p;
    std::memset(&p, 0, sizeof(p));
    for (int i = 0; i < nranks; ++i) {
        rc = check_comm(&comm[i]);
        if (rc != DLM_OK) return rc;
        if (comm[i].world != nranks || comm[i].rank != i || comm[i].out_mc != nullptr) return DLM_ERR_WORLD;
        if (comm[i].rows != comm[0].rows || comm[i].n != comm[0].n) return DLM_ERR_SHAPE;
        if (partial[i] == nullptr) return DLM_ERR_NULL;
        if (!aligned16(partial[i])) return DLM_ERR_ALIGN;
        fill_comm(&p.c[i], &comm[i]);
        p.partial[i] = static_cast<const __nv_bfloat16*>(partial[i]);
    }
    int grid = info.sms / nranks;
    if (comm[0].max_ctas > 0 && comm[0].max_ctas < grid) grid = comm[0].max_ctas;
    if (grid < 1) return DLM_ERR_GRID;
    return launch_reduce_loopback(p, grid, nranks, comm[0].n / kVec, {static_cast<cudaStream_t>(stream), false, true});
}

namespace {

// The DlmComm of an all-gather describes only the exchange: rank, world, recv (+ recv_mc), out, epochs, status.
int check_gather(const DlmComm* c, const void* x, int64_t bytes) {
    if (c == nullptr || x == nullptr) return DLM_ERR_NULL;
    if (c->world < 1 || c->world > DLM_MAX_WORLD || c->rank < 0 || c->rank >= c->world) return DLM_ERR_WORLD;
    if (bytes <= 0 || bytes % 16 || bytes > DLM_GATHER_MAX_BYTES) return DLM_ERR_SHAPE;
    if (c->out == nullptr || c->epochs == nullptr) return DLM_ERR_NULL;
    for (int s = 0; s < c->world; ++s) {
        if (c->recv[s] == nullptr) return DLM_ERR_NULL;
        if (!aligned16(c->recv[s])) return DLM_ERR_ALIGN;
    }
    if (!aligned16(x) || !aligned16(c->out) || !aligned16(c->recv_mc)) return DLM_ERR_ALIGN;
    if (c->timeout_ns < 0 || c->max_ctas < 0) return DLM_ERR_SHAPE;
    return DLM_OK;
}

void fill_gather(CommDev* d, const DlmComm* c, int64_t bytes) {
    std::memset(d, 0, sizeof(*d));
    for (int s = 0; s < c->world; ++s) d->recv[s] = static_cast<__nv_bfloat16*>(c->recv[s]);
    d->recv_mc = static_cast<__nv_bfloat16*>(c->recv_mc);
    d->out = static_cast<__nv_bfloat16*>(c->out);
    d->epochs = c->epochs;
    d->status = c->status;
    d->timeout_ns = c->timeout_ns > 0 ? c->timeout_ns : kDefaultTimeoutNs;
    d->rank = c->rank;
    d->world = c->world;
    d->rows = d->R = d->slot_rows = 1;
    d->n = static_cast<int>(bytes / 2);
    d->one_shot = 1;  // every rank receives every block whole (also with one rank: its own)
}

int gather_grid(int64_t bytes, int cap) {
    int grid = static_cast<int>((bytes / 16 + 255) / 256);
    if (grid > cap) grid = cap;
    return grid < 1 ? 1 : grid;
}

}  // namespace

int dlm_all_gather(const void* x, int64_t bytes, const DlmComm* comm, dlm_stream_t stream) {
    int rc = check_gather(comm, x, bytes);
    if (rc != DLM_OK) return rc;
    DeviceInfo info;
    rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    ReduceParams<1> p;
    fill_gather(&p.c[0], comm, bytes);
    p.partial[0] = static_cast<const __nv_bfloat16*>(x);
    const int cap = comm->max_ctas > 0 && comm->max_ctas < 32 ? comm->max_ctas : 32;
    return launch_gather(p, gather_grid(bytes, cap), {static_cast<cudaStream_t>(stream), comm->pdl != 0, false});
}

int dlm_all_gather_loopback(const void* const* x, int64_t bytes, const DlmComm* comm, int nranks, dlm_stream_t stream) {
    DeviceInfo info;
    int rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    if (x == nullptr || comm == nullptr) return DLM_ERR_NULL;
    if (nranks < 1 || nranks > DLM_MAX_WORLD) return DLM_ERR_WORLD;
    ReduceParams<kMaxWorld> p;
    std::memset(&p, 0, sizeof(p));
    for (int i = 0; i < nranks; ++i) {
        rc = check_gather(&comm[i], x[i], bytes);
        if (rc != DLM_OK) return rc;
        if (comm[i].world != nranks || comm[i].rank != i || comm[i].recv_mc != nullptr) return DLM_ERR_WORLD;
        fill_gather(&p.c[i], &comm[i], bytes);
        p.partial[i] = static_cast<const __nv_bfloat16*>(x[i]);
    }
    int cap = info.sms / nranks;
    if (cap > 16) cap = 16;
    if (comm[0].max_ctas > 0 && comm[0].max_ctas < cap) cap = comm[0].max_ctas;
    if (cap < 1) return DLM_ERR_GRID;
    return launch_gather_loopback(p, gather_grid(bytes, cap), nranks, {static_cast<cudaStream_t>(stream), false, true});
}

int dlm_gemm_bf16(const DlmGemm* gemm, void* out, int64_t ldo, int pdl, dlm_stream_t stream) {
    int rc = check_gemm(gemm);
    if (rc != DLM_OK) return rc;
    if (out == nullptr) return DLM_ERR_NULL;
    if (!aligned16(out) || ldo < gemm->n || ldo % 8) return DLM_ERR_ALIGN;
    DeviceInfo info;
    rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    RowparParams<1> p;
    std::memset(&p, 0, sizeof(p));
    int grid = 0;
    rc = fill_gemm(&p.g[0], gemm, 0, info.sms, &grid);
    if (rc != DLM_OK) return rc;
    p.g[0].out = static_cast<__nv_bfloat16*>(out);
    p.g[0].ldo = ldo;
    p.fused = 0;
    return launch_rowpar(p, grid, {static_cast<cudaStream_t>(stream), pdl != 0, false});
}

// ---------------------------------------------------------------------------------------------------------------------
// The entry point that allocates nothing.
//
// Its split-K scratch is this file-scope device array: DLM_NOALLOC_SCRATCH_BYTES of global memory that every GPU which
// loads the library holds until the process exits. In host code `g_noalloc_scratch` is only a stand-in for the symbol,
// not a device address; the address a kernel may use comes from cudaGetSymbolAddress, asked once per device with that
// device current (first call of the entry point on that device).
// ---------------------------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_noalloc_scratch[DLM_NOALLOC_SCRATCH_BYTES];

static int noalloc_scratch(void** ptr) {
    static void* cached[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return cuda_fail(err);
    if (dev < 0 || dev >= 64) return DLM_ERR_ARCH;
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (err != cudaSuccess) return cuda_fail(err);
        cached[dev] = p;
    }
    *ptr = cached[dev];
    return DLM_OK;
}

int dlm_gemm_bf16_noalloc(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw,
                          int64_t ldo, int splits, int token_tiles, int pdl, dlm_stream_t stream) {
    DlmGemm g;
    std::memset(&g, 0, sizeof(g));
    g.x = x, g.w = w, g.m = m, g.n = n, g.k = k, g.ldx = ldx, g.ldw = ldw;
    g.splits = splits, g.token_tiles = token_tiles, g.w_tiled = 0;
    g.workspace = reinterpret_cast<void*>(uintptr_t(256));  // placeholder for the argument checks only
    g.workspace_bytes = DLM_NOALLOC_SCRATCH_BYTES;
    int rc = check_gemm(&g);
    if (rc != DLM_OK) return rc;
    if (out == nullptr) return DLM_ERR_NULL;
    if (!aligned16(out) || ldo < n || ldo % 8) return DLM_ERR_ALIGN;
    const size_t per_split = static_cast<size_t>(m) * n * sizeof(float);
    // K cannot be split into more ranges than it has k-blocks: a larger request runs as that many (as dlm_gemm_bf16
    // does), and it is that number the scratch must hold.
    const int nkb = (k + kBlockK - 1) / kBlockK;
    if (g.splits > nkb) g.splits = splits = nkb;
    // An explicit request that does not fit is refused; splits the library picks are capped to what fits
    // (one split needs no partial tiles at all).
    if (splits > 1 && kWorkspaceHeader + splits * per_split > DLM_NOALLOC_SCRATCH_BYTES) return DLM_ERR_SCRATCH;
    DeviceInfo info;
    rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    void* scratch = nullptr;
    rc = noalloc_scratch(&scratch);
    if (rc != DLM_OK) return rc;
    g.workspace = scratch;
    if (g.splits == 0 || g.token_tiles == 0) {
        int t = 1, sp = 1;
        choose_tiling(m, n, k, info.sms, &t, &sp);
        if (g.token_tiles == 0) g.token_tiles = g.splits == 0 ? t : 1;
        if (g.splits == 0) g.splits = token_tiles == 0 ? sp : 1;
        while (g.splits > 1 && kWorkspaceHeader + g.splits * per_split > DLM_NOALLOC_SCRATCH_BYTES) --g.splits;
    }
    RowparParams<1> p;
    std::memset(&p, 0, sizeof(p));
    int grid = 0;
    rc = fill_gemm(&p.g[0], &g, 0, info.sms, &grid);
    if (rc != DLM_OK) return rc;
    p.g[0].out = static_cast<__nv_bfloat16*>(out);
    p.g[0].ldo = ldo;
    p.fused = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the last call left. The only part that must start at zero is the header (launch
    // generation and arrival counters); the partial tiles are fully rewritten before they are read.
    const cudaError_t err = cudaMemsetAsync(scratch, 0, kWorkspaceHeader, s);
    if (err != cudaSuccess) return cuda_fail(err);
    return launch_rowpar(p, grid, {s, pdl != 0, false});
}

static bool overlaps(const void* a, size_t a_bytes, const void* b, size_t b_bytes) {
    const uintptr_t a0 = reinterpret_cast<uintptr_t>(a), b0 = reinterpret_cast<uintptr_t>(b);
    return a != nullptr && b != nullptr && a0 < b0 + b_bytes && b0 < a0 + a_bytes;
}

static int check_pair(const DlmGemm* gemm, const DlmComm* comm) {
    int rc = check_gemm(gemm);
    if (rc == DLM_OK) rc = check_comm(comm);
    if (rc != DLM_OK) return rc;
    if (gemm->m != comm->rows || gemm->n != comm->n || comm->n > DLM_FUSED_MAX_N) return DLM_ERR_SHAPE;
    // The fused kernel re-arms `rearm` and fills `out` while other CTAs may still be loading x: the GEMM's input must
    // be neither (in the reference the GEMM is an earlier kernel, so there the aliasing is harmless).
    const size_t x_bytes = (static_cast<size_t>(gemm->m - 1) * gemm->ldx + gemm->k) * 2;
    const size_t out_bytes = static_cast<size_t>(comm->rows) * comm->n * 2;
    if (overlaps(gemm->x, x_bytes, comm->rearm, static_cast<size_t>(comm->rearm_bytes)) ||
        overlaps(gemm->x, x_bytes, comm->out, out_bytes))
        return DLM_ERR_OVERLAP;
    return DLM_OK;
}

int dlm_rowpar_bf16(const DlmGemm* gemm, const DlmComm* comm, dlm_stream_t stream) {
    int rc = check_pair(gemm, comm);
    if (rc != DLM_OK) return rc;
    DeviceInfo info;
    rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    RowparParams<1> p;
    std::memset(&p, 0, sizeof(p));
    int grid = 0;
    const int slot_rows = comm->one_shot && comm->world > 1 ? comm->rows : comm->rows / comm->world;  // rows this rank sums
    rc = fill_gemm(&p.g[0], gemm, comm->max_ctas, info.sms, &grid, slot_rows, comm->world == 1);
    if (rc != DLM_OK) return rc;
    fill_comm(&p.c[0], comm);
    p.fused = 1;
    return launch_rowpar(p, grid, {static_cast<cudaStream_t>(stream), comm->pdl != 0, false});
}

static int check_moe(const DlmMoe* m) {
    if (m == nullptr) return DLM_ERR_NULL;
    if (!m->act_codes || !m->act_scales || !m->amap || !m->counts || !m->w_codes || !m->w_scales || !m->g2 || !m->ids ||
        !m->weights || !m->workspace)
        return DLM_ERR_NULL;
    if (m->m < 1 || m->m > DLM_MAX_M || m->n < kBlockF || m->n % 256 || m->n > DLM_FUSED_MAX_N) return DLM_ERR_SHAPE;
    if (m->f < 64 || m->f % 64 || m->f > 4096 || m->top_k < 1 || m->top_k > 16) return DLM_ERR_SHAPE;
    if (m->m_max < 1 || m->m_max > 256 || m->e_local < 1 || m->e_local > 256) return DLM_ERR_SHAPE;
    if (m->lo < 0 || m->lo + m->e_local > m->e_total || m->w_tiled < 0 || m->w_tiled > 1) return DLM_ERR_SHAPE;
    if (!aligned16(m->act_codes) || !aligned16(m->w_codes) || !aligned16(m->w_scales) || !aligned16(m->shared) ||
        (reinterpret_cast<uintptr_t>(m->act_scales) & 3) || (reinterpret_cast<uintptr_t>(m->workspace) & 255))
        return DLM_ERR_ALIGN;
    if (static_cast<size_t>(m->workspace_bytes) < dlm_moe_workspace_bytes(m->m, m->n, m->top_k)) return DLM_ERR_WORKSPACE;
    return DLM_OK;
}

static int make_map_u8(CUtensorMap* map, const void* base, long long rows, int row_bytes, int box_rows) {
    EncodeTiled fn = encode_tiled();
    if (fn == nullptr) return DLM_ERR_CUDA;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
    const cuuint32_t box[2] = {128, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = 100000 + static_cast<int>(r);
        return DLM_ERR_CUDA;
    }
    return DLM_OK;
}

static int fill_moe(MoeDev* d, const DlmMoe* m) {
    std::memset(d, 0, sizeof(*d));
    int rc = DLM_OK;
    if (m->w_tiled) d->w_tiles = static_cast<const uint8_t*>(m->w_codes);
    else rc = make_map_u8(&d->tm_w, m->w_codes, static_cast<long long>(m->e_local) * m->n, m->f / 2, kBlockF);
    if (rc == DLM_OK) rc = make_map_u8(&d->tm_a, m->act_codes, static_cast<long long>(m->e_local) * m->m_max, m->f / 2, 8);
    if (rc != DLM_OK) return rc;
    d->a_scales = static_cast<const uint8_t*>(m->act_scales);
    d->w_scales = static_cast<const uint8_t*>(m->w_scales);
    d->amap = m->amap, d->counts = m->counts, d->g2 = m->g2, d->ids = m->ids, d->weights = m->weights;
    d->shared = static_cast<const __nv_bfloat16*>(m->shared);
    d->gen = static_cast<int*>(m->workspace);
    d->counters = d->gen + kEpochSlots;
    d->y = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(m->workspace) + kWorkspaceHeader);
    d->m = m->m, d->n = m->n, d->f = m->f, d->top_k = m->top_k, d->m_max = m->m_max;
    d->lo = m->lo, d->e_local = m->e_local, d->e_total = m->e_total;
    d->rows_cap = (m->m_max + 15) / 16 * 16;  // activation rows of one work item: at most 128
    if (d->rows_cap > 128) d->rows_cap = 128;
    d->stages = moe_stages(d->rows_cap);
    return DLM_OK;
}

size_t dlm_moe_workspace_bytes(int m, int n, int top_k) {
    if (m <= 0 || n <= 0 || top_k <= 0) return 0;
    return kWorkspaceHeader + static_cast<size_t>(m) * top_k * n * 2;
}

int dlm_moe_nvfp4(const DlmMoe* moe, void* out, int64_t ldo, int pdl, dlm_stream_t stream) {
    int rc = check_moe(moe);
    if (rc != DLM_OK) return rc;
    if (out == nullptr) return DLM_ERR_NULL;
    if (!aligned16(out) || ldo < moe->n || ldo % 8) return DLM_ERR_ALIGN;
    DeviceInfo info;
    rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    MoeParams<1> p;
    std::memset(&p, 0, sizeof(p));
    rc = fill_moe(&p.g[0], moe);
    if (rc != DLM_OK) return rc;
    p.g[0].out = static_cast<__nv_bfloat16*>(out);
    p.g[0].ldo = ldo;
    p.fused = 0;
    return launch_moe(p, info.sms, {static_cast<cudaStream_t>(stream), pdl != 0, false});
}

int dlm_rowpar_nvfp4_moe(const DlmMoe* moe, const DlmComm* comm, dlm_stream_t stream) {
    int rc = check_moe(moe);
    if (rc == DLM_OK) rc = check_comm(comm);
    if (rc != DLM_OK) return rc;
    if (moe->m != comm->rows || moe->n != comm->n) return DLM_ERR_SHAPE;
    DeviceInfo info;
    rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    MoeParams<1> p;
    std::memset(&p, 0, sizeof(p));
    rc = fill_moe(&p.g[0], moe);
    if (rc != DLM_OK) return rc;
    fill_comm(&p.c[0], comm);
    p.fused = 1;
    const int grid = comm->max_ctas > 0 && comm->max_ctas < info.sms ? comm->max_ctas : info.sms;
    return launch_moe(p, grid, {static_cast<cudaStream_t>(stream), comm->pdl != 0, false});
}

static int check_front(const DlmMoeFront* a) {
    if (a == nullptr) return DLM_ERR_NULL;
    if ((a->x == nullptr && (a->xq == nullptr || a->xs == nullptr)) || (a->x != nullptr && a->a1_inv == nullptr))
        return DLM_ERR_NULL;
    if (!a->packed || !a->w13_codes || !a->w13_scales || !a->g1 || !a->a2_inv || !a->ids || !a->weights || !a->counts ||
        !a->amap || !a->slot_codes || !a->slot_scales || !a->act_codes || !a->act_scales)
        return DLM_ERR_NULL;
    if (a->m < 1 || a->m > DLM_MAX_M || a->hidden < 256 || a->hidden % 256 || a->hidden > DLM_MAX_N) return DLM_ERR_SHAPE;
    if (a->f < 64 || a->f % 64 || a->f > 4096 || a->top_k < 1 || a->top_k > 16) return DLM_ERR_SHAPE;
    if (a->m_max < 1 || a->m_max > 256 || a->e_local < 1 || a->e_local > 256 || a->activation < 0 || a->activation > 1)
        return DLM_ERR_SHAPE;
    if (a->lo < 0 || a->lo + a->e_local > a->e_total || a->w13_tiled < 0 || a->w13_tiled > 1) return DLM_ERR_SHAPE;
    if (!aligned16(a->x) || !aligned16(a->xq) || !aligned16(a->xs) || !aligned16(a->w13_codes) ||
        !aligned16(a->w13_scales) || !aligned16(a->slot_codes) || !aligned16(a->slot_scales) ||
        !aligned16(a->act_codes) || (reinterpret_cast<uintptr_t>(a->act_scales) & 3))
        return DLM_ERR_ALIGN;
    return DLM_OK;
}

int dlm_moe_front_nvfp4(const DlmMoeFront* a, int pdl, dlm_stream_t stream) {
    int rc = check_front(a);
    if (rc != DLM_OK) return rc;
    DeviceInfo info;
    rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    PrepareDev prep;
    std::memset(&prep, 0, sizeof(prep));
    prep.x = static_cast<const __nv_bfloat16*>(a->x);
    prep.xq = static_cast<const uint8_t*>(a->xq), prep.xs = static_cast<const uint8_t*>(a->xs);
    prep.a1_inv = a->a1_inv, prep.packed = a->packed;
    prep.ids = a->ids, prep.weights = a->weights, prep.counts = a->counts, prep.amap = a->amap;
    prep.slot_codes = static_cast<uint8_t*>(a->slot_codes), prep.slot_scales = static_cast<uint8_t*>(a->slot_scales);
    prep.rows = a->m, prep.hidden = a->hidden, prep.top_k = a->top_k, prep.e_total = a->e_total;
    prep.lo = a->lo, prep.e_local = a->e_local, prep.m_max = a->m_max;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    rc = launch_moe_prepare(prep, {s, pdl != 0, false});
    if (rc != DLM_OK) return rc;
    // GEMM1 on the expert pipeline: the "output features" are the 2F interleaved gate / up rows, K is the hidden size.
    MoeParams<1> p;
    std::memset(&p, 0, sizeof(p));
    MoeDev* d = &p.g[0];
    if (a->w13_tiled) d->w_tiles = static_cast<const uint8_t*>(a->w13_codes);
    else rc = make_map_u8(&d->tm_w, a->w13_codes, static_cast<long long>(a->e_local) * 2 * a->f, a->hidden / 2, kBlockF);
    if (rc == DLM_OK)
        rc = make_map_u8(&d->tm_a, a->slot_codes, static_cast<long long>(a->e_local) * a->m_max, a->hidden / 2, 8);
    if (rc != DLM_OK) return rc;
    d->a_scales = static_cast<const uint8_t*>(a->slot_scales);
    d->w_scales = static_cast<const uint8_t*>(a->w13_scales);
    d->amap = a->amap, d->counts = a->counts, d->g2 = a->g1, d->a2_inv = a->a2_inv;
    d->aq_out = static_cast<uint8_t*>(a->act_codes), d->as_out = static_cast<uint8_t*>(a->act_scales);
    d->m = a->m, d->n = 2 * a->f, d->f = a->hidden, d->top_k = a->top_k, d->m_max = a->m_max;
    d->lo = a->lo, d->e_local = a->e_local, d->e_total = a->e_total;
    d->f_out = a->f, d->act_kind = a->activation;
    d->rows_cap = (a->m_max + 15) / 16 * 16;
    if (d->rows_cap > 128) d->rows_cap = 128;
    d->stages = moe_stages(d->rows_cap);
    p.fused = 0;
    return launch_moe_gate_up(p, info.sms, {s, true, false});  // always a dependent launch of the kernel above
}

int dlm_route_packed(const void* logits, const void* scale, int32_t* packed, int rows, int e, int top_k, int pdl,
                     dlm_stream_t stream) {
    if (logits == nullptr || scale == nullptr || packed == nullptr) return DLM_ERR_NULL;
    if (rows < 1 || e < 1 || e > 256 || top_k < 1 || top_k > 16 || top_k > e) return DLM_ERR_SHAPE;
    DeviceInfo info;
    const int rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    RouteDev r;
    r.logits = static_cast<const __nv_bfloat16*>(logits), r.scale = static_cast<const __nv_bfloat16*>(scale);
    r.packed = packed, r.rows = rows, r.e = e, r.top_k = top_k;
    return launch_route_packed(r, {static_cast<cudaStream_t>(stream), pdl != 0, false});
}

int dlm_abi_check_front(size_t sizeof_front) { return sizeof_front == sizeof(DlmMoeFront) ? DLM_OK : DLM_ERR_SHAPE; }

int dlm_rowpar_nvfp4_moe_loopback(const DlmMoe* moe, const DlmComm* comm, int nranks, dlm_stream_t stream) {
    if (moe == nullptr || comm == nullptr) return DLM_ERR_NULL;
    if (nranks < 1 || nranks > DLM_MAX_WORLD) return DLM_ERR_WORLD;
    MoeParams<kMaxWorld> p;
    std::memset(&p, 0, sizeof(p));
    for (int i = 0; i < nranks; ++i) {
        int rc = check_moe(&moe[i]);
        if (rc == DLM_OK) rc = check_comm(&comm[i]);
        if (rc != DLM_OK) return rc;
        if (comm[i].world != nranks || comm[i].rank != i || comm[i].out_mc != nullptr) return DLM_ERR_WORLD;
        if (moe[i].m != comm[i].rows || moe[i].n != comm[i].n || moe[i].m != moe[0].m || moe[i].n != moe[0].n ||
            moe[i].m_max != moe[0].m_max)
            return DLM_ERR_SHAPE;
    }
    DeviceInfo info;
    int rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    for (int i = 0; i < nranks; ++i) {
        rc = fill_moe(&p.g[i], &moe[i]);
        if (rc != DLM_OK) return rc;
        fill_comm(&p.c[i], &comm[i]);
    }
    p.fused = 1;
    int grid = info.sms / nranks;
    if (comm[0].max_ctas > 0 && comm[0].max_ctas < grid) grid = comm[0].max_ctas;
    if (grid < 1) return DLM_ERR_GRID;
    return launch_moe_loopback(p, grid, nranks, {static_cast<cudaStream_t>(stream), false, true});
}

int dlm_rowpar_bf16_loopback(const DlmGemm* gemm, const DlmComm* comm, int nranks, dlm_stream_t stream) {
    DeviceInfo info;
    int rc = device_info(&info);
    if (rc != DLM_OK) return rc;
    if (gemm == nullptr || comm == nullptr) return DLM_ERR_NULL;
    if (nranks < 1 || nranks > DLM_MAX_WORLD) return DLM_ERR_WORLD;
    RowparParams<kMaxWorld> p;
    std::memset(&p, 0, sizeof(p));
    const int per_rank = info.sms / nranks;
    int grid = 0;
    for (int i = 0; i < nranks; ++i) {
        rc = check_pair(&gemm[i], &comm[i]);
        if (rc != DLM_OK) return rc;
        if (comm[i].world != nranks || comm[i].rank != i || comm[i].out_mc != nullptr) return DLM_ERR_WORLD;
        if (gemm[i].m != gemm[0].m || gemm[i].n != gemm[0].n || gemm[i].k != gemm[0].k) return DLM_ERR_SHAPE;
        int cap = comm[0].max_ctas > 0 && comm[0].max_ctas < per_rank ? comm[0].max_ctas : per_rank;
        int gi = 0;
        rc = fill_gemm(&p.g[i], &gemm[i], cap, per_rank, &gi, comm[i].rows / comm[i].world, comm[i].world == 1);
        if (rc != DLM_OK) return rc;
        if (i > 0 && gi != grid) return DLM_ERR_SHAPE;
        grid = gi;
        fill_comm(&p.c[i], &comm[i]);
    }
    p.fused = 1;
    return launch_rowpar_loopback(p, grid, nranks, {static_cast<cudaStream_t>(stream), false, true});
}

size_t dlm_workspace_bytes(int m, int n, int k) {
    (void)k;
    if (m <= 0 || n <= 0) return 0;
    return kWorkspaceHeader +
           static_cast<size_t>(kMaxSplits) * static_cast<size_t>(m) * static_cast<size_t>(n) * sizeof(float);
}

int dlm_choose_tiling(int m, int n, int k, int max_ctas, int* token_tiles, int* splits) {
    if (token_tiles == nullptr || splits == nullptr) return DLM_ERR_NULL;
    if (m < 16 || m > DLM_MAX_M || m % 16 || n < kBlockF || n % kBlockF || k < kBlockK || k % 8) return DLM_ERR_SHAPE;
    DeviceInfo info;
    int sms = 148;
    if (device_info(&info) == DLM_OK) sms = info.sms;
    choose_tiling(m, n, k, max_ctas > 0 && max_ctas < sms ? max_ctas : sms, token_tiles, splits);
    return DLM_OK;
}

int dlm_status_read(int32_t* device_status, DlmStatus* out, dlm_stream_t stream) {
    if (device_status == nullptr || out == nullptr) return DLM_ERR_NULL;
    int32_t host[DLM_STATUS_WORDS];
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemcpyAsync(host, device_status, sizeof(host), cudaMemcpyDeviceToHost, s);
    if (err == cudaSuccess) err = cudaMemsetAsync(device_status, 0, sizeof(host), s);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    if (err != cudaSuccess) return cuda_fail(err);
    out->code = host[0];
    out->block = host[1] >> 8;
    out->slot = host[1] & 0xFF;
    out->phase = host[2];
    out->epoch = host[3];
    return DLM_OK;
}

int dlm_abi_check(size_t sizeof_comm, size_t sizeof_gemm, size_t sizeof_status) {
    return sizeof_comm == sizeof(DlmComm) && sizeof_gemm == sizeof(DlmGemm) && sizeof_status == sizeof(DlmStatus)
               ? DLM_OK
               : DLM_ERR_SHAPE;
}

int dlm_abi_check_moe(size_t sizeof_moe) { return sizeof_moe == sizeof(DlmMoe) ? DLM_OK : DLM_ERR_SHAPE; }

const char* dlm_strerror(int code) {
    switch (code) {
        case DLM_OK: return "ok";
        case DLM_ERR_SHAPE: return "unsupported shape (hidden size a multiple of 256, at most 8192; m a multiple of 16, at most 256; k a multiple of 64)";
        case DLM_ERR_ALIGN: return "address or leading dimension not 16-byte aligned";
        case DLM_ERR_WORLD: return "rows must split over ranks; at most 8 ranks; rank within the world";
        case DLM_ERR_NULL: return "required pointer is null";
        case DLM_ERR_GRID: return "grid cannot be co-resident on this GPU";
        case DLM_ERR_CUDA: return "CUDA call failed (dlm_last_cuda_error)";
        case DLM_ERR_WORKSPACE: return "workspace too small (dlm_workspace_bytes)";
        case DLM_ERR_TIMEOUT: return "device wait ran out: data from a rank never arrived";
        case DLM_ERR_ARCH: return "not an sm_100 device";
        case DLM_ERR_OVERLAP: return "the fused GEMM's input overlaps a buffer the same launch re-arms or writes (rearm, out)";
        case DLM_ERR_SCRATCH: return "requested K splits need more than the library's built-in scratch (DLM_NOALLOC_SCRATCH_BYTES)";
        default: return "unknown error";
    }
}

int dlm_last_cuda_error(void) { return g_last_cuda_error; }

int dlm_device_sms(void) {
    DeviceInfo info;
    const int rc = device_info(&info);
    return rc == DLM_OK || rc == DLM_ERR_ARCH ? info.sms : 0;
}

int dlm_device_arch(void) {
    DeviceInfo info;
    return device_info(&info) == DLM_OK ? 100 : 0;
}

int64_t dlm_launch_count(void) { return g_launches; }

}  // extern "C"
