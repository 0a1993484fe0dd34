// Stand-alone fused tensor-parallel reduction of a given BF16 partial: push reduce-scatter, rank-ordered FP32 sum
// (+ residual + RMSNorm), multicast all-gather, in-band arrival detection. One launch per call; every CTA pushes its
// share of the partial, re-arms its share of the stale buffers, then owns rows r = block, block + grid, ...
// Replaces reduce_kernel<NORM, RESIDUAL> of the reference (dlmrt/ops/csrc/tp_comm.cu:138-275) bit for bit.
#include "kernels.cuh"

namespace dlm {

int g_last_cuda_error = 0;
long long g_launches = 0;

// NR = 1: one rank per GPU (production). NR = 8: up to eight ranks emulated by one launch on one GPU, rank slot =
// blockIdx.y; the grid is launched cooperatively so that all ranks' CTAs are resident together.
// MAXT: 512 for hidden sizes up to 4096 (blocks of hidden / 8 threads), where the compiler may then use 128 registers
// per thread; 1024 for the rest.
template <int NR, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) reduce_kernel(const __grid_constant__ ReduceParams<NR> p) {
    const int slot = NR == 1 ? 0 : static_cast<int>(blockIdx.y);
    const CommDev& c = p.c[slot];
    __shared__ float scratch[64];
    pdl_launch_dependents();  // the next kernel may be set up while this one runs; it waits before it reads our output
    pdl_wait();
    const CommCtx x = comm_begin(c, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x), c.epochs[blockIdx.x],
                                 comm_failed(c));
    stamp(c, x, 0);
    push_partial(c, x, p.partial[slot]);
    stamp(c, x, 1);
    rearm_early(c, x);
    own_and_collect<(MAXT <= 512)>(c, x, scratch);  // re-arms late shares between its own and collect phases
    comm_end(c, x);
}

// All-gather of a small block of bytes (row statistics and the like) in the same barrier-free style: every rank stores
// its block into slot [e % 3][rank] of every rank's receive buffer (one multimem.st per 16 bytes, or one store per
// rank), re-arms the buffer peers write two invocations from now, and copies each slot into its own OUT
// [world][bytes] as the slot's vectors arrive. A vector has arrived once none of its four 32-bit words is all-ones,
// so the payload may be FP32, FP16 or BF16 values (arithmetic never produces those bit patterns) but not arbitrary
// integers. `c.n` is the block's size in 2-byte units (a multiple of 8), `c.rows` is 1.
template <int NR>
__global__ void __launch_bounds__(256, 1) gather_kernel(const __grid_constant__ ReduceParams<NR> p) {
    const int slot = NR == 1 ? 0 : static_cast<int>(blockIdx.y);
    const CommDev& c = p.c[slot];
    pdl_wait();
    const CommCtx x = comm_begin(c, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x), c.epochs[blockIdx.x],
                                 comm_failed(c));
    const int vecs = c.n / kVec;
    const int stride = x.blocks * blockDim.x;
    const int first = x.block * blockDim.x + threadIdx.x;
    for (int i = first; i < vecs; i += stride) {
        const uint4 v = *reinterpret_cast<const uint4*>(p.partial[slot] + static_cast<size_t>(i) * kVec);
        push_store(c, x, 0, i * kVec, v);
    }
    rearm(c, x, x.block, x.blocks);
    pdl_launch_dependents();
    const __nv_bfloat16* mine = c.recv[c.rank] + x.buf * x.buf_elems;
    for (int i = first; i < vecs * c.world; i += stride) {  // slot s = i / vecs, vector i % vecs
        const __nv_bfloat16* src = mine + static_cast<size_t>(i) * kVec;
        uint4 v;
        bool ok = !x.dead;
        while (ok) {
            v = load_volatile(src);
            if (v.x != 0xFFFFFFFFu && v.y != 0xFFFFFFFFu && v.z != 0xFFFFFFFFu && v.w != 0xFFFFFFFFu) break;
            if (globaltimer() > x.deadline) {
                report(c.status, kErrTimeout, i / vecs, kPhaseReceive, x.e);
                ok = false;
                break;
            }
        }
        if (ok) store_v4(c.out + static_cast<size_t>(i) * kVec, v);
    }
    comm_end(c, x);
}

template <int NR>
static int launch_gather_impl(const ReduceParams<NR>& p, dim3 grid, const LaunchOpts& o) {
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = dim3(256);
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
    const cudaError_t err = cudaLaunchKernelEx(&config, gather_kernel<NR>, p);
    if (err != cudaSuccess) {
        g_last_cuda_error = static_cast<int>(err);
        (void)cudaGetLastError();
        return -6;
    }
    ++g_launches;
    return 0;
}

int launch_gather(const ReduceParams<1>& p, int grid, const LaunchOpts& o) { return launch_gather_impl<1>(p, dim3(grid), o); }

int launch_gather_loopback(const ReduceParams<kMaxWorld>& p, int grid, int nranks, const LaunchOpts& o) {
    return launch_gather_impl<kMaxWorld>(p, dim3(grid, nranks), o);
}

template <int NR>
static int launch_impl(const ReduceParams<NR>& p, dim3 grid, int threads, const LaunchOpts& o) {
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = dim3(static_cast<unsigned>(threads));
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
    const cudaError_t err = threads <= 512 ? cudaLaunchKernelEx(&config, reduce_kernel<NR, 512>, p)
                                           : cudaLaunchKernelEx(&config, reduce_kernel<NR, 1024>, p);
    if (err != cudaSuccess) {
        g_last_cuda_error = static_cast<int>(err);
        (void)cudaGetLastError();
        return -6;
    }
    ++g_launches;
    return 0;
}

int launch_reduce(const ReduceParams<1>& p, int grid, int threads, const LaunchOpts& o) {
    return launch_impl<1>(p, dim3(grid), threads, o);
}

int launch_reduce_loopback(const ReduceParams<kMaxWorld>& p, int grid, int nranks, int threads, const LaunchOpts& o) {
    return launch_impl<kMaxWorld>(p, dim3(grid, nranks), threads, o);
}

}  // namespace dlm
