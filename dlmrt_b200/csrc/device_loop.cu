// Device-side loop around captured graphs: head -> WHILE(*remaining > 0 && *step < limit){parts...} -> ... -> tail.
//
// The fused kernels of this library keep all their state (invocation counters, split-K generations, arrival flags) in
// device memory, so a captured round can be re-executed by a conditional WHILE node without the host. This file builds
// that loop for callers that hand in captured graphs; it serves the three shapes the reference's block-graph module
// has (dlmrt/ops/csrc/block_graph.cu:29-129,131-210): one loop between a begin and a commit graph, several loops in
// sequence, and one loop whose body is a list of parts of which some run only while a device flag is positive.
//
// Described as data instead of three classes: a program is a head graph, `n_loops` loops, and a tail graph; a loop is
// a list of parts (child graphs, optionally guarded by an IF on a device flag) and the (remaining, step, limit)
// triple its WHILE condition reads. The condition is evaluated on entry and again after every pass of the body, so a
// loop whose `limit` is reached, or whose `remaining` is already zero, never runs its body; `limit` also bounds the
// number of passes of one execution, so no body can keep the GPU in the loop forever.
#include <cuda_runtime.h>

#include <new>

#include "../../include/dlmrt_b200.h"

namespace dlm {
extern int g_last_cuda_error;
}

namespace {

// Entry test of a loop, and the test after every pass. `passes` counts the passes of this execution: a body that
// fails to advance *step cannot spin the GPU forever, the loop ends after `limit` passes whatever the body does.
__global__ void loop_enter(cudaGraphConditionalHandle handle, const int* remaining, const int* step, int limit, int* passes) {
    *passes = 0;
    cudaGraphSetConditional(handle, (*remaining > 0 && *step < limit) ? 1u : 0u);
}

__global__ void loop_again(cudaGraphConditionalHandle handle, const int* remaining, const int* step, int limit, int* passes) {
    const int done = ++*passes;
    cudaGraphSetConditional(handle, (*remaining > 0 && *step < limit && done < limit) ? 1u : 0u);
}

__global__ void part_condition(cudaGraphConditionalHandle handle, const int* flag) {
    cudaGraphSetConditional(handle, *flag > 0 ? 1u : 0u);
}

struct Builder {
    cudaError_t err = cudaSuccess;
    bool ok() const { return err == cudaSuccess; }
    void run(cudaError_t e) {
        if (err == cudaSuccess) err = e;
    }

    // Appends `node` after `*last` (or as a root when *last is null) and makes it the new last node.
    cudaGraphNode_t child(cudaGraph_t graph, cudaGraphNode_t last, cudaGraph_t what) {
        cudaGraphNode_t node = nullptr;
        run(cudaGraphAddChildGraphNode(&node, graph, last ? &last : nullptr, last ? 1 : 0, what));
        return node;
    }

    cudaGraphNode_t kernel(cudaGraph_t graph, cudaGraphNode_t last, void* func, void** args) {
        cudaKernelNodeParams params{};
        params.func = func;
        params.gridDim = dim3(1);
        params.blockDim = dim3(1);
        params.kernelParams = args;
        cudaGraphNode_t node = nullptr;
        run(cudaGraphAddKernelNode(&node, graph, last ? &last : nullptr, last ? 1 : 0, &params));
        return node;
    }

    // A conditional node of `type` after `last`; returns the node and its (empty) body graph.
    cudaGraphNode_t conditional(cudaGraph_t graph, cudaGraphNode_t last, cudaGraphConditionalHandle handle,
                                cudaGraphConditionalNodeType type, cudaGraph_t* body) {
        cudaGraphNodeParams params{};
        params.type = cudaGraphNodeTypeConditional;
        params.conditional.handle = handle;
        params.conditional.type = type;
        params.conditional.size = 1;
        cudaGraphNode_t node = nullptr;
#if CUDART_VERSION >= 13000
        run(cudaGraphAddNode(&node, graph, last ? &last : nullptr, nullptr, last ? 1 : 0, &params));
#else
        run(cudaGraphAddNode(&node, graph, last ? &last : nullptr, last ? 1 : 0, &params));
#endif
        *body = ok() ? params.conditional.phGraph_out[0] : nullptr;
        return node;
    }
};

}  // namespace

struct DlmDeviceLoop {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int* passes = nullptr;  // one pass counter per loop, device memory owned by this object
};

extern "C" {

DLM_API int dlm_device_loop_create(void* head, const DlmLoop* loops, int n_loops, void* tail, DlmDeviceLoop** out) {
    if (!out) return DLM_ERR_NULL;
    *out = nullptr;
    if (n_loops < 0 || n_loops > DLM_MAX_LOOPS || (n_loops > 0 && !loops)) return DLM_ERR_SHAPE;
    for (int l = 0; l < n_loops; ++l) {
        const DlmLoop& loop = loops[l];
        if (loop.n_parts < 1 || loop.n_parts > DLM_MAX_LOOP_PARTS || loop.limit < 0) return DLM_ERR_SHAPE;
        if (!loop.parts || !loop.remaining || !loop.step) return DLM_ERR_NULL;
        for (int i = 0; i < loop.n_parts; ++i)
            if (!loop.parts[i].graph) return DLM_ERR_NULL;
    }
    DlmDeviceLoop* self = new (std::nothrow) DlmDeviceLoop();
    if (!self) return DLM_ERR_CUDA;
    Builder b;
    b.run(cudaGraphCreate(&self->graph, 0));
    if (n_loops > 0) b.run(cudaMalloc(&self->passes, sizeof(int) * n_loops));
    cudaGraphNode_t last = nullptr;
    if (b.ok() && head) last = b.child(self->graph, nullptr, static_cast<cudaGraph_t>(head));
    for (int l = 0; l < n_loops && b.ok(); ++l) {
        const DlmLoop& loop = loops[l];
        cudaGraphConditionalHandle handle{};
        b.run(cudaGraphConditionalHandleCreate(&handle, self->graph, 0, 0));
        const int* remaining = loop.remaining;
        const int* step = loop.step;
        int limit = loop.limit;
        int* passes = self->passes + l;
        void* args[] = {&handle, &remaining, &step, &limit, &passes};
        // Entry test, the WHILE node, and inside it the parts followed by the test again.
        last = b.kernel(self->graph, last, reinterpret_cast<void*>(loop_enter), args);
        cudaGraph_t body = nullptr;
        last = b.conditional(self->graph, last, handle, cudaGraphCondTypeWhile, &body);
        cudaGraphNode_t inner = nullptr;
        for (int i = 0; i < loop.n_parts && b.ok(); ++i) {
            cudaGraph_t part = static_cast<cudaGraph_t>(loop.parts[i].graph);
            if (!loop.parts[i].flag) {
                inner = b.child(body, inner, part);
            } else {
                cudaGraphConditionalHandle when{};
                b.run(cudaGraphConditionalHandleCreate(&when, body, 0, 0));
                const int* flag = loop.parts[i].flag;
                void* if_args[] = {&when, &flag};
                inner = b.kernel(body, inner, reinterpret_cast<void*>(part_condition), if_args);
                cudaGraph_t branch = nullptr;
                inner = b.conditional(body, inner, when, cudaGraphCondTypeIf, &branch);
                if (b.ok()) b.child(branch, nullptr, part);
            }
        }
        if (b.ok()) b.kernel(body, inner, reinterpret_cast<void*>(loop_again), args);
    }
    if (b.ok() && tail) b.child(self->graph, last, static_cast<cudaGraph_t>(tail));
    if (b.ok()) b.run(cudaGraphInstantiate(&self->exec, self->graph, 0));
    if (!b.ok()) {
        dlm::g_last_cuda_error = static_cast<int>(b.err);
        (void)cudaGetLastError();
        if (self->exec) cudaGraphExecDestroy(self->exec);
        if (self->graph) cudaGraphDestroy(self->graph);
        if (self->passes) cudaFree(self->passes);
        delete self;
        return DLM_ERR_CUDA;
    }
    *out = self;
    return DLM_OK;
}

DLM_API int dlm_device_loop_launch(DlmDeviceLoop* loop, void* stream) {
    if (!loop || !loop->exec) return DLM_ERR_NULL;
    const cudaError_t err = cudaGraphLaunch(loop->exec, static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) {
        dlm::g_last_cuda_error = static_cast<int>(err);
        (void)cudaGetLastError();
        return DLM_ERR_CUDA;
    }
    return DLM_OK;
}

DLM_API void dlm_device_loop_destroy(DlmDeviceLoop* loop) {
    if (!loop) return;
    if (loop->exec) cudaGraphExecDestroy(loop->exec);
    if (loop->graph) cudaGraphDestroy(loop->graph);
    if (loop->passes) cudaFree(loop->passes);
    delete loop;
}

}  // extern "C"
