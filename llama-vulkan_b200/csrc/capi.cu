// Context, memory and execution entry points of the C ABI.
#include <chrono>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"
#include "ctx.h"

struct lv_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint32_t kernel_nodes = 0;
};

namespace lv {

static thread_local std::string g_last_error;

int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    g_last_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
    return LV_ERR_CUDA;
}

}  // namespace lv

using namespace lv;

extern "C" const char* lv_last_error_string(void) { return g_last_error.c_str(); }

extern "C" int lv_device_count(int* count) {
    LV_REQUIRE(count, "null argument");
    *count = 0;
    LV_CUDA(cudaGetDeviceCount(count));
    return LV_OK;
}

extern "C" int lv_ctx_create(int device, lv_ctx** out) {
    LV_REQUIRE(out, "null argument");
    *out = nullptr;
    int n = 0;
    LV_CUDA(cudaGetDeviceCount(&n));
    LV_REQUIRE(device >= 0 && device < n, "no such CUDA device");
    LV_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop{};
    LV_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(LV_ERR_NOK, std::string("device is not sm_100 (B200): ") + prop.name);
    auto* ctx = new lv_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->max_smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
    cudaError_t e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->d_err, 256);
    if (e == cudaSuccess) e = cudaMemset(ctx->d_err, 0, 256);
    if (e == cudaSuccess) e = cudaMallocHost(&ctx->h_err, sizeof(uint32_t));
    if (e != cudaSuccess) {
        lv_ctx_destroy(ctx);
        return cuda_fail(e, "lv_ctx_create");
    }
    *ctx->h_err = 0;
    int rc = gemv_configure(ctx);
    if (rc == LV_OK) rc = attention_configure(ctx);
    if (rc == LV_OK) rc = gemm_tc_configure(ctx);
    if (rc != LV_OK) {
        lv_ctx_destroy(ctx);
        return rc;
    }
    *out = ctx;
    return LV_OK;
}

extern "C" int lv_ctx_destroy(lv_ctx* ctx) {
    if (!ctx) return LV_OK;
    cudaSetDevice(ctx->device);
    if (ctx->peer) lv_peer_destroy(ctx);
    if (ctx->comm) lv_comm_destroy(ctx);
    if (ctx->stream) { cudaStreamSynchronize(ctx->stream); cudaStreamDestroy(ctx->stream); }
    gemm_tc_release(ctx);
    if (ctx->d_err) cudaFree(ctx->d_err);
    if (ctx->h_err) cudaFreeHost(ctx->h_err);
    delete ctx;
    return LV_OK;
}

extern "C" void* lv_ctx_stream(lv_ctx* ctx) { return ctx ? ctx->stream : nullptr; }
extern "C" int lv_ctx_sm_count(lv_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

extern "C" int lv_arena_create(lv_ctx* ctx, size_t bytes, void** dptr) {
    LV_ENTER(ctx);
    LV_REQUIRE(dptr && bytes, "bad arena arguments");
    *dptr = nullptr;
    LV_CUDA(cudaMalloc(dptr, bytes));
    return LV_OK;
}

extern "C" int lv_arena_free(lv_ctx* ctx, void* dptr) {
    LV_ENTER(ctx);
    if (!dptr) return LV_OK;
    LV_CUDA(cudaStreamSynchronize(ctx->stream));
    LV_CUDA(cudaFree(dptr));
    return LV_OK;
}

extern "C" int lv_host_alloc(lv_ctx* ctx, size_t bytes, void** hptr) {
    LV_ENTER(ctx);
    LV_REQUIRE(hptr && bytes, "bad host allocation arguments");
    LV_CUDA(cudaMallocHost(hptr, bytes));
    return LV_OK;
}

extern "C" int lv_host_free(lv_ctx* ctx, void* hptr) {
    LV_ENTER(ctx);
    if (hptr) LV_CUDA(cudaFreeHost(hptr));
    return LV_OK;
}

extern "C" int lv_upload(lv_ctx* ctx, void* dst, const void* host_src, size_t bytes) {
    LV_ENTER(ctx);
    LV_REQUIRE(dst && host_src, "null argument");
    if (!bytes) return LV_OK;
    LV_CUDA(cudaMemcpyAsync(dst, host_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    LV_CUDA(cudaStreamSynchronize(ctx->stream));
    return LV_OK;
}

extern "C" int lv_download(lv_ctx* ctx, void* host_dst, const void* src, size_t bytes) {
    LV_ENTER(ctx);
    LV_REQUIRE(host_dst && src, "null argument");
    if (!bytes) return LV_OK;
    LV_CUDA(cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    LV_CUDA(cudaStreamSynchronize(ctx->stream));
    return LV_OK;
}

extern "C" int lv_upload_async(lv_ctx* ctx, void* dst, const void* pinned_src, size_t bytes) {
    LV_ENTER(ctx);
    LV_REQUIRE(dst && pinned_src, "null argument");
    if (!bytes) return LV_OK;
    LV_CUDA(cudaMemcpyAsync(dst, pinned_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return LV_OK;
}

extern "C" int lv_download_async(lv_ctx* ctx, void* pinned_dst, const void* src, size_t bytes) {
    LV_ENTER(ctx);
    LV_REQUIRE(pinned_dst && src, "null argument");
    if (!bytes) return LV_OK;
    LV_CUDA(cudaMemcpyAsync(pinned_dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return LV_OK;
}

extern "C" int lv_memset(lv_ctx* ctx, void* dst, int value, size_t bytes) {
    LV_ENTER(ctx);
    LV_REQUIRE(dst, "null argument");
    if (!bytes) return LV_OK;
    LV_CUDA(cudaMemsetAsync(dst, value, bytes, ctx->stream));
    return LV_OK;
}

extern "C" int lv_copy_d2d(lv_ctx* ctx, void* dst, const void* src, size_t bytes) {
    LV_ENTER(ctx);
    LV_REQUIRE(dst && src, "null argument");
    if (!bytes) return LV_OK;
    LV_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return LV_OK;
}

extern "C" int lv_graph_begin_capture(lv_ctx* ctx) {
    LV_ENTER(ctx);
    LV_REQUIRE(!ctx->capturing, "a capture is already open on this context");
    LV_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    ctx->api_mutex.lock();            // kept until lv_graph_end_capture (on this thread)
    return LV_OK;
}

extern "C" int lv_graph_end_capture(lv_ctx* ctx, lv_graph** out) {
    LV_ENTER(ctx);
    LV_REQUIRE(out, "null argument");
    LV_REQUIRE(ctx->capturing, "no capture is open on this context");
    *out = nullptr;
    ctx->capturing = false;
    cudaGraph_t graph = nullptr;
    const cudaError_t ended = cudaStreamEndCapture(ctx->stream, &graph);
    ctx->api_mutex.unlock();          // taken by lv_graph_begin_capture
    if (ended != cudaSuccess) return cuda_fail(ended, "cudaStreamEndCapture");
    auto* g = new lv_graph();
    g->graph = graph;
    size_t n_nodes = 0;
    if (cudaGraphGetNodes(graph, nullptr, &n_nodes) == cudaSuccess && n_nodes != 0) {
        std::vector<cudaGraphNode_t> nodes(n_nodes);
        if (cudaGraphGetNodes(graph, nodes.data(), &n_nodes) == cudaSuccess) {
            for (size_t i = 0; i < n_nodes; ++i) {
                cudaGraphNodeType t;
                if (cudaGraphNodeGetType(nodes[i], &t) == cudaSuccess && t == cudaGraphNodeTypeKernel) g->kernel_nodes++;
            }
        }
    }
    cudaError_t e = cudaGraphInstantiate(&g->exec, graph, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(graph);
        delete g;
        return cuda_fail(e, "cudaGraphInstantiate");
    }
    *out = g;
    return LV_OK;
}

extern "C" int lv_graph_launch(lv_ctx* ctx, lv_graph* g) {
    LV_ENTER(ctx);
    LV_REQUIRE(g && g->exec, "null graph");
    LV_CUDA(cudaGraphLaunch(g->exec, ctx->stream));
    return LV_OK;
}

extern "C" int lv_graph_kernel_nodes(lv_graph* g, uint32_t* out) {
    LV_REQUIRE(g && out, "null argument");
    *out = g->kernel_nodes;
    return LV_OK;
}

extern "C" int lv_graph_destroy(lv_graph* g) {
    if (!g) return LV_OK;
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    return LV_OK;
}

extern "C" int lv_stream_sync(lv_ctx* ctx, int timeout_ms) {
    LV_ENTER(ctx);                     // a capture that another thread has open ends first
    LV_REQUIRE(!ctx->capturing, "cannot wait for the stream while it is being captured");
    if (timeout_ms <= 0) {
        LV_CUDA(cudaStreamSynchronize(ctx->stream));
    } else {
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
        for (;;) {
            const cudaError_t q = cudaStreamQuery(ctx->stream);
            if (q == cudaSuccess) break;
            if (q != cudaErrorNotReady) return cuda_fail(q, "cudaStreamQuery");
            if (std::chrono::steady_clock::now() > deadline) return fail(LV_ERR_TIMEOUT, "stream did not drain in time");
            std::this_thread::yield();
        }
    }
    LV_CUDA(cudaMemcpyAsync(ctx->h_err, ctx->d_err, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    LV_CUDA(cudaStreamSynchronize(ctx->stream));
    if (*ctx->h_err != 0) {
        const uint32_t word = *ctx->h_err;
        cudaMemsetAsync(ctx->d_err, 0, sizeof(uint32_t), ctx->stream);
        return fail(LV_ERR_DEVICE_WAIT, "device error word " + std::to_string(word) +
                                            " (1 = copy wait lost, 2 = grid barrier lost, 4 = peer wait lost, 8 = index out of range)");
    }
    return LV_OK;
}
