// Context object behind the C ABI: one device, one stream, one error word.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <mutex>
#include <string>

#include "../../include/lv_b200.h"

struct lv_ctx {
    int device = 0;
    int sm_count = 0;
    int max_smem_optin = 0;
    cudaStream_t stream = nullptr;
    uint32_t* d_err = nullptr;        // device error word, see lv::ERR_* in common.cuh
    uint32_t* h_err = nullptr;        // pinned mirror used by lv_ctx_check
    cudaGraph_t capture_graph = nullptr;
    bool capturing = false;
    std::recursive_mutex api_mutex;   // see LV_ENTER
    void* comm = nullptr;             // ncclComm_t when a communicator is attached
    int comm_rank = 0, comm_size = 1;
    void* peer = nullptr;             // lv::PeerState of the peer-memory all-reduce
    bool peer_ready = false;
    void* tc_scratch = nullptr;       // partial accumulators of the K-split tensor-core products
    void* tc_counters = nullptr;
    bool tc_exact = false;            // batched q4_0 products with the exact hi/lo weight planes instead of one fp16 plane
    // exchange roles that lv_tp_arm_push / lv_tp_arm_pull set for the next GEMV-family launch
    struct {
        int push = -1, pull = -1;
        uint32_t epochs_per_step = 0, pull_rows = 0;
        float* x_out = nullptr;
    } tp_arm;
};

namespace lv {

// Records a message retrievable through lv_last_error_string (thread local).
int fail(int code, const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);
int gemv_configure(lv_ctx* ctx);
int attention_configure(lv_ctx* ctx);
int gemm_tc_configure(lv_ctx* ctx);
void gemm_tc_release(lv_ctx* ctx);
uint32_t* peer_step_counter(lv_ctx* ctx);
bool peer_windows(lv_ctx* ctx, float** windows, int* n_ranks, int* rank, uint32_t* capacity);   // the connected peer windows, if any          // device word counting evaluation steps, or null without a peer window

#define LV_CUDA(call)                                          \
    do {                                                       \
        cudaError_t e__ = (call);                              \
        if (e__ != cudaSuccess) return lv::cuda_fail(e__, #call); \
    } while (0)

// First statement of every entry point that takes a context.
// Entry points of one context are serialised: a stream capture keeps the context's lock from
// lv_graph_begin_capture to lv_graph_end_capture, so that no other thread can put work on (or
// synchronise) the capturing stream in between, which would invalidate the capture.
#define LV_ENTER(ctx)                                                        \
    if ((ctx) == nullptr) return lv::fail(LV_ERR_BAD_ARGUMENTS, "null context"); \
    std::lock_guard<std::recursive_mutex> lv_api_guard__((ctx)->api_mutex);  \
    LV_CUDA(cudaSetDevice((ctx)->device))

#define LV_REQUIRE(cond, msg)                                              \
    do {                                                                   \
        if (!(cond)) return lv::fail(LV_ERR_BAD_ARGUMENTS, std::string(msg)); \
    } while (0)

// Launches `kernel` on the context's stream with programmatic stream serialisation, so
// that it may begin while its predecessor drains (see pdl_wait in common.cuh).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(lv_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace lv
