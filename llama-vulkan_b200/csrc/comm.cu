// Multi-GPU exchange step of the tensor-parallel decoder: an fp32 sum
// all-reduce of `dim` floats after the wo and the w2 products.  The reference
// is single-device; this is the addition that shards it.  NCCL is loaded at
// run time (dlopen) so that the library itself has no link-time dependency on it.
#include <dlfcn.h>

#include <mutex>
#include <string>

#include "common.cuh"
#include "ctx.h"

namespace lv {

// The few NCCL declarations that are used (stable since NCCL 2.x).
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclFloat32 = 7 };
enum { ncclSum = 0 };

struct NcclApi {
    int (*GetUniqueId)(ncclUniqueId*);
    int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t);
    int (*CommDestroy)(ncclComm_t);
    int (*CommAbort)(ncclComm_t);
    int (*CommGetAsyncError)(ncclComm_t, int*);
    const char* (*GetErrorString)(int);
    bool ok = false;
};

static NcclApi g_nccl;
static std::once_flag g_nccl_once;

static void load_nccl() {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
#define LV_SYM(field, name) g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, name))
    LV_SYM(GetUniqueId, "ncclGetUniqueId");
    LV_SYM(CommInitRank, "ncclCommInitRank");
    LV_SYM(AllReduce, "ncclAllReduce");
    LV_SYM(CommDestroy, "ncclCommDestroy");
    LV_SYM(CommAbort, "ncclCommAbort");
    LV_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
    LV_SYM(GetErrorString, "ncclGetErrorString");
#undef LV_SYM
    g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.AllReduce && g_nccl.CommDestroy && g_nccl.CommAbort &&
                g_nccl.CommGetAsyncError && g_nccl.GetErrorString;
}

static int nccl_ready() {
    std::call_once(g_nccl_once, load_nccl);
    if (!g_nccl.ok) return fail(LV_ERR_COMM, "libnccl.so.2 could not be loaded");
    return LV_OK;
}

static int nccl_fail(int rc, const char* what) {
    return fail(LV_ERR_COMM, std::string(what) + ": " + (g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "NCCL error"));
}

}  // namespace lv

using namespace lv;

extern "C" int lv_comm_unique_id(uint8_t* out128) {
    LV_REQUIRE(out128, "null argument");
    if (int rc = nccl_ready()) return rc;
    ncclUniqueId id;
    const int rc = g_nccl.GetUniqueId(&id);
    if (rc != ncclSuccess) return nccl_fail(rc, "ncclGetUniqueId");
    memcpy(out128, id.internal, 128);
    return LV_OK;
}

extern "C" int lv_comm_init_rank(lv_ctx* ctx, const uint8_t* id128, int n_ranks, int rank) {
    LV_ENTER(ctx);
    LV_REQUIRE(id128 && n_ranks >= 1 && rank >= 0 && rank < n_ranks, "bad communicator arguments");
    LV_REQUIRE(ctx->comm == nullptr, "the context already has a communicator");
    if (int rc = nccl_ready()) return rc;
    ncclUniqueId id;
    memcpy(id.internal, id128, 128);
    ncclComm_t comm = nullptr;
    const int rc = g_nccl.CommInitRank(&comm, n_ranks, id, rank);
    if (rc != ncclSuccess) return nccl_fail(rc, "ncclCommInitRank");
    ctx->comm = comm;
    ctx->comm_rank = rank;
    ctx->comm_size = n_ranks;
    return LV_OK;
}

extern "C" int lv_allreduce_f32(lv_ctx* ctx, float* buf, size_t count) {
    LV_ENTER(ctx);
    LV_REQUIRE(buf && count, "bad all-reduce arguments");
    if (ctx->comm_size <= 1 || ctx->comm == nullptr) return LV_OK;          // single rank: nothing to exchange
    const int rc = g_nccl.AllReduce(buf, buf, count, ncclFloat32, ncclSum, static_cast<ncclComm_t>(ctx->comm), ctx->stream);
    if (rc != ncclSuccess) return nccl_fail(rc, "ncclAllReduce");
    return LV_OK;
}

extern "C" int lv_comm_status(lv_ctx* ctx) {
    LV_ENTER(ctx);
    if (ctx->comm == nullptr) return LV_OK;
    int async = ncclSuccess;
    const int rc = g_nccl.CommGetAsyncError(static_cast<ncclComm_t>(ctx->comm), &async);
    if (rc != ncclSuccess) return nccl_fail(rc, "ncclCommGetAsyncError");
    if (async != ncclSuccess) return nccl_fail(async, "asynchronous NCCL error");
    return LV_OK;
}

extern "C" int lv_comm_abort(lv_ctx* ctx) {
    LV_ENTER(ctx);
    if (ctx->comm == nullptr) return LV_OK;
    g_nccl.CommAbort(static_cast<ncclComm_t>(ctx->comm));
    ctx->comm = nullptr;
    ctx->comm_size = 1;
    ctx->comm_rank = 0;
    return LV_OK;
}

extern "C" int lv_comm_destroy(lv_ctx* ctx) {
    LV_ENTER(ctx);
    if (ctx->comm == nullptr) return LV_OK;
    cudaStreamSynchronize(ctx->stream);
    g_nccl.CommDestroy(static_cast<ncclComm_t>(ctx->comm));
    ctx->comm = nullptr;
    ctx->comm_size = 1;
    ctx->comm_rank = 0;
    return LV_OK;
}
