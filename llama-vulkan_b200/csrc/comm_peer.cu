// One-shot all-reduce over NVLink peer memory, fused with the residual add of the
// tensor-parallel decoder: residual += sum over ranks of partial.
//
// Every rank owns a receive window (cudaMalloc'd, exported with CUDA IPC) of
// 4 x n_ranks slots of `capacity` floats plus arrival flags.  Slot sets 0 and 1 belong to the
// exchanges fused into the GEMVs, sets 2 and 3 to the stand-alone kernel below: a step may mix the
// two mechanisms (the last exchange of a step without an output head uses this kernel), and with
// sets of its own this kernel can never overwrite a slot that a slower rank's GEMV is still reading.  A launch pushes the rank's
// partial vector into its slot of every rank's window with ordinary peer stores, publishes a
// flag per (rank, CTA), waits -- bounded -- for the flags of all ranks in its own window, and
// adds the slots from its own memory in rank order, so every rank computes bit-identical
// sums.  Its slots and flags alternate between two halves by launch parity, which is enough
// because a rank cannot start launch k + 2 before every rank has finished reading launch k.
// The reference is single-device; this replaces the NCCL all-reduce + add pair of the
// baseline path (lv_allreduce_f32 + lv_add_f32) with one kernel.
#include <cstdlib>
#include <string>

#include "common.cuh"
#include "ctx.h"
#include "gemv_stream.cuh"

namespace lv {

constexpr int kPeerMaxRanks = 8;
constexpr int kPeerCtas = 32;              // a batch of 64 rows is a megabyte per rank: four CTAs moved it at ~40 GB/s
constexpr int kPeerThreads = 256;

struct PeerWindowLayout {
    uint32_t capacity;        // floats per slot
    __host__ __device__ size_t slot_floats(int n_ranks) const { return size_t(kTpSlotSets) * n_ranks * capacity; }
    // slots, the flags of the stand-alone kernel (2 x 8 x 32 words), the flags of the exchanges fused into the GEMV
    __host__ __device__ size_t bytes(int n_ranks) const {
        return slot_floats(n_ranks) * sizeof(float) + size_t(kTpLegacyFlagWords) * sizeof(uint32_t) +
               size_t(2) * kTpMaxRanks * kTpFlagCtas * sizeof(uint32_t) + size_t(kTpFlagCtas) * sizeof(uint32_t) /* local flags */ + 256;
    }
};

struct PeerParams {
    float* window[kPeerMaxRanks];     // window[r]: rank r's receive window as seen from this GPU
    int rank, n_ranks;
    uint32_t capacity;
    uint32_t* epoch;                  // device word of this rank: launches completed so far
    uint32_t* err;
};

__device__ __forceinline__ uint32_t* window_flags(float* window, int n_ranks, uint32_t capacity) {
    return reinterpret_cast<uint32_t*>(window + size_t(kTpSlotSets) * n_ranks * capacity);
}

// grid = kPeerCtas; CTA c owns the float4 indices c, c + kPeerCtas, ... of the vector
__global__ void __launch_bounds__(kPeerThreads) allreduce_add_peer_kernel(float* __restrict__ residual, const float* __restrict__ partial,
                                                                         uint32_t count, const PeerParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t epoch = *p.epoch + 1;                 // this launch's number, the same on every rank
    const uint32_t half = epoch & 1u;
    const uint32_t n4 = count / 4;
    const size_t my_slot = (size_t(2 + half) * p.n_ranks + p.rank) * p.capacity;      // slot sets 2 and 3

    // push this rank's slice into its slot of every window (its own included)
    for (uint32_t i = blockIdx.x * kPeerThreads + threadIdx.x; i < n4; i += kPeerCtas * kPeerThreads) {
        const float4 v = reinterpret_cast<const float4*>(partial)[i];
        for (int r = 0; r < p.n_ranks; ++r) reinterpret_cast<float4*>(p.window[r] + my_slot)[i] = v;
    }
    // the barrier orders the CTA's stores before the release stores of the flags, whose system-scope
    // release covers them (a system fence in every thread is far more expensive)
    __syncthreads();
    if (threadIdx.x < uint32_t(p.n_ranks)) {
        uint32_t* flags = window_flags(p.window[threadIdx.x], p.n_ranks, p.capacity);
        st_release_sys(&flags[(half * kPeerMaxRanks + p.rank) * kPeerCtas + blockIdx.x], epoch);
    }
    // wait for every rank's slice of this CTA to land in this rank's window
    __shared__ uint32_t s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < uint32_t(p.n_ranks)) {
        const uint32_t* flag = &window_flags(p.window[p.rank], p.n_ranks, p.capacity)[(half * kPeerMaxRanks + threadIdx.x) * kPeerCtas + blockIdx.x];
        const long long t0 = clock64();
        while (ld_acquire_sys(flag) != epoch) {
            if (*reinterpret_cast<volatile uint32_t*>(p.err) != 0 || clock64() - t0 > kWaitCycleLimit) {
                atomicOr(p.err, ERR_PEER_TIMEOUT);
                s_ok = 0;
                break;
            }
        }
    }
    __syncthreads();
    if (s_ok) {
        const float* base = p.window[p.rank] + size_t(2 + half) * p.n_ranks * p.capacity;
        for (uint32_t i = blockIdx.x * kPeerThreads + threadIdx.x; i < n4; i += kPeerCtas * kPeerThreads) {
            float4 acc = reinterpret_cast<float4*>(residual)[i];
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < p.n_ranks; ++r) {              // fixed order: identical on every rank
                const float4 v = __ldcg(reinterpret_cast<const float4*>(base + size_t(r) * p.capacity) + i);
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            acc.x += sum.x; acc.y += sum.y; acc.z += sum.z; acc.w += sum.w;
            reinterpret_cast<float4*>(residual)[i] = acc;
        }
    }
    // the last CTA to finish advances the launch counter
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t done = atomicAdd(p.epoch + 1, 1u);
        if (done == kPeerCtas - 1) {
            p.epoch[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(p.epoch) = epoch;
        }
    }
}

static_assert(kTpLegacyFlagWords == 2 * kPeerMaxRanks * kPeerCtas && kTpMaxRanks == kPeerMaxRanks, "window layout");

struct PeerState {
    PeerParams params{};
    void* own_window = nullptr;
    void* opened[kPeerMaxRanks] = {nullptr};
    uint32_t* d_epoch = nullptr;
};

}  // namespace lv

using namespace lv;

extern "C" size_t lv_peer_window_bytes(int n_ranks, uint32_t capacity_floats) {
    if (n_ranks < 1 || n_ranks > kPeerMaxRanks || capacity_floats == 0 || capacity_floats % 4) return 0;
    return PeerWindowLayout{capacity_floats}.bytes(n_ranks);
}

extern "C" int lv_peer_window_create(lv_ctx* ctx, int n_ranks, uint32_t capacity_floats, uint8_t* handle64) {
    LV_ENTER(ctx);
    LV_REQUIRE(handle64 && ctx->peer == nullptr, "bad peer window arguments");
    const size_t bytes = lv_peer_window_bytes(n_ranks, capacity_floats);
    LV_REQUIRE(bytes != 0, "n_ranks must be 1..8 and the capacity a multiple of 4 floats");
    auto* st = new PeerState();
    cudaError_t e = cudaMalloc(&st->own_window, bytes);
    if (e == cudaSuccess) e = cudaMemset(st->own_window, 0, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&st->d_epoch, 256);
    if (e == cudaSuccess) e = cudaMemset(st->d_epoch, 0, 256);
    cudaIpcMemHandle_t h{};
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, st->own_window);
    if (e != cudaSuccess) {
        cudaFree(st->own_window);
        cudaFree(st->d_epoch);
        delete st;
        return cuda_fail(e, "lv_peer_window_create");
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    st->params.capacity = capacity_floats;
    st->params.n_ranks = n_ranks;
    st->params.epoch = st->d_epoch;
    st->params.err = ctx->d_err;
    ctx->peer = st;
    return LV_OK;
}

extern "C" int lv_peer_connect(lv_ctx* ctx, int rank, const uint8_t* handles /* n_ranks x 64 */) {
    LV_ENTER(ctx);
    auto* st = static_cast<PeerState*>(ctx->peer);
    LV_REQUIRE(st && handles && rank >= 0 && rank < st->params.n_ranks, "bad peer connect arguments");
    st->params.rank = rank;
    for (int r = 0; r < st->params.n_ranks; ++r) {
        if (r == rank) {
            st->params.window[r] = static_cast<float*>(st->own_window);
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + size_t(r) * 64, 64);
        void* ptr = nullptr;
        LV_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        st->opened[r] = ptr;
        st->params.window[r] = static_cast<float*>(ptr);
    }
    ctx->peer_ready = true;
    return LV_OK;
}

extern "C" int lv_allreduce_add_f32(lv_ctx* ctx, float* residual, float* partial, size_t count) {
    LV_ENTER(ctx);
    LV_REQUIRE(residual && partial && count, "bad all-reduce arguments");
    auto* st = static_cast<PeerState*>(ctx->peer);
    if (st != nullptr && ctx->peer_ready) {
        LV_REQUIRE(count % 4 == 0 && count <= st->params.capacity, "vector longer than the peer window's slots or not a multiple of 4");
        LV_REQUIRE((reinterpret_cast<uintptr_t>(residual) & 15u) == 0 && (reinterpret_cast<uintptr_t>(partial) & 15u) == 0, "vectors must be 16-byte aligned");
        LV_CUDA(launch_pdl(ctx, allreduce_add_peer_kernel, dim3(kPeerCtas), dim3(kPeerThreads), 0, residual,
                           static_cast<const float*>(partial), uint32_t(count), st->params));
        return LV_OK;
    }
    // baseline: NCCL (or nothing, on one rank), then the add
    if (int rc = lv_allreduce_f32(ctx, partial, count)) return rc;
    return lv_add_f32(ctx, residual, partial, count);
}

namespace lv {

// The connected windows of a context, for kernels that run their own exchange in them (lv_decode_step uses slot
// sets 0 and 1, like the exchanges fused into the GEMVs, which it replaces).  False without connected windows.
bool peer_windows(lv_ctx* ctx, float** windows, int* n_ranks, int* rank, uint32_t* capacity) {
    auto* st = static_cast<PeerState*>(ctx->peer);
    if (st == nullptr || !ctx->peer_ready) return false;
    for (int r = 0; r < st->params.n_ranks; ++r) windows[r] = st->params.window[r];
    *n_ranks = st->params.n_ranks;
    *rank = st->params.rank;
    *capacity = st->params.capacity;
    return true;
}

uint32_t* peer_step_counter(lv_ctx* ctx) {
    auto* st = static_cast<PeerState*>(ctx->peer);
    return (st != nullptr && ctx->peer_ready) ? st->d_epoch + 2 : nullptr;
}

// Fills the exchange part of a GEMV launch from the roles armed on the context and disarms them.
int peer_take_armed(lv_ctx* ctx, TpParams* tp, uint32_t pull_ctas) {
    *tp = TpParams{};
    tp->push_exchange = tp->pull_exchange = -1;
    auto& arm = ctx->tp_arm;
    if (arm.push < 0 && arm.pull < 0) return LV_OK;
    auto* st = static_cast<PeerState*>(ctx->peer);
    const bool ready = st != nullptr && ctx->peer_ready;
    if (ready) {
        for (int r = 0; r < st->params.n_ranks; ++r) tp->window[r] = st->params.window[r];
        tp->rank = st->params.rank;
        tp->n_ranks = st->params.n_ranks;
        tp->capacity = st->params.capacity;
        tp->step = st->d_epoch + 2;
        tp->epochs_per_step = arm.epochs_per_step;
        tp->push_exchange = arm.push;
        tp->pull_exchange = arm.pull;
        tp->pull_ctas = pull_ctas;
        tp->x_out = arm.x_out;
        // summing once per GPU instead of in every CTA is off unless LV_TP_TWO_PHASE=1 asks for it
        const char* force = getenv("LV_TP_TWO_PHASE");
        tp->two_phase = force != nullptr && (force[0] == '0' || force[0] == '1') ? uint32_t(force[0] - '0')
                                                                                  : uint32_t(st->params.n_ranks >= kTpTwoPhaseRanks);
    }
    arm.push = arm.pull = -1;
    arm.x_out = nullptr;
    if (!ready) return fail(LV_ERR_BAD_ARGUMENTS, "an exchange was armed but the peer windows are not connected");
    return LV_OK;
}

}  // namespace lv

extern "C" int lv_tp_arm_push(lv_ctx* ctx, int exchange, uint32_t epochs_per_step) {
    LV_ENTER(ctx);
    LV_REQUIRE(ctx->peer_ready, "peer windows are not connected");
    LV_REQUIRE(exchange >= 0 && uint32_t(exchange) < epochs_per_step, "exchange index out of range");
    ctx->tp_arm.push = exchange;
    ctx->tp_arm.epochs_per_step = epochs_per_step;
    return LV_OK;
}

extern "C" int lv_tp_arm_pull(lv_ctx* ctx, int exchange, uint32_t epochs_per_step, uint32_t producer_rows, float* x_out) {
    LV_ENTER(ctx);
    LV_REQUIRE(ctx->peer_ready, "peer windows are not connected");
    LV_REQUIRE(exchange >= 0 && uint32_t(exchange) < epochs_per_step, "exchange index out of range");
    LV_REQUIRE(producer_rows != 0 && producer_rows % 4 == 0, "producer rows must be a non-zero multiple of 4");
    LV_REQUIRE(x_out != nullptr && (reinterpret_cast<uintptr_t>(x_out) & 15u) == 0, "x_out null or not 16-byte aligned");
    ctx->tp_arm.pull = exchange;
    ctx->tp_arm.epochs_per_step = epochs_per_step;
    ctx->tp_arm.pull_rows = producer_rows;
    ctx->tp_arm.x_out = x_out;
    return LV_OK;
}

extern "C" int lv_peer_destroy(lv_ctx* ctx) {
    LV_ENTER(ctx);
    auto* st = static_cast<PeerState*>(ctx->peer);
    if (!st) return LV_OK;
    cudaStreamSynchronize(ctx->stream);
    for (void* p : st->opened) if (p) cudaIpcCloseMemHandle(p);
    cudaFree(st->own_window);
    cudaFree(st->d_epoch);
    delete st;
    ctx->peer = nullptr;
    ctx->peer_ready = false;
    return LV_OK;
}
