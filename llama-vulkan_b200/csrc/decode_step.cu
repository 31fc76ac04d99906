// One decoded token in ONE launch.
//
// Replaces the whole recorded command list of a single-token step of the reference
// (llava_command_buffer::record_execution, llava_command_buffer.cpp:29-45, which runs
// llava_layer::execute, llava_layer.cpp:39-75, for every layer and then the final normalisation and
// output matrix) by a persistent kernel: one CTA per SM, all CTAs resident together (cooperative
// launch), every CTA walking the same list of operations
//
//     embedding row;  per layer: QKV -> attention -> wo (+residual) -> gate/up (SiLU) -> w2 (+residual);
//     final norm + output head;  argmax + bookkeeping
//
// on its own share of the rows of each matrix.  What this buys over one kernel per operation:
//
//   * The weight stream never stops.  Every warp owns a two-stage shared-memory ring that it fills with
//     TMA loads of its work items (4 rows x 64 blocks); a warp that has finished its items of one
//     operation at once requests its first items of the NEXT operation -- weights depend on nothing --
//     so HBM keeps delivering while the CTA waits for the operation's input vector.
//   * Operations hand their results over through "flag-in-data" vectors in global memory (L2): every
//     element is an 8-byte word {value, epoch} written with one store, so a consumer that polls the
//     vector sees each element either old or complete and needs no fence, no flag and no second trip:
//     one L2 round trip from the last producer's store to every consumer having the data.  The epoch
//     is step * operations-per-step + operation + 1 and never repeats, so nothing is ever cleared.
//   * No grid-wide barrier and no kernel boundary between operations; the activation records of
//     an input vector are built while the first weights of the operation are already in shared memory.
//
// Arithmetic is that of the per-operation kernels (gemv_stream.cuh, attention.cu): activations as
// fixed-point digit records, exact int32 block sums (dp4a), fp32 row accumulation; attention with the
// reference's un-rotated f16 cache rotated by distance through the cos/sin table.
//
// Every wait is bounded (kWaitCycleLimit); a lost wait sets the context's error word, every CTA
// then leaves at its next wait, after letting its own outstanding copies land.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "ctx.h"
#include "gemv_stream.cuh"
#include "tmap.h"

namespace lv {

constexpr int kStepMaxLayers = 96;
constexpr int kStepNchMax = 4;              // attention chunks per head, at most
constexpr int kStepAttRec = 132;            // flag-in-data words of one (head, chunk) partial: 128 outputs, max, exp-sum, 2 unused
constexpr int kStepChunkRowsMax = 2048;     // rows of one attention chunk, at most
constexpr int kStepPartFloats = 2048;       // row-segment partial sums of one operation of one CTA
constexpr uint32_t kStepRot = 128;
constexpr int kStepMaxRanks = 8;
constexpr int kStepKeyBatch = 8;            // cache rows per warp whose loads are in flight together
constexpr int kStepValuePrefetch = 2;       // value rows per thread fetched before the scores

enum : int { OP_QKV = 0, OP_WO = 1, OP_GU = 2, OP_W2 = 3, OP_HEAD = 4 };

// One layer as the kernel sees it (device memory, copied to shared memory by every CTA).
// Matrices are addressed as row ranges of the tensor map of their row size: row0 = first row.
struct StepLayerDev {
    uint32_t row_k, row_q, row_v, row_o, row_3, row_1, row_2, pad;
    const uint8_t* w_k; const uint8_t* w_q; const uint8_t* w_v; const uint8_t* w_o;
    const uint8_t* w_3; const uint8_t* w_1; const uint8_t* w_2;
    const float* attn_norm; const float* ffn_norm;
    __half* k_cache; __half* v_cache;
    uint64_t pad2;
};
static_assert(sizeof(StepLayerDev) % 16 == 0, "the layer table is copied in 16-byte units");

// Tensor maps, one per (row size, box height):
//   [0] rows of dim columns, box of 4 rows      (wk, wq, wv, output)
//   [1] rows of dim columns, box of 2 rows      (w3 / w1: two rows of each per work item)
//   [2] rows of k_2 columns, box of 4 rows      (w2)
//   [3] rows of k_o columns, box of 4 rows      (wo; the same view as [0] on one GPU)
struct StepMaps { CUtensorMap m[4]; };

struct StepParams {
    // dim: length of the residual stream.  The rest is this rank's share (equal to the model's on one GPU): dq rows of
    // each of wq / wk / wv = width of its cache rows = heads * 128; ff rows of w1 / w3; k_o, k_2 columns of the wo / w2
    // shards (dq and ff padded with zero blocks to the shard's row length)
    uint32_t dim, dq, ff, heads, k_o, k_2, n_layers, vocab, ctx_rows;
    uint32_t row_bytes_d, row_bytes_f, row_bytes_o;     // bytes of a row of dim / k_2 / k_o columns
    // tensor parallelism: n_ranks > 1 -> wo and w2 produce partial rows that every rank sums.  xw[r]: the exchange
    // vectors in rank r's peer window as seen from this GPU, [2 sets][n_ranks senders][xw_stride words]
    int n_ranks, rank;
    uint64_t* xw[kStepMaxRanks];
    uint32_t xw_stride;
    const StepLayerDev* layers;
    const uint8_t* emb; int emb_type;
    const float* final_norm;
    const uint8_t* head_w; uint32_t head_row0;
    const float* rope;
    uint32_t* config; uint32_t* token_log; uint32_t log_capacity;
    float* logits; uint32_t* argmax_out; volatile uint32_t* host_token;
    uint64_t* x_ll;      // [2][dim]   residual stream after wo (0) and after w2 (1)
    uint64_t* qkv_ll;    // [3][dim]   k, q, v of the current token
    uint64_t* att_ll;    // [heads][kStepNchMax][kStepAttRec]
    uint64_t* g_ll;      // [ff]
    uint64_t* amax_ll;   // [grid][2]
    uint32_t* step;      // launches completed with this workspace
    uint32_t* err;
    uint32_t* tp_step;   // step counter of a peer window (sharded contexts), or null
    int with_head;
    unsigned long long* trace;   // null, or [operation][CTA][kStepTracePoints] nanosecond timestamps (lv_step_plan_set_trace)
};

constexpr int kStepTracePoints = 5;     // per operation: begin, attention done, records ready, items done, rows handed over

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ---- flag-in-data words -------------------------------------------------------------------------

__device__ __forceinline__ void ll_store(uint64_t* p, float v, uint32_t epoch) {
    const uint64_t w = (uint64_t(epoch) << 32) | uint64_t(__float_as_uint(v));
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}

// The same across NVLink: a peer's window is written with system-scope stores and read with system-scope loads.
__device__ __forceinline__ void ll_store_sys(uint64_t* p, float v, uint32_t epoch) {
    const uint64_t w = (uint64_t(epoch) << 32) | uint64_t(__float_as_uint(v));
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}

__device__ __forceinline__ bool ll_try4_sys(const uint64_t* __restrict__ buf, uint32_t e, uint32_t epoch, float4& out) {
    uint64_t a, b, c, d;
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(buf + e) : "memory");
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(c), "=l"(d) : "l"(buf + e + 2) : "memory");
    out = make_float4(__uint_as_float(uint32_t(a)), __uint_as_float(uint32_t(b)), __uint_as_float(uint32_t(c)), __uint_as_float(uint32_t(d)));
    return (uint32_t(a >> 32) == epoch) & (uint32_t(b >> 32) == epoch) & (uint32_t(c >> 32) == epoch) & (uint32_t(d >> 32) == epoch);
}

__device__ __forceinline__ void ll_store_u32(uint64_t* p, uint32_t v, uint32_t epoch) {
    const uint64_t w = (uint64_t(epoch) << 32) | uint64_t(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}

__device__ __forceinline__ void ll_load2(const uint64_t* p, uint64_t& a, uint64_t& b) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

// Words e .. e+3 (e a multiple of 4), fetched once; true when all four carry `epoch`.
__device__ __forceinline__ bool ll_try4(const uint64_t* __restrict__ buf, uint32_t e, uint32_t epoch, float4& out) {
    uint64_t a, b, c, d;
    ll_load2(buf + e, a, b);
    ll_load2(buf + e + 2, c, d);
    out = make_float4(__uint_as_float(uint32_t(a)), __uint_as_float(uint32_t(b)), __uint_as_float(uint32_t(c)), __uint_as_float(uint32_t(d)));
    return (uint32_t(a >> 32) == epoch) & (uint32_t(b >> 32) == epoch) & (uint32_t(c >> 32) == epoch) & (uint32_t(d >> 32) == epoch);
}

// Bounded polling: returns false (and records the failure) when the words do not arrive.
struct Poll {
    long long t0;
    uint32_t spins;
    uint32_t* err;
    __device__ __forceinline__ explicit Poll(uint32_t* e) : t0(0), spins(0), err(e) {}
    // call after a failed try; false = give up
    __device__ __forceinline__ bool again() {
        if (spins == 0) t0 = clock64();
        if ((++spins & 63u) == 0) {
            if (*reinterpret_cast<volatile uint32_t*>(err) != 0) return false;
            if (clock64() - t0 > kWaitCycleLimit) {
                atomicOr(err, ERR_GRID_BARRIER_TIMEOUT);
                return false;
            }
        }
        return true;
    }
};

__device__ __forceinline__ bool ll_wait4(const uint64_t* __restrict__ buf, uint32_t e, uint32_t epoch, float4& out, uint32_t* err) {
    if (ll_try4(buf, e, epoch, out)) return true;
    Poll poll(err);
    while (poll.again())
        if (ll_try4(buf, e, epoch, out)) return true;
    return false;
}

// Lets the outstanding copies of a warp's ring land (bounded), whatever the error word says.
__device__ __forceinline__ void mbar_drain(uint64_t* bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_test(bar, parity))
        if (clock64() - t0 > 20000000ll) break;
}

// emit_block_record out of line: the step kernel calls it from a dozen places and its code size matters more than a call
__device__ __noinline__ void emit_record(uint8_t* __restrict__ xrec, float4 v, uint32_t e, int lane) { emit_block_record(xrec, v, e, lane); }

// ---- geometry of one weight operation for this CTA -------------------------------------------------

struct OpGeo {
    uint32_t K, nb, nseg, n_items, cta_first, cta_groups, groups_per_mat;
    uint32_t row0[3];
    const uint8_t* w[3];
    uint32_t row_bytes;
    int kind;
};

// What a warp needs to request the items of one operation; one per warp in shared memory (the request cursor
// runs ahead of the operation the CTA is working on, and registers are short).
struct ReqGeo {
    uint32_t kind, nseg, nb, n_items, cta_first, groups_per_mat, row_bytes, pad;
    uint32_t row0[4];
    const uint8_t* w[4];
};
static_assert(sizeof(ReqGeo) == 80, "request geometry layout");

__device__ __forceinline__ OpGeo op_geo(const StepParams& p, const StepLayerDev* __restrict__ tab, uint32_t s) {
    OpGeo g;
    uint32_t groups;
    if (s >= 4u * p.n_layers) {
        g.kind = OP_HEAD;
        g.K = p.dim; g.row_bytes = p.row_bytes_d;
        g.row0[0] = p.head_row0; g.w[0] = p.head_w;
        groups = p.vocab / 4;
        g.groups_per_mat = groups;
    } else {
        const StepLayerDev& L = tab[s >> 2];
        g.kind = int(s & 3u);
        if (g.kind == OP_QKV) {
            g.K = p.dim; g.row_bytes = p.row_bytes_d;
            g.row0[0] = L.row_k; g.row0[1] = L.row_q; g.row0[2] = L.row_v;
            g.w[0] = L.w_k; g.w[1] = L.w_q; g.w[2] = L.w_v;
            g.groups_per_mat = p.dq / 4;
            groups = 3 * g.groups_per_mat;
        } else if (g.kind == OP_WO) {
            g.K = p.k_o; g.row_bytes = p.row_bytes_o;
            g.row0[0] = L.row_o; g.w[0] = L.w_o;
            groups = p.dim / 4;
            g.groups_per_mat = groups;
        } else if (g.kind == OP_GU) {
            g.K = p.dim; g.row_bytes = p.row_bytes_d;
            g.row0[0] = L.row_3; g.row0[1] = L.row_1;
            g.w[0] = L.w_3; g.w[1] = L.w_1;
            groups = p.ff / 2;                     // two rows of each of the two matrices per group
            g.groups_per_mat = groups;
        } else {
            g.K = p.k_2; g.row_bytes = p.row_bytes_f;
            g.row0[0] = L.row_2; g.w[0] = L.w_2;
            groups = p.dim / 4;
            g.groups_per_mat = groups;
        }
    }
    g.nb = g.K / 32;
    g.nseg = (g.nb + kSegBlocks - 1) / kSegBlocks;
    g.cta_first = uint32_t(uint64_t(groups) * blockIdx.x / gridDim.x);
    g.cta_groups = uint32_t(uint64_t(groups) * (blockIdx.x + 1) / gridDim.x) - g.cta_first;
    g.n_items = g.cta_groups * g.nseg;
    return g;
}

// Attention chunks per head at position P: a chunk per 64 rows up to kStepNchMax, and no more chunks than
// the grid has CTAs for.
__device__ __forceinline__ uint32_t att_chunks(uint32_t P, uint32_t heads) {
    uint32_t n = (P + 1 + 63) / 64;
    const uint32_t cap = min(uint32_t(kStepNchMax), max(1u, gridDim.x / heads));
    return min(max(n, 1u), cap);
}

// ---- the kernel ---------------------------------------------------------------------------------------

template <int QT>
struct StepSmem {
    static constexpr int kWarps = QTraits<QT>::kWarps;
    static constexpr size_t kStage = size_t(4) * kSegBlocks * QTraits<QT>::kBlockBytes;
    static constexpr size_t kRing = size_t(kWarps) * kStages * kStage;
    static constexpr size_t kBars = 512 + size_t(kWarps) * sizeof(ReqGeo), kScratch = 256, kPart = size_t(kStepPartFloats) * 4;
    static constexpr size_t kAttScratch = size_t(kStepChunkRowsMax) * 4 + 3 * 512 + size_t(kWarps) * 2 * kStepRot * 4 + 256;
    __host__ __device__ static size_t table_bytes(uint32_t n_layers) { return size_t(n_layers) * sizeof(StepLayerDev); }
    __host__ __device__ static size_t rec_bytes(uint32_t kmax) {
        const size_t r = size_t(kmax / 64) * kPairBytes;
        return (r > kAttScratch ? r : kAttScratch + 15) / 16 * 16;
    }
    __host__ __device__ static size_t total(uint32_t dim, uint32_t kmax, uint32_t n_layers) {
        return kRing + kBars + kScratch + kPart + size_t(dim) * 4 + rec_bytes(kmax) + table_bytes(n_layers);
    }
};

template <int QT, bool TMAP>
__global__ void __launch_bounds__(QTraits<QT>::kWarps * 32, 1) lv_decode_step_kernel(const StepParams p, const __grid_constant__ StepMaps maps) {
    using Q = QTraits<QT>;
    using S = StepSmem<QT>;
    constexpr int W = Q::kWarps;
    constexpr int NS = 4;
    constexpr int kStreamStride = kSegBlocks * Q::kBlockBytes;
    constexpr size_t kStage = S::kStage;
    constexpr int kThreads = W * 32;
    constexpr int kRowGroups = kThreads / 16;
    constexpr int kNormIters = (6144 + kThreads * 4 - 1) / (kThreads * 4);     // float4s per thread that cover a residual stream of up to 6144

    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kRing);
    float* scratch = reinterpret_cast<float*>(smem + S::kRing + S::kBars);
    float* part = reinterpret_cast<float*>(smem + S::kRing + S::kBars + S::kScratch);
    float* xres = reinterpret_cast<float*>(smem + S::kRing + S::kBars + S::kScratch + S::kPart);
    uint8_t* xrec = reinterpret_cast<uint8_t*>(xres + p.dim);
    const uint32_t kmax = max(p.dim, p.k_2);
    const StepLayerDev* tab = reinterpret_cast<const StepLayerDev*>(xrec + S::rec_bytes(kmax));

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t* my_ring = smem + size_t(warp) * kStages * kStage;
    uint64_t* my_bars = bars + warp * kStages;
    ReqGeo* rq = reinterpret_cast<ReqGeo*>(smem + S::kRing + 512) + warp;
    __shared__ uint32_t s_flag;
    __shared__ float s_x0[2];

    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&my_bars[s], 1);
        fence_mbar_init();
    }
    {   // the layer table: weights and caches of every layer
        const uint4* src = reinterpret_cast<const uint4*>(p.layers);
        uint4* dst = reinterpret_cast<uint4*>(const_cast<StepLayerDev*>(tab));
        for (uint32_t i = threadIdx.x; i < S::table_bytes(p.n_layers) / 16; i += kThreads) dst[i] = src[i];
    }
    if (threadIdx.x == 0) s_flag = 1;
    __syncthreads();

    const uint64_t policy = l2_policy_evict_first();
    const uint32_t n_wops = 4u * p.n_layers + (p.with_head ? 1u : 0u);      // operations that stream weights

    // ---- the warp's request cursor: runs two items ahead of its consume cursor, across operations ----
    uint32_t is = 0;                 // operation of the next request
    uint32_t ij = warp;              // item of the next request inside that operation
    uint32_t i_items;                // items of that operation for this CTA
    int islot = 0;
    uint32_t outstanding = 0;        // requests not yet consumed (0..2)

    auto load_req = [&](uint32_t s) {
        const OpGeo g = op_geo(p, tab, s);
        __syncwarp();
        if (lane == 0) {
            rq->kind = uint32_t(g.kind); rq->nseg = g.nseg; rq->nb = g.nb; rq->n_items = g.n_items; rq->cta_first = g.cta_first;
            rq->groups_per_mat = g.groups_per_mat; rq->row_bytes = g.row_bytes;
            rq->row0[0] = g.row0[0]; rq->row0[1] = g.kind == OP_QKV || g.kind == OP_GU ? g.row0[1] : 0u; rq->row0[2] = g.kind == OP_QKV ? g.row0[2] : 0u;
            rq->w[0] = g.w[0]; rq->w[1] = g.kind == OP_QKV || g.kind == OP_GU ? g.w[1] : nullptr; rq->w[2] = g.kind == OP_QKV ? g.w[2] : nullptr;
        }
        __syncwarp();
        return g.n_items;
    };
    i_items = load_req(0);

    auto request_next = [&]() {
        while (is < n_wops && ij >= i_items) {
            ++is;
            if (is < n_wops) i_items = load_req(is);
            ij = warp;
        }
        if (is >= n_wops) return;
        const uint32_t nseg = rq->nseg, kind = rq->kind;
        const uint32_t gl = ij / nseg, seg = ij - gl * nseg;
        const uint32_t gg = rq->cta_first + gl;
        uint8_t* dst = my_ring + islot * kStage;
        uint64_t* bar = &my_bars[islot];
        if constexpr (TMAP) {
            if (lane == 0) {
                const int x = int(seg * (kStreamStride / 8));
                mbar_expect_tx(bar, NS * kStreamStride);                    // whole boxes, zero fill included
                if (kind == OP_GU) {
                    const int y = int(gg * 2);
                    tma_load_2d(dst, &maps.m[1], x, int(rq->row0[0]) + y, bar, policy);
                    tma_load_2d(dst + 2 * kStreamStride, &maps.m[1], x, int(rq->row0[1]) + y, bar, policy);
                } else {
                    const uint32_t gpm = rq->groups_per_mat;
                    const uint32_t m = kind == OP_QKV ? gg / gpm : 0u;
                    const int y = int(rq->row0[m] + (gg - m * gpm) * 4);
                    if (kind == OP_W2) tma_load_2d(dst, &maps.m[2], x, y, bar, policy);
                    else if (kind == OP_WO) tma_load_2d(dst, &maps.m[3], x, y, bar, policy);
                    else tma_load_2d(dst, &maps.m[0], x, y, bar, policy);
                }
            }
        } else {
            const uint32_t segblocks = min(uint32_t(kSegBlocks), rq->nb - seg * kSegBlocks);
            const uint32_t bytes = segblocks * Q::kBlockBytes;
            if (lane == 0) mbar_expect_tx(bar, NS * bytes);
            __syncwarp();
            if (lane < NS) {
                const uint8_t* base;
                uint32_t row;
                if (kind == OP_GU) {
                    base = rq->w[lane >> 1];
                    row = gg * 2 + (lane & 1);
                } else {
                    const uint32_t gpm = rq->groups_per_mat;
                    const uint32_t m = kind == OP_QKV ? gg / gpm : 0u;
                    base = rq->w[m];
                    row = (gg - m * gpm) * 4 + lane;
                }
                bulk_g2s_stream(dst + lane * kStreamStride, base + size_t(row) * rq->row_bytes + size_t(seg) * kStreamStride, bytes, bar, policy);
            }
        }
        ij += W;
        islot ^= 1;
        ++outstanding;
    };
    request_next();
    request_next();

    int cslot = 0;
    uint32_t cparity = 0;
    bool ok = true;

    // leaves the kernel after a lost wait: the warp's own copies in flight land first
    auto drain = [&]() {
        for (uint32_t k = 0; k < outstanding; ++k) {
            mbar_drain(&my_bars[cslot], cparity);
            cslot ^= 1;
            cparity ^= uint32_t(cslot == 0);
        }
        outstanding = 0;
    };

    // ---- this step ----------------------------------------------------------------------------
    pdl_wait();
    const uint32_t step = *p.step;
    const uint32_t epochs_per_step = 5u * p.n_layers + 2u;
    const uint32_t epoch0 = step * epochs_per_step + 1u;         // + index of the producing operation
    const uint32_t P = p.config[0];
    uint32_t token = (P < p.log_capacity) ? p.token_log[P] : 0u;
    if (P >= p.ctx_rows || P >= p.log_capacity || token >= p.vocab) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(p.err, ERR_BAD_INDEX);
        ok = false;
    }
    if (*reinterpret_cast<volatile uint32_t*>(p.err) != 0) ok = false;
    if (!ok) { drain(); return; }

    // embedding row of the token -> residual stream (llava_session.cpp:219-223, llava_buffer.cpp:360-394)
    {
        const uint32_t nbk = p.dim / 32;
        if (p.emb_type == T_F32) {
            const float* src = reinterpret_cast<const float*>(p.emb) + size_t(token) * p.dim;
            for (uint32_t i = threadIdx.x; i < p.dim; i += kThreads) xres[i] = src[i];
        } else {
            const uint32_t bb = p.emb_type == T_Q4_0 ? kQ4BlockBytes : kQ8BlockBytes;
            const uint8_t* row = p.emb + size_t(token) * nbk * bb;
            for (uint32_t b = threadIdx.x; b < nbk; b += kThreads) {
                const uint8_t* blk = row + size_t(b) * bb;
                const float d = half_bits_to_float(uint32_t(blk[0]) | (uint32_t(blk[1]) << 8));
                if (p.emb_type == T_Q4_0) {
                    for (int j = 0; j < 16; ++j) {
                        const int qv = blk[2 + j];
                        xres[b * 32 + j] = static_cast<float>((qv & 0xf) - 8) * d;
                        xres[b * 32 + j + 16] = static_cast<float>((qv >> 4) - 8) * d;
                    }
                } else {
                    for (int j = 0; j < 32; ++j) xres[b * 32 + j] = static_cast<float>(static_cast<int8_t>(blk[2 + j])) * d;
                }
            }
        }
    }
    __syncthreads();

    uint32_t norm_count = 0;                 // normalised inputs staged so far (selects the entry of s_x0)
    if (threadIdx.x == 0) { s_x0[0] = xres[0]; s_x0[1] = xres[0]; }
    __syncthreads();
    const uint32_t nch = att_chunks(P, p.heads);
    const float att_scale = rsqrtf(float(kStepRot));

    for (uint32_t s = 0; s < n_wops && ok; ++s) {
        const OpGeo g = op_geo(p, tab, s);
        const uint32_t layer = s >> 2;
        const StepLayerDev& L = tab[min(layer, p.n_layers - 1)];
        // index of this operation among the step's producers: layer * 5 + {QKV 0, attention 1, wo 2, gate/up 3, w2 4}; head = 5 n_layers
        const uint32_t prod = g.kind == OP_HEAD ? 5u * p.n_layers : layer * 5u + (g.kind == OP_QKV ? 0u : uint32_t(g.kind) + 1u);
        const uint32_t my_epoch = epoch0 + prod;
        unsigned long long* tr = (p.trace != nullptr && threadIdx.x == 0) ? p.trace + (size_t(s) * gridDim.x + blockIdx.x) * kStepTracePoints : nullptr;
        if (tr) tr[0] = global_ns();

        // ================= attention of this layer (before wo): CTAs that own a (head, chunk) unit =================
        if (g.kind == OP_WO) {
            const uint32_t att_epoch = epoch0 + layer * 5u + 1u, qkv_epoch = epoch0 + layer * 5u;
            float* s_e = reinterpret_cast<float*>(xrec);                               // [chunk rows] scores, then exponentials
            float* s_q = s_e + kStepChunkRowsMax;                                       // [128] query of the head
            float* s_k = s_q + kStepRot;                                                // [128] new key row, rounded to half
            float* s_v = s_k + kStepRot;                                                // [128] new value row, rounded to half
            float* s_red = s_v + kStepRot;                                              // [W*2][128] partial outputs
            float* s_l = s_red + size_t(kRowGroups) * kStepRot;                         // [W*2] partial exp-sums
            for (uint32_t u = blockIdx.x; u < p.heads * nch && ok; u += gridDim.x) {
                const uint32_t h = u / nch, c = u - h * nch;
                const uint32_t csz = (P + 1 + nch - 1) / nch;
                const uint32_t p0 = c * csz;
                const uint32_t n = min(csz, P + 1 - p0);                                // rows p0 .. p0+n-1, all <= P
                const bool has_new = p0 + n - 1 == P;                                   // the chunk ends with the row of this token
                const uint32_t n_old = has_new ? n - 1 : n;                             // rows that come from the cache
                const __half* kc = L.k_cache + size_t(h) * kStepRot;
                const __half* vc = L.v_cache + size_t(h) * kStepRot;
                // value rows do not depend on this layer's QKV product: fetch the first ones now
                const int d8 = (threadIdx.x & 15) * 8, rg = threadIdx.x >> 4;
                uint4 vpre[kStepValuePrefetch];
#pragma unroll
                for (int j = 0; j < kStepValuePrefetch; ++j) {
                    const uint32_t i = rg + kRowGroups * j;
                    vpre[j] = i < n_old ? *reinterpret_cast<const uint4*>(vc + size_t(p0 + i) * p.dq + d8) : make_uint4(0, 0, 0, 0);
                }
                // q, and the new k and v rows, of this head from the QKV operation (order k, q, v)
                if (threadIdx.x < 96) {
                    const uint32_t which = threadIdx.x >> 5, e4 = (threadIdx.x & 31) * 4;
                    float4 v;
                    if (!ll_wait4(p.qkv_ll, which * p.dq + h * kStepRot + e4, qkv_epoch, v, p.err)) s_flag = 0;
                    if (which != 1) {      // the cache holds halves (copy_to_cache.comp:35): attention sees the rounded row
                        v.x = __half2float(__float2half_rn(v.x)); v.y = __half2float(__float2half_rn(v.y));
                        v.z = __half2float(__float2half_rn(v.z)); v.w = __half2float(__float2half_rn(v.w));
                    }
                    float* dst = which == 0 ? s_k : which == 1 ? s_q : s_v;
                    *reinterpret_cast<float4*>(dst + e4) = v;
                }
                __syncthreads();
                if (s_flag == 0) { ok = false; break; }
                // ---- scores (mhsa.comp:42-57): warp w takes rows w, w + W, ...; a lane owns two (even, odd) pairs ----
                const float4 q4 = *reinterpret_cast<const float4*>(s_q + 4 * lane);
                for (uint32_t i0 = warp; i0 < n; i0 += W * kStepKeyBatch) {
                    uint2 kraw[kStepKeyBatch];
                    float4 cs[kStepKeyBatch];
#pragma unroll
                    for (int b = 0; b < kStepKeyBatch; ++b) {
                        const uint32_t i = i0 + b * W;
                        if (i < n_old) {
                            kraw[b] = *reinterpret_cast<const uint2*>(kc + size_t(p0 + i) * p.dq + 4 * lane);
                            cs[b] = *reinterpret_cast<const float4*>(p.rope + size_t(P - (p0 + i)) * kStepRot + 4 * lane);
                        }
                    }
#pragma unroll
                    for (int b = 0; b < kStepKeyBatch; ++b) {
                        const uint32_t i = i0 + b * W;
                        if (i >= n) break;
                        float2 k01, k23;
                        float4 t;
                        if (i < n_old) {
                            k01 = __half22float2(*reinterpret_cast<const __half2*>(&kraw[b].x));
                            k23 = __half22float2(*reinterpret_cast<const __half2*>(&kraw[b].y));
                            t = cs[b];
                        } else {            // the row of this token: distance 0, cos 1, sin 0
                            const float4 kn = *reinterpret_cast<const float4*>(s_k + 4 * lane);
                            k01 = make_float2(kn.x, kn.y);
                            k23 = make_float2(kn.z, kn.w);
                            t = *reinterpret_cast<const float4*>(p.rope + 4 * lane);
                        }
                        const float rx0 = t.x * k01.x + t.y * k01.y, ry0 = -t.y * k01.x + t.x * k01.y;
                        const float rx1 = t.z * k23.x + t.w * k23.y, ry1 = -t.w * k23.x + t.z * k23.y;
                        float sc = q4.x * rx0 + q4.y * ry0;
                        sc += q4.z * rx1 + q4.w * ry1;
                        sc = warp_sum(sc);
                        if (lane == 0) s_e[i] = sc * att_scale;
                    }
                }
                __syncthreads();
                // ---- chunk maximum (every warp on its own), exponentials, weighted values (softmax.comp, kqv_matching.comp) ----
                float m = -INFINITY;
                for (uint32_t i = lane; i < n; i += 32) m = fmaxf(m, s_e[i]);
                m = warp_max(m);
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                float lsum = 0.f;
                auto add_row = [&](const uint4& raw, float e) {
                    const __half2* v2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 f = __half22float2(v2[k]);
                        acc[2 * k] = fmaf(f.x, e, acc[2 * k]);
                        acc[2 * k + 1] = fmaf(f.y, e, acc[2 * k + 1]);
                    }
                };
#pragma unroll
                for (int j = 0; j < kStepValuePrefetch; ++j) {
                    const uint32_t i = rg + kRowGroups * j;
                    if (i < n_old) {
                        const float e = __expf(s_e[i] - m);
                        lsum += e;
                        add_row(vpre[j], e);
                    }
                }
                for (uint32_t i = rg + kRowGroups * kStepValuePrefetch; i < n_old; i += kRowGroups) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(vc + size_t(p0 + i) * p.dq + d8);
                    const float e = __expf(s_e[i] - m);
                    lsum += e;
                    add_row(raw, e);
                }
                if (has_new && rg == int((n - 1) % kRowGroups)) {                       // the row of this token, from shared memory
                    const float e = __expf(s_e[n - 1] - m);
                    lsum += e;
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[k] = fmaf(s_v[d8 + k], e, acc[k]);
                }
                *reinterpret_cast<float4*>(&s_red[rg * kStepRot + d8]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                *reinterpret_cast<float4*>(&s_red[rg * kStepRot + d8 + 4]) = make_float4(acc[4], acc[5], acc[6], acc[7]);
                if ((threadIdx.x & 15) == 0) s_l[rg] = lsum;
                __syncthreads();
                uint64_t* rec = p.att_ll + (size_t(h) * kStepNchMax + c) * kStepAttRec;
                if (threadIdx.x < kStepRot) {
                    float o = 0.f, l = 0.f;
                    for (int r = 0; r < kRowGroups; ++r) {
                        o += s_red[r * kStepRot + threadIdx.x];
                        l += s_l[r];
                    }
                    ll_store(rec + threadIdx.x, o, att_epoch);
                    if (threadIdx.x == 0) {           // words 128 .. 131 travel together: maximum, exp-sum, two unused
                        ll_store(rec + kStepRot, m, att_epoch);
                        ll_store(rec + kStepRot + 1, l, att_epoch);
                        ll_store(rec + kStepRot + 2, 0.f, att_epoch);
                        ll_store(rec + kStepRot + 3, 0.f, att_epoch);
                    }
                }
                __syncthreads();              // the scratch is reused by the next unit / by the records
            }
            if (!ok) break;
        }
        if (tr) tr[1] = global_ns();

        // ================= input vector -> activation records =================
        if (g.kind == OP_QKV || g.kind == OP_GU || g.kind == OP_HEAD) {
            // The input is the residual stream (length dim, kept in xres) and is normalised: normalize.comp:39-63 split
            // as in stage_activations -- records hold x * w, rsqrt(var) multiplies the finished rows.  The norm weights
            // are requested first: they depend on nothing and arrive while the vector is being polled.
            const uint32_t K = p.dim;
            const float* norm_w = g.kind == OP_QKV ? L.attn_norm : g.kind == OP_GU ? L.ffn_norm : p.final_norm;
            const bool from_smem = g.kind == OP_QKV && layer == 0;                  // the embedding row is in xres already
            const uint64_t* src = g.kind == OP_GU ? p.x_ll : p.x_ll + p.dim;       // after wo / after w2
            const uint32_t src_epoch = g.kind == OP_GU     ? epoch0 + layer * 5u + 2u
                                       : g.kind == OP_HEAD ? epoch0 + (p.n_layers - 1) * 5u + 4u
                                                           : epoch0 + (layer - 1) * 5u + 4u;
            float4 v[kNormIters], w[kNormIters];
            float x0;
            bool mine = true;
#pragma unroll
            for (int i = 0; i < kNormIters; ++i) {
                const uint32_t e = uint32_t(i) * (kThreads * 4) + threadIdx.x * 4;
                w[i] = e < K ? *reinterpret_cast<const float4*>(norm_w + e) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if (from_smem) {
#pragma unroll
                for (int i = 0; i < kNormIters; ++i) {
                    const uint32_t e = uint32_t(i) * (kThreads * 4) + threadIdx.x * 4;
                    v[i] = e < K ? *reinterpret_cast<const float4*>(xres + e) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                x0 = xres[0];
            } else if (p.n_ranks > 1) {
                // input = residual + the partial rows of every rank, added in rank order (the same bits on every rank).
                // The partials arrive in this rank's window: set 0 after wo, set 1 after w2.  One float4 of the vector at
                // a time, the words of all ranks in flight together.
                const uint64_t* base = p.xw[p.rank] + size_t(g.kind == OP_GU ? 0u : 1u) * p.n_ranks * p.xw_stride;
                x0 = s_x0[norm_count & 1u];            // a shift near the data, the same on every thread: the residual's first element one operation ago
#pragma unroll
                for (int i = 0; i < kNormIters; ++i) {
                    const uint32_t e = uint32_t(i) * (kThreads * 4) + threadIdx.x * 4;
                    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (e >= K || !mine) continue;
                    float4 t[kStepMaxRanks];
                    uint32_t pending = (1u << p.n_ranks) - 1u;
                    Poll poll(p.err);
                    for (;;) {
#pragma unroll
                        for (int r = 0; r < kStepMaxRanks; ++r)
                            if ((pending >> r) & 1u)
                                if (ll_try4_sys(base + size_t(r) * p.xw_stride, e, src_epoch, t[r])) pending &= ~(1u << r);
                        if (pending == 0) break;
                        if (!poll.again()) { mine = false; break; }
                    }
                    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int r = 0; r < kStepMaxRanks; ++r)
                        if (r < p.n_ranks) { sum.x += t[r].x; sum.y += t[r].y; sum.z += t[r].z; sum.w += t[r].w; }
                    const float4 old = *reinterpret_cast<const float4*>(xres + e);
                    v[i] = make_float4(old.x + sum.x, old.y + sum.y, old.z + sum.z, old.w + sum.w);
                    *reinterpret_cast<float4*>(xres + e) = v[i];
                    if (e == 0) s_x0[(norm_count + 1u) & 1u] = v[i].x;
                }
            } else {
                // every word of the thread is requested before any is examined; stragglers are polled again
                uint32_t pending = 0;
                float4 first;
                if (!ll_try4(src, 0, src_epoch, first)) pending |= 1u << kNormIters;
#pragma unroll
                for (int i = 0; i < kNormIters; ++i) {
                    const uint32_t e = uint32_t(i) * (kThreads * 4) + threadIdx.x * 4;
                    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (e < K && !ll_try4(src, e, src_epoch, v[i])) pending |= 1u << i;
                }
                if (pending != 0) {
                    Poll poll(p.err);
                    while (pending != 0) {
                        if (!poll.again()) { mine = false; break; }
                        if ((pending >> kNormIters) && ll_try4(src, 0, src_epoch, first)) pending &= ~(1u << kNormIters);
#pragma unroll
                        for (int i = 0; i < kNormIters; ++i) {
                            if (pending & (1u << i)) {
                                const uint32_t e = uint32_t(i) * (kThreads * 4) + threadIdx.x * 4;
                                if (ll_try4(src, e, src_epoch, v[i])) pending &= ~(1u << i);
                            }
                        }
                    }
                }
                x0 = first.x;
#pragma unroll
                for (int i = 0; i < kNormIters; ++i) {
                    const uint32_t e = uint32_t(i) * (kThreads * 4) + threadIdx.x * 4;
                    if (e < K) *reinterpret_cast<float4*>(xres + e) = v[i];
                }
            }
            float s1 = 0.f, s2 = 0.f;
#pragma unroll
            for (int i = 0; i < kNormIters; ++i)
                if (uint32_t(i) * (kThreads * 4) + threadIdx.x * 4 < K) norm_accumulate(v[i], x0, s1, s2);
            norm_publish(s1, s2, scratch);
#pragma unroll
            for (int i = 0; i < kNormIters; ++i) {
                const uint32_t e = uint32_t(i) * (kThreads * 4) + threadIdx.x * 4;
                if (e >= K) break;              // whole warps leave together: dim is a multiple of 128
                emit_record(xrec, make_float4(v[i].x * w[i].x, v[i].y * w[i].y, v[i].z * w[i].z, v[i].w * w[i].w), e, lane);
            }
            if (!mine) s_flag = 0;
            ++norm_count;
        } else if (g.kind == OP_WO) {
            // attention output of element e: the chunks of its head combined (the last step of flash decoding)
            const uint32_t att_epoch = epoch0 + layer * 5u + 1u;
            bool mine = true;
            for (uint32_t e = threadIdx.x * 4; e < p.k_o; e += kThreads * 4) {
                if (e >= p.dq) {                 // columns that pad the shard's rows: zero weights, zero records
                    emit_record(xrec, make_float4(0.f, 0.f, 0.f, 0.f), e, lane);
                    continue;
                }
                const uint32_t h = e / kStepRot, j = e - h * kStepRot;
                const uint64_t* rec = p.att_ll + size_t(h) * kStepNchMax * kStepAttRec;
                float4 o[kStepNchMax];
                float mc[kStepNchMax], lc[kStepNchMax];
                float M = -INFINITY;
#pragma unroll
                for (uint32_t c = 0; c < uint32_t(kStepNchMax); ++c) {
                    o[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                    mc[c] = -INFINITY; lc[c] = 0.f;
                    if (c < nch && mine) {
                        float4 ml;
                        if (!ll_wait4(rec + c * kStepAttRec + j, 0, att_epoch, o[c], p.err) ||
                            !ll_wait4(rec + c * kStepAttRec + kStepRot, 0, att_epoch, ml, p.err)) {
                            mine = false;
                        } else {
                            mc[c] = ml.x; lc[c] = ml.y;
                            M = fmaxf(M, ml.x);
                        }
                    }
                }
                float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
                float den = 0.f;
#pragma unroll
                for (uint32_t c = 0; c < uint32_t(kStepNchMax); ++c) {
                    if (c < nch) {
                        const float wgt = nch == 1 ? 1.0f : __expf(mc[c] - M);
                        num.x = fmaf(o[c].x, wgt, num.x); num.y = fmaf(o[c].y, wgt, num.y);
                        num.z = fmaf(o[c].z, wgt, num.z); num.w = fmaf(o[c].w, wgt, num.w);
                        den = fmaf(lc[c], wgt, den);
                    }
                }
                const float rden = 1.0f / den;
                emit_record(xrec, make_float4(num.x * rden, num.y * rden, num.z * rden, num.w * rden), e, lane);
            }
            if (!mine) s_flag = 0;
        } else {
            // w2: the gated activations of the whole FFN width
            const uint32_t K = p.k_2, Kin = p.ff;       // columns of the shard; those beyond the FFN rows of this rank are padding
            const uint32_t src_epoch = epoch0 + layer * 5u + 3u;
            bool mine = true;
            for (uint32_t chunk = 0; chunk < K; chunk += kThreads * 4 * kActIters) {
                float4 v[kActIters];
                uint32_t pending = 0;
#pragma unroll
                for (int i = 0; i < kActIters; ++i) {
                    const uint32_t e = chunk + uint32_t(i) * (kThreads * 4) + threadIdx.x * 4;
                    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (e < Kin && !ll_try4(p.g_ll, e, src_epoch, v[i])) pending |= 1u << i;
                }
                if (pending != 0) {
                    Poll poll(p.err);
                    while (pending != 0) {
                        if (!poll.again()) { mine = false; break; }
#pragma unroll
                        for (int i = 0; i < kActIters; ++i) {
                            if (pending & (1u << i)) {
                                const uint32_t e = chunk + uint32_t(i) * (kThreads * 4) + threadIdx.x * 4;
                                if (ll_try4(p.g_ll, e, src_epoch, v[i])) pending &= ~(1u << i);
                            }
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < kActIters; ++i) {
                    const uint32_t e = chunk + uint32_t(i) * (kThreads * 4) + threadIdx.x * 4;
                    if (e >= K) break;              // whole warps leave together: ff is a multiple of 128
                    emit_record(xrec, v[i], e, lane);
                }
            }
            if (!mine) s_flag = 0;
        }
        __syncthreads();
        if (s_flag == 0) { ok = false; break; }
        if (tr) tr[2] = global_ns();

        // ================= this warp's items of the operation =================
        for (uint32_t cj = warp; cj < g.n_items; cj += W) {
            if (!mbar_wait(&my_bars[cslot], cparity, p.err)) { ok = false; break; }
            const uint32_t gl = cj / g.nseg, seg = cj - gl * g.nseg;
            const uint32_t segblocks = min(uint32_t(kSegBlocks), g.nb - seg * kSegBlocks);
            const uint8_t* stage = my_ring + cslot * kStage;
            float acc[NS];
#pragma unroll
            for (int i = 0; i < NS; ++i) acc[i] = 0.f;
            if (uint32_t(lane) * 2 < segblocks) {
                PairX px;
                load_pair_x(px, xrec + size_t(seg * (kSegBlocks / 2) + lane) * kPairBytes);
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                    const uint32_t* sw = reinterpret_cast<const uint32_t*>(stage + i * kStreamStride) + lane * Q::kPairWords;
                    acc[i] = dot_pair<QT>(sw, px);
                }
            }
            __syncwarp();
            --outstanding;
            cslot ^= 1;
            cparity ^= uint32_t(cslot == 0);
            request_next();                       // refills the stage just read, possibly with an item of a later operation
            const float u = warp_sum4(acc[0], acc[1], acc[2], acc[3], lane);
            if ((lane & 7) == 0) part[size_t(cj) * NS + (lane >> 3)] = u;
        }
        if (!__syncthreads_and(ok)) { ok = false; break; }
        if (tr) tr[3] = global_ns();

        // ================= one thread per row: segments added in order, epilogue, hand-over =================
        {
            const uint32_t rows_per_group = g.kind == OP_GU ? 2u : 4u;
            const uint32_t n_rows = g.cta_groups * rows_per_group;
            const bool normed = g.kind == OP_QKV || g.kind == OP_GU || g.kind == OP_HEAD;
            const float factor = (normed && threadIdx.x < n_rows) ? norm_factor(scratch, g.K) : 1.0f;
            float best = 0.f;
            uint32_t best_i = 0xffffffffu;
            for (uint32_t t = threadIdx.x; t < n_rows; t += kThreads) {
                const uint32_t gl = t / rows_per_group, rr = t - gl * rows_per_group;
                const float* srcp = part + size_t(gl) * g.nseg * NS;
                const uint32_t gg = g.cta_first + gl;
                if (g.kind == OP_GU) {
                    float up = 0.f, gate = 0.f;
                    for (uint32_t sg = 0; sg < g.nseg; ++sg) {
                        up += srcp[sg * NS + rr];
                        gate += srcp[sg * NS + rr + 2];
                    }
                    up *= factor;
                    gate *= factor;
                    ll_store(p.g_ll + gg * 2 + rr, up * gate / (__expf(-gate) + 1.0f), my_epoch);      // matmul_silu_ff.comp:95
                    continue;
                }
                float v = 0.f;
                for (uint32_t sg = 0; sg < g.nseg; ++sg) v += srcp[sg * NS + rr];
                v *= factor;
                if (g.kind == OP_QKV) {
                    const uint32_t m = gg / g.groups_per_mat, row = (gg - m * g.groups_per_mat) * 4 + rr;
                    ll_store(p.qkv_ll + m * p.dq + row, v, my_epoch);
                    if (m != 1) {                                                                      // copy_to_cache.comp:35
                        __half* cache = m == 0 ? L.k_cache : L.v_cache;
                        cache[size_t(P) * p.dq + row] = __float2half_rn(v);
                    }
                } else if (g.kind == OP_WO) {
                    const uint32_t row = gg * 4 + rr;
                    if (p.n_ranks > 1) {
                        for (int r = 0; r < p.n_ranks; ++r) ll_store_sys(p.xw[r] + size_t(p.rank) * p.xw_stride + row, v, my_epoch);
                    } else {
                        ll_store(p.x_ll + row, xres[row] + v, my_epoch);                               // matmul.glsl:68-70
                    }
                } else if (g.kind == OP_W2) {
                    const uint32_t row = gg * 4 + rr;
                    if (p.n_ranks > 1) {
                        for (int r = 0; r < p.n_ranks; ++r)
                            ll_store_sys(p.xw[r] + (size_t(p.n_ranks) + p.rank) * p.xw_stride + row, v, my_epoch);
                    } else {
                        ll_store(p.x_ll + p.dim + row, xres[row] + v, my_epoch);
                    }
                } else {
                    const uint32_t row = gg * 4 + rr;
                    p.logits[row] = v;
                    if (v == v && (best_i == 0xffffffffu || v > best)) { best = v; best_i = row; }     // rows ascend: a tie keeps the lower index
                }
            }
            if (g.kind == OP_HEAD) {
                // first index of the maximum over this CTA's rows (NaN never wins), handed to CTA 0
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                    const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
                    if (oi != 0xffffffffu && (best_i == 0xffffffffu || ov > best || (ov == best && oi < best_i))) { best = ov; best_i = oi; }
                }
                float* s_val = scratch;
                uint32_t* s_idx = reinterpret_cast<uint32_t*>(scratch + 32);
                __syncthreads();
                if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
                __syncthreads();
                if (threadIdx.x == 0) {
                    for (int w2 = 1; w2 < W; ++w2) {
                        const float ov = s_val[w2];
                        const uint32_t oi = s_idx[w2];
                        if (oi != 0xffffffffu && (best_i == 0xffffffffu || ov > best || (ov == best && oi < best_i))) { best = ov; best_i = oi; }
                    }
                    ll_store(p.amax_ll + size_t(blockIdx.x) * 2, best, my_epoch);
                    ll_store_u32(p.amax_ll + size_t(blockIdx.x) * 2 + 1, best_i, my_epoch);
                }
            }
            __syncthreads();          // partials, scratch and records are rewritten by the next operation
        }
        if (tr) tr[4] = global_ns();
    }

    if (!ok) { drain(); return; }

    // ================= bookkeeping of the step: CTA 0 =================
    if (blockIdx.x == 0) {
        uint32_t token_out = 0;
        if (p.with_head) {
            const uint32_t head_epoch = epoch0 + 5u * p.n_layers;
            float best = 0.f;
            uint32_t best_i = 0xffffffffu;
            bool mine = true;
            // CTA order is row order, so a tie keeps the lower index (llava_session.cpp:145-151)
            for (uint32_t c = threadIdx.x; c < gridDim.x && mine; c += kThreads) {
                uint64_t a, b;
                Poll poll(p.err);
                for (;;) {
                    ll_load2(p.amax_ll + size_t(c) * 2, a, b);
                    if (uint32_t(a >> 32) == head_epoch && uint32_t(b >> 32) == head_epoch) break;
                    if (!poll.again()) { mine = false; break; }
                }
                if (!mine) break;
                const float ov = __uint_as_float(uint32_t(a));
                const uint32_t oi = uint32_t(b);
                if (oi != 0xffffffffu && (best_i == 0xffffffffu || ov > best || (ov == best && oi < best_i))) { best = ov; best_i = oi; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
                if (oi != 0xffffffffu && (best_i == 0xffffffffu || ov > best || (ov == best && oi < best_i))) { best = ov; best_i = oi; }
            }
            float* s_val = scratch;
            uint32_t* s_idx = reinterpret_cast<uint32_t*>(scratch + 32);
            if (!mine) s_flag = 0;
            if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
            __syncthreads();
            if (s_flag == 0) return;
            if (threadIdx.x == 0) {
                for (int w2 = 1; w2 < W; ++w2) {
                    const float ov = s_val[w2];
                    const uint32_t oi = s_idx[w2];
                    if (oi != 0xffffffffu && (best_i == 0xffffffffu || ov > best || (ov == best && oi < best_i))) { best = ov; best_i = oi; }
                }
                // the reference's scan returns 0 when nothing improves on element 0, which includes a NaN there
                const float first = p.logits[0];          // written by this CTA (row 0 is its own)
                token_out = (best_i == 0xffffffffu || first != first) ? 0u : best_i;
            }
        }
        if (threadIdx.x == 0) {
            if (p.with_head) {
                const uint32_t at = P + 1;
                if (at < p.log_capacity) p.token_log[at] = token_out;
                else atomicOr(p.err, ERR_BAD_INDEX);
                if (p.argmax_out != nullptr) *p.argmax_out = token_out;
            }
            for (int i = 0; i < 4; ++i) p.config[i] = P + 1;                         // llava_session.cpp:224-225
            *p.step = step + 1;
            if (p.tp_step != nullptr) *p.tp_step += 1;
            if (p.with_head && p.host_token != nullptr) {
                *p.host_token = token_out;
                __threadfence_system();
            }
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------------

int make_weight_map(CUtensorMap* out, const void* base, uint32_t rows, uint32_t row_bytes, uint32_t box_rows, uint32_t seg_bytes);

}  // namespace lv

using namespace lv;

struct lv_step_plan {
    lv_ctx* ctx = nullptr;
    StepParams params{};
    StepMaps maps{};
    int wtype = 0;
    bool tmap = false;
    size_t smem = 0;
    int grid = 0;
    void* d_layers = nullptr;
    void* d_ws = nullptr;
    void* d_trace = nullptr;
    size_t trace_words = 0;
};

// The dynamic shared memory a kernel may ask for is the opt-in limit less its static shared memory.
template <int QT, bool TMAP>
static int step_configure_one(lv_ctx* ctx, size_t need) {
    cudaFuncAttributes fa{};
    LV_CUDA(cudaFuncGetAttributes(&fa, lv_decode_step_kernel<QT, TMAP>));
    const size_t room = size_t(ctx->max_smem_optin) - fa.sharedSizeBytes;
    if (need > room) return fail(LV_ERR_BAD_ARGUMENTS, "lv_step_plan_create: the model needs " + std::to_string(need) + " bytes of shared memory per CTA, " + std::to_string(room) + " are available");
    LV_CUDA(cudaFuncSetAttribute(lv_decode_step_kernel<QT, TMAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(room)));
    return LV_OK;
}

template <int QT>
static int step_configure(lv_ctx* ctx, size_t need) {
    if (int rc = step_configure_one<QT, true>(ctx, need)) return rc;
    return step_configure_one<QT, false>(ctx, need);
}

template <int QT, bool TMAP>
static int step_launch(const lv_step_plan* plan, const StepParams& p) {
    lv_ctx* ctx = plan->ctx;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(plan->grid);
    cfg.blockDim = dim3(QTraits<QT>::kWarps * 32);
    cfg.dynamicSmemBytes = plan->smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;          // all CTAs resident together, or the launch fails
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, lv_decode_step_kernel<QT, TMAP>, p, plan->maps);
    if (e == cudaErrorNotSupported || e == cudaErrorInvalidValue) {
        // a stream capture that refuses the cooperative attribute: one CTA per SM on a GPU of its own is resident
        // together anyway, and every wait in the kernel is bounded
        (void)cudaGetLastError();
        cfg.numAttrs = 0;
        e = cudaLaunchKernelEx(&cfg, lv_decode_step_kernel<QT, TMAP>, p, plan->maps);
    }
    if (e != cudaSuccess) return cuda_fail(e, "lv_decode_step launch");
    return LV_OK;
}

extern "C" int lv_step_plan_create(lv_ctx* ctx, const lv_step_model* m, lv_step_plan** out) {
    LV_ENTER(ctx);
    LV_REQUIRE(m && out && m->layers, "null argument");
    *out = nullptr;
    LV_REQUIRE(m->wtype == T_Q4_0 || m->wtype == T_Q8_0, "layer matrices must be q4_0 (2) or q8_0 (8)");
    LV_REQUIRE(m->emb_type == T_Q4_0 || m->emb_type == T_Q8_0 || m->emb_type == T_F32, "unsupported embedding type");
    LV_REQUIRE(m->n_layers >= 1 && m->n_layers <= uint32_t(kStepMaxLayers), "layer count out of range");
    LV_REQUIRE(m->dim % 256 == 0 && m->ff % 256 == 0 && m->dim >= 256 && m->dim <= 6144 && m->heads * kStepRot == m->dim,
               "need dim = heads * 128 <= 6144, dim and ff multiples of 256");
    LV_REQUIRE(m->vocab % 4 == 0 && m->vocab >= 4 && m->ctx_rows >= 1 && m->ctx_rows <= uint32_t(kStepChunkRowsMax), "vocab / context out of range");
    LV_REQUIRE(m->weights_base && m->tok_embeddings && m->norm && m->output && m->rope_table, "null model pointer");
    // this rank's share
    const uint32_t ranks = m->tp_ranks > 1 ? m->tp_ranks : 1u;
    LV_REQUIRE(ranks <= uint32_t(kStepMaxRanks) && m->tp_rank < ranks, "rank out of range");
    LV_REQUIRE(m->heads % ranks == 0 && (m->ff / ranks) % 4 == 0 && m->ff % ranks == 0, "heads and ff must divide evenly over the ranks");
    const uint32_t dq = m->dim / ranks, heads = m->heads / ranks, ff = m->ff / ranks;
    const uint32_t k_o = ranks > 1 ? m->shard_cols_o : m->dim, k_2 = ranks > 1 ? m->shard_cols_2 : m->ff;
    LV_REQUIRE(k_o % 256 == 0 && k_2 % 256 == 0 && k_o >= dq && k_2 >= ff, "shard rows must be padded to multiples of 256 columns");
    float* windows[kStepMaxRanks] = {nullptr};
    int w_ranks = 0, w_rank = 0;
    uint32_t w_capacity = 0;
    if (ranks > 1) {
        LV_REQUIRE(peer_windows(ctx, windows, &w_ranks, &w_rank, &w_capacity), "a sharded step needs connected peer windows");
        LV_REQUIRE(uint32_t(w_ranks) == ranks && uint32_t(w_rank) == m->tp_rank, "the peer windows belong to another rank layout");
        LV_REQUIRE(w_capacity >= 2 * m->dim, "peer window slots too small for the exchange vectors");
    }
    const uint32_t bb = m->wtype == T_Q4_0 ? kQ4BlockBytes : kQ8BlockBytes;
    const uint32_t rb_d = m->dim / 32 * bb, rb_f = k_2 / 32 * bb, rb_o = k_o / 32 * bb;
    const int grid = ctx->sm_count;
    // shares: every operation gives each CTA whole groups of 4 rows; partial sums and row threads must fit
    auto nseg_of = [](uint32_t K) { return (K / 32 + kSegBlocks - 1) / kSegBlocks; };
    auto share = [&](uint32_t groups) { return (groups + grid - 1) / grid; };
    const uint32_t worst_part = std::max(std::max(share(3 * dq / 4) * nseg_of(m->dim), share(ff / 2) * nseg_of(m->dim)),
                                         std::max(std::max(share(m->dim / 4) * nseg_of(k_2), share(m->dim / 4) * nseg_of(k_o)),
                                                  share(m->vocab / 4) * nseg_of(m->dim))) * 4;
    LV_REQUIRE(worst_part <= uint32_t(kStepPartFloats), "too many rows per CTA for the partial-sum buffer");

    auto* plan = new lv_step_plan();
    plan->ctx = ctx;
    plan->wtype = m->wtype;
    plan->grid = grid;
    const uint32_t kmax = std::max(m->dim, k_2);
    plan->smem = m->wtype == T_Q4_0 ? StepSmem<T_Q4_0>::total(m->dim, kmax, m->n_layers) : StepSmem<T_Q8_0>::total(m->dim, kmax, m->n_layers);
    // every matrix is a row range of the 2-D view [arena bytes / row size][row size] of the weight arena
    const uint8_t* base = static_cast<const uint8_t*>(m->weights_base);
    bool aligned = (reinterpret_cast<uintptr_t>(base) & 15u) == 0;
    auto row_of = [&](const void* w, uint32_t rb, uint64_t rows, uint32_t* out_row) {
        const uint8_t* q = static_cast<const uint8_t*>(w);
        if (q == nullptr || q < base || size_t(q - base) + rows * rb > m->weights_bytes || size_t(q - base) % rb != 0) { aligned = false; return; }
        *out_row = uint32_t(size_t(q - base) / rb);
    };
    std::vector<StepLayerDev> tab(m->n_layers);
    for (uint32_t l = 0; l < m->n_layers; ++l) {
        const lv_step_layer& a = m->layers[l];
        StepLayerDev& d = tab[l];
        memset(&d, 0, sizeof d);
        if (!(a.wq && a.wk && a.wv && a.wo && a.w1 && a.w2 && a.w3 && a.attention_norm && a.ffn_norm && a.k_cache && a.v_cache)) {
            delete plan;
            return fail(LV_ERR_BAD_ARGUMENTS, "lv_step_plan_create: null pointer in layer " + std::to_string(l));
        }
        row_of(a.wk, rb_d, dq, &d.row_k); row_of(a.wq, rb_d, dq, &d.row_q); row_of(a.wv, rb_d, dq, &d.row_v);
        row_of(a.wo, rb_o, m->dim, &d.row_o); row_of(a.w3, rb_d, ff, &d.row_3); row_of(a.w1, rb_d, ff, &d.row_1);
        row_of(a.w2, rb_f, m->dim, &d.row_2);
        d.w_k = static_cast<const uint8_t*>(a.wk); d.w_q = static_cast<const uint8_t*>(a.wq); d.w_v = static_cast<const uint8_t*>(a.wv);
        d.w_o = static_cast<const uint8_t*>(a.wo); d.w_3 = static_cast<const uint8_t*>(a.w3); d.w_1 = static_cast<const uint8_t*>(a.w1);
        d.w_2 = static_cast<const uint8_t*>(a.w2);
        d.attn_norm = a.attention_norm; d.ffn_norm = a.ffn_norm;
        d.k_cache = static_cast<__half*>(a.k_cache); d.v_cache = static_cast<__half*>(a.v_cache);
        for (const void* q : {a.wq, a.wk, a.wv, a.wo, a.w1, a.w2, a.w3, static_cast<const void*>(a.attention_norm), static_cast<const void*>(a.ffn_norm),
                              static_cast<const void*>(a.k_cache), static_cast<const void*>(a.v_cache)})
            if (reinterpret_cast<uintptr_t>(q) & 15u) {
                delete plan;
                return fail(LV_ERR_BAD_ARGUMENTS, "lv_step_plan_create: pointers must be 16-byte aligned");
            }
    }
    StepParams& p = plan->params;
    p.dim = m->dim; p.dq = dq; p.ff = ff; p.heads = heads; p.k_o = k_o; p.k_2 = k_2;
    p.n_layers = m->n_layers; p.vocab = m->vocab; p.ctx_rows = m->ctx_rows;
    p.row_bytes_d = rb_d; p.row_bytes_f = rb_f; p.row_bytes_o = rb_o;
    p.n_ranks = int(ranks); p.rank = int(m->tp_rank);
    for (uint32_t r = 0; r < ranks && ranks > 1; ++r) p.xw[r] = reinterpret_cast<uint64_t*>(windows[r]);
    p.xw_stride = w_capacity / 2;                  // a slot of `capacity` floats, counted in 8-byte words
    p.emb = static_cast<const uint8_t*>(m->tok_embeddings); p.emb_type = m->emb_type;
    p.final_norm = m->norm;
    p.head_w = static_cast<const uint8_t*>(m->output);
    row_of(m->output, rb_d, m->vocab, &p.head_row0);
    p.rope = m->rope_table;
    p.err = ctx->d_err;
    // tiled loads need boxes of at most 256 eight-byte elements (q4_0: 144; q8_0: 272 -> bulk copies) and every matrix on the row grid
    constexpr uint32_t seg_q4 = kSegBlocks * kQ4BlockBytes;
    static const char* no_tmap = getenv("LV_GEMV_NO_TENSOR_MAP");
    plan->tmap = m->wtype == T_Q4_0 && aligned && rb_d % 16 == 0 && rb_f % 16 == 0 && rb_o % 16 == 0 && !(no_tmap != nullptr && no_tmap[0] == '1');
    if (plan->tmap) {
        const uint64_t rows_d = m->weights_bytes / rb_d, rows_f = m->weights_bytes / rb_f, rows_o = m->weights_bytes / rb_o;
        int rc = LV_OK;
        if (rows_d > 0xffffffffull || rows_f > 0xffffffffull || rows_o > 0xffffffffull) rc = fail(LV_ERR_BAD_ARGUMENTS, "weight arena too large for the tensor maps");
        if (rc == LV_OK) rc = make_weight_map(&plan->maps.m[0], base, uint32_t(rows_d), rb_d, 4, seg_q4);
        if (rc == LV_OK) rc = make_weight_map(&plan->maps.m[1], base, uint32_t(rows_d), rb_d, 2, seg_q4);
        if (rc == LV_OK) rc = make_weight_map(&plan->maps.m[2], base, uint32_t(rows_f), rb_f, 4, seg_q4);
        if (rc == LV_OK) rc = make_weight_map(&plan->maps.m[3], base, uint32_t(rows_o), rb_o, 4, seg_q4);
        if (rc != LV_OK) { delete plan; return rc; }
    } else if (rb_d % 16 != 0 || rb_f % 16 != 0 || rb_o % 16 != 0) {
        delete plan;
        return fail(LV_ERR_BAD_ARGUMENTS, "lv_step_plan_create: row sizes must be multiples of 16 bytes");
    }
    // device copies: the layer table and the workspace of flag-in-data vectors
    const size_t ws_words = size_t(2) * m->dim + size_t(3) * dq + size_t(heads) * kStepNchMax * kStepAttRec + ff + size_t(grid) * 2 + 64;
    cudaError_t e = cudaMalloc(&plan->d_layers, tab.size() * sizeof(StepLayerDev));
    if (e == cudaSuccess) e = cudaMemcpy(plan->d_layers, tab.data(), tab.size() * sizeof(StepLayerDev), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMalloc(&plan->d_ws, ws_words * 8);
    if (e == cudaSuccess) e = cudaMemset(plan->d_ws, 0, ws_words * 8);
    if (e != cudaSuccess) {
        cudaFree(plan->d_layers);
        cudaFree(plan->d_ws);
        delete plan;
        return cuda_fail(e, "lv_step_plan_create");
    }
    p.layers = static_cast<const StepLayerDev*>(plan->d_layers);
    uint64_t* ws = static_cast<uint64_t*>(plan->d_ws);
    p.x_ll = ws; ws += size_t(2) * m->dim;
    p.qkv_ll = ws; ws += size_t(3) * dq;
    p.att_ll = ws; ws += size_t(heads) * kStepNchMax * kStepAttRec;
    p.g_ll = ws; ws += (ff + 3) / 4 * 4;
    p.amax_ll = ws; ws += size_t(grid) * 2;
    p.step = reinterpret_cast<uint32_t*>(ws);
    int rc = m->wtype == T_Q4_0 ? step_configure<T_Q4_0>(ctx, plan->smem) : step_configure<T_Q8_0>(ctx, plan->smem);
    if (rc != LV_OK) { lv_step_plan_destroy(plan); return rc; }
    *out = plan;
    return LV_OK;
}

extern "C" int lv_step_plan_set_trace(lv_step_plan* plan, int on) {
    LV_REQUIRE(plan && plan->ctx, "null plan");
    LV_CUDA(cudaSetDevice(plan->ctx->device));
    LV_CUDA(cudaStreamSynchronize(plan->ctx->stream));
    if (on && plan->d_trace == nullptr) {
        plan->trace_words = size_t(4 * plan->params.n_layers + 1) * plan->grid * kStepTracePoints;
        LV_CUDA(cudaMalloc(&plan->d_trace, plan->trace_words * 8));
        LV_CUDA(cudaMemset(plan->d_trace, 0, plan->trace_words * 8));
    } else if (!on && plan->d_trace != nullptr) {
        cudaFree(plan->d_trace);
        plan->d_trace = nullptr;
        plan->trace_words = 0;
    }
    return LV_OK;
}

extern "C" int lv_step_plan_read_trace(lv_step_plan* plan, uint64_t* out, size_t max_words, uint32_t* n_ops, uint32_t* n_ctas, uint32_t* n_points) {
    LV_REQUIRE(plan && plan->ctx && out && plan->d_trace, "no trace to read");
    LV_REQUIRE(max_words >= plan->trace_words, "trace buffer too small");
    LV_CUDA(cudaSetDevice(plan->ctx->device));
    LV_CUDA(cudaStreamSynchronize(plan->ctx->stream));
    LV_CUDA(cudaMemcpy(out, plan->d_trace, plan->trace_words * 8, cudaMemcpyDeviceToHost));
    if (n_ops) *n_ops = 4 * plan->params.n_layers + 1;
    if (n_ctas) *n_ctas = uint32_t(plan->grid);
    if (n_points) *n_points = kStepTracePoints;
    return LV_OK;
}

extern "C" int lv_step_plan_destroy(lv_step_plan* plan) {
    if (!plan) return LV_OK;
    if (plan->ctx) {
        cudaSetDevice(plan->ctx->device);
        cudaStreamSynchronize(plan->ctx->stream);
    }
    cudaFree(plan->d_layers);
    cudaFree(plan->d_ws);
    cudaFree(plan->d_trace);
    delete plan;
    return LV_OK;
}

extern "C" int lv_decode_step(lv_ctx* ctx, const lv_step_plan* plan, uint32_t* config, uint32_t* token_log, uint32_t log_capacity,
                              float* logits, uint32_t* argmax_out, uint32_t* host_token, int with_head) {
    LV_ENTER(ctx);
    LV_REQUIRE(plan && plan->ctx == ctx && config && token_log && log_capacity, "bad decode step arguments");
    LV_REQUIRE(!with_head || logits, "a step with the output head needs a logits buffer");
    StepParams p = plan->params;
    p.config = config;
    p.token_log = token_log;
    p.log_capacity = log_capacity;
    p.logits = logits;
    p.argmax_out = argmax_out;
    p.host_token = static_cast<volatile uint32_t*>(host_token);
    p.with_head = with_head ? 1 : 0;
    p.tp_step = peer_step_counter(ctx);
    p.trace = static_cast<unsigned long long*>(plan->d_trace);
    if (plan->wtype == T_Q4_0) return plan->tmap ? step_launch<T_Q4_0, true>(plan, p) : step_launch<T_Q4_0, false>(plan, p);
    return step_launch<T_Q8_0, false>(plan, p);
}
