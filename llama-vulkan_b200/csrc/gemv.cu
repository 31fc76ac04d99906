// Quantised GEMV entry points (lv_gemv, lv_gemv_silu and the norm-fused forms).
// Replaces shaders/matmul.glsl, matmul_q8.glsl, matmul_silu_ff*.comp and their
// matmul_{add_,}{dim,ff}* wrappers of the reference.
#include "ctx.h"
#include "gemv_stream.cuh"

namespace lv {

// Shared memory map of one CTA:
//   [ring: warps x stages x kStageBytes][mbarriers][reduction scratch][activations, padded]
constexpr size_t kRingBytes = size_t(kGemvWarps) * kStages * kStageBytes;
constexpr size_t kBarBytes = 128;
constexpr size_t kScratchBytes = 256;

static size_t gemv_smem_bytes(uint32_t K) {
    return kRingBytes + kBarBytes + kScratchBytes + size_t(K / 32) * kXPad * sizeof(float);
}

template <int QT, bool SILU>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kernel(const GemvParams p) {
    using Q = QTraits<QT>;
    constexpr int kRowsPerItem = SILU ? 2 : 4;
    constexpr int kStreamStride = Q::kSegBlocks * Q::kBlockBytes;   // bytes between streams in a stage

    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kRingBytes);
    float* scratch = reinterpret_cast<float*>(smem + kRingBytes + kBarBytes);
    float* xs = reinterpret_cast<float*>(smem + kRingBytes + kBarBytes + kScratchBytes);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t z = blockIdx.y;
    const uint32_t nb = p.K / 32;
    const uint32_t nseg = (nb + Q::kSegBlocks - 1) / Q::kSegBlocks;

    // groups of kRowsPerItem rows, numbered across the (up to three) matrices
    const uint32_t g0 = p.m[0].rows / kRowsPerItem;
    const uint32_t g1 = g0 + (p.n_mat > 1 ? p.m[1].rows / kRowsPerItem : 0);
    const uint32_t g2 = g1 + (p.n_mat > 2 ? p.m[2].rows / kRowsPerItem : 0);
    const uint32_t gw = blockIdx.x * kGemvWarps + warp;
    const uint32_t gstride = gridDim.x * kGemvWarps;
    const uint32_t my_groups = gw < g2 ? (g2 - gw + gstride - 1) / gstride : 0;
    const uint32_t total = my_groups * nseg;

    uint8_t* my_ring = ring + size_t(warp) * kStages * kStageBytes;
    uint64_t* my_bars = bars + warp * kStages;

    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&my_bars[s], 1);
        fence_mbar_init();
    }
    __syncwarp();

    const uint64_t policy = l2_policy_evict_first();

    // lane 0: start the copies of work item t into ring slot `slot`
    auto issue = [&](uint32_t t, int slot) {
        const uint32_t gg = gw + (t / nseg) * gstride;
        const uint32_t seg = t % nseg;
        const int mi = gg < g0 ? 0 : (gg < g1 ? 1 : 2);
        const uint32_t lg = gg - (mi == 0 ? 0 : (mi == 1 ? g0 : g1));
        const GemvMatrix& M = p.m[mi];
        const uint32_t segblocks = min(uint32_t(Q::kSegBlocks), nb - seg * Q::kSegBlocks);
        const uint32_t bytes = segblocks * Q::kBlockBytes;
        const size_t col_off = size_t(seg) * kStreamStride;
        uint8_t* dst = my_ring + slot * kStageBytes;
        mbar_expect_tx(&my_bars[slot], kStreams * bytes);
        if constexpr (SILU) {
            const size_t r0 = size_t(lg) * 2 * p.row_bytes + col_off;
            bulk_g2s_stream(dst + 0 * kStreamStride, M.w + r0, bytes, &my_bars[slot], policy);
            bulk_g2s_stream(dst + 1 * kStreamStride, M.w_gate + r0, bytes, &my_bars[slot], policy);
            bulk_g2s_stream(dst + 2 * kStreamStride, M.w + r0 + p.row_bytes, bytes, &my_bars[slot], policy);
            bulk_g2s_stream(dst + 3 * kStreamStride, M.w_gate + r0 + p.row_bytes, bytes, &my_bars[slot], policy);
        } else {
            const size_t r0 = size_t(lg) * 4 * p.row_bytes + col_off;
            if (nseg == 1 && p.row_bytes == uint32_t(kStreamStride)) {
                bulk_g2s_stream(dst, M.w + r0, 4 * bytes, &my_bars[slot], policy);   // four whole rows, contiguous
            } else {
#pragma unroll
                for (int i = 0; i < kStreams; ++i)
                    bulk_g2s_stream(dst + i * kStreamStride, M.w + r0 + size_t(i) * p.row_bytes, bytes, &my_bars[slot], policy);
            }
        }
    };

    if (lane == 0) {
        for (uint32_t t = 0; t < uint32_t(kStages) && t < total; ++t) issue(t, int(t));
    }

    // activations (optionally normalised) while the first weight bytes are in flight
    stage_activations(xs, p.x + size_t(z) * p.K, p.norm_w, p.K, scratch);
    __syncthreads();

    float acc[kStreams] = {0.f, 0.f, 0.f, 0.f};
    for (uint32_t t = 0; t < total; ++t) {
        const int slot = int(t % kStages);
        const uint32_t parity = (t / kStages) & 1u;
        if (!mbar_wait(&my_bars[slot], parity, p.err)) break;

        const uint32_t seg = t % nseg;
        const uint32_t segblocks = min(uint32_t(Q::kSegBlocks), nb - seg * Q::kSegBlocks);
        const uint32_t npairs = segblocks / 2;
        const uint8_t* stage = my_ring + slot * kStageBytes;

        for (uint32_t pp = lane; pp < npairs; pp += 32) {
            float x[64];
            const float4* xb = reinterpret_cast<const float4*>(xs + size_t(seg * Q::kSegBlocks + 2 * pp) * kXPad);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 a = xb[i];
                x[4 * i] = a.x; x[4 * i + 1] = a.y; x[4 * i + 2] = a.z; x[4 * i + 3] = a.w;
                const float4 b = xb[kXPad / 4 + i];
                x[32 + 4 * i] = b.x; x[32 + 4 * i + 1] = b.y; x[32 + 4 * i + 2] = b.z; x[32 + 4 * i + 3] = b.w;
            }
#pragma unroll
            for (int i = 0; i < kStreams; ++i) {
                const uint32_t* sw = reinterpret_cast<const uint32_t*>(stage + i * kStreamStride) + size_t(pp) * Q::kPairWords;
                acc[i] += dot_pair<QT>(sw, x);
            }
        }
        __syncwarp();
        if (lane == 0 && t + kStages < total) issue(t + kStages, slot);

        if (seg == nseg - 1) {
            const uint32_t gg = gw + (t / nseg) * gstride;
            const int mi = gg < g0 ? 0 : (gg < g1 ? 1 : 2);
            const uint32_t lg = gg - (mi == 0 ? 0 : (mi == 1 ? g0 : g1));
            const GemvMatrix& M = p.m[mi];
            const float u = warp_sum4(acc[0], acc[1], acc[2], acc[3], lane);
            float v = u;
            uint32_t row;
            bool writer;
            if constexpr (SILU) {
                // streams: (w3 r0, w1 r0, w3 r1, w1 r1); lanes 0 and 16 finish rows r0 and r1
                const float gate = __shfl_xor_sync(0xffffffffu, u, 8);
                v = u * gate / (expf(-gate) + 1.0f);                 // matmul_silu_ff.comp:95
                row = lg * 2 + (lane >> 4);
                writer = (lane & 15) == 0;
            } else {
                row = lg * 4 + (lane >> 3);
                writer = (lane & 7) == 0;
            }
            if (writer) {
                if (M.epilogue == EPI_STORE_F16_AT_POS) {
                    __half* cache = static_cast<__half*>(M.out);
                    const uint32_t slot_row = *p.pos + z;
                    if (slot_row < p.ctx_rows) cache[size_t(slot_row) * M.rows + row] = __float2half_rn(v);   // copy_to_cache.comp:35
                    else atomicOr(p.err, ERR_BAD_INDEX);
                } else {
                    float* o = static_cast<float*>(M.out) + size_t(z) * M.rows + row;
                    *o = (M.epilogue == EPI_ADD) ? (*o + v) : v;                       // matmul.glsl:68-72
                }
            }
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        }
    }
}

template <int QT, bool SILU>
static int launch_gemv(lv_ctx* ctx, const GemvParams& p, uint32_t batch) {
    constexpr int rpi = SILU ? 2 : 4;
    uint32_t groups = 0;
    for (int i = 0; i < p.n_mat; ++i) groups += p.m[i].rows / rpi;
    const size_t smem = gemv_smem_bytes(p.K);
    LV_REQUIRE(smem <= size_t(ctx->max_smem_optin), "lv_gemv: K too large for the shared-memory activation buffer");
    auto kern = gemv_kernel<QT, SILU>;
    const uint32_t ctas = min(uint32_t(ctx->sm_count), (groups + kGemvWarps - 1) / kGemvWarps);
    dim3 grid(ctas, batch);
    kern<<<grid, kGemvThreads, smem, ctx->stream>>>(p);
    LV_CUDA(cudaGetLastError());
    return LV_OK;
}

static int check_matrix_args(const void* const* ws, int nw, int wtype, uint32_t cols, uint32_t rows_mult,
                             const uint32_t* rows, uint32_t batch, uint32_t* row_bytes) {
    LV_REQUIRE(wtype == T_Q4_0 || wtype == T_Q8_0, "matrix type must be q4_0 (2) or q8_0 (8)");
    LV_REQUIRE(cols != 0 && cols % 256 == 0, "cols must be a non-zero multiple of 256");
    LV_REQUIRE(batch >= 1 && batch <= 65535, "batch out of range");
    for (int i = 0; i < nw; ++i) {
        LV_REQUIRE(ws[i] != nullptr && (reinterpret_cast<uintptr_t>(ws[i]) & 15u) == 0, "matrix pointer null or not 16-byte aligned");
        LV_REQUIRE(rows[i] != 0 && rows[i] % rows_mult == 0, "rows must be a non-zero multiple of 4");
    }
    *row_bytes = cols / 32 * (wtype == T_Q4_0 ? kQ4BlockBytes : kQ8BlockBytes);
    return LV_OK;
}

// Raises the dynamic shared-memory limit of every instantiation; called once
// per context with its device current.
int gemv_configure(lv_ctx* ctx) {
    const int lim = ctx->max_smem_optin;
    LV_CUDA(cudaFuncSetAttribute(gemv_kernel<T_Q4_0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    LV_CUDA(cudaFuncSetAttribute(gemv_kernel<T_Q4_0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    LV_CUDA(cudaFuncSetAttribute(gemv_kernel<T_Q8_0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    LV_CUDA(cudaFuncSetAttribute(gemv_kernel<T_Q8_0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    return LV_OK;
}

static int gemv_dispatch(lv_ctx* ctx, const GemvParams& p, int wtype, bool silu, uint32_t batch) {
    if (wtype == T_Q4_0) return silu ? launch_gemv<T_Q4_0, true>(ctx, p, batch) : launch_gemv<T_Q4_0, false>(ctx, p, batch);
    return silu ? launch_gemv<T_Q8_0, true>(ctx, p, batch) : launch_gemv<T_Q8_0, false>(ctx, p, batch);
}

}  // namespace lv

using namespace lv;

static int gemv_single(lv_ctx* ctx, float* out, const void* W, int wtype, const float* x, const float* norm_w,
                       uint32_t rows, uint32_t cols, uint32_t batch, bool add) {
    LV_ENTER(ctx);
    LV_REQUIRE(out && x, "null argument");
    GemvParams p{};
    const void* ws[1] = {W};
    if (int rc = check_matrix_args(ws, 1, wtype, cols, 4, &rows, batch, &p.row_bytes)) return rc;
    p.m[0] = {static_cast<const uint8_t*>(W), nullptr, out, rows, add ? EPI_ADD : EPI_STORE};
    p.n_mat = 1;
    p.x = x;
    p.norm_w = norm_w;
    p.K = cols;
    p.err = ctx->d_err;
    return gemv_dispatch(ctx, p, wtype, false, batch);
}

extern "C" int lv_gemv(lv_ctx* ctx, float* out, const void* W, int wtype, const float* x, uint32_t rows,
                       uint32_t cols, uint32_t batch, int add) {
    return gemv_single(ctx, out, W, wtype, x, nullptr, rows, cols, batch, add != 0);
}

extern "C" int lv_norm_gemv(lv_ctx* ctx, float* out, const void* W, int wtype, const float* x, const float* norm_w,
                            uint32_t rows, uint32_t cols, uint32_t batch) {
    return gemv_single(ctx, out, W, wtype, x, norm_w, rows, cols, batch, false);
}

extern "C" int lv_gemv_silu(lv_ctx* ctx, float* out, const void* w3, const void* w1, int wtype, const float* x,
                            uint32_t rows, uint32_t cols, uint32_t batch) {
    return lv_norm_gate_up_silu(ctx, out, w3, w1, wtype, x, nullptr, rows, cols, batch);
}

extern "C" int lv_norm_gate_up_silu(lv_ctx* ctx, float* out, const void* w3, const void* w1, int wtype,
                                    const float* x, const float* norm_w, uint32_t ff, uint32_t dim, uint32_t batch) {
    LV_ENTER(ctx);
    LV_REQUIRE(out && x, "null argument");
    GemvParams p{};
    const void* ws[2] = {w3, w1};
    const uint32_t rows[2] = {ff, ff};
    if (int rc = check_matrix_args(ws, 2, wtype, dim, 2, rows, batch, &p.row_bytes)) return rc;
    p.m[0] = {static_cast<const uint8_t*>(w3), static_cast<const uint8_t*>(w1), out, ff, EPI_STORE};
    p.n_mat = 1;
    p.x = x;
    p.norm_w = norm_w;
    p.K = dim;
    p.err = ctx->d_err;
    return gemv_dispatch(ctx, p, wtype, true, batch);
}

extern "C" int lv_norm_qkv_kvappend(lv_ctx* ctx, float* q_out, void* k_cache, void* v_cache, const void* wq,
                                    const void* wk, const void* wv, int wtype, const float* x, const float* norm_w,
                                    const uint32_t* pos, uint32_t dim, uint32_t batch, uint32_t ctx_rows) {
    LV_ENTER(ctx);
    LV_REQUIRE(q_out && k_cache && v_cache && x && pos, "null argument");
    LV_REQUIRE(ctx_rows >= batch, "cache smaller than the batch");
    GemvParams p{};
    const void* ws[3] = {wk, wq, wv};
    const uint32_t rows[3] = {dim, dim, dim};
    if (int rc = check_matrix_args(ws, 3, wtype, dim, 4, rows, batch, &p.row_bytes)) return rc;
    // same order as the reference records them: K, Q, V (llava_layer.cpp:54-56)
    p.m[0] = {static_cast<const uint8_t*>(wk), nullptr, k_cache, dim, EPI_STORE_F16_AT_POS};
    p.m[1] = {static_cast<const uint8_t*>(wq), nullptr, q_out, dim, EPI_STORE};
    p.m[2] = {static_cast<const uint8_t*>(wv), nullptr, v_cache, dim, EPI_STORE_F16_AT_POS};
    p.n_mat = 3;
    p.x = x;
    p.norm_w = norm_w;
    p.pos = pos;
    p.ctx_rows = ctx_rows;
    p.K = dim;
    p.err = ctx->d_err;
    return gemv_dispatch(ctx, p, wtype, false, batch);
}
