// Quantised GEMV entry points (lv_gemv, lv_gemv_silu and the norm-fused forms).
// Replaces shaders/matmul.glsl, matmul_q8.glsl, matmul_silu_ff*.comp and their
// matmul_{add_,}{dim,ff}* wrappers of the reference.
#include <cuda.h>

#include <cstdlib>
#include <string>

#include "ctx.h"
#include "gemv_stream.cuh"
#include "tmap.h"

namespace lv {

// Shared memory map of one CTA:
//   [ring: warps x stages x stage bytes][mbarriers][reduction scratch][item partials][activation records]
constexpr size_t kBarBytes = 512;          // kStages mbarriers for each of up to 32 warps
constexpr size_t kScratchBytes = 256;
constexpr int kPartialFloats = 2048;          // per-round row-segment partial sums
constexpr size_t kPartialBytes = kPartialFloats * sizeof(float);

template <int QT, int NS>
__host__ __device__ constexpr size_t stage_bytes() { return size_t(NS) * kSegBlocks * QTraits<QT>::kBlockBytes; }

template <int QT, int NS, int W>
static size_t gemv_smem_bytes(uint32_t K) {
    return size_t(W) * kStages * stage_bytes<QT, NS>() + kBarBytes + kScratchBytes + kPartialBytes + size_t(K / 64) * kPairBytes;
}

// NS row streams per work item: NS consecutive rows, or NS/2 rows of each of the
// two matrices of the SiLU-gated pair (streams ordered w3 r0, w1 r0, w3 r1, w1 r1).
//
// A CTA takes a contiguous share of the row groups.  Its work items are (row group, segment of
// 64 blocks) pairs dealt to the warps round robin, which balances the warps to within one
// item; an item's NS partial sums go to shared memory and, once all items of a round are done,
// one thread per row adds the segments in order and applies the epilogue (deterministic).
// Tensor maps of the (up to three) matrices and, for the SiLU pair, of the gate matrix: 2-D
// tiled views [rows][row_bytes / 8] of 8-byte elements with a box of NS (or NS/2) rows x 64
// blocks, so that ONE TMA instruction fills a stage.  (One bulk copy per row stream -- four per
// stage -- is limited by the per-instruction cost of the TMA unit, about 65 cycles for 1152
// bytes, to ~5 TB/s whatever the source; measured with weights resident in L2.)
struct GemvMaps {
    CUtensorMap m[3];
    CUtensorMap gate;
};

template <int QT, int NS, bool SILU, int W, bool TMAP>
__global__ void __launch_bounds__(W * 32, W <= 8 && QT == T_Q4_0 ? 2 : 1) lv_qrow_stream_kernel(const GemvParams p, const __grid_constant__ GemvMaps maps) {
    using Q = QTraits<QT>;
    constexpr int kWarps = W;
    static_assert(size_t(W) * kStages * sizeof(uint64_t) <= kBarBytes, "mbarrier area too small for this many warps");
    static_assert(W <= 32, "block_sum supports at most 32 warps");
    constexpr int kRowsPerItem = SILU ? NS / 2 : NS;
    constexpr int kStreamStride = kSegBlocks * Q::kBlockBytes;   // bytes between streams in a stage
    constexpr size_t kStage = stage_bytes<QT, NS>();
    constexpr size_t kRing = size_t(kWarps) * kStages * kStage;

    pdl_launch_dependents();
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kRing);
    float* scratch = reinterpret_cast<float*>(smem + kRing + kBarBytes);
    float* part = reinterpret_cast<float*>(smem + kRing + kBarBytes + kScratchBytes);
    uint8_t* xrec = smem + kRing + kBarBytes + kScratchBytes + kPartialBytes;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t z = blockIdx.y;
    const uint32_t nb = p.K / 32;
    const uint32_t nseg = (nb + kSegBlocks - 1) / kSegBlocks;

    // groups of kRowsPerItem rows, numbered across the (up to three) matrices
    const uint32_t g0 = p.m[0].rows / kRowsPerItem;
    const uint32_t g1 = g0 + (p.n_mat > 1 ? p.m[1].rows / kRowsPerItem : 0);
    const uint32_t g2 = g1 + (p.n_mat > 2 ? p.m[2].rows / kRowsPerItem : 0);
    const uint32_t cta_first = uint32_t(uint64_t(g2) * blockIdx.x / gridDim.x);
    const uint32_t cta_groups = uint32_t(uint64_t(g2) * (blockIdx.x + 1) / gridDim.x) - cta_first;
    const uint32_t n_items = cta_groups * nseg;
    // a round = as many whole groups as the partial buffer holds
    const uint32_t groups_per_round = max(1u, uint32_t(kPartialFloats) / (nseg * NS));

    uint8_t* my_ring = smem + size_t(warp) * kStages * kStage;
    uint64_t* my_bars = bars + warp * kStages;

    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&my_bars[s], 1);
        fence_mbar_init();
    }
    __syncwarp();

    const uint64_t policy = l2_policy_evict_first();

    // which matrix a group belongs to, and its index inside that matrix
    auto locate = [&](uint32_t gg, uint32_t& lg) -> const GemvMatrix& {
        if (gg < g0) { lg = gg; return p.m[0]; }
        if (gg < g1) { lg = gg - g0; return p.m[1]; }
        lg = gg - g1;
        return p.m[2];
    };

    // starts the copies of item j into ring slot `slot`.  Stage layout: NS streams of 64 blocks;
    // plain: rows r .. r+NS-1; SiLU pair, tensor maps: w3 rows then w1 rows; SiLU pair, bulk
    // copies: (w3 r0, w1 r0, w3 r1, w1 r1).
    auto issue = [&](uint32_t j, int slot) {
        const uint32_t gl = j / nseg, seg = j - gl * nseg;
        uint32_t lg;
        const GemvMatrix& M = locate(cta_first + gl, lg);
        uint8_t* dst = my_ring + slot * kStage;
        if constexpr (TMAP) {
            if (lane == 0) {
                const uint32_t gg = cta_first + gl;
                const int x = int(seg * (kStreamStride / 8)), y = int(lg * kRowsPerItem);
                mbar_expect_tx(&my_bars[slot], NS * kStreamStride);                     // the whole box, zero fill included
                // the maps are addressed with constant indices so that they stay in parameter space
                if (gg < g0) tma_load_2d(dst, &maps.m[0], x, y, &my_bars[slot], policy);
                else if (gg < g1) tma_load_2d(dst, &maps.m[1], x, y, &my_bars[slot], policy);
                else tma_load_2d(dst, &maps.m[2], x, y, &my_bars[slot], policy);
                if constexpr (SILU) tma_load_2d(dst + (NS / 2) * kStreamStride, &maps.gate, x, y, &my_bars[slot], policy);
            }
        } else {
            const uint32_t segblocks = min(uint32_t(kSegBlocks), nb - seg * kSegBlocks);
            const uint32_t bytes = segblocks * Q::kBlockBytes;
            if (lane == 0) mbar_expect_tx(&my_bars[slot], NS * bytes);
            __syncwarp();
            if (lane < NS) {
                const uint8_t* base;
                uint32_t row;
                if constexpr (SILU) {
                    base = (lane & 1) ? M.w_gate : M.w;
                    row = lg * kRowsPerItem + (lane >> 1);
                } else {
                    base = M.w;
                    row = lg * kRowsPerItem + lane;
                }
                bulk_g2s_stream(dst + lane * kStreamStride, base + size_t(row) * p.row_bytes + size_t(seg) * kStreamStride, bytes,
                                &my_bars[slot], policy);
            }
        }
    };

    // the issue cursor runs kStages items ahead of the consume cursor
    uint32_t ij = warp;
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
        if (ij < n_items) {
            issue(ij, s);
            ij += kWarps;
        }
    }

    // weights never depend on the previous kernel; everything below does
    pdl_wait();
    // a CTA that finishes in one round knows its output rows now: fetch what an add-in-place
    // epilogue adds to before the long part instead of after it
    const bool early_rows = cta_groups <= groups_per_round && cta_groups * kRowsPerItem <= blockDim.x;
    float resid = 0.f;
    if (early_rows && threadIdx.x < cta_groups * kRowsPerItem) {
        const uint32_t gl = threadIdx.x / kRowsPerItem, rr = threadIdx.x - gl * kRowsPerItem;
        uint32_t lg;
        const GemvMatrix& M = locate(cta_first + gl, lg);
        if (M.epilogue == EPI_ADD) resid = static_cast<const float*>(M.out)[size_t(z) * M.rows + lg * kRowsPerItem + rr];
    }
    const bool tp_pull = p.tp.n_ranks > 0 && p.tp.pull_exchange >= 0;
    const bool tp_push = p.tp.n_ranks > 0 && p.tp.push_exchange >= 0;
    bool ok = true;
    if (tp_pull) {
        // wait until every CTA of every rank's producer launch has delivered its rows to this rank's window
        const uint32_t epoch = tp_epoch(p.tp, p.tp.pull_exchange);
        // four flags per acquire load: ranks x CTAs / 4 loads (296 at 8 ranks of 148 CTAs) fit one round of the CTA's
        // threads, where a load per flag took up to three acquire round trips in a row
        const uint32_t quads = (p.tp.pull_ctas + 3) / 4, total = uint32_t(p.tp.n_ranks) * quads;
        for (uint32_t idx = threadIdx.x; idx < total && ok; idx += blockDim.x) {
            const uint32_t src = idx / quads, cta = (idx - src * quads) * 4;
            const uint32_t* flag = tp_flag(p.tp, p.tp.rank, p.tp.pull_exchange, int(src), cta);
            const uint32_t live = p.tp.pull_ctas - cta;                  // words of this quad that a producer CTA writes
            const long long t0 = clock64();
            for (;;) {
                const uint4 f = ld_acquire_sys_v4(flag);
                if (f.x == epoch && (live < 2 || f.y == epoch) && (live < 3 || f.z == epoch) && (live < 4 || f.w == epoch)) break;
                if (*reinterpret_cast<volatile uint32_t*>(p.err) != 0 || clock64() - t0 > kWaitCycleLimit) {
                    atomicOr(p.err, ERR_PEER_TIMEOUT);
                    ok = false;
                    break;
                }
            }
        }
        ok = __syncthreads_and(ok);
    }
    const float* x_in = p.x + size_t(z) * p.K;
    bool sum_slots = true;
    if (tp_pull && p.tp.two_phase != 0) {
        // many ranks: summing all slots in every CTA would read (ranks + 1) vectors 148 times from L2.
        // Instead every CTA sums one slice of the vector into x_out, publishes a flag, and all CTAs then
        // stage the finished sum.  (All CTAs of the grid become resident: the kernel before this one
        // waits for nothing, and a successor cannot start before every CTA of this grid has.)
        const uint32_t epoch = tp_epoch(p.tp, p.tp.pull_exchange);
        const uint32_t n4 = p.K / 4, per = (n4 + gridDim.x - 1) / gridDim.x;
        const uint32_t begin = min(n4, blockIdx.x * per), end = min(n4, begin + per);
        for (uint32_t i = begin + threadIdx.x; i < end && ok; i += blockDim.x) {
            float4 v = reinterpret_cast<const float4*>(x_in)[i];
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < p.tp.n_ranks; ++r) {                     // rank order: the same bits on every rank
                const float4 t = __ldcg(reinterpret_cast<const float4*>(tp_slot(p.tp, p.tp.rank, p.tp.pull_exchange, r)) + i);
                sum.x += t.x; sum.y += t.y; sum.z += t.z; sum.w += t.w;
            }
            v.x += sum.x; v.y += sum.y; v.z += sum.z; v.w += sum.w;
            reinterpret_cast<float4*>(p.tp.x_out)[i] = v;
        }
        __syncthreads();
        if (threadIdx.x == 0) st_release_gpu(tp_local_flag(p.tp, blockIdx.x), epoch);
        for (uint32_t idx = threadIdx.x; idx < gridDim.x && ok; idx += blockDim.x) {
            const uint32_t* flag = tp_local_flag(p.tp, idx);
            const long long t0 = clock64();
            while (ld_acquire_gpu(flag) != epoch) {
                if (*reinterpret_cast<volatile uint32_t*>(p.err) != 0 || clock64() - t0 > kWaitCycleLimit) {
                    atomicOr(p.err, ERR_PEER_TIMEOUT);
                    ok = false;
                    break;
                }
            }
        }
        ok = __syncthreads_and(ok);
        x_in = p.tp.x_out;
        sum_slots = false;
    }
    // activation records (optionally normalised) while the first weight bytes are in flight
    stage_activations(xrec, x_in, p.norm_w, p.K, scratch, p.tp, sum_slots);
    __syncthreads();

    int slot = 0;
    uint32_t parity = 0;
    uint32_t cj = warp;
    for (uint32_t round_first = 0; round_first < cta_groups; round_first += groups_per_round) {
        const uint32_t round_groups = min(groups_per_round, cta_groups - round_first);
        const uint32_t item_base = round_first * nseg, item_end = (round_first + round_groups) * nseg;
        while (ok && cj < item_end) {
            if (!mbar_wait(&my_bars[slot], parity, p.err)) { ok = false; break; }
            const uint32_t gl = cj / nseg, seg = cj - gl * nseg;
            const uint32_t segblocks = min(uint32_t(kSegBlocks), nb - seg * kSegBlocks);
            const uint8_t* stage = my_ring + slot * kStage;
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
            if (ij < n_items) {
                issue(ij, slot);
                ij += kWarps;
            }
            slot ^= 1;
            parity ^= uint32_t(slot == 0);
            float* dst = part + size_t(cj - item_base) * NS;
            if constexpr (NS == 4) {
                const float u = warp_sum4(acc[0], acc[1], acc[2], acc[3], lane);
                if ((lane & 7) == 0) dst[lane >> 3] = u;
            } else {
                const float u = warp_sum2(acc[0], acc[1], lane);
                if ((lane & 15) == 0) dst[lane >> 4] = u;
            }
            cj += kWarps;
        }
        __syncthreads();
        // one thread per row of the round: add its segments in order, then the epilogue
        const bool finishing = threadIdx.x < round_groups * kRowsPerItem;
        const float factor = (p.norm_w != nullptr && finishing) ? norm_factor(scratch, p.K) : 1.0f;
        for (uint32_t t = threadIdx.x; t < round_groups * kRowsPerItem; t += blockDim.x) {
            const uint32_t gl = t / kRowsPerItem, rr = t - gl * kRowsPerItem;
            const float* src = part + size_t(gl) * nseg * NS;
            float v;
            if constexpr (SILU) {
                float up = 0.f, gate = 0.f;
                constexpr int kUp = TMAP ? 1 : 2, kGateOff = TMAP ? NS / 2 : 1;     // stream of row rr: up, gate
                for (uint32_t sg = 0; sg < nseg; ++sg) {
                    up += src[sg * NS + kUp * rr];
                    gate += src[sg * NS + kUp * rr + kGateOff];
                }
                up *= factor;
                gate *= factor;
                v = up * gate / (expf(-gate) + 1.0f);                   // matmul_silu_ff.comp:95
            } else {
                v = 0.f;
                for (uint32_t sg = 0; sg < nseg; ++sg) v += src[sg * NS + rr];
                v *= factor;
            }
            uint32_t lg;
            const GemvMatrix& M = locate(cta_first + round_first + gl, lg);
            const uint32_t row = lg * kRowsPerItem + rr;
            if (tp_push) {
                // this rank's partial product of the row goes to its slot of every rank's window
                for (int r = 0; r < p.tp.n_ranks; ++r) tp_slot(p.tp, r, p.tp.push_exchange, p.tp.rank)[row] = v;
            } else if (M.epilogue == EPI_STORE_F16_AT_POS) {
                __half* cache = static_cast<__half*>(M.out);
                const uint32_t slot_row = *p.pos + z;
                if (slot_row < p.ctx_rows) cache[size_t(slot_row) * M.rows + row] = __float2half_rn(v);   // copy_to_cache.comp:35
                else atomicOr(p.err, ERR_BAD_INDEX);
            } else {
                float* o = static_cast<float*>(M.out) + size_t(z) * M.rows + row;
                *o = (M.epilogue == EPI_ADD) ? ((early_rows ? resid : *o) + v) : v;   // matmul.glsl:68-72
            }
        }
        if (round_first + groups_per_round < cta_groups) __syncthreads();        // partials are reused by the next round
    }
    if (tp_push) {
        // the rows are out: one flag per CTA in every rank's window.  The barrier orders the CTA's row
        // stores before the few release stores below, whose system-scope release covers them all (a
        // system fence in every thread costs ~10 us here)
        __syncthreads();
        if (threadIdx.x < uint32_t(p.tp.n_ranks))
            st_release_sys(tp_flag(p.tp, int(threadIdx.x), p.tp.push_exchange, p.tp.rank, blockIdx.x), tp_epoch(p.tp, p.tp.push_exchange));
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

int make_weight_map(CUtensorMap* out, const void* base, uint32_t rows, uint32_t row_bytes, uint32_t box_rows, uint32_t seg_bytes) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(LV_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {row_bytes / 8, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {seg_bytes / 8, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LV_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
    return LV_OK;
}

// Tiled view of `rank` dimensions over 8-byte elements: dims[0] is the contiguous one, strides[i] (bytes) belongs to
// dims[i + 1].  No swizzle, no interleave, out-of-range elements read as zero.
int make_tiled_map(CUtensorMap* out, const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides, const uint32_t* box) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(LV_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t d[5], st[4];
    cuuint32_t b[5], el[5];
    for (uint32_t i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; el[i] = 1; }
    for (uint32_t i = 0; i + 1 < rank; ++i) st[i] = strides[i];
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT64, rank, const_cast<void*>(base), d, st, b, el, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LV_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
    return LV_OK;
}

template <int QT, int NS, bool SILU, int W>
static int launch_gemv(lv_ctx* ctx, const GemvParams& p, uint32_t batch, uint32_t groups, uint32_t ctas_per_sm = 1) {
    const size_t smem = gemv_smem_bytes<QT, NS, W>(p.K);
    LV_REQUIRE(smem <= size_t(ctx->max_smem_optin), "lv_gemv: K too large for the shared-memory activation buffer");
    const uint32_t ctas = min(uint32_t(ctx->sm_count) * ctas_per_sm, groups);
    dim3 grid(ctas, batch);
    constexpr uint32_t seg_bytes = kSegBlocks * QTraits<QT>::kBlockBytes;
    // the tiled form needs a box of at most 256 eight-byte elements (q4_0: 144) and rows of a multiple of 16 bytes
    static const char* no_tmap = getenv("LV_GEMV_NO_TENSOR_MAP");
    const bool tmap = seg_bytes / 8 <= 256 && p.row_bytes % 16 == 0 && !(no_tmap != nullptr && no_tmap[0] == '1');
    GemvMaps maps{};
    if (tmap) {
        constexpr uint32_t box_rows = SILU ? NS / 2 : NS;
        for (int i = 0; i < p.n_mat; ++i)
            if (int rc = make_weight_map(&maps.m[i], p.m[i].w, p.m[i].rows, p.row_bytes, box_rows, seg_bytes)) return rc;
        if (SILU)
            if (int rc = make_weight_map(&maps.gate, p.m[0].w_gate, p.m[0].rows, p.row_bytes, box_rows, seg_bytes)) return rc;
        LV_CUDA(launch_pdl(ctx, lv_qrow_stream_kernel<QT, NS, SILU, W, true>, grid, dim3(W * 32), smem, p, maps));
    } else {
        LV_CUDA(launch_pdl(ctx, lv_qrow_stream_kernel<QT, NS, SILU, W, false>, grid, dim3(W * 32), smem, p, maps));
    }
    return LV_OK;
}

static bool gemv_two_per_sm() {
    static const bool on = []() {
        const char* e = getenv("LV_GEMV_TWO_PER_SM");
        return e != nullptr && e[0] == '1';
    }();
    return on;
}

template <int QT, bool SILU>
static int launch_gemv_pick_streams(lv_ctx* ctx, const GemvParams& p, uint32_t batch) {
    uint32_t rows = 0;
    for (int i = 0; i < p.n_mat; ++i) rows += p.m[i].rows;
    // four streams per item reuse each activation record twice as often as two; measured on B200
    // this wins for every decoder shape (gate/up 12.1 vs 14.5 us, wq 4.7 vs 5.6 us; 4096x11008, where
    // two streams would balance the warps better, is a tie), so the two-stream form is kept only for
    // matrices with fewer row groups than SMs
    const uint32_t groups4 = SILU ? rows / 2 : rows / 4;
    constexpr int W = QTraits<QT>::kWarps;      // 20 warps instead of 16 measured no faster
    if constexpr (QT == T_Q4_0) {
        // Two CTAs of eight warps per SM instead of one of sixteen: the slots of an SM turn over one CTA at a time, so the
        // first CTAs of the next launch (programmatic dependent launch) become resident and start their weight copies while
        // the last CTAs of this one are still in their row pass.  Needs the shared memory of two CTAs: four rows per item
        // while the activation records are small, two rows for the FFN-wide inputs.
        if (gemv_two_per_sm() && p.tp.n_ranks == 0 && groups4 >= 2 * uint32_t(ctx->sm_count)) {
            constexpr size_t kHalf = 113 * 1024;
            if (gemv_smem_bytes<QT, 4, 8>(p.K) <= kHalf) return launch_gemv<QT, 4, SILU, 8>(ctx, p, batch, groups4, 2);
            if (gemv_smem_bytes<QT, 2, 8>(p.K) <= kHalf) return launch_gemv<QT, 2, SILU, 8>(ctx, p, batch, groups4 * 2, 2);
        }
    }
    if (groups4 >= uint32_t(ctx->sm_count)) return launch_gemv<QT, 4, SILU, W>(ctx, p, batch, groups4);
    return launch_gemv<QT, 2, SILU, W>(ctx, p, batch, groups4 * 2);
}

// Raises the dynamic shared-memory limit of every instantiation; called once
// per context with its device current.
int gemv_configure(lv_ctx* ctx) {
    const int lim = ctx->max_smem_optin;
#define LV_CFG1(QT, NS, SILU, W)                                                                                              \
    LV_CUDA(cudaFuncSetAttribute(lv_qrow_stream_kernel<QT, NS, SILU, W, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));         \
    LV_CUDA(cudaFuncSetAttribute(lv_qrow_stream_kernel<QT, NS, SILU, W, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim))
#define LV_CFG(QT, SILU)                       \
    LV_CFG1(QT, 4, SILU, QTraits<QT>::kWarps); \
    LV_CFG1(QT, 2, SILU, QTraits<QT>::kWarps)
    LV_CFG(T_Q4_0, false); LV_CFG(T_Q4_0, true); LV_CFG(T_Q8_0, false); LV_CFG(T_Q8_0, true);
    LV_CFG(T_Q4_0_V1, false); LV_CFG(T_Q4_0_V1, true);
    LV_CFG1(T_Q4_0, 4, false, 8); LV_CFG1(T_Q4_0, 2, false, 8); LV_CFG1(T_Q4_0, 4, true, 8); LV_CFG1(T_Q4_0, 2, true, 8);
#undef LV_CFG
#undef LV_CFG1
    return LV_OK;
}

static int check_matrix_args(const void* const* ws, int nw, int wtype, uint32_t cols, uint32_t rows_mult,
                             const uint32_t* rows, uint32_t batch, uint32_t* row_bytes, const float* x, const float* norm_w) {
    LV_REQUIRE(wtype == T_Q4_0 || wtype == T_Q8_0 || wtype == T_Q4_0_V1, "matrix type must be q4_0 (2), q8_0 (8) or version-1 q4_0 (258)");
    LV_REQUIRE(cols != 0 && cols % 256 == 0, "cols must be a non-zero multiple of 256");
    LV_REQUIRE(batch >= 1 && batch <= 65535, "batch out of range");
    LV_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(norm_w) & 15u) == 0,
               "activation and norm vectors must be 16-byte aligned");
    for (int i = 0; i < nw; ++i) {
        LV_REQUIRE(ws[i] != nullptr && (reinterpret_cast<uintptr_t>(ws[i]) & 15u) == 0, "matrix pointer null or not 16-byte aligned");
        LV_REQUIRE(rows[i] != 0 && rows[i] % rows_mult == 0, "rows must be a non-zero multiple of 4");
    }
    *row_bytes = cols / 32 * (wtype == T_Q4_0 ? kQ4BlockBytes : wtype == T_Q8_0 ? kQ8BlockBytes : kQ4V1BlockBytes);
    return LV_OK;
}

int peer_take_armed(lv_ctx* ctx, TpParams* tp, uint32_t pull_ctas);

// CTAs of a plain (one matrix, no SiLU pair) GEMV launch over `rows` rows; mirrors launch_gemv_pick_streams.
static uint32_t plain_gemv_ctas(const lv_ctx* ctx, uint32_t rows) {
    const uint32_t groups4 = rows / 4;
    return groups4 >= uint32_t(ctx->sm_count) ? uint32_t(ctx->sm_count) : min(uint32_t(ctx->sm_count), groups4 * 2);
}

static int gemv_dispatch(lv_ctx* ctx, GemvParams& p, int wtype, bool silu, uint32_t batch) {
    if (int rc = peer_take_armed(ctx, &p.tp, plain_gemv_ctas(ctx, ctx->tp_arm.pull_rows))) return rc;
    if (p.tp.n_ranks > 0) {
        LV_REQUIRE(batch == 1, "an exchange fused into a GEMV needs batch 1");
        LV_REQUIRE(p.tp.pull_ctas <= uint32_t(kTpFlagCtas), "too many producer CTAs for the flag area");
        if (p.tp.push_exchange >= 0) {
            LV_REQUIRE(p.n_mat == 1 && !silu && p.m[0].rows <= p.tp.capacity, "a pushing GEMV has one matrix whose rows fit a window slot");
            LV_REQUIRE(plain_gemv_ctas(ctx, p.m[0].rows) <= uint32_t(kTpFlagCtas), "too many CTAs for the flag area");
        }
        if (p.tp.pull_exchange >= 0) {
            LV_REQUIRE(p.K <= p.tp.capacity, "input longer than a window slot");
            LV_REQUIRE(ctx->sm_count <= kTpFlagCtas, "too many CTAs for the flag area");
        }
    }
    if (wtype == T_Q4_0) return silu ? launch_gemv_pick_streams<T_Q4_0, true>(ctx, p, batch) : launch_gemv_pick_streams<T_Q4_0, false>(ctx, p, batch);
    if (wtype == T_Q4_0_V1) return silu ? launch_gemv_pick_streams<T_Q4_0_V1, true>(ctx, p, batch) : launch_gemv_pick_streams<T_Q4_0_V1, false>(ctx, p, batch);
    return silu ? launch_gemv_pick_streams<T_Q8_0, true>(ctx, p, batch) : launch_gemv_pick_streams<T_Q8_0, false>(ctx, p, batch);
}

}  // namespace lv

using namespace lv;

static int gemv_single(lv_ctx* ctx, float* out, const void* W, int wtype, const float* x, const float* norm_w,
                       uint32_t rows, uint32_t cols, uint32_t batch, bool add) {
    LV_ENTER(ctx);
    LV_REQUIRE(out && x, "null argument");
    GemvParams p{};
    const void* ws[1] = {W};
    if (int rc = check_matrix_args(ws, 1, wtype, cols, 4, &rows, batch, &p.row_bytes, x, norm_w)) return rc;
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
    if (int rc = check_matrix_args(ws, 2, wtype, dim, 2, rows, batch, &p.row_bytes, x, norm_w)) return rc;
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
                                    const uint32_t* pos, uint32_t rows_each, uint32_t dim, uint32_t batch,
                                    uint32_t ctx_rows) {
    LV_ENTER(ctx);
    LV_REQUIRE(q_out && k_cache && v_cache && x && pos, "null argument");
    LV_REQUIRE(ctx_rows >= batch, "cache smaller than the batch");
    GemvParams p{};
    const void* ws[3] = {wk, wq, wv};
    const uint32_t rows[3] = {rows_each, rows_each, rows_each};
    if (int rc = check_matrix_args(ws, 3, wtype, dim, 4, rows, batch, &p.row_bytes, x, norm_w)) return rc;
    // same order as the reference records them: K, Q, V (llava_layer.cpp:54-56)
    p.m[0] = {static_cast<const uint8_t*>(wk), nullptr, k_cache, rows_each, EPI_STORE_F16_AT_POS};
    p.m[1] = {static_cast<const uint8_t*>(wq), nullptr, q_out, rows_each, EPI_STORE};
    p.m[2] = {static_cast<const uint8_t*>(wv), nullptr, v_cache, rows_each, EPI_STORE_F16_AT_POS};
    p.n_mat = 3;
    p.x = x;
    p.norm_w = norm_w;
    p.pos = pos;
    p.ctx_rows = ctx_rows;
    p.K = dim;
    p.err = ctx->d_err;
    return gemv_dispatch(ctx, p, wtype, false, batch);
}
