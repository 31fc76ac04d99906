// Batched (multi-token) matrix products on the tcgen05 tensor cores.
//
// The decode step multiplies every matrix by one activation vector (gemv.cu).  When a prompt
// is evaluated, several tokens share each matrix, the contraction becomes dense and the
// reference's per-token shader dispatches (matmul.glsl with a batch in gl_WorkGroupID.z,
// llava_command_buffer.cpp:61-132) are replaced by one pass over the weights:
//
//   out[z][r] = sum_k W[r][k] * x[z][k]        r: 128 rows per CTA, z < Z <= 64
//
// A operand: the q4_0 / q8_0 blocks of 128 rows, fetched by 2-D tensor-map TMA loads into a
// raw ring, dequantised by sixteen warps into K-major fp16 tiles with the 128-byte swizzle.
// A weight (q - 8) * d (q4_0) or q * d (q8_0) needs up to 14 / 19 significant bits, so it is
// written as an exact pair hi = fp16(w), lo = w - hi.  B operand: the activations as an
// exact-to-22-bits pair of fp16 planes that lv_act_split_f16 writes tile by tile in the
// swizzled order, so that one bulk copy per 64 columns of K brings a ready B tile (the lo
// plane's rows follow the hi plane's, so one tile of 2Z rows serves both).  One thread issues,
// per 64 columns of K, four K=16 steps of two tcgen05.mma: W_hi x [x_hi; x_lo] (N = 2Z) and
// W_lo x x_hi (N = Z) into three 128 x Z fp32 accumulators in tensor memory (lo*lo is below
// fp32 resolution; two such banks are used in turn).  Four warps read the accumulators back
// with tcgen05.ld, add them and apply the epilogue (store / add to the residual / f16 cache
// rows at the position / SiLU gate of a row pair).
//
// A matrix with few row tiles (wo, w2: 32-40) is also split along K, up to four CTAs per tile:
// the kernel is bound by shared-memory traffic (each weight is written once and read once as two
// fp16 planes), which only more SMs relieve.  The CTAs of a tile leave their partial accumulators
// in a scratch buffer; the last to arrive adds them in split order (deterministic) and applies
// the epilogue.
//
// Three forms of the A operand (template parameter FORM; 1 for q4_0 only):
//   exact (FORM = 0)      the hi/lo pair described above, one 64-column tile per producer step;
//   fast  (FORM = 1, 2)   hi = fp16(w) alone: a weight is rounded to 11 significant bits (relative error <= 2^-12, none
//                         for q4_0 weights with q - 8 in {0, +-1, +-2, +-4, -8}); the activations keep both planes.
//                         One producer step covers four tiles of K (a whole raw stage): a warp handles 8 rows x 4 tiles,
//                         so that its 32-bit loads of the 144-byte raw rows and its 16-byte tile stores are free of bank
//                         conflicts, a thread dequantises the two blocks of one tile of one row, and one MMA per K step
//                         (W_hi x [x_hi; x_lo]) replaces two.  Any matrix is split along K so that the CTAs fill the SMs
//                         in whole waves.  Form 1 keeps the tile in shared memory as described; form 2 (the default)
//                         stores it from the producers' registers into tensor memory and gives it to the MMA as its
//                         TMEM operand (see the producer branch below).
//
// Every wait is bounded (common.cuh); a lost wait sets the context's error word, the CTA
// drains and frees its tensor memory.
#include <cuda.h>

#include <cstdlib>
#include <string>

#include "common.cuh"
#include "ctx.h"
#include "gemv_stream.cuh"
#include "tmap.h"

namespace lv {

constexpr int kTcRows = 128;                   // rows of W per CTA = M of the MMA
constexpr int kTcMaxZ = 64;                    // tokens per launch = N of the MMA (padded to 16)
constexpr int kTcChunkK = 64;                  // K per A/B tile: 64 fp16 = one 128-byte swizzle row
constexpr int kTcRawBlocks = 8;                // q-blocks of a row per raw stage (4 tiles of K)
constexpr int kTcRawStages = 2;
constexpr int kTcSlots = 3;
constexpr int kTcTileBytes = kTcRows * kTcChunkK * 2;                 // 16384: one fp16 plane of A
constexpr int kTcSlotBytes = 2 * kTcTileBytes;                        // 32768: hi and lo planes of A
constexpr int kTcMaxBStages = 16;
constexpr int kTcBanks = 2;                    // accumulator sets used in turn, to halve the length of each fp32 chain
constexpr int kTcProducerWarps = 16;           // two groups of 8: even and odd tiles of K
constexpr int kTcGroupWarps = 8;
constexpr int kTcThreads = (kTcProducerWarps + 3) * 32;               // + TMA warp + two MMA warps (the second issues in form 2 only)

template <int QT> struct TcTraits;
template <> struct TcTraits<T_Q4_0> {
    static constexpr int kBlockBytes = kQ4BlockBytes;
    static constexpr int kBRingBytes = 65536;  // ring of B tiles (hi and lo planes, 2 zpad rows of 128 bytes each)
};
template <> struct TcTraits<T_Q8_0> {
    static constexpr int kBlockBytes = kQ8BlockBytes;
    static constexpr int kBRingBytes = 49152;  // the raw ring is larger, the B ring shorter
};
template <int QT> __host__ __device__ constexpr int tc_raw_row_bytes() { return kTcRawBlocks * TcTraits<QT>::kBlockBytes; }       // 144 / 272
template <int QT> __host__ __device__ constexpr int tc_raw_stage() { return kTcRows * tc_raw_row_bytes<QT>(); }                   // 18432 / 34816
constexpr int kTcFastGroup = 4;                // fast form: tiles of K per producer step (= one raw stage)
constexpr int kTcFastBufs = 2;
constexpr int kTcFastBufBytes = kTcFastGroup * kTcTileBytes;          // 65536
constexpr int kTcFastBRingBytes = 49152;
// FORM: 0 exact (hi/lo tiles in shared memory), 1 fast (one fp16 plane in shared memory), 2 fast with the weight tile in
// tensor memory (written by the producers with tcgen05.st and read by the MMA as its TMEM operand: the tile never passes
// through shared memory, which is what bounds forms 0 and 1; the freed 128 KB hold eight activation stages)
constexpr int kTcTmemBRingBytes = 131072;
constexpr int kTcTmemScratchBytes = 8192;      // the epilogue's gate exchange
template <int QT, int FORM> __host__ __device__ constexpr int tc_a_bytes() {
    return FORM == 2 ? kTcTmemScratchBytes : (FORM == 1 ? kTcFastBufs * kTcFastBufBytes : kTcSlots * kTcSlotBytes);
}
template <int QT, int FORM> __host__ __device__ constexpr int tc_b_ring_bytes() {
    return FORM == 2 ? kTcTmemBRingBytes : (FORM == 1 ? kTcFastBRingBytes : TcTraits<QT>::kBRingBytes);
}
template <int QT, int FORM = 0> __host__ __device__ constexpr size_t tc_smem_bytes() {
    return 1024 /* alignment slack */ + size_t(tc_a_bytes<QT, FORM>()) + tc_b_ring_bytes<QT, FORM>() + size_t(kTcRawStages) * tc_raw_stage<QT>() + 512;
}

struct GemmTcParams {
    GemvMatrix m[3];         // same meaning as in the GEMV; w_gate set = SiLU pair (64 + 64 rows per CTA)
    int n_mat;
    const uint32_t* pos;     // device word for EPI_STORE_F16_AT_POS
    uint32_t K;
    uint32_t Z;              // tokens (columns actually written)
    uint32_t zpad;           // Z rounded up to 16 = N of the MMA
    uint32_t ctx_rows;
    const __half* xh;        // split activations, one contiguous pre-swizzled B tile per 64 columns of K (act_split_kernel)
    uint32_t splits;         // CTAs that share one tile of rows, each taking a contiguous range of K
    float* scratch;          // splits > 1: partial accumulators [tile][split][zpad][128]
    uint32_t* counters;      // splits > 1: arrivals per tile (zero between launches)
    uint32_t* err;
    const lv_group_member* group;   // non-null: token z is member z of a group step; cache rows go to its own caches at its own position
};

struct GemmTcMaps {
    CUtensorMap w[3];
    CUtensorMap gate;
};

__device__ __forceinline__ void tma_load_2d_plain(void* smem_dst, const void* tensor_map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(tensor_map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], fp16 inputs, fp32 accumulation; issued by one thread.
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The same with the A operand in tensor memory (lane = row, one 32-bit column per two fp16 along K).
__device__ __forceinline__ void tc_mma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 fp16) with the
// 128-byte swizzle: 8-row groups 1024 bytes apart, descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr) {
    return uint64_t((smem_addr >> 4) & 0x3fffu) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) |
           (uint64_t(2) << 61);
}

// Where the 16-byte chunk `c` (0..7) of row `r` lives inside a swizzled tile.
__device__ __forceinline__ uint32_t tc_swizzled(uint32_t r, uint32_t c) {
    return (r >> 3) * 1024u + (r & 7u) * 128u + ((c ^ (r & 7u)) << 4);
}

// Eight nibbles of one word -> exact (hi, lo) fp16 pairs of (q - 8) * d.
// Output order: e[0] = elements (4k, 4k+1), e[1] = (4k+2, 4k+3), e[2] = (16+4k, 17+4k), e[3] = (18+4k, 19+4k).
__device__ __forceinline__ void dequant_word(uint32_t w, __half2 d2, __half2 (&hi)[4], __half2 (&lo)[4]) {
    const uint32_t v01 = __byte_perm(w, 0u, 0x4140), v23 = __byte_perm(w, 0u, 0x4342);       // (b0, b1), (b2, b3) in 16-bit lanes
    const uint32_t raw[4] = {(v01 & 0x000f000fu) | 0x64006400u, (v23 & 0x000f000fu) | 0x64006400u,
                             ((v01 >> 4) & 0x000f000fu) | 0x64006400u, ((v23 >> 4) & 0x000f000fu) | 0x64006400u};   // 1024 + q
    const __half2 off = __floats2half2_rn(1032.0f, 1032.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 q = __hsub2(*reinterpret_cast<const __half2*>(&raw[i]), off);      // q - 8, exact
        hi[i] = __hmul2(q, d2);
        lo[i] = __hfma2(q, d2, __hneg2(hi[i]));                                            // exact remainder
    }
}

// Eight nibbles of one word -> fp16((q - 8) * d), same output order as dequant_word.
__device__ __forceinline__ void dequant_word_hi(uint32_t w, __half2 d2, uint32_t (&hi)[4]) {
    const uint32_t v01 = __byte_perm(w, 0u, 0x4140), v23 = __byte_perm(w, 0u, 0x4342);
    const uint32_t raw[4] = {(v01 & 0x000f000fu) | 0x64006400u, (v23 & 0x000f000fu) | 0x64006400u,
                             ((v01 >> 4) & 0x000f000fu) | 0x64006400u, ((v23 >> 4) & 0x000f000fu) | 0x64006400u};
    const __half2 off = __floats2half2_rn(1032.0f, 1032.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 h = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&raw[i]), off), d2);
        hi[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
}

// Four int8 of one word -> exact (hi, lo) fp16 pairs of q * d: e[0] = elements (4k, 4k+1), e[1] = (4k+2, 4k+3).
__device__ __forceinline__ void dequant_word_q8(uint32_t w, __half2 d2, __half2 (&hi)[2], __half2 (&lo)[2]) {
    const uint32_t u = w ^ 0x80808080u;                                       // q + 128 as unsigned bytes
    const uint32_t raw[2] = {__byte_perm(u, 0x64646464u, 0x4140), __byte_perm(u, 0x64646464u, 0x4342)};   // 1024 + 128 + q
    const __half2 off = __floats2half2_rn(1152.0f, 1152.0f);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const __half2 q = __hsub2(*reinterpret_cast<const __half2*>(&raw[i]), off);      // q, exact
        hi[i] = __hmul2(q, d2);
        lo[i] = __hfma2(q, d2, __hneg2(hi[i]));                                            // exact remainder (q * d has <= 19 bits)
    }
}

// Four int8 of one word -> fp16(q * d): out[0] = elements (4k, 4k+1), out[1] = (4k+2, 4k+3).
__device__ __forceinline__ void dequant_word_q8_hi(uint32_t w, __half2 d2, uint32_t (&out)[2]) {
    const uint32_t u = w ^ 0x80808080u;                                       // q + 128 as unsigned bytes
    const uint32_t raw[2] = {__byte_perm(u, 0x64646464u, 0x4140), __byte_perm(u, 0x64646464u, 0x4342)};   // 1024 + 128 + q
    const __half2 off = __floats2half2_rn(1152.0f, 1152.0f);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const __half2 h = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&raw[i]), off), d2);
        out[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
}

template <int QT, int FORM>
__global__ void __launch_bounds__(kTcThreads, 1) gemm_tc_kernel(const GemmTcParams p, const __grid_constant__ GemmTcMaps maps) {
    constexpr bool FAST = FORM != 0, TMEMA = FORM == 2;
    static_assert(FORM != 1 || QT == T_Q4_0, "the shared-memory fast form exists for q4_0 only");
    pdl_launch_dependents();
    extern __shared__ uint8_t smem_raw[];
    // swizzled tiles need 1024-byte alignment
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    uint8_t* slots = smem;
    constexpr int kRawRowBytes = tc_raw_row_bytes<QT>(), kRawStage = tc_raw_stage<QT>(), kBRingBytes = tc_b_ring_bytes<QT, FORM>();
    constexpr int kTileWords = kRawRowBytes / 16;                    // 32-bit words of one 64-column tile of a row: 9 / 17
    uint8_t* bring = smem + tc_a_bytes<QT, FORM>();
    uint8_t* rawring = bring + kBRingBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(rawring + kTcRawStages * kRawStage);
    uint64_t* raw_full = bars;                       // [2]
    uint64_t* raw_empty = bars + 2;                  // [2]
    uint64_t* slot_full = bars + 4;                  // [3]
    uint64_t* slot_empty = bars + 7;                 // [3]
    uint64_t* acc_full = bars + 10;
    uint64_t* b_full = bars + 12;                    // [16]
    uint64_t* b_empty = bars + 28;                   // [16]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 44);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool pair = p.m[0].w_gate != nullptr;
    const uint32_t rows_per_cta = pair ? kTcRows / 2 : kTcRows;

    // which matrix this CTA works on, and its first row there
    // (a last tile may reach past the matrix: the tensor map fills the missing rows with zero blocks and the epilogue
    // leaves them out)
    uint32_t t0 = (p.m[0].rows + rows_per_cta - 1) / rows_per_cta;
    uint32_t t1 = t0 + (p.n_mat > 1 ? (p.m[1].rows + rows_per_cta - 1) / rows_per_cta : 0);
    int mi = 0;
    const uint32_t tile_all = blockIdx.x / p.splits, split = blockIdx.x - tile_all * p.splits;
    uint32_t tile = tile_all;
    if (tile >= t1) { mi = 2; tile -= t1; }
    else if (tile >= t0) { mi = 1; tile -= t0; }
    const GemvMatrix& M = p.m[mi];
    const uint32_t row0 = tile * rows_per_cta;

    // this CTA's share of K, in groups of four 64-column tiles (one raw stage each)
    const uint32_t groups_all = p.K / (4 * kTcChunkK);
    const uint32_t g_begin = groups_all * split / p.splits, n_groups = groups_all * (split + 1) / p.splits - g_begin;
    const uint32_t n_chunks = 4 * n_groups;
    const uint32_t b_bytes = 2u * p.zpad * kTcChunkK * 2u;
    uint32_t nb = min(uint32_t(kTcMaxBStages), uint32_t(kBRingBytes) / b_bytes);               // B stages: 3-4 (zpad 64) .. 16
    if constexpr (FORM == 2) nb &= ~1u;                   // 8 (zpad 64) .. 16, even: see the MMA warps
    // accumulator columns of a bank: [0, zpad) hi*hi, [zpad, 2 zpad) hi*lo, [2 zpad, 3 zpad) lo*hi; two banks;
    // the allocation is a power of two >= 32
    const uint32_t bank_cols = (FAST ? 2u : 3u) * p.zpad;
    // form 2: accumulators in columns [0, 256), the two weight buffers (4 tiles x 32 columns each) in [256, 512)
    constexpr uint32_t kTmemABase = 256, kTmemTileCols = kTcChunkK / 2;
    const uint32_t tmem_cols = TMEMA ? 512u
                               : (FAST ? (p.zpad <= 16 ? 64u : (p.zpad <= 32 ? 128u : 256u)) : (p.zpad <= 16 ? 128u : (p.zpad <= 32 ? 256u : 512u)));

    // one barrier per thread (a single thread takes about a microsecond for all of them)
    if (threadIdx.x < 44) {
        const int i = int(threadIdx.x);
        uint32_t count = 1;                                             // raw_full, slot_empty, acc_full, b_full, b_empty
        if (i >= 2 && i < 4) count = kTcProducerWarps;                  // raw_empty
        else if (i >= 4 && i < 7) count = FAST ? kTcProducerWarps : kTcGroupWarps;      // slot_full
        else if (TMEMA && i >= 7 && i <= 10) count = 2;                 // slot_empty, acc_full: both MMA-issuing lanes commit
        mbar_init(&bars[i], count);
        fence_mbar_init();
    }
    if (warp == kTcProducerWarps + 1) {
        // the MMA warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    auto issue_raw = [&](uint32_t g) {
        const int rs = int(g % kTcRawStages);
        uint8_t* dst = rawring + rs * kRawStage;
        const int x = int((g_begin + g) * (kRawRowBytes / 8));
        mbar_expect_tx(&raw_full[rs], kRawStage);
        const CUtensorMap* wm = mi == 0 ? &maps.w[0] : (mi == 1 ? &maps.w[1] : &maps.w[2]);
        if (pair) {
            tma_load_2d_plain(dst, &maps.w[0], x, int(row0), &raw_full[rs]);                              // w3 rows -> tile rows 0..63
            tma_load_2d_plain(dst + (kTcRows / 2) * kRawRowBytes, &maps.gate, x, int(row0), &raw_full[rs]);      // w1 rows -> 64..127
        } else {
            tma_load_2d_plain(dst, wm, x, int(row0), &raw_full[rs]);
        }
    };

    bool ok = true;

    if (warp == kTcProducerWarps) {
        // ---------------- TMA warp: one lane feeds the raw ring and the B tiles ----------------
        if (lane == 0) {
            issue_raw(0);
            if (n_groups > 1) issue_raw(1);
            pdl_wait();                                    // the activations come from the previous kernel
            // the two rings advance independently: a raw stage is refilled as soon as the producers have taken it into
            // registers, a B stage as soon as its MMAs have completed, whichever comes first
            uint32_t g_next = min(uint32_t(kTcRawStages), n_groups), c_next = 0, idle = 0, bs = 0, b_wait_phase = 0;
            long long t_idle = 0;
            while (ok && (g_next < n_groups || c_next < n_chunks)) {
                bool progressed = false;
                if (g_next < n_groups && mbar_poll(&raw_empty[g_next % kTcRawStages], ((g_next / kTcRawStages) - 1) & 1u)) {
                    issue_raw(g_next++);
                    progressed = true;
                }
                if (c_next < n_chunks) {
                    // stage bs was last freed in the round before this one: its phase parity is b_wait_phase
                    if (c_next < nb || mbar_poll(&b_empty[bs], b_wait_phase)) {
                        mbar_expect_tx(&b_full[bs], b_bytes);
                        bulk_g2s(bring + bs * b_bytes, reinterpret_cast<const uint8_t*>(p.xh) + size_t(4 * g_begin + c_next) * b_bytes, b_bytes, &b_full[bs]);
                        ++c_next;
                        if (++bs == nb) { bs = 0; if (c_next > nb) b_wait_phase ^= 1u; }
                        progressed = true;
                    }
                }
                if (progressed) {
                    idle = 0;
                } else if ((++idle & 0xffu) == 0) {                 // bounded like mbar_wait
                    if (idle == 0x100u) t_idle = clock64();
                    if (*reinterpret_cast<volatile uint32_t*>(p.err) != 0) ok = false;
                    else if (clock64() - t_idle > kWaitCycleLimit) { atomicOr(p.err, ERR_MBAR_TIMEOUT); ok = false; }
                }
            }
        }
    } else if (warp == kTcProducerWarps + 1 || warp == kTcProducerWarps + 2) {
        // ---------------- MMA warps: one lane each issues tensor-core work ------------------------
        // Forms 0 and 1: the first warp issues everything.  Form 2: the issue loop of a single in-order thread (barrier
        // wait, four MMAs, commit: ~0.25 us per tile) is longer than the producers' step, so two lanes share it: lane 0 of
        // the first warp takes the even tiles of K into accumulator bank 0, lane 0 of the second the odd ones into bank 1.
        // That needs an EVEN number of activation stages, so that a stage is always consumed by the same lane: with an odd
        // number the two lanes would use a stage in turn, and a lane that runs ahead would find its barrier showing the
        // completed phase of the same parity two uses earlier and take stale data for its tile.
        const uint32_t issuer = uint32_t(warp) - (kTcProducerWarps + 1);
        if (lane == 0 && (TMEMA || issuer == 0)) {
            // instruction descriptors: fp32 accumulator, fp16 A and B, both K-major, M = 128, N = 2 zpad / zpad
            const uint32_t idesc_common = (1u << 4) | ((uint32_t(kTcRows) >> 4) << 24);
            const uint32_t idesc_wide = idesc_common | (((2u * p.zpad) >> 3) << 17);
            const uint32_t idesc_narrow = idesc_common | ((p.zpad >> 3) << 17);
            const uint64_t a_desc0 = tc_smem_desc(smem_u32(slots)), b_desc0 = tc_smem_desc(smem_u32(bring));
            if constexpr (TMEMA) {
                static_assert(kTcBanks == 2 && kTcFastGroup % 2 == 0, "two issuing lanes, one accumulator bank each");
                uint32_t bs = issuer, b_phase = 0;             // stage and phase of this lane's next tile (nb is even and >= 2)
                const uint32_t bank = tmem_base + issuer * bank_cols;
                bool first = true;
                for (uint32_t g = 0; g < n_groups && ok; ++g) {
                    const uint32_t ab = g % kTcFastBufs;
                    ok = mbar_wait(&slot_full[ab], (g / kTcFastBufs) & 1u, p.err);
                    uint32_t a_tmem = tmem_base + kTmemABase + (ab * kTcFastGroup + issuer) * kTmemTileCols;
                    for (uint32_t t = issuer; t < uint32_t(kTcFastGroup) && ok; t += 2) {
                        ok = mbar_wait(&b_full[bs], b_phase, p.err);
                        if (!ok) break;
                        tc_fence_after_sync();
                        const uint64_t b_desc = b_desc0 + ((bs * b_bytes) >> 4);
#pragma unroll
                        for (int k = 0; k < kTcChunkK / 16; ++k)          // 16 fp16 along K = 2 address units of B = 8 TMEM columns of A
                            tc_mma_f16_ta(bank, a_tmem + 8u * k, b_desc + 2u * k, idesc_wide, (!first || k != 0) ? 1u : 0u);
                        first = false;
                        tc_commit(&b_empty[bs]);
                        a_tmem += 2u * kTmemTileCols;
                        bs += 2;
                        if (bs >= nb) { bs -= nb; b_phase ^= 1u; }
                    }
                    if (ok) tc_commit(&slot_empty[ab]);
                }
            } else
            if constexpr (FAST) {
                uint32_t bs = 0, b_phase = 0;                  // B stage and its phase, advanced without divisions
                for (uint32_t g = 0; g < n_groups && ok; ++g) {
                    const uint32_t ab = g % kTcFastBufs;
                    ok = mbar_wait(&slot_full[ab], (g / kTcFastBufs) & 1u, p.err);
                    // descriptors differ from the first tile's only in the address field (units of 16 bytes; the whole
                    // shared memory stays below the field's 256 KB)
                    uint64_t a_desc = a_desc0 + ((ab * uint32_t(kTcFastBufBytes)) >> 4);
                    uint32_t a_tmem = tmem_base + kTmemABase + ab * (kTcFastGroup * kTmemTileCols);
                    for (uint32_t t = 0; t < uint32_t(kTcFastGroup) && ok; ++t) {
                        const uint32_t c = g * kTcFastGroup + t;
                        ok = mbar_wait(&b_full[bs], b_phase, p.err);
                        if (!ok) break;
                        tc_fence_after_sync();
                        const uint64_t b_desc = b_desc0 + ((bs * b_bytes) >> 4);
                        const uint32_t bank = tmem_base + (c % kTcBanks) * bank_cols;
#pragma unroll
                        for (int k = 0; k < kTcChunkK / 16; ++k) {        // 16 fp16 along K = 32 bytes = 2 address units = 8 TMEM columns
                            const uint32_t acc = (c >= uint32_t(kTcBanks) || k != 0) ? 1u : 0u;
                            if constexpr (TMEMA) tc_mma_f16_ta(bank, a_tmem + 8u * k, b_desc + 2u * k, idesc_wide, acc);
                            else tc_mma_f16(bank, a_desc + 2u * k, b_desc + 2u * k, idesc_wide, acc);
                        }
                        tc_commit(&b_empty[bs]);
                        a_desc += uint32_t(kTcTileBytes) >> 4;
                        a_tmem += kTmemTileCols;
                        if (++bs == nb) { bs = 0; b_phase ^= 1u; }
                    }
                    if (ok) tc_commit(&slot_empty[ab]);
                }
            } else {
            uint32_t bs = 0, b_phase = 0;
            for (uint32_t c = 0; c < n_chunks && ok; ++c) {
                const int s = int(c % kTcSlots);
                ok = mbar_wait(&b_full[bs], b_phase, p.err) && mbar_wait(&slot_full[s], (c / kTcSlots) & 1u, p.err);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t a_hi = a_desc0 + ((uint32_t(s) * uint32_t(kTcSlotBytes)) >> 4), a_lo = a_hi + (kTcTileBytes >> 4);
                const uint64_t b_all = b_desc0 + ((bs * b_bytes) >> 4);       // rows 0..zpad-1: x_hi, zpad..2 zpad-1: x_lo
                const uint32_t bank = tmem_base + (c % kTcBanks) * bank_cols;
#pragma unroll
                for (int k = 0; k < kTcChunkK / 16; ++k) {                    // 16 fp16 along K inside the swizzled row = 2 address units
                    const uint32_t acc = (c >= uint32_t(kTcBanks) || k != 0) ? 1u : 0u;
                    tc_mma_f16(bank, a_hi + 2u * k, b_all + 2u * k, idesc_wide, acc);
                    tc_mma_f16(bank + 2u * p.zpad, a_lo + 2u * k, b_all + 2u * k, idesc_narrow, acc);
                }
                tc_commit(&slot_empty[s]);                                   // arrive when these MMAs have read the tiles
                tc_commit(&b_empty[bs]);
                if (++bs == nb) { bs = 0; b_phase ^= 1u; }
            }
            }
            if (ok) tc_commit(acc_full);
        }
    } else {
        // ---------------- producer warps: q4_0 blocks -> swizzled fp16 hi/lo tiles ---------------
        if constexpr (TMEMA) {
            // A warp can reach only its own quarter of the tensor memory's lanes (32 (warp % 4) ..): lane = tile row.  Warp w
            // handles rows 32 (w % 4) .. + 31 of tile w / 4 of every raw stage; a thread dequantises the two blocks of its row
            // into 32 registers (two fp16 each, in element order) and stores them as 32 columns of its lane.
            const uint32_t tr_row = (uint32_t(warp) & 3u) * 32u + uint32_t(lane), tt = uint32_t(warp) >> 2;
            for (uint32_t g = 0; g < n_groups && ok; ++g) {
                const int rs = int(g % kTcRawStages);
                ok = mbar_wait(&raw_full[rs], (g / kTcRawStages) & 1u, p.err);
                if (!ok) break;
                // the tile's two blocks (36 / 68 bytes) start at byte 36 t / 68 t of the raw row: 16-byte loads from the chunk
                // that holds the first byte (rows are 9 / 17 chunks apart, so a quarter warp's loads fall into different
                // banks); the tile then starts t words into the loaded words
                constexpr int kTileWordsQ = kRawRowBytes / 16;                 // words of a tile: 9 / 17
                constexpr int kLoadChunks = (kTileWordsQ + 3 + 3) / 4;          // 3 / 5
                uint32_t L[4 * kLoadChunks];
                {
                    const uint4* src = reinterpret_cast<const uint4*>(rawring + rs * kRawStage + tr_row * kRawRowBytes) +
                                       (QT == T_Q4_0 ? 2u : 4u) * tt;
#pragma unroll
                    for (int i = 0; i < kLoadChunks; ++i) {
                        const uint4 v = src[i];
                        L[4 * i] = v.x; L[4 * i + 1] = v.y; L[4 * i + 2] = v.z; L[4 * i + 3] = v.w;
                    }
                }
                uint32_t w[kTileWordsQ];
                switch (tt) {                      // (t is the same for the whole warp)
                    case 0:
#pragma unroll
                        for (int i = 0; i < kTileWordsQ; ++i) w[i] = L[i];
                        break;
                    case 1:
#pragma unroll
                        for (int i = 0; i < kTileWordsQ; ++i) w[i] = L[i + 1];
                        break;
                    case 2:
#pragma unroll
                        for (int i = 0; i < kTileWordsQ; ++i) w[i] = L[i + 2];
                        break;
                    default:
#pragma unroll
                        for (int i = 0; i < kTileWordsQ; ++i) w[i] = L[i + 3];
                        break;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[rs]);
                // registers of the row: column j of the tile = elements 2j, 2j + 1 (block 0: columns 0..15, block 1: 16..31)
                uint32_t cols[32];
                constexpr int kQW = (kTileWordsQ - 1) / 2;                      // payload words of a block: 4 / 8
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    // block 0: scale in the low half of word 0, payload shifted by two bytes; block 1: scale in the high half
                    // of the middle word, payload word-aligned
                    uint32_t q[kQW];
#pragma unroll
                    for (int k = 0; k < kQW; ++k) q[k] = b == 0 ? __funnelshift_r(w[k], w[k + 1], 16) : w[kQW + 1 + k];
                    const uint32_t dbits = b == 0 ? (w[0] & 0xffffu) : (w[kQW] >> 16);
                    const __half2 d2 = __half2half2(__ushort_as_half(static_cast<unsigned short>(dbits)));
                    if constexpr (QT == T_Q4_0) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            uint32_t hi[4];
                            dequant_word_hi(q[k], d2, hi);          // (4k, 4k+1), (4k+2, 4k+3), (16+4k, 17+4k), (18+4k, 19+4k)
                            cols[16 * b + 2 * k] = hi[0];
                            cols[16 * b + 2 * k + 1] = hi[1];
                            cols[16 * b + 8 + 2 * k] = hi[2];
                            cols[16 * b + 8 + 2 * k + 1] = hi[3];
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            uint32_t hi[2];
                            dequant_word_q8_hi(q[k], d2, hi);       // int8 payload in element order: (4k, 4k+1), (4k+2, 4k+3)
                            cols[16 * b + 2 * k] = hi[0];
                            cols[16 * b + 2 * k + 1] = hi[1];
                        }
                    }
                }
                const uint32_t ab = g % kTcFastBufs;
                if (g >= uint32_t(kTcFastBufs)) {
                    ok = mbar_wait(&slot_empty[ab], ((g / kTcFastBufs) - 1) & 1u, p.err);
                    if (!ok) break;
                }
                tc_fence_after_sync();
                const uint32_t taddr = tmem_base + ((uint32_t(warp) & 3u) * 32u << 16) + kTmemABase + (ab * kTcFastGroup + tt) * kTmemTileCols;
                asm volatile(
                    "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                    "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                    ::"r"(taddr), "r"(cols[0]), "r"(cols[1]), "r"(cols[2]), "r"(cols[3]), "r"(cols[4]), "r"(cols[5]), "r"(cols[6]), "r"(cols[7]),
                      "r"(cols[8]), "r"(cols[9]), "r"(cols[10]), "r"(cols[11]), "r"(cols[12]), "r"(cols[13]), "r"(cols[14]), "r"(cols[15]),
                      "r"(cols[16]), "r"(cols[17]), "r"(cols[18]), "r"(cols[19]), "r"(cols[20]), "r"(cols[21]), "r"(cols[22]), "r"(cols[23]),
                      "r"(cols[24]), "r"(cols[25]), "r"(cols[26]), "r"(cols[27]), "r"(cols[28]), "r"(cols[29]), "r"(cols[30]), "r"(cols[31])
                    : "memory");
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&slot_full[ab]);
            }
        } else if constexpr (FAST) {
            // a warp: 8 rows x the 4 tiles of a raw stage; the word offsets 36 r + 9 t of its lanes fall into 32 different banks
            const uint32_t fr = uint32_t(warp) * 8u + (uint32_t(lane) & 7u), ft = uint32_t(lane) >> 3;
            for (uint32_t g = 0; g < n_groups && ok; ++g) {
                const int rs = int(g % kTcRawStages);
                ok = mbar_wait(&raw_full[rs], (g / kTcRawStages) & 1u, p.err);
                if (!ok) break;
                uint32_t w[9];
                {
                    const uint32_t* src = reinterpret_cast<const uint32_t*>(rawring + rs * kRawStage + fr * kRawRowBytes) + 9u * ft;
#pragma unroll
                    for (int i = 0; i < 9; ++i) w[i] = src[i];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[rs]);
                const uint32_t ab = g % kTcFastBufs;
                if (g >= uint32_t(kTcFastBufs)) {
                    ok = mbar_wait(&slot_empty[ab], ((g / kTcFastBufs) - 1) & 1u, p.err);
                    if (!ok) break;
                }
                uint8_t* a_tile = slots + ab * kTcFastBufBytes + ft * kTcTileBytes;
                // block 0: bytes 0-1 scale, 2-17 nibbles; block 1: bytes 18-19 scale, 20-35 nibbles
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    uint32_t q[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) q[k] = b == 0 ? __funnelshift_r(w[k], w[k + 1], 16) : w[5 + k];
                    const uint32_t dbits = b == 0 ? (w[0] & 0xffffu) : (w[4] >> 16);
                    const __half2 d2 = __half2half2(__ushort_as_half(static_cast<unsigned short>(dbits)));
                    uint32_t hi[4][4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) dequant_word_hi(q[k], d2, hi[k]);
                    // 16-byte chunks of the block in element order: 0-7 (low nibbles of words 0, 1), 8-15, 16-23 (high nibbles), 24-31
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        const int k0 = (cc & 1) * 2, part = (cc >> 1) * 2;
                        *reinterpret_cast<uint4*>(a_tile + tc_swizzled(fr, uint32_t(b * 4 + cc))) =
                            make_uint4(hi[k0][part], hi[k0][part + 1], hi[k0 + 1][part], hi[k0 + 1][part + 1]);
                    }
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&slot_full[ab]);
            }
        } else {
        const uint32_t r = threadIdx.x & (kTcRows - 1);       // tile row of this thread
        const uint32_t khalf = (threadIdx.x >> 7) & 1u;       // which block of a 64-column tile
        const uint32_t jpar = threadIdx.x >> 8;               // producer group: even or odd tiles of K
        for (uint32_t g = 0; g < n_groups && ok; ++g) {
            const int rs = int(g % kTcRawStages);
            ok = mbar_wait(&raw_full[rs], (g / kTcRawStages) & 1u, p.err);
            if (!ok) break;
            // the two tiles of this group that the thread's producer group owns (tiles jpar and jpar + 2 of the
            // four): kTileWords words each, taken out of the row with 16-byte loads
            uint32_t w[2][kTileWords];
            const uint4* src = reinterpret_cast<const uint4*>(rawring + rs * kRawStage + r * kRawRowBytes);
            {
                uint32_t all[4 * kTileWords];
#pragma unroll
                for (int i = 0; i < kTileWords; ++i) {
                    const uint4 v = src[i];
                    all[4 * i] = v.x; all[4 * i + 1] = v.y; all[4 * i + 2] = v.z; all[4 * i + 3] = v.w;
                }
#pragma unroll
                for (int i = 0; i < kTileWords; ++i) {
                    w[0][i] = jpar ? all[kTileWords + i] : all[i];
                    w[1][i] = jpar ? all[3 * kTileWords + i] : all[2 * kTileWords + i];
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&raw_empty[rs]);       // the row is in registers
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const uint32_t c = g * 4 + jpar + 2 * jj;
                const int s = int(c % kTcSlots);
                if (c >= kTcSlots) {
                    ok = mbar_wait(&slot_empty[s], ((c / kTcSlots) - 1) & 1u, p.err);
                    if (!ok) break;
                }
                // even block of the tile: scale in the low half of word 0, payload shifted by two bytes;
                // odd block: scale in the high half of the middle word, payload word-aligned
                constexpr int kQWords = (kTileWords - 1) / 2;         // payload words of a block: 4 (nibbles) / 8 (int8)
                uint32_t q[kQWords];
                uint32_t dbits;
                if (khalf == 0) {
                    dbits = w[jj][0] & 0xffffu;
#pragma unroll
                    for (int k = 0; k < kQWords; ++k) q[k] = __funnelshift_r(w[jj][k], w[jj][k + 1], 16);
                } else {
                    dbits = w[jj][kQWords] >> 16;
#pragma unroll
                    for (int k = 0; k < kQWords; ++k) q[k] = w[jj][kQWords + 1 + k];
                }
                const __half dh = __ushort_as_half(static_cast<unsigned short>(dbits));
                const __half2 d2 = __half2half2(dh);
                uint8_t* a_hi = slots + s * kTcSlotBytes;
                uint8_t* a_lo = a_hi + kTcTileBytes;
                if constexpr (QT == T_Q4_0) {
                    __half2 hi[4][4], lo[4][4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) dequant_word(q[k], d2, hi[k], lo[k]);
                    // 16-byte chunks of the block: elements 0-7 (words 0,1 low nibbles), 8-15, 16-23 (high nibbles), 24-31
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        const int k0 = (cc & 1) * 2, part = (cc >> 1) * 2;     // words k0, k0+1; low (0) or high (2) nibbles
                        const uint32_t at = tc_swizzled(r, khalf * 4 + cc);
                        uint4 vh, vl;
                        vh.x = *reinterpret_cast<uint32_t*>(&hi[k0][part]); vh.y = *reinterpret_cast<uint32_t*>(&hi[k0][part + 1]);
                        vh.z = *reinterpret_cast<uint32_t*>(&hi[k0 + 1][part]); vh.w = *reinterpret_cast<uint32_t*>(&hi[k0 + 1][part + 1]);
                        vl.x = *reinterpret_cast<uint32_t*>(&lo[k0][part]); vl.y = *reinterpret_cast<uint32_t*>(&lo[k0][part + 1]);
                        vl.z = *reinterpret_cast<uint32_t*>(&lo[k0 + 1][part]); vl.w = *reinterpret_cast<uint32_t*>(&lo[k0 + 1][part + 1]);
                        *reinterpret_cast<uint4*>(a_hi + at) = vh;
                        *reinterpret_cast<uint4*>(a_lo + at) = vl;
                    }
                } else {
                    // int8 payload in element order: chunk cc = elements 8cc .. 8cc+7 = words 2cc, 2cc+1
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        __half2 hi0[2], lo0[2], hi1[2], lo1[2];
                        dequant_word_q8(q[2 * cc], d2, hi0, lo0);
                        dequant_word_q8(q[2 * cc + 1], d2, hi1, lo1);
                        const uint32_t at = tc_swizzled(r, khalf * 4 + cc);
                        uint4 vh, vl;
                        vh.x = *reinterpret_cast<uint32_t*>(&hi0[0]); vh.y = *reinterpret_cast<uint32_t*>(&hi0[1]);
                        vh.z = *reinterpret_cast<uint32_t*>(&hi1[0]); vh.w = *reinterpret_cast<uint32_t*>(&hi1[1]);
                        vl.x = *reinterpret_cast<uint32_t*>(&lo0[0]); vl.y = *reinterpret_cast<uint32_t*>(&lo0[1]);
                        vl.z = *reinterpret_cast<uint32_t*>(&lo1[0]); vl.w = *reinterpret_cast<uint32_t*>(&lo1[1]);
                        *reinterpret_cast<uint4*>(a_hi + at) = vh;
                        *reinterpret_cast<uint4*>(a_lo + at) = vl;
                    }
                }
                fence_proxy_async();                           // make the tile visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&slot_full[s]);
            }
        }
        }
        // ---------------- epilogue: warps 0-3 own accumulator rows 32w .. 32w+31 -----------------
        // 16 tokens z0 .. z0+15 of one output row (tile row tr)
        auto store_plain = [&](uint32_t tr, uint32_t z0, const float (&r32)[16]) {
                const uint32_t row = row0 + tr;
                if (row >= M.rows) return;
                if (M.epilogue == EPI_STORE_F16_AT_POS && p.group != nullptr) {
                    // matrix 0 is wk, matrix 2 is wv (lv_gemm_tc_qkv_kvappend_group)
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t z = z0 + i;
                        if (z < p.Z) {
                            const lv_group_member& m = p.group[z];
                            __half* cache = static_cast<__half*>(mi == 0 ? m.k_cache : m.v_cache);
                            const uint32_t at = *m.pos;
                            if (at < p.ctx_rows) cache[size_t(at) * M.rows + row] = __float2half_rn(r32[i]);
                            else atomicOr(p.err, ERR_BAD_INDEX);
                        }
                    }
                } else if (M.epilogue == EPI_STORE_F16_AT_POS) {
                    __half* cache = static_cast<__half*>(M.out);
                    const uint32_t first = *p.pos;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t z = z0 + i;
                        if (z < p.Z) {
                            if (first + z < p.ctx_rows) cache[size_t(first + z) * M.rows + row] = __float2half_rn(r32[i]);
                            else atomicOr(p.err, ERR_BAD_INDEX);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t z = z0 + i;
                        if (z < p.Z) {
                            float* o = static_cast<float*>(M.out) + size_t(z) * M.rows + row;
                            *o = (M.epilogue == EPI_ADD) ? (*o + r32[i]) : r32[i];                   // matmul.glsl:68-72
                        }
                    }
                }
            };
        auto store_pair = [&](uint32_t tr, uint32_t z0, const float (&up)[16], const float (&gate)[16]) {
                const uint32_t row = row0 + tr;
                if (row >= M.rows) return;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint32_t z = z0 + i;
                    if (z < p.Z) static_cast<float*>(M.out)[size_t(z) * M.rows + row] = up[i] * gate[i] / (expf(-gate[i]) + 1.0f);   // matmul_silu_ff.comp:95
                }
            };
        uint32_t* s_last = tmem_slot + 1;
        if (warp < 4) {
            pdl_wait();
            if (ok) ok = mbar_wait(acc_full, 0u, p.err);
            tc_fence_after_sync();
            float* gate_s = reinterpret_cast<float*>(slots);      // [64][17] floats, free once the accumulator is complete
            const uint32_t tr = uint32_t(warp * 32 + lane);       // tile row
            float* my_partial = p.scratch + (size_t(tile_all) * p.splits + split) * p.zpad * kTcRows;
            for (uint32_t z0 = 0; z0 < p.zpad; z0 += 16) {
                float v[16];
                if (ok) {
                    const uint32_t taddr = tmem_base + (uint32_t(warp * 32) << 16) + z0;
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                    const uint32_t banks_used = min(uint32_t(kTcBanks), n_chunks);
                    for (uint32_t b = 0; b < banks_used; ++b) {
                        constexpr int kAcc = FAST ? 2 : 3;
                        uint32_t u[3][16];
#pragma unroll
                        for (int a = 0; a < kAcc; ++a) {
                            asm volatile(
                                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                                : "=r"(u[a][0]), "=r"(u[a][1]), "=r"(u[a][2]), "=r"(u[a][3]), "=r"(u[a][4]), "=r"(u[a][5]), "=r"(u[a][6]),
                                  "=r"(u[a][7]), "=r"(u[a][8]), "=r"(u[a][9]), "=r"(u[a][10]), "=r"(u[a][11]), "=r"(u[a][12]), "=r"(u[a][13]),
                                  "=r"(u[a][14]), "=r"(u[a][15])
                                : "r"(taddr + b * bank_cols + uint32_t(a) * p.zpad));
                        }
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 16; ++i) {    // the small cross terms first, then the main one
                            if constexpr (FAST) v[i] += __uint_as_float(u[1][i]) + __uint_as_float(u[0][i]);
                            else v[i] += (__uint_as_float(u[1][i]) + __uint_as_float(u[2][i])) + __uint_as_float(u[0][i]);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                }
                if (p.splits > 1) {
                    // leave the partial sums for the last CTA of the tile
#pragma unroll
                    for (int i = 0; i < 16; ++i) my_partial[size_t(z0 + i) * kTcRows + tr] = v[i];
                } else if (pair) {
                    // rows 64..127 carry the gate (w1) of rows 0..63
                    if (tr >= 64) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) gate_s[(tr - 64) * 17 + i] = v[i];
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (tr < 64 && ok) {
                        float gate[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) gate[i] = gate_s[tr * 17 + i];
                        store_pair(tr, z0, v, gate);
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                } else if (ok) {
                    store_plain(tr, z0, v);
                }
            }
            if (p.splits > 1) {
                // the last of the tile's CTAs to get here adds the partial sums in split order and finishes the rows
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (tr == 0) {
                    __threadfence();
                    const uint32_t prev = atomicAdd(&p.counters[tile_all], 1u);
                    *s_last = (prev + 1 == p.splits) ? 1u : 0u;
                    if (prev + 1 == p.splits) p.counters[tile_all] = 0;         // ready for the next launch
                }
            }
        }
        if (p.splits > 1) {
            // all sixteen producer warps share the pass over the partial sums: a quarter of the tokens each
            asm volatile("bar.sync 2, 512;" ::: "memory");
            if (*reinterpret_cast<volatile uint32_t*>(s_last) != 0 && ok) {
                pdl_wait();                                   // warps 4-15 have not waited for the previous kernel yet
                __threadfence();
                const uint32_t tr = threadIdx.x & (kTcRows - 1), zq = threadIdx.x >> 7;
                const float* base = p.scratch + size_t(tile_all) * p.splits * p.zpad * kTcRows;
                for (uint32_t z0 = 16u * zq; z0 < p.zpad; z0 += 64u) {
                    if (pair) {
                        if (tr < 64) {
                            float up[16], gate[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) { up[i] = 0.f; gate[i] = 0.f; }
                            for (uint32_t sp = 0; sp < p.splits; ++sp) {
                                const float* q = base + (size_t(sp) * p.zpad + z0) * kTcRows;
                                float a[16], b[16];
#pragma unroll
                                for (int i = 0; i < 16; ++i) { a[i] = __ldcg(q + size_t(i) * kTcRows + tr); b[i] = __ldcg(q + size_t(i) * kTcRows + tr + 64); }
#pragma unroll
                                for (int i = 0; i < 16; ++i) { up[i] += a[i]; gate[i] += b[i]; }
                            }
                            store_pair(tr, z0, up, gate);
                        }
                    } else {
                        float v[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = 0.f;
                        for (uint32_t sp = 0; sp < p.splits; ++sp) {
                            const float* q = base + (size_t(sp) * p.zpad + z0) * kTcRows;
                            float a[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) a[i] = __ldcg(q + size_t(i) * kTcRows + tr);
#pragma unroll
                            for (int i = 0; i < 16; ++i) v[i] += a[i];
                        }
                        store_plain(tr, z0, v);
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kTcProducerWarps + 1) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// x (optionally normalised, normalize.comp:39-63) as two fp16 planes, hi = fp16(v), lo = fp16(v - hi), laid out
// as the B tiles the product kernel copies verbatim into shared memory: for every 64 columns of K one
// contiguous tile of 2 zpad rows x 128 bytes (rows 0..zpad-1: hi of token z, rows zpad..: lo), each row's eight
// 16-byte units stored at unit ^ (row & 7) -- the 128-byte swizzle the tensor core's descriptors expect.
// Grid: zpad CTAs; tokens z >= Z are zero so that the padded columns
// of the product are defined.  A thread converts one unit of eight values.
// K_used <= K: the rows of x hold K_used values (row stride K_used); columns from K_used on are zero (the padding of a
// tensor-parallel column shard).
__global__ void __launch_bounds__(512) act_split_kernel(__half* __restrict__ xh, const float* __restrict__ x,
                                                        const float* __restrict__ norm_w, uint32_t K, uint32_t K_used, uint32_t Z, uint32_t zpad) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[64];
    const uint32_t z = blockIdx.x;
    const float* xr = x + size_t(z) * K_used;
    float factor = 1.0f;
    if (z < Z && norm_w != nullptr) {
        float part = 0.f;
        for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) part += xr[i];
        const float mean = block_sum(part, scratch) / static_cast<float>(K);
        part = 0.f;
        for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) {
            const float c = xr[i] - mean;
            part = fmaf(c, c, part);
        }
        factor = 1.0f / sqrtf(block_sum(part, scratch) / static_cast<float>(K));        // no epsilon
    }
    for (uint32_t unit = threadIdx.x; unit < K / 8; unit += blockDim.x) {
        float v[8];
        if (z < Z && 8 * unit < K_used) {
            const float4 a = *reinterpret_cast<const float4*>(xr + 8 * unit), b = *reinterpret_cast<const float4*>(xr + 8 * unit + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            if (norm_w != nullptr) {
                const float4 wa = *reinterpret_cast<const float4*>(norm_w + 8 * unit), wb = *reinterpret_cast<const float4*>(norm_w + 8 * unit + 4);
                const float w8[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = (v[i] * w8[i]) * factor;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
        }
        __half2 hi[4], lo[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half h0 = __float2half_rn(v[2 * i]), h1 = __float2half_rn(v[2 * i + 1]);
            hi[i] = __halves2half2(h0, h1);
            lo[i] = __halves2half2(__float2half_rn(v[2 * i] - __half2float(h0)), __float2half_rn(v[2 * i + 1] - __half2float(h1)));
        }
        const uint32_t chunk = unit >> 3, u = unit & 7u;
        const size_t tile = size_t(chunk) * 2 * zpad * 64;                   // halves
        const size_t at_hi = tile + size_t(z) * 64 + ((u ^ (z & 7u)) << 3);
        const size_t at_lo = at_hi + size_t(zpad) * 64;                      // zpad is a multiple of 8: same swizzle key
        *reinterpret_cast<uint4*>(xh + at_hi) = *reinterpret_cast<const uint4*>(hi);
        *reinterpret_cast<uint4*>(xh + at_lo) = *reinterpret_cast<const uint4*>(lo);
    }
}

constexpr size_t kTcScratchBytes = size_t(32) << 20;
constexpr uint32_t kTcMaxTiles = 1024;

void gemm_tc_release(lv_ctx* ctx) {
    cudaFree(ctx->tc_scratch);
    cudaFree(ctx->tc_counters);
    ctx->tc_scratch = nullptr;
    ctx->tc_counters = nullptr;
}

int gemm_tc_configure(lv_ctx* ctx) {
    LV_CUDA(cudaMalloc(&ctx->tc_scratch, kTcScratchBytes));
    LV_CUDA(cudaMalloc(&ctx->tc_counters, kTcMaxTiles * sizeof(uint32_t)));
    LV_CUDA(cudaMemset(ctx->tc_counters, 0, kTcMaxTiles * sizeof(uint32_t)));
    LV_REQUIRE(size_t(ctx->max_smem_optin) >= tc_smem_bytes<T_Q4_0>() && size_t(ctx->max_smem_optin) >= tc_smem_bytes<T_Q8_0>(),
               "device has too little shared memory for the batched product");
    constexpr size_t kFastSmem = tc_smem_bytes<T_Q4_0, 1>();
    LV_REQUIRE(size_t(ctx->max_smem_optin) >= kFastSmem, "device has too little shared memory for the batched product");
    LV_CUDA((cudaFuncSetAttribute(gemm_tc_kernel<T_Q4_0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(tc_smem_bytes<T_Q4_0>()))));
    LV_CUDA((cudaFuncSetAttribute(gemm_tc_kernel<T_Q4_0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kFastSmem))));
    constexpr size_t kTmemSmem = tc_smem_bytes<T_Q4_0, 2>();
    LV_REQUIRE(size_t(ctx->max_smem_optin) >= kTmemSmem, "device has too little shared memory for the batched product");
    LV_CUDA((cudaFuncSetAttribute(gemm_tc_kernel<T_Q4_0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kTmemSmem))));
    constexpr size_t kTmemSmem8 = tc_smem_bytes<T_Q8_0, 2>();
    LV_REQUIRE(size_t(ctx->max_smem_optin) >= kTmemSmem8, "device has too little shared memory for the batched product");
    LV_CUDA((cudaFuncSetAttribute(gemm_tc_kernel<T_Q8_0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kTmemSmem8))));
    LV_CUDA((cudaFuncSetAttribute(gemm_tc_kernel<T_Q8_0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(tc_smem_bytes<T_Q8_0>()))));
    const char* exact = getenv("LV_GEMM_TC_EXACT");
    ctx->tc_exact = exact != nullptr && exact[0] == '1';
    return LV_OK;
}

template <int QT>
static int launch_gemm_tc_typed(lv_ctx* ctx, GemmTcParams& p, const __half* xh) {
    LV_REQUIRE(p.K != 0 && p.K % 256 == 0, "cols must be a non-zero multiple of 256");
    LV_REQUIRE(p.Z >= 1 && p.Z <= uint32_t(kTcMaxZ), "batch of the tensor-core product must be 1..64");
    LV_REQUIRE(xh != nullptr && (reinterpret_cast<uintptr_t>(xh) & 15u) == 0, "split activations null or not 16-byte aligned");
    p.zpad = (p.Z + 15u) & ~15u;
    const bool pair = p.m[0].w_gate != nullptr;
    const uint32_t rows_per_cta = pair ? kTcRows / 2 : kTcRows;
    const uint32_t row_bytes = p.K / 32 * TcTraits<QT>::kBlockBytes;
    GemmTcMaps maps{};
    uint32_t tiles = 0;
    for (int i = 0; i < p.n_mat; ++i) {
        LV_REQUIRE(p.m[i].w != nullptr && (reinterpret_cast<uintptr_t>(p.m[i].w) & 15u) == 0, "matrix pointer null or not 16-byte aligned");
        LV_REQUIRE(p.m[i].rows != 0 && p.m[i].rows % 32 == 0, "rows must be a non-zero multiple of 32");
        if (int rc = make_weight_map(&maps.w[i], p.m[i].w, p.m[i].rows, row_bytes, rows_per_cta, tc_raw_row_bytes<QT>())) return rc;
        tiles += (p.m[i].rows + rows_per_cta - 1) / rows_per_cta;
    }
    if (pair) {
        LV_REQUIRE((reinterpret_cast<uintptr_t>(p.m[0].w_gate) & 15u) == 0, "matrix pointer not 16-byte aligned");
        if (int rc = make_weight_map(&maps.gate, p.m[0].w_gate, p.m[0].rows, row_bytes, rows_per_cta, tc_raw_row_bytes<QT>())) return rc;
    }
    p.xh = xh;
    const uint32_t groups_all = p.K / (4 * kTcChunkK);
    const bool fast = !ctx->tc_exact;
    uint32_t splits = 1;
    auto fits = [&](uint32_t s) {
        return groups_all / s >= 2 && tiles <= kTcMaxTiles && size_t(tiles) * s * p.zpad * kTcRows * sizeof(float) <= kTcScratchBytes;
    };
    if (fast) {
        // every CTA holds an SM to itself, so the launch runs in waves of sm_count CTAs; a CTA costs a fixed part (set-up,
        // filling its rings, the epilogue or the pass over the partial sums: about three group steps) plus its share of K
        float best = 1e30f;
        for (uint32_t s = 1; s <= 8 && fits(s); ++s) {
            const uint32_t waves = (tiles * s + uint32_t(ctx->sm_count) - 1) / uint32_t(ctx->sm_count);
            const float cost = float(waves) * (3.0f + (s > 1 ? 0.5f : 0.0f) + float(groups_all) / float(s));
            if (cost < best) { best = cost; splits = s; }
        }
    } else {
        // few row tiles: up to four CTAs per tile, each with at least two raw stages of K, as far as SMs and scratch allow
        while (splits < 4 && tiles * (splits + 1) <= uint32_t(ctx->sm_count) && fits(splits + 1)) ++splits;
    }
    static const char* no_split = getenv("LV_GEMM_TC_NO_SPLIT");
    if (no_split != nullptr && no_split[0] == '1') splits = 1;
    p.splits = splits;
    p.scratch = static_cast<float*>(ctx->tc_scratch);
    p.counters = static_cast<uint32_t*>(ctx->tc_counters);
    tiles *= splits;
    if (fast) {
        static const char* smem_tiles = getenv("LV_GEMM_TC_SMEM_TILES");
        if constexpr (QT == T_Q4_0) {
            if (smem_tiles != nullptr && smem_tiles[0] == '1') {
                constexpr size_t kFastSmem = tc_smem_bytes<T_Q4_0, 1>();
                LV_CUDA((launch_pdl(ctx, gemm_tc_kernel<T_Q4_0, 1>, dim3(tiles), dim3(kTcThreads), kFastSmem, p, maps)));
                return LV_OK;
            }
        }
        constexpr size_t kTmemSmem = tc_smem_bytes<QT, 2>();
        LV_CUDA((launch_pdl(ctx, gemm_tc_kernel<QT, 2>, dim3(tiles), dim3(kTcThreads), kTmemSmem, p, maps)));
        return LV_OK;
    }
    LV_CUDA((launch_pdl(ctx, gemm_tc_kernel<QT, 0>, dim3(tiles), dim3(kTcThreads), tc_smem_bytes<QT>(), p, maps)));
    return LV_OK;
}

static int launch_gemm_tc(lv_ctx* ctx, GemmTcParams& p, const __half* xh, int wtype) {
    LV_REQUIRE(wtype == T_Q4_0 || wtype == T_Q8_0, "matrix type must be q4_0 (2) or q8_0 (8)");
    return wtype == T_Q4_0 ? launch_gemm_tc_typed<T_Q4_0>(ctx, p, xh) : launch_gemm_tc_typed<T_Q8_0>(ctx, p, xh);
}

}  // namespace lv

using namespace lv;

extern "C" size_t lv_act_split_bytes(uint32_t cols, uint32_t batch) {
    return size_t(2) * ((batch + 15u) & ~15u) * cols * sizeof(__half);
}

extern "C" int lv_gemm_tc_set_exact(lv_ctx* ctx, int exact) {
    LV_ENTER(ctx);
    ctx->tc_exact = exact != 0;
    return LV_OK;
}

extern "C" int lv_act_split_f16_padded(lv_ctx* ctx, void* xh, const float* x, const float* norm_w, uint32_t cols_used, uint32_t cols,
                                       uint32_t batch) {
    LV_ENTER(ctx);
    LV_REQUIRE(xh && x && cols && batch >= 1 && batch <= uint32_t(kTcMaxZ), "bad act_split arguments");
    LV_REQUIRE(cols_used != 0 && cols_used <= cols && cols_used % 8 == 0 && cols % 64 == 0, "act_split: cols a multiple of 64, cols_used of 8 and at most cols");
    LV_REQUIRE(norm_w == nullptr || cols_used == cols, "act_split: a normalised input has no padding");
    const uint32_t zpad = (batch + 15u) & ~15u;
    LV_CUDA(launch_pdl(ctx, act_split_kernel, dim3(zpad), dim3(512), 0, static_cast<__half*>(xh), x, norm_w, cols, cols_used, batch, zpad));
    return LV_OK;
}

extern "C" int lv_act_split_f16(lv_ctx* ctx, void* xh, const float* x, const float* norm_w, uint32_t cols, uint32_t batch) {
    return lv_act_split_f16_padded(ctx, xh, x, norm_w, cols, cols, batch);
}

extern "C" int lv_gemm_tc(lv_ctx* ctx, float* out, const void* W, int wtype, const void* xh, uint32_t rows, uint32_t cols,
                          uint32_t batch, int add) {
    LV_ENTER(ctx);
    LV_REQUIRE(out && W, "null argument");
    GemmTcParams p{};
    p.m[0] = {static_cast<const uint8_t*>(W), nullptr, out, rows, add ? EPI_ADD : EPI_STORE};
    p.n_mat = 1;
    p.K = cols;
    p.Z = batch;
    p.err = ctx->d_err;
    return launch_gemm_tc(ctx, p, static_cast<const __half*>(xh), wtype);
}

extern "C" int lv_gemm_tc_silu(lv_ctx* ctx, float* out, const void* w3, const void* w1, int wtype, const void* xh, uint32_t ff,
                               uint32_t dim, uint32_t batch) {
    LV_ENTER(ctx);
    LV_REQUIRE(out && w3 && w1, "null argument");
    GemmTcParams p{};
    p.m[0] = {static_cast<const uint8_t*>(w3), static_cast<const uint8_t*>(w1), out, ff, EPI_STORE};
    p.n_mat = 1;
    p.K = dim;
    p.Z = batch;
    p.err = ctx->d_err;
    return launch_gemm_tc(ctx, p, static_cast<const __half*>(xh), wtype);
}

extern "C" int lv_gemm_tc_qkv_kvappend(lv_ctx* ctx, float* q_out, void* k_cache, void* v_cache, const void* wq, const void* wk,
                                       const void* wv, int wtype, const void* xh, const uint32_t* pos, uint32_t rows_each,
                                       uint32_t dim, uint32_t batch, uint32_t ctx_rows) {
    LV_ENTER(ctx);
    LV_REQUIRE(q_out && k_cache && v_cache && wq && wk && wv && pos, "null argument");
    LV_REQUIRE(ctx_rows >= batch, "cache smaller than the batch");
    GemmTcParams p{};
    p.m[0] = {static_cast<const uint8_t*>(wk), nullptr, k_cache, rows_each, EPI_STORE_F16_AT_POS};
    p.m[1] = {static_cast<const uint8_t*>(wq), nullptr, q_out, rows_each, EPI_STORE};
    p.m[2] = {static_cast<const uint8_t*>(wv), nullptr, v_cache, rows_each, EPI_STORE_F16_AT_POS};
    p.n_mat = 3;
    p.pos = pos;
    p.ctx_rows = ctx_rows;
    p.K = dim;
    p.Z = batch;
    p.err = ctx->d_err;
    return launch_gemm_tc(ctx, p, static_cast<const __half*>(xh), wtype);
}

extern "C" int lv_gemm_tc_qkv_kvappend_group(lv_ctx* ctx, float* q_out, const void* wq, const void* wk, const void* wv, int wtype,
                                             const void* xh, const lv_group_member* members, uint32_t rows_each, uint32_t dim,
                                             uint32_t n, uint32_t ctx_rows) {
    LV_ENTER(ctx);
    LV_REQUIRE(q_out && wq && wk && wv && members, "null argument");
    GemmTcParams p{};
    // the cache pointers come from the members; `out` of the two cache matrices only has to be non-null
    p.m[0] = {static_cast<const uint8_t*>(wk), nullptr, q_out, rows_each, EPI_STORE_F16_AT_POS};
    p.m[1] = {static_cast<const uint8_t*>(wq), nullptr, q_out, rows_each, EPI_STORE};
    p.m[2] = {static_cast<const uint8_t*>(wv), nullptr, q_out, rows_each, EPI_STORE_F16_AT_POS};
    p.n_mat = 3;
    p.group = members;
    p.ctx_rows = ctx_rows;
    p.K = dim;
    p.Z = n;
    p.err = ctx->d_err;
    return launch_gemm_tc(ctx, p, static_cast<const __half*>(xh), wtype);
}
