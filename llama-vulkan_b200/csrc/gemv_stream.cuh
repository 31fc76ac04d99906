// Warp-level streaming GEMV over GGML q4_0 / q8_0 block rows (ggjt v3 layout,
// f16 scale followed by 16 nibble bytes or 32 int8).
//
// Replaces the reference's matmul.glsl / matmul_q8.glsl / matmul_silu_ff*.comp
// family.  Each warp owns a private two-stage ring in shared memory that it
// fills with bulk (TMA) copies of its "row streams" (consecutive rows, or rows
// of the two matrices of the SiLU-gated pair) and drains with all 32 lanes: a
// lane handles a pair of adjacent blocks (36 B / 68 B, an odd number of 32-bit
// words, hence bank-conflict free).
//
// Arithmetic.  B200 has about three issue slots per weight at the HBM
// roofline, so widening every nibble to fp32 cannot keep up.  Instead each
// block of 32 activations is turned, once per CTA, into fixed point
// X_e = rint(x_e * S / max|x|), S = 31 * 2^16, split into three balanced
// base-256 digits (X = a*2^16 + b*2^8 + c, every digit an int8, |a| <= 32), and
// the inner sums sum_e q_e * X_e are formed exactly in int32 with dp4a (the
// bound on a keeps 15 * 32 * |X| below 2^31).  The block result is converted
// to fp32 once and multiplied by d * max|x| / S; rows are accumulated in fp32
// and lanes combined by shuffles in a fixed order.  The only rounding beyond
// fp32 is that of x_e to about 22 bits relative to its block maximum, of the
// order of the reordering noise of an fp32 accumulation.
#pragma once

#include "common.cuh"

namespace lv {

constexpr int kStages = 2;                 // ring depth per warp
constexpr int kSegBlocks = 64;             // blocks of one row per stage (32 lane pairs)
constexpr int kPairBytes = 208;            // activation record of one block pair in shared memory:
                                           //   a[64] b[64] c[64] int8, T8[2] int32, scale[2] f32
constexpr int kMaxStreams = 4;

template <int QT> struct QTraits;
template <> struct QTraits<T_Q4_0> {
    static constexpr int kBlockBytes = kQ4BlockBytes;
    static constexpr int kPairWords = 9;
    static constexpr int kWarps = 16;                 // consumer warps per CTA
};
template <> struct QTraits<T_Q4_0_V1> {
    static constexpr int kBlockBytes = kQ4V1BlockBytes;
    static constexpr int kPairWords = 10;                // an even stride: two lanes share a bank (the layout of old files; not tuned)
    static constexpr int kWarps = 16;
};
template <> struct QTraits<T_Q8_0> {
    static constexpr int kBlockBytes = kQ8BlockBytes;
    static constexpr int kPairWords = 17;
    static constexpr int kWarps = 8;
};

// largest fixed-point magnitude of an activation: top digit at most 31 (32 after the rounding
// slack of the approximate reciprocal)
constexpr float kFixedOne = 31.0f * 65536.0f;

// What to do with a finished row.
enum : int { EPI_STORE = 0, EPI_ADD = 1, EPI_STORE_F16_AT_POS = 2 };

struct GemvMatrix {
    const uint8_t* w;      // first matrix (w3 for the SiLU pair)
    const uint8_t* w_gate; // second matrix of the SiLU pair (w1), else null
    void* out;             // f32 [batch][rows] or f16 cache [ctx][rows]
    uint32_t rows;
    int epilogue;
};

// Tensor-parallel exchange fused into the GEMV (see comm_peer.cu for the window layout).
// A producer launch (push_exchange >= 0) sends its finished row sums -- this rank's partial
// products -- into its slot of every rank's receive window instead of storing them, and
// publishes one flag per CTA.  A consumer launch (pull_exchange >= 0) waits for the flags of
// all ranks in its own window and builds its input as x + sum over ranks of the slots.
constexpr int kTpMaxRanks = 8;
constexpr int kTpSlotSets = 4;         // slot sets of a window: 0 and 1 alternate for the exchanges fused into the GEMVs,
                                       // 2 and 3 for the stand-alone all-reduce kernel, so the two never share a slot
constexpr int kTpFlagCtas = 256;       // flags per (exchange parity, source rank)
constexpr int kTpLegacyFlagWords = 512; // flag words of the stand-alone all-reduce kernel that precede these
constexpr int kTpTwoPhaseRanks = 64;   // ranks from which a consumer launch would sum the slots once per GPU instead of once per CTA:
                                       // never by default -- on 2 GPUs the extra intra-GPU flag round costs 5 us per exchange

struct TpParams {
    float* window[kTpMaxRanks];   // window[r]: rank r's receive window as seen from this GPU
    int rank, n_ranks;            // n_ranks == 0: no exchange in this launch
    uint32_t capacity;            // floats per slot
    const uint32_t* step;         // device word: evaluation steps completed by this context
    uint32_t epochs_per_step;     // exchanges in one step; epoch = step * epochs_per_step + exchange + 1
    int push_exchange;            // producer side, -1 = none
    int pull_exchange;            // consumer side, -1 = none
    uint32_t pull_ctas;           // CTAs of the producer launch of the consumed exchange
    float* x_out;                 // consumer: the summed input is stored here (the new residual stream)
    uint32_t two_phase;           // consumer: sum the slots once per GPU (slice per CTA + local flags) instead of in every CTA
};

__device__ __forceinline__ float* tp_slot(const TpParams& t, int r_window, int exchange, int src) {
    return t.window[r_window] + (size_t(exchange & 1) * t.n_ranks + src) * t.capacity;
}

__device__ __forceinline__ uint32_t* tp_flag(const TpParams& t, int r_window, int exchange, int src, uint32_t cta) {
    uint32_t* flags = reinterpret_cast<uint32_t*>(t.window[r_window] + size_t(kTpSlotSets) * t.n_ranks * t.capacity) + kTpLegacyFlagWords;
    return flags + (size_t(exchange & 1) * kTpMaxRanks + src) * kTpFlagCtas + cta;
}

// Flag of CTA `cta` of a consumer launch on this GPU: its slice of the summed input is in x_out.
__device__ __forceinline__ uint32_t* tp_local_flag(const TpParams& t, uint32_t cta) {
    uint32_t* flags = reinterpret_cast<uint32_t*>(t.window[t.rank] + size_t(kTpSlotSets) * t.n_ranks * t.capacity) + kTpLegacyFlagWords;
    return flags + size_t(2) * kTpMaxRanks * kTpFlagCtas + cta;
}

__device__ __forceinline__ uint32_t tp_epoch(const TpParams& t, int exchange) {
    return *t.step * t.epochs_per_step + uint32_t(exchange) + 1u;
}

struct GemvParams {
    TpParams tp;
    GemvMatrix m[3];
    int n_mat;
    const float* x;          // [batch][K]
    const float* norm_w;     // non-null: x is normalised first (normalize.comp arithmetic)
    const uint32_t* pos;     // device word: tokens already in the cache
    uint32_t K;              // columns
    uint32_t row_bytes;
    uint32_t ctx_rows;       // rows of the f16 caches (bound for *pos + z)
    uint32_t* err;
};

__device__ __forceinline__ int dp4a_us(uint32_t a_u8x4, uint32_t b_s8x4, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_s8x4), "r"(c));
    return d;
}

__device__ __forceinline__ int dp4a_ss(uint32_t a_s8x4, uint32_t b_s8x4, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_s8x4), "r"(b_s8x4), "r"(c));
    return d;
}

// Activation record of one block pair as a lane holds it in registers.
struct PairX {
    uint32_t a[16], b[16], c[16];   // digit words: [0..7] block 0 (elements 4k..4k+3), [8..15] block 1
    int t8[2];                      // 8 * sum_e X_e per block (the q4_0 offset of 8, folded in once)
    float scale[2];                 // max|x| / 2^F per block
};

__device__ __forceinline__ void load_pair_x(PairX& px, const uint8_t* __restrict__ rec) {
    const uint4* r = reinterpret_cast<const uint4*>(rec);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 va = r[i], vb = r[4 + i], vc = r[8 + i];
        px.a[4 * i] = va.x; px.a[4 * i + 1] = va.y; px.a[4 * i + 2] = va.z; px.a[4 * i + 3] = va.w;
        px.b[4 * i] = vb.x; px.b[4 * i + 1] = vb.y; px.b[4 * i + 2] = vb.z; px.b[4 * i + 3] = vb.w;
        px.c[4 * i] = vc.x; px.c[4 * i + 1] = vc.y; px.c[4 * i + 2] = vc.z; px.c[4 * i + 3] = vc.w;
    }
    const uint4 meta = r[12];
    px.t8[0] = int(meta.x); px.t8[1] = int(meta.y);
    px.scale[0] = __uint_as_float(meta.z); px.scale[1] = __uint_as_float(meta.w);
}

// sum_e (nibble_e - 8) * X_e of one q4_0 block, exactly.  q: the 16 nibble bytes
// (byte j carries element j in the low and element j + 16 in the high nibble).
__device__ __forceinline__ int block_sum_q4(const uint32_t (&q)[4], const uint32_t* __restrict__ a,
                                            const uint32_t* __restrict__ b, const uint32_t* __restrict__ c, int t8) {
    int al = 0, bl = 0, cl = 0, ah = 0, bh = 0, ch = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t lo = q[k] & 0x0f0f0f0fu;          // elements 4k..4k+3
        const uint32_t hi = q[k] & 0xf0f0f0f0u;          // elements 16+4k.., scaled by 16
        al = dp4a_us(lo, a[k], al); bl = dp4a_us(lo, b[k], bl); cl = dp4a_us(lo, c[k], cl);
        ah = dp4a_us(hi, a[4 + k], ah); bh = dp4a_us(hi, b[4 + k], bh); ch = dp4a_us(hi, c[4 + k], ch);
    }
    // the high-nibble sums are exact multiples of 16
    const int hi_ab = (ah * 256 + bh) >> 4;
    return ((al * 256 + bl + hi_ab) * 256 + cl + (ch >> 4)) - t8;
}

// sum_e int8_e * X_e of one q8_0 block.  The exact integer can exceed 2^31, so the two upper
// digits and the lowest one are converted separately (the first conversion rounds to 24 bits,
// like any fp32 accumulation would).
__device__ __forceinline__ float block_sum_q8(const uint32_t (&q)[8], const uint32_t* __restrict__ a,
                                              const uint32_t* __restrict__ b, const uint32_t* __restrict__ c) {
    int sa = 0, sb = 0, sc = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        sa = dp4a_ss(q[k], a[k], sa); sb = dp4a_ss(q[k], b[k], sb); sc = dp4a_ss(q[k], c[k], sc);
    }
    return fmaf(static_cast<float>(sa * 256 + sb), 256.0f, static_cast<float>(sc));
}

// Contribution of one lane's block pair to one row stream.
template <int QT>
__device__ __forceinline__ float dot_pair(const uint32_t* __restrict__ sw, const PairX& px) {
    if constexpr (QT == T_Q4_0_V1) {
        // ggjt v1 (llava_buffer.cpp:350-359): words 0 and 5 are the f32 scales, byte j of a block holds elements 2j and 2j+1.
        // The records keep the elements in natural order, four per word; the low nibbles of a weight word meet the even
        // elements of two record words, the high nibbles the odd ones.
        uint32_t w[10];
#pragma unroll
        for (int i = 0; i < 10; ++i) w[i] = sw[i];
        float out = 0.f;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            const uint32_t* q = &w[5 * blk + 1];
            const uint32_t* a = &px.a[8 * blk];
            const uint32_t* b = &px.b[8 * blk];
            const uint32_t* c = &px.c[8 * blk];
            int al = 0, bl = 0, cl = 0, ah = 0, bh = 0, ch = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                // word k: bytes 4k..4k+3 = elements 8k..8k+7, which the natural-order records hold in words 2k and 2k+1
                // (v3 layout of px: words 0..3 elements 0..15, words 4..7 elements 16..31)
                const int r0 = 2 * k, r1 = 2 * k + 1;
                const uint32_t lo = q[k] & 0x0f0f0f0fu, hi = q[k] & 0xf0f0f0f0u;
                const uint32_t ae = __byte_perm(a[r0], a[r1], 0x6420), ao = __byte_perm(a[r0], a[r1], 0x7531);
                const uint32_t be = __byte_perm(b[r0], b[r1], 0x6420), bo = __byte_perm(b[r0], b[r1], 0x7531);
                const uint32_t ce = __byte_perm(c[r0], c[r1], 0x6420), co = __byte_perm(c[r0], c[r1], 0x7531);
                al = dp4a_us(lo, ae, al); bl = dp4a_us(lo, be, bl); cl = dp4a_us(lo, ce, cl);
                ah = dp4a_us(hi, ao, ah); bh = dp4a_us(hi, bo, bh); ch = dp4a_us(hi, co, ch);
            }
            const int hi_ab = (ah * 256 + bh) >> 4;
            const int sum = ((al * 256 + bl + hi_ab) * 256 + cl + (ch >> 4)) - px.t8[blk];
            out = fmaf(static_cast<float>(sum), __uint_as_float(w[5 * blk]) * px.scale[blk], out);
        }
        return out;
    } else if constexpr (QT == T_Q4_0) {
        uint32_t w[9];
#pragma unroll
        for (int i = 0; i < 9; ++i) w[i] = sw[i];
        // block 0: bytes 0-1 scale, 2-17 nibbles; block 1: bytes 18-19 scale, 20-35 nibbles
        uint32_t q0[4], q1[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            q0[k] = __funnelshift_r(w[k], w[k + 1], 16);
            q1[k] = w[5 + k];
        }
        const float d0 = half_bits_to_float(w[0] & 0xffffu) * px.scale[0];
        const float d1 = half_bits_to_float(w[4] >> 16) * px.scale[1];
        const int i0 = block_sum_q4(q0, &px.a[0], &px.b[0], &px.c[0], px.t8[0]);
        const int i1 = block_sum_q4(q1, &px.a[8], &px.b[8], &px.c[8], px.t8[1]);
        return fmaf(static_cast<float>(i0), d0, static_cast<float>(i1) * d1);
    } else {
        uint32_t w[17];
#pragma unroll
        for (int i = 0; i < 17; ++i) w[i] = sw[i];
        // block 0: bytes 0-1 scale, 2-33 int8; block 1: bytes 34-35 scale, 36-67 int8
        uint32_t q0[8], q1[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            q0[k] = __funnelshift_r(w[k], w[k + 1], 16);
            q1[k] = w[9 + k];
        }
        const float d0 = half_bits_to_float(w[0] & 0xffffu) * px.scale[0];
        const float d1 = half_bits_to_float(w[8] >> 16) * px.scale[1];
        const float f0 = block_sum_q8(q0, &px.a[0], &px.b[0], &px.c[0]);
        const float f1 = block_sum_q8(q1, &px.a[8], &px.b[8], &px.c[8]);
        return fmaf(f0, d0, f1 * d1);
    }
}

// Sums four per-lane values across the warp.  Afterwards lanes 8s..8s+7 hold
// the total of value s.  Fixed combination order, hence deterministic.
__device__ __forceinline__ float warp_sum4(float a0, float a1, float a2, float a3, int lane) {
    const bool up16 = lane & 16;
    float s0 = up16 ? a2 : a0, s1 = up16 ? a3 : a1;
    const float t0 = up16 ? a0 : a2, t1 = up16 ? a1 : a3;
    s0 += __shfl_xor_sync(0xffffffffu, t0, 16);
    s1 += __shfl_xor_sync(0xffffffffu, t1, 16);
    const bool up8 = lane & 8;
    float u = up8 ? s1 : s0;
    const float v = up8 ? s0 : s1;
    u += __shfl_xor_sync(0xffffffffu, v, 8);
    u += __shfl_xor_sync(0xffffffffu, u, 4);
    u += __shfl_xor_sync(0xffffffffu, u, 2);
    u += __shfl_xor_sync(0xffffffffu, u, 1);
    return u;
}

// Same for two values: lanes 0-15 end up with the total of a0, lanes 16-31 with a1.
__device__ __forceinline__ float warp_sum2(float a0, float a1, int lane) {
    const bool up16 = lane & 16;
    float u = up16 ? a1 : a0;
    const float v = up16 ? a0 : a1;
    u += __shfl_xor_sync(0xffffffffu, v, 16);
    u += __shfl_xor_sync(0xffffffffu, u, 8);
    u += __shfl_xor_sync(0xffffffffu, u, 4);
    u += __shfl_xor_sync(0xffffffffu, u, 2);
    u += __shfl_xor_sync(0xffffffffu, u, 1);
    return u;
}

// Three balanced base-256 digits of four fixed-point values, packed as int8x4 words.
// Adding 128 * (2^16 + 2^8 + 1) makes every digit of the sum non-negative, so the digits are
// the bytes of the sum; flipping bit 7 of each byte subtracts the 128 again and leaves int8
// digits whose weighted sum is the original value.
__device__ __forceinline__ void digit_words(int X0, int X1, int X2, int X3, uint32_t& wa, uint32_t& wb, uint32_t& wc) {
    constexpr int kBias = 128 * (65536 + 256 + 1);
    const uint32_t Y0 = uint32_t(X0 + kBias), Y1 = uint32_t(X1 + kBias), Y2 = uint32_t(X2 + kBias), Y3 = uint32_t(X3 + kBias);
    const uint32_t p01 = __byte_perm(Y0, Y1, 0x5140), p23 = __byte_perm(Y2, Y3, 0x5140);   // (c0 c1 b0 b1), (c2 c3 b2 b3)
    const uint32_t q01 = __byte_perm(Y0, Y1, 0x0062), q23 = __byte_perm(Y2, Y3, 0x0062);   // (a0 a1 . .), (a2 a3 . .)
    wc = __byte_perm(p01, p23, 0x5410) ^ 0x80808080u;
    wb = __byte_perm(p01, p23, 0x7632) ^ 0x80808080u;
    wa = __byte_perm(q01, q23, 0x5410) ^ 0x80808080u;
}

// Builds the activation records of all K/64 block pairs in shared memory.
// A thread owns four consecutive elements (one 16-byte load), eight adjacent
// lanes own a block.  Everything a thread needs is fetched before anything
// depends on it, so the vector costs one trip to L2.
//
// With norm_w the reference's normalisation (shaders/normalize.comp:39-63:
// m = mean(x), v = mean((x-m)^2), out = x * w * rsqrt(v); no epsilon, numerator
// not centred) is split in two.  The records hold x * w: the fixed-point digits
// of a block do not change when the whole vector is multiplied by a constant,
// only the block scales do.  The constant rsqrt(v) multiplies the finished row
// sums instead (norm_factor below), which takes the block-wide reduction and
// the square root off the path to the first weight.  Mean and variance come
// from one pass over values shifted by x[0] (sum d, sum d^2 with d = x - x[0]),
// which is the same quantity without the cancellation of sum x^2 - n*mean^2.
// `scratch` holds 64 floats: the per-warp partial sums.
constexpr int kActIters = 7;     // float4s per thread held at once (7 * 2048 >= 13824 with 16 warps)

// Contribution of four consecutive elements to the sums from which norm_factor() forms the variance:
// s1 += sum d, s2 += sum d^2 with d = x - x0 (any x0 gives the same variance; one near the data avoids
// the cancellation of sum x^2 - n * mean^2).
__device__ __forceinline__ void norm_accumulate(const float4& v, float x0, float& s1, float& s2) {
    const float a = v.x - x0, b = v.y - x0, c = v.z - x0, d = v.w - x0;
    s1 += (a + b) + (c + d);
    s2 += (a * a + b * b) + (c * c + d * d);
}

// Per-warp sums go to scratch ([0..31] sum d, [32..63] sum d^2); norm_factor() adds them up after a CTA barrier.
__device__ __forceinline__ void norm_publish(float s1, float s2, float* scratch) {
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if ((threadIdx.x & 31) == 0) { scratch[threadIdx.x >> 5] = s1; scratch[32 + (threadIdx.x >> 5)] = s2; }
}

// Writes this thread's part of the activation record of the block that holds elements e .. e+3 (e a multiple
// of 4; the eight lanes that own a block call this together).
__device__ __forceinline__ void emit_block_record(uint8_t* __restrict__ xrec, const float4& v, uint32_t e, int lane) {
    float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
    // an approximate quotient is enough: the record keeps whatever integers come out, and
    // their scale is off by an fp32 rounding or two at most
    const float inv = m > 1e-30f ? __fdividef(kFixedOne, m) : 0.f;     // smaller blocks count as zero
    const int X0 = __float2int_rn(v.x * inv), X1 = __float2int_rn(v.y * inv);   // |X| <= 31 * 2^16 (+ slack)
    const int X2 = __float2int_rn(v.z * inv), X3 = __float2int_rn(v.w * inv);
    uint32_t wa, wb, wc;
    digit_words(X0, X1, X2, X3, wa, wb, wc);
    int T = (X0 + X1) + (X2 + X3);
    T += __shfl_xor_sync(0xffffffffu, T, 1);
    T += __shfl_xor_sync(0xffffffffu, T, 2);
    T += __shfl_xor_sync(0xffffffffu, T, 4);
    const uint32_t blk = e >> 5;
    uint8_t* rec = xrec + size_t(blk >> 1) * kPairBytes;
    const uint32_t at = (blk & 1) * 32 + (lane & 7) * 4;
    *reinterpret_cast<uint32_t*>(rec + at) = wa;
    *reinterpret_cast<uint32_t*>(rec + 64 + at) = wb;
    *reinterpret_cast<uint32_t*>(rec + 128 + at) = wc;
    if ((lane & 7) == 0) {
        reinterpret_cast<int*>(rec + 192)[blk & 1] = 8 * T;
        reinterpret_cast<float*>(rec + 200)[blk & 1] = m * (1.0f / kFixedOne);
    }
}

__device__ __forceinline__ void stage_activations(uint8_t* __restrict__ xrec, const float* __restrict__ x,
                                                  const float* __restrict__ norm_w, uint32_t K, float* scratch,
                                                  const TpParams& tp, bool sum_slots) {
    const int lane = threadIdx.x & 31;
    const uint32_t stride = blockDim.x * 4;
    const bool pull = sum_slots && tp.n_ranks > 0 && tp.pull_exchange >= 0;

    for (uint32_t chunk = 0; chunk < K; chunk += stride * kActIters) {
        float4 v[kActIters], w[kActIters];
#pragma unroll
        for (int i = 0; i < kActIters; ++i) {
            const uint32_t e = chunk + uint32_t(i) * stride + threadIdx.x * 4;
            v[i] = e < K ? *reinterpret_cast<const float4*>(x + e) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (pull) {
            // input = x + the partial products of all ranks, added in rank order (the same bits on every
            // rank); the slots are read from L2, where the peers' stores land
            float4 sum[kActIters];
#pragma unroll
            for (int i = 0; i < kActIters; ++i) sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < tp.n_ranks; ++r) {
                const float* slot = tp_slot(tp, tp.rank, tp.pull_exchange, r);
#pragma unroll
                for (int i = 0; i < kActIters; ++i) {
                    const uint32_t e = chunk + uint32_t(i) * stride + threadIdx.x * 4;
                    if (e < K) {
                        const float4 t = __ldcg(reinterpret_cast<const float4*>(slot + e));
                        sum[i].x += t.x; sum[i].y += t.y; sum[i].z += t.z; sum[i].w += t.w;
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < kActIters; ++i) {
                const uint32_t e = chunk + uint32_t(i) * stride + threadIdx.x * 4;
                v[i].x += sum[i].x; v[i].y += sum[i].y; v[i].z += sum[i].z; v[i].w += sum[i].w;
                if (e < K && blockIdx.x == 0 && blockIdx.y == 0 && tp.x_out != nullptr) *reinterpret_cast<float4*>(tp.x_out + e) = v[i];
            }
        }
        if (norm_w != nullptr) {
            // normalised inputs have length dim, which always fits one chunk
            const float x0 = x[0];
#pragma unroll
            for (int i = 0; i < kActIters; ++i) {
                const uint32_t e = chunk + uint32_t(i) * stride + threadIdx.x * 4;
                w[i] = e < K ? *reinterpret_cast<const float4*>(norm_w + e) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float s1 = 0.f, s2 = 0.f;
#pragma unroll
            for (int i = 0; i < kActIters; ++i) {
                if (chunk + uint32_t(i) * stride + threadIdx.x * 4 < K) norm_accumulate(v[i], x0, s1, s2);
            }
            norm_publish(s1, s2, scratch);
#pragma unroll
            for (int i = 0; i < kActIters; ++i) {
                v[i].x *= w[i].x; v[i].y *= w[i].y; v[i].z *= w[i].z; v[i].w *= w[i].w;
            }
        }
#pragma unroll
        for (int i = 0; i < kActIters; ++i) {
            const uint32_t e = chunk + uint32_t(i) * stride + threadIdx.x * 4;
            if (e >= K) break;              // K is a multiple of 32: the eight lanes of a block leave together
            emit_block_record(xrec, v[i], e, lane);
        }
    }
}

// rsqrt of the variance from the partial sums stage_activations left in scratch; call after a
// CTA barrier.  The warps' sums are added in warp order, so every thread gets the same bits.
__device__ __forceinline__ float norm_factor(const float* scratch, uint32_t K) {
    const int nwarps = (blockDim.x + 31) >> 5;
    float s1 = 0.f, s2 = 0.f;
    for (int w = 0; w < nwarps; ++w) { s1 += scratch[w]; s2 += scratch[32 + w]; }
    const float md = s1 / static_cast<float>(K);                          // mean - x[0]
    const float var = s2 / static_cast<float>(K) - md * md;
    return 1.0f / sqrtf(var);
}

}  // namespace lv
