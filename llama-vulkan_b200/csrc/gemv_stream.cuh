// Warp-level streaming GEMV over GGML q4_0 / q8_0 block rows (ggjt v3 layout,
// f16 scale followed by 16 nibble bytes or 32 int8).
//
// Replaces the reference's matmul.glsl / matmul_q8.glsl / matmul_silu_ff*.comp
// family.  Each warp owns a private two-stage ring in shared memory that it
// fills with bulk (TMA) copies of four "row streams" (four consecutive rows,
// or two rows of each of two matrices for the SiLU-gated pair) and drains with
// all 32 lanes: a lane handles a pair of adjacent blocks (36 B / 68 B, an odd
// number of 32-bit words, hence bank-conflict free), keeps the 64 matching
// activations in registers and reuses them for all four streams.  Nibbles are
// widened in registers, accumulation is fp32, the block scale multiplies the
// 32-term partial sum once (as the reference shaders do), lanes are combined by
// shuffles in a fixed order.
#pragma once

#include "common.cuh"

namespace lv {

constexpr int kGemvWarps = 8;              // consumer warps per CTA
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kStreams = 4;                // row streams per work item
constexpr int kStages = 2;                 // ring depth per warp
constexpr int kStageBytes = 9216;          // 4 streams x 2304 B
constexpr int kXPad = 36;                  // floats per activation block in shared memory (32 + 4 pad)

template <int QT> struct QTraits;
template <> struct QTraits<T_Q4_0> {
    static constexpr int kBlockBytes = kQ4BlockBytes;
    static constexpr int kSegBlocks = 128;                  // blocks per row segment (2304 B)
    static constexpr int kPairWords = 9;
};
template <> struct QTraits<T_Q8_0> {
    static constexpr int kBlockBytes = kQ8BlockBytes;
    static constexpr int kSegBlocks = 64;                   // 2176 B
    static constexpr int kPairWords = 17;
};

// What to do with a finished row.
enum : int { EPI_STORE = 0, EPI_ADD = 1, EPI_STORE_F16_AT_POS = 2 };

struct GemvMatrix {
    const uint8_t* w;      // first matrix (w3 for the SiLU pair)
    const uint8_t* w_gate; // second matrix of the SiLU pair (w1), else null
    void* out;             // f32 [batch][rows] or f16 cache [ctx][rows]
    uint32_t rows;
    int epilogue;
};

struct GemvParams {
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

// 32 dequantised-weight x activation products of one q4_0 block.  `q` holds the
// 16 nibble bytes: byte j carries element j (low nibble) and j+16 (high).
__device__ __forceinline__ float dot_block_q4(const uint32_t (&q)[4], const float* __restrict__ x) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t lo = q[k] & 0x0f0f0f0fu;
        const uint32_t hi = (q[k] >> 4) & 0x0f0f0f0fu;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // byte j -> 0x4B0000nn = 2^23 + n; subtracting 2^23 + 8 gives n - 8 exactly
            const float fl = __uint_as_float(__byte_perm(lo, 0x4b000000u, 0x7540 + j)) - 8388616.0f;
            const float fh = __uint_as_float(__byte_perm(hi, 0x4b000000u, 0x7540 + j)) - 8388616.0f;
            s = fmaf(fl, x[4 * k + j], s);
            s = fmaf(fh, x[16 + 4 * k + j], s);
        }
    }
    return s;
}

// Same for one q8_0 block: 32 signed bytes in element order.
__device__ __forceinline__ float dot_block_q8(const uint32_t (&q)[8], const float* __restrict__ x) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const uint32_t biased = q[k] ^ 0x80808080u;      // byte + 128
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float f = __uint_as_float(__byte_perm(biased, 0x4b000000u, 0x7540 + j)) - 8388736.0f;   // 2^23 + 128
            s = fmaf(f, x[4 * k + j], s);
        }
    }
    return s;
}

// Partial dot product of one lane's block pair for one row stream.
template <int QT>
__device__ __forceinline__ float dot_pair(const uint32_t* __restrict__ sw, const float (&x)[64]) {
    if constexpr (QT == T_Q4_0) {
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
        const float d0 = half_bits_to_float(w[0] & 0xffffu);
        const float d1 = half_bits_to_float(w[4] >> 16);
        return dot_block_q4(q0, &x[0]) * d0 + dot_block_q4(q1, &x[32]) * d1;
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
        const float d0 = half_bits_to_float(w[0] & 0xffffu);
        const float d1 = half_bits_to_float(w[8] >> 16);
        return dot_block_q8(q0, &x[0]) * d0 + dot_block_q8(q1, &x[32]) * d1;
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

// Copies activations into the padded shared layout (block b at float b*kXPad).
// With norm_w the reference's normalisation is applied on the way
// (shaders/normalize.comp:39-63): m = mean(x), v = mean((x-m)^2),
// out = x * w * rsqrt(v); no epsilon, numerator not centred.
__device__ __forceinline__ void stage_activations(float* __restrict__ xs, const float* __restrict__ x,
                                                  const float* __restrict__ norm_w, uint32_t K, float* scratch) {
    float factor = 1.f;
    if (norm_w != nullptr) {
        float part = 0.f;
        for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) part += x[i];
        const float mean = block_sum(part, scratch) / static_cast<float>(K);
        part = 0.f;
        for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) {
            const float c = x[i] - mean;
            part = fmaf(c, c, part);
        }
        factor = 1.0f / sqrtf(block_sum(part, scratch) / static_cast<float>(K));
    }
    for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) {
        float v = x[i];
        if (norm_w != nullptr) v = (v * norm_w[i]) * factor;
        xs[(i >> 5) * kXPad + (i & 31)] = v;
    }
}

}  // namespace lv
