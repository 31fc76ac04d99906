// Small element-wise and reduction kernels: normalisation, cache append, copy,
// add, embedding-row dequantisation, argmax.
#include <algorithm>

#include "common.cuh"
#include "ctx.h"

namespace lv {

// shaders/normalize.comp:34-63: one CTA per batch row.
__global__ void __launch_bounds__(1024) norm_kernel(float* __restrict__ out, const float* __restrict__ x,
                                                    const float* __restrict__ w, uint32_t dim) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[64];
    const float* xr = x + size_t(blockIdx.x) * dim;
    float* orow = out + size_t(blockIdx.x) * dim;
    float part = 0.f;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) part += xr[i];
    const float mean = block_sum(part, scratch) / static_cast<float>(dim);
    part = 0.f;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) {
        const float c = xr[i] - mean;
        part = fmaf(c, c, part);
    }
    const float factor = 1.0f / sqrtf(block_sum(part, scratch) / static_cast<float>(dim));   // no epsilon
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) orow[i] = (xr[i] * w[i]) * factor;
}

// shaders/copy_to_cache.comp:29-37
__global__ void kv_append_kernel(__half* __restrict__ cache, const float* __restrict__ x, const uint32_t* __restrict__ pos,
                                 uint32_t dim, uint32_t ctx_rows, uint32_t* err) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t z = blockIdx.y;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t row = *pos + z;
    if (row >= ctx_rows) {               // never write outside the cache
        if (i == 0) atomicOr(err, ERR_BAD_INDEX);
        return;
    }
    if (i < dim) cache[size_t(row) * dim + i] = __float2half_rn(x[size_t(z) * dim + i]);
}

__global__ void copy_kernel(float* __restrict__ dst, const float* __restrict__ src, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) dst[i] = src[i];
}

__global__ void add_kernel(float* __restrict__ a, const float* __restrict__ b, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) a[i] += b[i];
}

// llava_buffer.cpp:360-370 (q4_0 v3), :387-394 (q8_0 v3), :377-381 (f32).
// One CTA per row; one thread per block of 32 weights.
// group != null: row z belongs to member z (its own token log and position).
__global__ void dequant_rows_kernel(float* __restrict__ out, const uint8_t* __restrict__ table, int wtype,
                                    const uint32_t* __restrict__ ids, const uint32_t* __restrict__ first, uint32_t cols,
                                    uint32_t vocab, uint32_t* err, const lv_group_member* __restrict__ group) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t z = blockIdx.x;
    uint32_t id = group != nullptr ? group[z].token_log[*group[z].pos] : ids[(first ? *first : 0u) + z];
    if (id >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, ERR_BAD_INDEX);
        id = 0;
    }
    float* o = out + size_t(z) * cols;
    if (wtype == T_F32) {
        const float* src = reinterpret_cast<const float*>(table) + size_t(id) * cols;
        for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) o[i] = src[i];
        return;
    }
    const uint32_t nb = cols / 32;
    if (wtype == T_Q4_0_V1) {       // llava_buffer.cpp:350-359: f32 scale, byte j = elements 2j (low nibble) and 2j+1
        const uint8_t* row = table + size_t(id) * nb * kQ4V1BlockBytes;
        for (uint32_t b = threadIdx.x; b < nb; b += blockDim.x) {
            const uint8_t* blk = row + size_t(b) * kQ4V1BlockBytes;
            const float d = *reinterpret_cast<const float*>(blk);
            for (int j = 0; j < 16; ++j) {
                const int qv = blk[4 + j];
                o[b * 32 + 2 * j] = static_cast<float>((qv & 0xf) - 8) * d;
                o[b * 32 + 2 * j + 1] = static_cast<float>((qv >> 4) - 8) * d;
            }
        }
        return;
    }
    const uint32_t bb = wtype == T_Q4_0 ? kQ4BlockBytes : kQ8BlockBytes;
    const uint8_t* row = table + size_t(id) * nb * bb;
    for (uint32_t b = threadIdx.x; b < nb; b += blockDim.x) {
        const uint8_t* blk = row + size_t(b) * bb;
        const float d = half_bits_to_float(uint32_t(blk[0]) | (uint32_t(blk[1]) << 8));
        if (wtype == T_Q4_0) {
            for (int j = 0; j < 16; ++j) {
                const int qv = blk[2 + j];
                o[b * 32 + j] = static_cast<float>((qv & 0xf) - 8) * d;
                o[b * 32 + j + 16] = static_cast<float>((qv >> 4) - 8) * d;
            }
        } else {
            for (int j = 0; j < 32; ++j) o[b * 32 + j] = static_cast<float>(static_cast<int8_t>(blk[2 + j])) * d;
        }
    }
}

// llava_session.cpp:144-152: m = 0; for every i: if (v[i] > v[m]) m = i.
// Equivalent parallel form: the lowest index holding the maximum of the
// non-NaN entries; 0 if v[0] is NaN (nothing compares greater than it) or if
// there is no such entry.
constexpr uint32_t kNoIndex = 0xffffffffu;

__device__ __forceinline__ void argmax_merge(float& best, uint32_t& bi, float ov, uint32_t oi) {
    if (oi == kNoIndex) return;
    if (bi == kNoIndex || ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
}

// First index of the maximum of v[0..n) over a 1024-thread CTA; the result is valid in thread 0.
// Elements that are NaN never win; kNoIndex if every element is NaN.  A thread looks at its
// elements in ascending order and keeps a candidate only on a strict improvement, and the merges
// prefer the lower index among equals, so the lowest index of the maximum comes out
// (llava_session.cpp:145-151).  All loads of a thread are issued before the first compare.
__device__ __forceinline__ uint32_t block_argmax(const float* __restrict__ v, uint32_t n, float* s_val, uint32_t* s_idx) {
    constexpr int kVec = 8;                                   // float4 loads in flight per thread
    float best = 0.f;
    uint32_t bi = kNoIndex;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(v) & 15u) == 0;
    const uint32_t n4 = vec_ok ? n / 4 : 0;
    for (uint32_t base = 0; base < n4; base += blockDim.x * kVec) {
        float4 q[kVec];
#pragma unroll
        for (int k = 0; k < kVec; ++k) {
            const uint32_t i = base + k * blockDim.x + threadIdx.x;
            q[k] = i < n4 ? __ldcg(reinterpret_cast<const float4*>(v) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < kVec; ++k) {
            const uint32_t i = base + k * blockDim.x + threadIdx.x;
            if (i < n4) {
                const float e[4] = {q[k].x, q[k].y, q[k].z, q[k].w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (e[j] == e[j] && (bi == kNoIndex || e[j] > best)) { best = e[j]; bi = 4 * i + j; }
            }
        }
    }
    for (uint32_t i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) {
        const float x = v[i];
        if (x == x && (bi == kNoIndex || x > best || (x == best && i < bi))) { best = x; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_merge(best, bi, ov, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        best = lane < nw ? s_val[lane] : 0.f;
        bi = lane < nw ? s_idx[lane] : kNoIndex;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_merge(best, bi, ov, oi);
        }
    }
    return bi;
}

// The reference returns index 0 when the scan never improves on element 0, which includes a NaN
// in element 0 (every comparison with it is false).
__device__ __forceinline__ uint32_t argmax_result(uint32_t bi, const float* v) {
    const float first = v[0];
    return (bi == kNoIndex || first != first) ? 0u : bi;
}

__global__ void __launch_bounds__(1024) argmax_kernel(uint32_t* __restrict__ out, const float* __restrict__ v, uint32_t n) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_val[32];
    __shared__ uint32_t s_idx[32];
    const uint32_t bi = block_argmax(v, n, s_val, s_idx);
    if (threadIdx.x == 0) *out = argmax_result(bi, v);
}

// argmax and the step's bookkeeping in one launch: the winner goes to token_log[old count + batch]
// (input of the next step), to *argmax_out and, when given, to a word of mapped host memory.
__global__ void __launch_bounds__(1024) argmax_advance_kernel(const float* __restrict__ v, uint32_t n, uint32_t* config,
                                                              uint32_t* token_log, uint32_t batch, uint32_t log_capacity,
                                                              uint32_t* argmax_out, volatile uint32_t* host_token, uint32_t* tp_step,
                                                              uint32_t* err) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_val[32];
    __shared__ uint32_t s_idx[32];
    const uint32_t count = threadIdx.x == 0 ? config[0] : 0u;           // in flight together with the logits
    const uint32_t bi = block_argmax(v, n, s_val, s_idx);
    if (threadIdx.x == 0) {
        const uint32_t token = argmax_result(bi, v);
        const uint32_t at = count + batch;
        if (at < log_capacity) token_log[at] = token;
        else atomicOr(err, ERR_BAD_INDEX);
        if (argmax_out != nullptr) *argmax_out = token;
        for (int i = 0; i < 4; ++i) config[i] = count + batch;
        if (tp_step != nullptr) *tp_step += 1;          // numbers the exchanges of the next step (sharded contexts)
        if (host_token != nullptr) {
            *host_token = token;
            __threadfence_system();
        }
    }
}

// The same for the members of a group step: CTA z works on logits row z and member z.
__global__ void __launch_bounds__(1024) argmax_advance_group_kernel(const float* __restrict__ logits, uint32_t n,
                                                                    const lv_group_member* __restrict__ group, uint32_t log_capacity,
                                                                    uint32_t* out_tokens, volatile uint32_t* host_tokens, uint32_t* err) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_val[32];
    __shared__ uint32_t s_idx[32];
    const uint32_t z = blockIdx.x;
    const float* v = logits + size_t(z) * n;
    const uint32_t count = threadIdx.x == 0 ? group[z].pos[0] : 0u;
    const uint32_t bi = block_argmax(v, n, s_val, s_idx);
    if (threadIdx.x == 0) {
        const uint32_t token = argmax_result(bi, v);
        if (count + 1 < log_capacity) group[z].token_log[count + 1] = token;
        else atomicOr(err, ERR_BAD_INDEX);
        for (int i = 0; i < 4; ++i) group[z].pos[i] = count + 1;
        if (out_tokens != nullptr) out_tokens[z] = token;
        if (host_tokens != nullptr) {
            host_tokens[z] = token;
            __threadfence_system();
        }
    }
}

__global__ void decode_advance_kernel(uint32_t* config, const uint32_t* argmax, uint32_t* token_log, uint32_t batch,
                                      uint32_t log_capacity, uint32_t* tp_step, uint32_t* err) {
    pdl_launch_dependents();
    pdl_wait();
    if (argmax != nullptr && token_log != nullptr) {
        const uint32_t at = config[0] + batch;
        if (at < log_capacity) token_log[at] = *argmax;
        else atomicOr(err, ERR_BAD_INDEX);
    }
    for (int i = 0; i < 4; ++i) config[i] += batch;
    if (tp_step != nullptr) *tp_step += 1;
}

}  // namespace lv

using namespace lv;

extern "C" int lv_decode_advance(lv_ctx* ctx, uint32_t* config, const uint32_t* argmax, uint32_t* token_log,
                                 uint32_t batch, uint32_t log_capacity) {
    LV_ENTER(ctx);
    LV_REQUIRE(config && batch, "bad advance arguments");
    LV_CUDA(launch_pdl(ctx, decode_advance_kernel, dim3(1), dim3(1), 0, config, argmax, token_log, batch, log_capacity,
                       peer_step_counter(ctx), ctx->d_err));
    return LV_OK;
}

extern "C" int lv_argmax_advance(lv_ctx* ctx, const float* v, uint32_t n, uint32_t* config, uint32_t* token_log,
                                 uint32_t batch, uint32_t log_capacity, uint32_t* argmax_out, uint32_t* host_token) {
    LV_ENTER(ctx);
    LV_REQUIRE(v && n && config && token_log && batch, "bad argmax_advance arguments");
    LV_CUDA(launch_pdl(ctx, argmax_advance_kernel, dim3(1), dim3(1024), 0, v, n, config, token_log, batch, log_capacity,
                       argmax_out, static_cast<volatile uint32_t*>(host_token), peer_step_counter(ctx), ctx->d_err));
    return LV_OK;
}

extern "C" int lv_argmax_advance_group(lv_ctx* ctx, const float* logits, uint32_t vocab, const lv_group_member* members, uint32_t n,
                                       uint32_t log_capacity, uint32_t* out_tokens, uint32_t* host_tokens) {
    LV_ENTER(ctx);
    LV_REQUIRE(logits && vocab && members && n, "bad argmax_advance arguments");
    LV_CUDA(launch_pdl(ctx, argmax_advance_group_kernel, dim3(n), dim3(1024), 0, logits, vocab, members, log_capacity, out_tokens,
                       static_cast<volatile uint32_t*>(host_tokens), ctx->d_err));
    return LV_OK;
}

extern "C" int lv_norm_f32(lv_ctx* ctx, float* out, const float* x, const float* w, uint32_t dim, uint32_t batch) {
    LV_ENTER(ctx);
    LV_REQUIRE(out && x && w && dim && batch, "bad norm arguments");
    LV_CUDA(launch_pdl(ctx, norm_kernel, dim3(batch), dim3(1024), 0, out, x, w, dim));
    return LV_OK;
}

extern "C" int lv_kv_append_f16(lv_ctx* ctx, void* cache, const float* x, const uint32_t* pos, uint32_t dim,
                                uint32_t batch, uint32_t ctx_rows) {
    LV_ENTER(ctx);
    LV_REQUIRE(cache && x && pos && dim && batch && batch <= 65535, "bad kv_append arguments");
    dim3 grid((dim + 255) / 256, batch);
    LV_CUDA(launch_pdl(ctx, kv_append_kernel, grid, dim3(256), 0, static_cast<__half*>(cache), x, pos, dim, ctx_rows, ctx->d_err));
    return LV_OK;
}

extern "C" int lv_copy_f32(lv_ctx* ctx, float* dst, const float* src, size_t count) {
    LV_ENTER(ctx);
    LV_REQUIRE(dst && src, "null argument");
    if (count == 0) return LV_OK;
    const unsigned blocks = static_cast<unsigned>(std::min<size_t>((count + 255) / 256, 4096));
    LV_CUDA(launch_pdl(ctx, copy_kernel, dim3(blocks), dim3(256), 0, dst, src, count));
    return LV_OK;
}

extern "C" int lv_add_f32(lv_ctx* ctx, float* a, const float* b, size_t count) {
    LV_ENTER(ctx);
    LV_REQUIRE(a && b, "null argument");
    if (count == 0) return LV_OK;
    const unsigned blocks = static_cast<unsigned>(std::min<size_t>((count + 255) / 256, 4096));
    LV_CUDA(launch_pdl(ctx, add_kernel, dim3(blocks), dim3(256), 0, a, b, count));
    return LV_OK;
}

extern "C" int lv_dequant_rows(lv_ctx* ctx, float* out, const void* table, int wtype, const uint32_t* token_ids,
                               const uint32_t* first, uint32_t cols, uint32_t vocab, uint32_t n) {
    LV_ENTER(ctx);
    LV_REQUIRE(out && table && token_ids && n && vocab, "bad dequant arguments");
    LV_REQUIRE(wtype == T_F32 || wtype == T_Q4_0 || wtype == T_Q8_0 || wtype == T_Q4_0_V1, "unsupported table type");
    LV_REQUIRE(cols && cols % 32 == 0, "cols must be a multiple of 32");
    LV_CUDA(launch_pdl(ctx, dequant_rows_kernel, dim3(n), dim3(256), 0, out, static_cast<const uint8_t*>(table), wtype, token_ids, first, cols, vocab, ctx->d_err,
                       static_cast<const lv_group_member*>(nullptr)));
    return LV_OK;
}

extern "C" int lv_dequant_rows_group(lv_ctx* ctx, float* out, const void* table, int wtype, const lv_group_member* members,
                                     uint32_t cols, uint32_t vocab, uint32_t n) {
    LV_ENTER(ctx);
    LV_REQUIRE(out && table && members && n && vocab, "bad dequant arguments");
    LV_REQUIRE(wtype == T_F32 || wtype == T_Q4_0 || wtype == T_Q8_0 || wtype == T_Q4_0_V1, "unsupported table type");
    LV_REQUIRE(cols && cols % 32 == 0, "cols must be a multiple of 32");
    LV_CUDA(launch_pdl(ctx, dequant_rows_kernel, dim3(n), dim3(256), 0, out, static_cast<const uint8_t*>(table), wtype,
                       static_cast<const uint32_t*>(nullptr), static_cast<const uint32_t*>(nullptr), cols, vocab, ctx->d_err, members));
    return LV_OK;
}

extern "C" int lv_argmax_f32(lv_ctx* ctx, uint32_t* out_index, const float* v, uint32_t n) {
    LV_ENTER(ctx);
    LV_REQUIRE(out_index && v && n, "bad argmax arguments");
    LV_CUDA(launch_pdl(ctx, argmax_kernel, dim3(1), dim3(1024), 0, out_index, v, n));
    return LV_OK;
}
