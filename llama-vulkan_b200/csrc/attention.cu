// Attention over the un-rotated f16 KV cache.  Replaces shaders/mhsa.comp,
// softmax.comp and kqv_matching.comp of the reference, both as three separate
// ops (same buffers as the reference's) and as one fused launch.
//
// The reference keeps K un-rotated in the cache and rotates it at attention
// time by the relative distance (mhsa.comp:42-55).  cos/sin of
// distance * 10000^(-i/(rot/2)) come from a table indexed by distance that the
// host builds once in double precision.
#include <math.h>

#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "ctx.h"

namespace lv {

constexpr int kAttnThreads = 256;
constexpr int kAttnChunk = 64;   // cache rows per CTA of the fused kernel
constexpr int kRot = 128;        // head size; the reference supports only 128 (dim 4096/5120)

// Score of one (query head, cache row) pair, computed by a full warp: each
// lane owns two adjacent (even, odd) pairs.  Returns the sum on every lane.
// Arithmetic of mhsa.comp:42-57 with q in the role the shader calls raw_K.
__device__ __forceinline__ float rope_score(const float4 q4, const __half* __restrict__ krow, const float* __restrict__ cs, int lane) {
    // krow: 128 halves of this head; cs: [rot/2][2] floats for this distance
    const uint2 kraw = *reinterpret_cast<const uint2*>(krow + 4 * lane);
    const float4 c = *reinterpret_cast<const float4*>(cs + 4 * lane);   // (cos0, sin0, cos1, sin1)
    const float2 k01 = __half22float2(*reinterpret_cast<const __half2*>(&kraw.x));
    const float2 k23 = __half22float2(*reinterpret_cast<const __half2*>(&kraw.y));
    const float rx0 = c.x * k01.x + c.y * k01.y, ry0 = -c.y * k01.x + c.x * k01.y;
    const float rx1 = c.z * k23.x + c.w * k23.y, ry1 = -c.w * k23.x + c.z * k23.y;
    float s = q4.x * rx0 + q4.y * ry0;
    s += q4.z * rx1 + q4.w * ry1;
    return warp_sum(s);
}

// ---- separate ops -------------------------------------------------------------------------

// scores[z][p][h] for p <= P, 0 above.  One warp per (p, h).
__global__ void __launch_bounds__(kAttnThreads) attn_scores_kernel(float* __restrict__ scores, const __half* __restrict__ kc,
                                                                  const float* __restrict__ q, const uint32_t* __restrict__ pos,
                                                                  const float* __restrict__ table, uint32_t backlog, uint32_t heads) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const uint32_t z = blockIdx.y;
    const uint32_t P = *pos + z;
    const uint32_t dim = heads * kRot;
    const uint32_t idx = blockIdx.x * (kAttnThreads / 32) + (threadIdx.x >> 5);   // p * heads + h
    if (idx >= backlog * heads) return;
    const uint32_t p = idx / heads, h = idx % heads;
    float s = 0.f;
    if (p <= P) {
        const float4 q4 = *reinterpret_cast<const float4*>(q + size_t(z) * dim + h * kRot + 4 * lane);
        s = rope_score(q4, kc + size_t(p) * dim + h * kRot, table + size_t(P - p) * kRot, lane);
    }
    if (lane == 0) scores[(size_t(z) * backlog + p) * heads + h] = s;
}

// In-place masked softmax over p for each (z, h).  One warp per (z, h).
__global__ void __launch_bounds__(kAttnThreads) softmax_kernel(float* __restrict__ scores, const uint32_t* __restrict__ pos,
                                                              uint32_t backlog, uint32_t heads, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const uint32_t z = blockIdx.y;
    const uint32_t P = *pos + z;
    const uint32_t h = blockIdx.x * (kAttnThreads / 32) + (threadIdx.x >> 5);
    if (h >= heads) return;
    float* s = scores + size_t(z) * backlog * heads + h;
    float m = -INFINITY;
    for (uint32_t p = lane; p <= P && p < backlog; p += 32) m = fmaxf(m, s[size_t(p) * heads] * scale);
    m = warp_max(m);
    float sum = 0.f;
    for (uint32_t p = lane; p < backlog; p += 32) {
        // exp(s * scale) / sum exp(s * scale) == exp(s * scale - m) / sum exp(s * scale - m)
        const float a = (p <= P) ? expf(s[size_t(p) * heads] * scale - m) : 0.f;   // softmax.comp:34-37
        s[size_t(p) * heads] = a;
        sum += a;
    }
    sum = warp_sum(sum);
    for (uint32_t p = lane; p < backlog; p += 32) s[size_t(p) * heads] /= sum;
}

// v_out[z][d] = sum_p V[p][d] * probs[z][p][d / rot].  One thread per d, two halves of p per CTA.
__global__ void __launch_bounds__(kAttnThreads) attn_values_kernel(float* __restrict__ vout, const __half* __restrict__ vc,
                                                                  const float* __restrict__ probs, uint32_t backlog, uint32_t heads) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float part[kRot];
    const uint32_t z = blockIdx.y, h = blockIdx.x;
    const uint32_t dim = heads * kRot;
    const int d = threadIdx.x & (kRot - 1), half = threadIdx.x >> 7;
    const float* pr = probs + size_t(z) * backlog * heads + h;
    float acc = 0.f;
    for (uint32_t p = half; p < backlog; p += 2) {
        const float w = pr[size_t(p) * heads];
        if (w != 0.f) acc = fmaf(__half2float(vc[size_t(p) * dim + h * kRot + d]), w, acc);
    }
    if (half == 1) part[d] = acc;
    __syncthreads();
    if (half == 0) vout[size_t(z) * dim + h * kRot + d] = acc + part[d];
}

// ---- fused ---------------------------------------------------------------------------------

// Scratch layout (floats): for each (z, h, chunk): kRot partial outputs, then
// the chunk's running maximum and exp-sum; after all of those one u32 arrival
// counter per (z, h).
struct AttnScratch {
    float* partial;      // [batch][heads][nchunks][kRot + 2]
    uint32_t* counters;  // [batch][heads]
};

__host__ __device__ inline size_t attn_partial_floats(uint32_t heads, uint32_t nchunks, uint32_t batch) {
    return size_t(batch) * heads * nchunks * (kRot + 2);
}

// grid (heads, nchunks, batch).  CTA (h, c, z) covers cache rows [c*64, c*64+64)
// up to P; the last CTA of a (z, h) to finish combines the chunks.
__global__ void __launch_bounds__(kAttnThreads) attention_fused_kernel(float* __restrict__ out, const float* __restrict__ q,
                                                                      const __half* __restrict__ kc, const __half* __restrict__ vc,
                                                                      const uint32_t* __restrict__ pos, const float* __restrict__ table,
                                                                      float* __restrict__ partial, uint32_t* __restrict__ counters,
                                                                      uint32_t heads, uint32_t nchunks, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_e[kAttnChunk];
    __shared__ float s_part[kRot];
    __shared__ float s_red[2];
    __shared__ uint32_t s_last;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t h = blockIdx.x, c = blockIdx.y, z = blockIdx.z;
    const uint32_t P = *pos + z;
    const uint32_t dim = heads * kRot;
    const uint32_t active = P / kAttnChunk + 1;          // chunks that hold at least one row <= P
    if (c >= active) return;
    const uint32_t p0 = c * kAttnChunk;
    const uint32_t n = min(uint32_t(kAttnChunk), P + 1 - p0);

    // scores of this chunk: 8 warps x 8 rows
    const float4 q4 = *reinterpret_cast<const float4*>(q + size_t(z) * dim + h * kRot + 4 * lane);
    for (uint32_t i = warp; i < uint32_t(kAttnChunk); i += kAttnThreads / 32) {
        float s = -INFINITY;
        if (i < n) {
            const uint32_t p = p0 + i;
            s = rope_score(q4, kc + size_t(p) * dim + h * kRot, table + size_t(P - p) * kRot, lane) * scale;
        }
        if (lane == 0) s_e[i] = s;
    }
    __syncthreads();
    // chunk maximum and exponentials
    if (warp == 0) {
        const float a = s_e[lane], b = s_e[lane + 32];
        const float m = warp_max(fmaxf(a, b));
        const float ea = (lane < n) ? expf(a - m) : 0.f;
        const float eb = (lane + 32 < n) ? expf(b - m) : 0.f;
        s_e[lane] = ea;
        s_e[lane + 32] = eb;
        const float l = warp_sum(ea + eb);
        if (lane == 0) { s_red[0] = m; s_red[1] = l; }
    }
    __syncthreads();
    // weighted values: thread = (d, half of the rows)
    const int d = threadIdx.x & (kRot - 1), half = threadIdx.x >> 7;
    float acc = 0.f;
    for (uint32_t i = half; i < n; i += 2) acc = fmaf(__half2float(vc[size_t(p0 + i) * dim + h * kRot + d]), s_e[i], acc);
    if (half == 1) s_part[d] = acc;
    __syncthreads();
    float* my = partial + ((size_t(z) * heads + h) * nchunks + c) * (kRot + 2);
    if (half == 0) {
        acc += s_part[d];
        if (active == 1) {
            out[size_t(z) * dim + h * kRot + d] = acc / s_red[1];
            return;
        }
        my[d] = acc;
        if (d == 0) { my[kRot] = s_red[0]; my[kRot + 1] = s_red[1]; }
    } else if (active == 1) {
        return;
    }
    // publish, then find out whether this CTA is the last of its (z, h)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t prev = atomicAdd(&counters[z * heads + h], 1u);
        s_last = (prev + 1 == active) ? 1u : 0u;
        if (s_last) counters[z * heads + h] = 0;          // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x < kRot) {
        const float* base = partial + (size_t(z) * heads + h) * nchunks * (kRot + 2);
        float M = -INFINITY;
        for (uint32_t j = 0; j < active; ++j) M = fmaxf(M, __ldcg(base + size_t(j) * (kRot + 2) + kRot));
        float num = 0.f, den = 0.f;
        for (uint32_t j = 0; j < active; ++j) {
            const float* pj = base + size_t(j) * (kRot + 2);
            const float w = expf(__ldcg(pj + kRot) - M);
            num = fmaf(__ldcg(pj + threadIdx.x), w, num);
            den = fmaf(__ldcg(pj + kRot + 1), w, den);
        }
        out[size_t(z) * dim + h * kRot + threadIdx.x] = num / den;
    }
}

int attention_configure(lv_ctx*) { return LV_OK; }

// Scratch of lv_attention_fused_static.  It lives in the library image: every GPU that loads
// the library holds these bytes until the process exits, whether or not the entry point is used.
constexpr size_t kStaticScratchBytes = size_t(1) << 20;
static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

// In host code the name above is only a handle for the symbol, not an address a kernel can
// use; the device address is looked up once per device, with that device current.
constexpr int kMaxDevices = 64;
static void* g_static_scratch_addr[kMaxDevices] = {nullptr};
static std::mutex g_static_scratch_mutex;

static int static_scratch_for(lv_ctx* ctx, void** out) {
    if (ctx->device < 0 || ctx->device >= kMaxDevices) return fail(LV_ERR_BAD_ARGUMENTS, "device index out of range");
    std::lock_guard<std::mutex> guard(g_static_scratch_mutex);
    if (g_static_scratch_addr[ctx->device] == nullptr) {
        void* p = nullptr;
        LV_CUDA(cudaGetSymbolAddress(&p, g_attn_static_scratch));      // cudaSetDevice(ctx->device) was done by LV_ENTER
        g_static_scratch_addr[ctx->device] = p;
    }
    *out = g_static_scratch_addr[ctx->device];
    return LV_OK;
}

}  // namespace lv

using namespace lv;

extern "C" int lv_rope_table_build(lv_ctx* ctx, float* table, uint32_t max_ctx, uint32_t rot) {
    LV_ENTER(ctx);
    LV_REQUIRE(table && max_ctx && rot && rot % 2 == 0, "bad rope table arguments");
    const uint32_t half_rot = rot / 2;
    std::vector<float> host(size_t(max_ctx) * half_rot * 2);
    for (uint32_t i = 0; i < half_rot; ++i) {
        // pow(10000.0, -float(i)/float(2*QUARTERROT)), mhsa.comp:47
        const float theta = static_cast<float>(pow(10000.0, static_cast<double>(-static_cast<float>(i) / static_cast<float>(half_rot))));
        for (uint32_t dist = 0; dist < max_ctx; ++dist) {
            const float d_theta = static_cast<float>(dist) * theta;
            host[(size_t(dist) * half_rot + i) * 2] = static_cast<float>(cos(static_cast<double>(d_theta)));
            host[(size_t(dist) * half_rot + i) * 2 + 1] = static_cast<float>(sin(static_cast<double>(d_theta)));
        }
    }
    LV_CUDA(cudaStreamSynchronize(ctx->stream));
    LV_CUDA(cudaMemcpy(table, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice));
    return LV_OK;
}

static int check_attn_shape(uint32_t backlog, uint32_t heads, uint32_t rot, uint32_t batch) {
    LV_REQUIRE(rot == uint32_t(kRot), "head size must be 128");
    LV_REQUIRE(heads >= 1 && heads <= 1024 && backlog >= 1 && batch >= 1 && batch <= 65535, "attention shape out of range");
    return LV_OK;
}

extern "C" int lv_attn_scores_rope(lv_ctx* ctx, float* scores, const void* k_cache, const float* q, const uint32_t* pos,
                                   const float* rope_table, uint32_t backlog, uint32_t heads, uint32_t rot, uint32_t batch) {
    LV_ENTER(ctx);
    LV_REQUIRE(scores && k_cache && q && pos && rope_table, "null argument");
    if (int rc = check_attn_shape(backlog, heads, rot, batch)) return rc;
    const uint32_t warps = backlog * heads;
    dim3 grid((warps + kAttnThreads / 32 - 1) / (kAttnThreads / 32), batch);
    LV_CUDA(launch_pdl(ctx, attn_scores_kernel, grid, dim3(kAttnThreads), 0, scores, static_cast<const __half*>(k_cache), q, pos, rope_table, backlog, heads));
    return LV_OK;
}

extern "C" int lv_softmax_masked(lv_ctx* ctx, float* scores, const uint32_t* pos, uint32_t backlog, uint32_t heads,
                                 uint32_t rot, uint32_t batch) {
    LV_ENTER(ctx);
    LV_REQUIRE(scores && pos, "null argument");
    if (int rc = check_attn_shape(backlog, heads, rot, batch)) return rc;
    dim3 grid((heads + kAttnThreads / 32 - 1) / (kAttnThreads / 32), batch);
    LV_CUDA(launch_pdl(ctx, softmax_kernel, grid, dim3(kAttnThreads), 0, scores, pos, backlog, heads, 1.0f / sqrtf(static_cast<float>(rot))));
    return LV_OK;
}

extern "C" int lv_attn_values(lv_ctx* ctx, float* v_out, const void* v_cache, const float* probs, uint32_t backlog,
                              uint32_t heads, uint32_t rot, uint32_t batch) {
    LV_ENTER(ctx);
    LV_REQUIRE(v_out && v_cache && probs, "null argument");
    if (int rc = check_attn_shape(backlog, heads, rot, batch)) return rc;
    dim3 grid(heads, batch);
    LV_CUDA(launch_pdl(ctx, attn_values_kernel, grid, dim3(kAttnThreads), 0, v_out, static_cast<const __half*>(v_cache), probs, backlog, heads));
    return LV_OK;
}

extern "C" size_t lv_attention_scratch_bytes(uint32_t heads, uint32_t rot, uint32_t max_ctx, uint32_t batch) {
    if (rot != uint32_t(kRot) || heads == 0 || max_ctx == 0 || batch == 0) return 0;
    const uint32_t nchunks = (max_ctx + kAttnChunk - 1) / kAttnChunk;
    return attn_partial_floats(heads, nchunks, batch) * sizeof(float) + size_t(batch) * heads * sizeof(uint32_t);
}

extern "C" int lv_attention_fused(lv_ctx* ctx, float* out, const float* q, const void* k_cache, const void* v_cache,
                                  const uint32_t* pos, const float* rope_table, void* scratch, uint32_t heads,
                                  uint32_t rot, uint32_t max_ctx, uint32_t batch) {
    LV_ENTER(ctx);
    LV_REQUIRE(out && q && k_cache && v_cache && pos && rope_table && scratch, "null argument");
    if (int rc = check_attn_shape(max_ctx, heads, rot, batch)) return rc;
    const uint32_t nchunks = (max_ctx + kAttnChunk - 1) / kAttnChunk;
    float* partial = static_cast<float*>(scratch);
    uint32_t* counters = reinterpret_cast<uint32_t*>(partial + attn_partial_floats(heads, nchunks, batch));
    dim3 grid(heads, nchunks, batch);
    LV_CUDA(launch_pdl(ctx, attention_fused_kernel, grid, dim3(kAttnThreads), 0, out, q, static_cast<const __half*>(k_cache),
                       static_cast<const __half*>(v_cache), pos, rope_table, partial, counters, heads, nchunks,
                       1.0f / sqrtf(static_cast<float>(rot))));
    return LV_OK;
}

extern "C" size_t lv_attention_static_scratch_limit(void) { return kStaticScratchBytes; }

extern "C" int lv_attention_fused_static(lv_ctx* ctx, float* out, const float* q, const void* k_cache, const void* v_cache,
                                         const uint32_t* pos, const float* rope_table, uint32_t heads, uint32_t rot,
                                         uint32_t max_ctx, uint32_t batch) {
    LV_ENTER(ctx);
    LV_REQUIRE(out && q && k_cache && v_cache && pos && rope_table, "null argument");
    if (int rc = check_attn_shape(max_ctx, heads, rot, batch)) return rc;
    const size_t need = lv_attention_scratch_bytes(heads, rot, max_ctx, batch);
    if (need == 0 || need > kStaticScratchBytes)
        return fail(LV_ERR_BAD_ARGUMENTS, "lv_attention_fused_static: heads x context x batch needs " + std::to_string(need) +
                                              " bytes of scratch, the built-in buffer holds " + std::to_string(kStaticScratchBytes) +
                                              "; use lv_attention_fused with caller-provided scratch");
    void* scratch = nullptr;
    if (int rc = static_scratch_for(ctx, &scratch)) return rc;
    const uint32_t nchunks = (max_ctx + kAttnChunk - 1) / kAttnChunk;
    float* partial = static_cast<float*>(scratch);
    uint32_t* counters = reinterpret_cast<uint32_t*>(partial + attn_partial_floats(heads, nchunks, batch));
    // the buffer keeps whatever the last call left; only the arrival counters must start at zero
    LV_CUDA(cudaMemsetAsync(counters, 0, size_t(batch) * heads * sizeof(uint32_t), ctx->stream));
    dim3 grid(heads, nchunks, batch);
    LV_CUDA(launch_pdl(ctx, attention_fused_kernel, grid, dim3(kAttnThreads), 0, out, q, static_cast<const __half*>(k_cache),
                       static_cast<const __half*>(v_cache), pos, rope_table, partial, counters, heads, nchunks,
                       1.0f / sqrtf(static_cast<float>(rot))));
    return LV_OK;
}
