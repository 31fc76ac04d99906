// Attention over the un-rotated f16 KV cache.  Replaces shaders/mhsa.comp,
// softmax.comp and kqv_matching.comp of the reference, both as three separate
// ops (same buffers as the reference's) and as one fused launch.
//
// The reference keeps K un-rotated in the cache and rotates it at attention
// time by the relative distance (mhsa.comp:42-55).  cos/sin of
// distance * 10000^(-i/(rot/2)) come from a table indexed by distance that the
// host builds once in double precision.
#include <math.h>

#include <cstdlib>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "ctx.h"

namespace lv {

constexpr int kAttnThreads = 256;  // the three separate ops
constexpr int kFusedThreads = 512;  // 128 registers per thread: room to keep every load of a step in flight
constexpr int kAttnChunk = 256;    // cache rows per CTA of the fused kernel (16 per warp)
constexpr int kScoreIters = kAttnChunk / (kFusedThreads / 32) / 4;   // row batches per warp: four rows at a time, 8 lanes each
constexpr int kValueRows = kAttnChunk / (kFusedThreads / 16);        // rows per thread in the value pass
constexpr int kRowGroups = kFusedThreads / 16;   // 16 threads x 8 dims cover a row of one head
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

// grid (heads, nchunks, batch).  CTA (h, c, z) covers cache rows [c*256, c*256+256)
// up to P; contexts of up to 256 rows need one CTA per head and no combine, longer
// ones end with the last CTA of a (z, h) combining the chunks.
//
// The kernel is a short chain of dependent steps on little data, so each step
// issues all of its global loads before using any of them (one trip to L2 per
// step): scores with 8 lanes per cache row (16 elements each, both of a warp's
// row batches in flight together), values with 16 threads per row (8 dims each)
// and four rows per thread in flight.
// Shared-memory staging of the score inputs: the chunk's key rows and the rows of the rotation table
// it needs are brought in by bulk (TMA) copies and the scores are computed from shared memory.  With
// plain loads the kernel spent a fifth of its samples throttled on the load/store queue (28 16-byte
// loads per thread).
//   STAGED = 2 (grids of at most one CTA per SM): the table rows of the chunk's distances, one
//     contiguous range, in one copy of up to 128 KB; key rows padded to 320 bytes so that the two
//     rows a half-warp reads with 8-byte loads fall on different banks.
//   STAGED = 1 (larger grids: long contexts, batches; two CTAs per SM): only 41 table rows -- those
//     of the distances 0..31 and of the up to nine multiples of 32 the chunk spans -- and
//     cos/sin((32 A + B) theta) from the angle-addition formulas (exact for A = 0, else a few units
//     in the last place beside the table's own rounding); key rows unpadded.
//   STAGED = 0: plain loads.
constexpr int kStagedKeyStride = 320;
constexpr size_t kStagedTableBytes = size_t(kAttnChunk) * kRot * sizeof(float);              // 131072
constexpr size_t kStagedSmemBytes = kStagedTableBytes + size_t(kAttnChunk) * kStagedKeyStride;  // + 81920
constexpr int kCompactARows = kAttnChunk / 32 + 1;                                            // multiples of 32 a chunk can span
constexpr size_t kCompactTableBytes = size_t(32 + kCompactARows) * kRot * sizeof(float);      // 20992
constexpr size_t kCompactSmemBytes = kCompactTableBytes + size_t(kAttnChunk) * kRot * sizeof(__half);   // + 65536

template <int MIN_CTAS_PER_SM, int STAGED>
__global__ void __launch_bounds__(kFusedThreads, MIN_CTAS_PER_SM) attention_fused_kernel(float* __restrict__ out, const float* __restrict__ q,
                                                                       const __half* kc, const __half* vc,
                                                                       const uint32_t* __restrict__ pos, const float* __restrict__ table,
                                                                       float* __restrict__ partial, uint32_t* __restrict__ counters,
                                                                       uint32_t heads, uint32_t nchunks, uint32_t max_ctx, float scale,
                                                                       uint32_t* err, const lv_group_member* __restrict__ group) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_e[kAttnChunk];
    __shared__ __align__(16) float s_v[kRowGroups][kRot];
    __shared__ float s_l[kRowGroups];
    __shared__ uint32_t s_last;
    __shared__ __align__(8) uint64_t s_bar;
    extern __shared__ __align__(128) uint8_t staged[];       // STAGED: [table rows][key rows]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t h = blockIdx.x, c = blockIdx.y, z = blockIdx.z;
    // a group step: query row z belongs to member z, with its own caches and position
    if (group != nullptr) {
        kc = static_cast<const __half*>(group[z].k_cache);
        vc = static_cast<const __half*>(group[z].v_cache);
    }
    const uint32_t P = group != nullptr ? *group[z].pos : *pos + z;
    if (P >= max_ctx) {
        // the position lies outside the caches and the rotation table: report it and touch nothing
        // (neither `out` nor the arrival counters), like the cache append does
        if (threadIdx.x == 0 && h == 0 && c == 0) atomicOr(err, ERR_BAD_INDEX);
        return;
    }
    const uint32_t dim = heads * kRot;
    const uint32_t active = P / kAttnChunk + 1;          // chunks that hold at least one row <= P
    if (c >= active) return;
    const uint32_t p0 = c * kAttnChunk;
    const uint32_t n = min(uint32_t(kAttnChunk), P + 1 - p0);

    // The value rows do not depend on the scores.  The staged variant with one CTA per SM has the
    // registers to fetch them first, so that they arrive while the keys are staged and the scores
    // computed; the others (64 registers, or plain loads) fetch them after the scores, before the barrier.
    const int d8 = (threadIdx.x & 15) * 8, rg = threadIdx.x >> 4;
    uint4 vraw[kValueRows];
    auto load_values = [&]() {
#pragma unroll
        for (int j = 0; j < kValueRows; ++j) {
            const uint32_t i = min(uint32_t(rg + kRowGroups * j), n - 1);
            vraw[j] = *reinterpret_cast<const uint4*>(vc + size_t(p0 + i) * dim + h * kRot + d8);
        }
    };
    if constexpr (STAGED == 2) load_values();

    // ---- scores: warp w owns rows 16w .. 16w+15, lane group g = lane / 8 one row per pass -----
    if constexpr (STAGED != 0) {
        const int sub = lane & 7, g = lane >> 3;
        constexpr bool kCompact = STAGED == 1;
        constexpr int kKeyStride = kCompact ? kRot * int(sizeof(__half)) : kStagedKeyStride;
        float* ttile = reinterpret_cast<float*>(staged);
        uint8_t* ktile = staged + (kCompact ? kCompactTableBytes : kStagedTableBytes);
        // distances of the chunk's rows: d_min .. d_min + n - 1, row i at distance d_min + (n - 1 - i)
        const uint32_t d_min = P - p0 - (n - 1);
        const uint32_t a_first = d_min >> 5, a_count = ((d_min + n - 1) >> 5) - a_first + 1;      // compact: multiples of 32 spanned
        if (threadIdx.x == 0) {
            mbar_init(&s_bar, 1);
            fence_mbar_init();
            const uint32_t table_bytes = kCompact ? (32u + a_count) * kRot * uint32_t(sizeof(float)) : n * kRot * uint32_t(sizeof(float));
            mbar_expect_tx(&s_bar, n * kRot * uint32_t(sizeof(__half)) + table_bytes);
        }
        __syncthreads();
        // key row p0 + t -> ktile row t
        if (threadIdx.x < n)
            bulk_g2s(ktile + threadIdx.x * kKeyStride, kc + size_t(p0 + threadIdx.x) * dim + h * kRot, kRot * sizeof(__half), &s_bar);
        if constexpr (kCompact) {
            // table rows 0..31 -> ttile rows 0..31; rows 32 (a_first + t) -> ttile row 32 + t
            if (threadIdx.x == 0) bulk_g2s(ttile, table, 32 * kRot * sizeof(float), &s_bar);
            if (threadIdx.x >= 32 && threadIdx.x < 32 + a_count)
                bulk_g2s(ttile + size_t(threadIdx.x) * kRot, table + size_t(32u * (a_first + threadIdx.x - 32)) * kRot, kRot * sizeof(float), &s_bar);
        } else {
            // table rows of the distances d_min .. d_min + n - 1 -> ttile rows 0 .. n-1
            if (threadIdx.x == 0) bulk_g2s(ttile, table + size_t(d_min) * kRot, n * kRot * uint32_t(sizeof(float)), &s_bar);
        }
        // this lane's part of q: float4 number sub + 8 m, i.e. pairs 2 (sub + 8 m) and 2 (sub + 8 m) + 1
        float4 qv[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) qv[m] = *reinterpret_cast<const float4*>(q + size_t(z) * dim + h * kRot + (sub + 8 * m) * 4);
        const bool ok = mbar_wait(&s_bar, 0u, err);
#pragma unroll
        for (int it = 0; it < kScoreIters; ++it) {
            const uint32_t i = warp * (4 * kScoreIters) + it * 4 + g;
            const uint32_t ic = min(i, n - 1);                        // rows past n are computed and discarded
            const uint8_t* krow = ktile + ic * kKeyStride;
            const uint32_t d = d_min + (n - 1 - ic);
            const float* trow = kCompact ? ttile + size_t(d & 31u) * kRot : ttile + size_t(n - 1 - ic) * kRot;
            const float* arow = ttile + size_t(32u + (d >> 5) - a_first) * kRot;          // compact only
            float sacc = 0.f;
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const int f = sub + 8 * m;
                const uint2 kk = *reinterpret_cast<const uint2*>(krow + f * 8);           // 4 halves = 2 pairs
                float4 t = *reinterpret_cast<const float4*>(trow + f * 4);                // (cos, sin) of the two pairs
                if constexpr (kCompact) {
                    // (cos, sin)((32 A + B) theta) from the rows of 32 A and of B
                    const float4 a = *reinterpret_cast<const float4*>(arow + f * 4);
                    const float c0 = fmaf(a.x, t.x, -(a.y * t.y)), s0 = fmaf(a.y, t.x, a.x * t.y);
                    const float c1 = fmaf(a.z, t.z, -(a.w * t.w)), s1 = fmaf(a.w, t.z, a.z * t.w);
                    t = make_float4(c0, s0, c1, s1);
                }
                const float2 ka = __half22float2(*reinterpret_cast<const __half2*>(&kk.x));
                const float2 kb = __half22float2(*reinterpret_cast<const __half2*>(&kk.y));
                const float4 qq = qv[m];
                // mhsa.comp:42-57
                const float rx0 = t.x * ka.x + t.y * ka.y, ry0 = -t.y * ka.x + t.x * ka.y;
                const float rx1 = t.z * kb.x + t.w * kb.y, ry1 = -t.w * kb.x + t.z * kb.y;
                sacc += qq.x * rx0 + qq.y * ry0;
                sacc += qq.z * rx1 + qq.w * ry1;
            }
            sacc += __shfl_xor_sync(0xffffffffu, sacc, 4);
            sacc += __shfl_xor_sync(0xffffffffu, sacc, 2);
            sacc += __shfl_xor_sync(0xffffffffu, sacc, 1);
            if (sub == 0) s_e[i] = (i < n && ok) ? sacc * scale : -INFINITY;
        }
    } else {
        const int sub = lane & 7, g = lane >> 3;
        const float* qh = q + size_t(z) * dim + h * kRot + sub * 16;
        float4 qv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) qv[j] = *reinterpret_cast<const float4*>(qh + 4 * j);
        uint4 kraw[kScoreIters][2];
        float4 cs[kScoreIters][4];
#pragma unroll
        for (int it = 0; it < kScoreIters; ++it) {
            const uint32_t i = warp * (4 * kScoreIters) + it * 4 + g;
            const uint32_t p = p0 + min(i, n - 1);                 // clamped: rows past n are computed and discarded
            const __half* krow = kc + size_t(p) * dim + h * kRot + sub * 16;
            kraw[it][0] = *reinterpret_cast<const uint4*>(krow);
            kraw[it][1] = *reinterpret_cast<const uint4*>(krow + 8);
            const float* t = table + size_t(P - p) * kRot + sub * 16;
#pragma unroll
            for (int j = 0; j < 4; ++j) cs[it][j] = *reinterpret_cast<const float4*>(t + 4 * j);
        }
#pragma unroll
        for (int it = 0; it < kScoreIters; ++it) {
            const uint32_t i = warp * (4 * kScoreIters) + it * 4 + g;
            const __half2* k2 = reinterpret_cast<const __half2*>(&kraw[it][0]);      // 8 (even, odd) pairs
            float sacc = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // pairs 2j and 2j+1 of this lane: q (x, y, z, w), cos/sin (x, y, z, w) -- mhsa.comp:42-57
                const float2 ka = __half22float2(k2[2 * j]), kb = __half22float2(k2[2 * j + 1]);
                const float4 t = cs[it][j], qq = qv[j];
                const float rx0 = t.x * ka.x + t.y * ka.y, ry0 = -t.y * ka.x + t.x * ka.y;
                const float rx1 = t.z * kb.x + t.w * kb.y, ry1 = -t.w * kb.x + t.z * kb.y;
                sacc += qq.x * rx0 + qq.y * ry0;
                sacc += qq.z * rx1 + qq.w * ry1;
            }
            sacc += __shfl_xor_sync(0xffffffffu, sacc, 4);
            sacc += __shfl_xor_sync(0xffffffffu, sacc, 2);
            sacc += __shfl_xor_sync(0xffffffffu, sacc, 1);
            if (sub == 0) s_e[i] = i < n ? sacc * scale : -INFINITY;
        }
    }
    // ---- weighted values: thread = (8 dims, one of 32 row groups), rows rg, rg+32, ... -----------
    if constexpr (STAGED != 2) load_values();              // (the one-CTA-per-SM staged variant issued these loads before the scores)
    __syncthreads();                                       // s_e holds the scaled scores
    // ---- chunk maximum (every warp on its own) and the exponentials a thread needs ---------------
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < kAttnChunk / 32; ++k) m = fmaxf(m, s_e[lane + 32 * k]);
    m = warp_max(m);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float lsum = 0.f;
#pragma unroll
    for (int j = 0; j < kValueRows; ++j) {
        const uint32_t i = rg + kRowGroups * j;
        const float e = i < n ? expf(s_e[i] - m) : 0.f;
        lsum += e;
        const __half2* v2 = reinterpret_cast<const __half2*>(&vraw[j]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __half22float2(v2[k]);
            acc[2 * k] = fmaf(f.x, e, acc[2 * k]);
            acc[2 * k + 1] = fmaf(f.y, e, acc[2 * k + 1]);
        }
    }
    *reinterpret_cast<float4*>(&s_v[rg][d8]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(&s_v[rg][d8 + 4]) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if ((threadIdx.x & 15) == 0) s_l[rg] = lsum;           // the exp-sum of this row group's rows
    __syncthreads();
    float* my = partial + ((size_t(z) * heads + h) * nchunks + c) * (kRot + 2);
    if (threadIdx.x < kRot) {
        float o = 0.f, l = 0.f;
#pragma unroll 16
        for (int r = 0; r < kRowGroups; ++r) {
            o += s_v[r][threadIdx.x];
            l += s_l[r];
        }
        if (active == 1) {
            out[size_t(z) * dim + h * kRot + threadIdx.x] = o / l;
        } else {
            my[threadIdx.x] = o;
            if (threadIdx.x == 0) { my[kRot] = m; my[kRot + 1] = l; }
        }
    }
    if (active == 1) return;
    // publish, then find out whether this CTA is the last of its (z, h).  The barrier orders the
    // CTA's partial stores before thread 0's fence, which makes them visible before the count
    // (one fence instead of one per thread).
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t prev = atomicAdd(&counters[z * heads + h], 1u);
        s_last = (prev + 1 == active) ? 1u : 0u;
        if (s_last) {
            counters[z * heads + h] = 0;                  // ready for the next launch
            __threadfence();                              // the count was seen: order the reads below after it
        }
    }
    __syncthreads();
    if (!s_last) return;
    // the other chunks' partials are read from L2 (__ldcg), where their stores are by now
    if (threadIdx.x < kRot) {
        const float* base = partial + (size_t(z) * heads + h) * nchunks * (kRot + 2);
        // lane j of every warp fetches chunk j's (max, sum): at most 32 chunks
        const bool mine = uint32_t(lane) < active;
        // the first eight chunks' outputs travel together with the (max, sum) pairs: one trip to L2
        float oj[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) oj[u] = (uint32_t(u) < active) ? __ldcg(base + size_t(u) * (kRot + 2) + threadIdx.x) : 0.f;
        const float mj = mine ? __ldcg(base + size_t(lane) * (kRot + 2) + kRot) : -INFINITY;
        const float lj = mine ? __ldcg(base + size_t(lane) * (kRot + 2) + kRot + 1) : 0.f;
        const float M = warp_max(mj);
        const float wj = mine ? expf(mj - M) : 0.f;
        const float den = warp_sum(lj * wj);
        float num = 0.f;
        for (uint32_t j0 = 0; j0 < active; j0 += 8) {
            if (j0 != 0) {
#pragma unroll
                for (int u = 0; u < 8; ++u) oj[u] = (j0 + u < active) ? __ldcg(base + size_t(j0 + u) * (kRot + 2) + threadIdx.x) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) num = fmaf(oj[u], __shfl_sync(0xffffffffu, wj, (j0 + u) & 31), num);
        }
        out[size_t(z) * dim + h * kRot + threadIdx.x] = num / den;
    }
}

int attention_configure(lv_ctx* ctx) {
    LV_REQUIRE(size_t(ctx->max_smem_optin) >= kStagedSmemBytes + 18 * 1024, "device has too little shared memory for the staged attention kernel");
    LV_CUDA(cudaFuncSetAttribute(attention_fused_kernel<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kStagedSmemBytes)));
    LV_CUDA(cudaFuncSetAttribute(attention_fused_kernel<2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kCompactSmemBytes)));
    return LV_OK;
}

// Grids of at most one CTA per SM stage key rows and the exact table rows in shared memory; larger
// ones (context beyond ~1280 rows, batches) stage key rows and the compact table, two CTAs per SM.
static int launch_attention_fused(lv_ctx* ctx, dim3 grid, float* out, const float* q, const void* k_cache, const void* v_cache,
                                  const uint32_t* pos, const float* rope_table, float* partial, uint32_t* counters, uint32_t heads,
                                  uint32_t nchunks, uint32_t max_ctx, uint32_t rot, const lv_group_member* group = nullptr) {
    const float scale = 1.0f / sqrtf(static_cast<float>(rot));
    static const char* no_stage = getenv("LV_ATTENTION_NO_STAGING");
    // the compact table variant always copies the table rows of distances 0..31
    const bool staged = !(no_stage != nullptr && no_stage[0] == '1') && max_ctx >= 32;
    const bool big = grid.x * grid.y * grid.z > uint32_t(ctx->sm_count);
    if (!staged) {
        if (big) {
            LV_CUDA(launch_pdl(ctx, attention_fused_kernel<2, 0>, grid, dim3(kFusedThreads), 0, out, q, static_cast<const __half*>(k_cache),
                               static_cast<const __half*>(v_cache), pos, rope_table, partial, counters, heads, nchunks, max_ctx, scale, ctx->d_err, group));
        } else {
            LV_CUDA(launch_pdl(ctx, attention_fused_kernel<1, 0>, grid, dim3(kFusedThreads), 0, out, q, static_cast<const __half*>(k_cache),
                               static_cast<const __half*>(v_cache), pos, rope_table, partial, counters, heads, nchunks, max_ctx, scale, ctx->d_err, group));
        }
    } else if (big) {
        LV_CUDA(launch_pdl(ctx, attention_fused_kernel<2, 1>, grid, dim3(kFusedThreads), kCompactSmemBytes, out, q,
                           static_cast<const __half*>(k_cache), static_cast<const __half*>(v_cache), pos, rope_table, partial, counters,
                           heads, nchunks, max_ctx, scale, ctx->d_err, group));
    } else {
        LV_CUDA(launch_pdl(ctx, attention_fused_kernel<1, 2>, grid, dim3(kFusedThreads), kStagedSmemBytes, out, q,
                           static_cast<const __half*>(k_cache), static_cast<const __half*>(v_cache), pos, rope_table, partial, counters,
                           heads, nchunks, max_ctx, scale, ctx->d_err, group));
    }
    return LV_OK;
}

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
    if (int rc = launch_attention_fused(ctx, grid, out, q, k_cache, v_cache, pos, rope_table, partial, counters, heads, nchunks, max_ctx, rot)) return rc;
    return LV_OK;
}

extern "C" int lv_attention_fused_group(lv_ctx* ctx, float* out, const float* q, const lv_group_member* members, const float* rope_table,
                                        void* scratch, uint32_t heads, uint32_t rot, uint32_t max_ctx, uint32_t n) {
    LV_ENTER(ctx);
    LV_REQUIRE(out && q && members && rope_table && scratch, "null argument");
    if (int rc = check_attn_shape(max_ctx, heads, rot, n)) return rc;
    const uint32_t nchunks = (max_ctx + kAttnChunk - 1) / kAttnChunk;
    float* partial = static_cast<float*>(scratch);
    uint32_t* counters = reinterpret_cast<uint32_t*>(partial + attn_partial_floats(heads, nchunks, n));
    dim3 grid(heads, nchunks, n);
    return launch_attention_fused(ctx, grid, out, q, nullptr, nullptr, nullptr, rope_table, partial, counters, heads, nchunks, max_ctx, rot, members);
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
    if (int rc = launch_attention_fused(ctx, grid, out, q, k_cache, v_cache, pos, rope_table, partial, counters, heads, nchunks, max_ctx, rot)) return rc;
    return LV_OK;
}
