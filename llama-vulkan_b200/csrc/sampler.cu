// The sampler of the reference on the device.
//
// llava_session::get_last_predicted_token (llava_session.cpp:154-194) reads the 32000 logits back and, on
// the host, applies the repeat penalty (to token 13 only), the temperature, turns the logits into
// probabilities without subtracting the maximum, keeps the tokens whose probability is at least 0.5^mu
// (mirostat v2 style), draws one of them in proportion to its probability and moves mu.  Here one
// 1024-thread CTA does the same on the logits where they are and returns four bytes.
//
// The draw: the reference uses std::discrete_distribution over the kept probabilities with a
// std::mt19937; this kernel inverts the cumulative distribution of the same kept probabilities (in index
// order) at a uniform variate from a counter-based generator (Philox 4x32, 10 rounds) keyed by the
// session's seed.  Same distribution, different stream of random numbers.
#include <math.h>

#include "common.cuh"
#include "ctx.h"

namespace lv {

constexpr int kSampleThreads = 1024;
constexpr int kSamplePerThread = 32;        // consecutive logits per thread: 32768 >= any vocabulary accepted here
constexpr uint32_t kNoToken = 0xffffffffu;

// sampler constants, llava_session.h:70-76
constexpr uint32_t kRepeatLastN = 64;
constexpr float kRepeatPenalty = 1.1f, kAlphaFrequency = 0.1f, kAlphaPresence = 0.0f, kTemp = 0.8f;
constexpr float kMirostatTau = 5.0f, kMirostatEta = 0.1f;

__device__ __forceinline__ uint32_t mulhi32(uint32_t a, uint32_t b) { return __umulhi(a, b); }

// Philox 4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"): first word of the block
// for counter (c0, c1, 0, 0) and key (k0, k1).
__device__ __forceinline__ uint32_t philox_first_word(uint32_t c0, uint32_t c1, uint32_t k0, uint32_t k1) {
    uint32_t x0 = c0, x1 = c1, x2 = 0u, x3 = 0u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = mulhi32(0xD2511F53u, x0), lo0 = 0xD2511F53u * x0;
        const uint32_t hi1 = mulhi32(0xCD9E8D57u, x2), lo1 = 0xCD9E8D57u * x2;
        const uint32_t y0 = hi1 ^ x1 ^ k0, y1 = lo1, y2 = hi0 ^ x3 ^ k1, y3 = lo0;
        x0 = y0; x1 = y1; x2 = y2; x3 = y3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return x0;
}

// state: {mu (f32 bits), seed, draws so far, unused}
// report (may be null): {kept count, kept probability sum (f32 bits), probability of the drawn token (f32 bits), uniform variate (f32 bits)}
__global__ void __launch_bounds__(kSampleThreads) sample_mirostat_kernel(const float* __restrict__ logits, uint32_t n, const uint32_t* __restrict__ token_log,
                                                                        const uint32_t* __restrict__ n_tokens_word, uint32_t* state, float forced_u,
                                                                        uint32_t* __restrict__ log_slot_base, uint32_t log_capacity,
                                                                        uint32_t* out_token, volatile uint32_t* host_token, uint32_t* report, uint32_t* err) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_f[64];
    __shared__ uint32_t s_u[64];
    __shared__ float s_total, s_kept_sum, s_target;
    __shared__ uint32_t s_pick, s_last_kept;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t n_tokens = *n_tokens_word;
    const float mu = __uint_as_float(state[0]);

    // tokens equal to 13 among the last 64 (llava_session.cpp:157-160)
    uint32_t count13 = 0;
    {
        const uint32_t first = n_tokens > kRepeatLastN ? n_tokens - kRepeatLastN : 0u;
        if (threadIdx.x < kRepeatLastN && first + threadIdx.x < n_tokens) count13 = token_log[first + threadIdx.x] == 13u ? 1u : 0u;
        count13 = __syncthreads_count(count13 != 0u);
    }

    const uint32_t base = threadIdx.x * kSamplePerThread;
    // exp(logit / temp) of four consecutive tokens, with the penalty on token 13; recomputed in each of the three
    // passes below (the logits stay in L1) rather than held in 32 registers per thread
    auto weights4 = [&](uint32_t i) -> float4 {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i + 3 < n) v = *reinterpret_cast<const float4*>(logits + i);
        else {
            if (i < n) v.x = logits[i];
            if (i + 1 < n) v.y = logits[i + 1];
            if (i + 2 < n) v.z = logits[i + 2];
        }
        if (i == 12u && count13 != 0u) {                                      // token 13 is v.y; llava_session.cpp:161-166
            float x = v.y;
            x = x <= 0.f ? x * kRepeatPenalty : x / kRepeatPenalty;
            x -= kAlphaFrequency * float(count13) + kAlphaPresence;
            v.y = x;
        }
        // no maximum subtracted, llava_session.cpp:169-172
        v.x = i < n ? expf(v.x / kTemp) : 0.f;
        v.y = i + 1 < n ? expf(v.y / kTemp) : 0.f;
        v.z = i + 2 < n ? expf(v.z / kTemp) : 0.f;
        v.w = i + 3 < n ? expf(v.w / kTemp) : 0.f;
        return v;
    };
    float local = 0.f;
#pragma unroll 2
    for (int k = 0; k < kSamplePerThread; k += 4) {
        const float4 v = weights4(base + k);
        local += v.x; local += v.y; local += v.z; local += v.w;
    }
    // total: thread sums in index order, then warps, then the block, always in the same order
    float t = warp_sum(local);
    if (lane == 0) s_f[warp] = t;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int w = 0; w < kSampleThreads / 32; ++w) tot += s_f[w];
        s_total = tot;
        s_pick = kNoToken;
        s_last_kept = 0;
    }
    __syncthreads();
    const float total = s_total;
    const float cut = powf(0.5f, mu);                                         // llava_session.cpp:174
    float kept_local = 0.f;
    uint32_t kept_n = 0, last_kept = kNoToken;
#pragma unroll 2
    for (int k = 0; k < kSamplePerThread; k += 4) {
        const float4 v = weights4(base + k);
        const float q[4] = {v.x / total, v.y / total, v.z / total, v.w / total};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (base + k + j < n && q[j] >= cut) { kept_local += q[j]; ++kept_n; last_kept = base + k + j; }     // llava_session.cpp:176-185
        }
    }
    // exclusive prefix of the kept mass over threads (thread order is index order): within the warp, then across warps
    float incl = kept_local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    uint32_t cnt = kept_n;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    uint32_t lk = last_kept == kNoToken ? 0u : last_kept + 1u;                // 0 = none; max over the block gives the last kept index + 1
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lk = max(lk, __shfl_xor_sync(0xffffffffu, lk, o));
    if (lane == 31) s_f[warp] = incl;
    if (lane == 0) { s_u[warp] = cnt; s_u[32 + warp] = lk; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float run = 0.f;
        uint32_t c = 0, l = 0;
        for (int w = 0; w < kSampleThreads / 32; ++w) {
            const float v = s_f[w];
            s_f[w] = run;                                                     // mass before warp w
            run += v;
            c += s_u[w];
            l = max(l, s_u[32 + w]);
        }
        s_kept_sum = run;
        s_last_kept = l;
        float u = forced_u;
        if (!(u >= 0.f && u < 1.f)) u = float(philox_first_word(state[2], 0u, state[1], 0x6c763230u) >> 8) * (1.0f / 16777216.0f);
        s_target = u * run;
        if (report != nullptr) { report[0] = c; report[1] = __float_as_uint(run); report[3] = __float_as_uint(u); }
    }
    __syncthreads();
    const float target = s_target;
    float cum = s_f[warp] + (incl - kept_local);                              // kept mass before this thread
    uint32_t mine = kNoToken;
    if (kept_n != 0u) {
#pragma unroll 2
        for (int k = 0; k < kSamplePerThread; k += 4) {
            const float4 v = weights4(base + k);
            const float q[4] = {v.x / total, v.y / total, v.z / total, v.w / total};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (base + k + j < n && q[j] >= cut) {
                    cum += q[j];
                    if (mine == kNoToken && cum > target) mine = base + k + j;   // first kept token whose cumulative mass passes the target
                }
            }
        }
    }
    if (mine != kNoToken) atomicMin(&s_pick, mine);
    __syncthreads();
    uint32_t pick = s_pick;
    if (pick == kNoToken && s_last_kept != 0u) pick = s_last_kept - 1u;       // rounding left the target at or beyond the total: the last kept token
    // the owner of the drawn token knows its probability
    if (pick != kNoToken && pick >= base && pick < base + kSamplePerThread) {
        const float4 v = weights4(pick & ~3u);
        const float w4[4] = {v.x, v.y, v.z, v.w};
        const float q = w4[pick & 3u] / total;
        const float kept_sum = s_kept_sum;
        state[0] = __float_as_uint(mu + kMirostatEta * (kMirostatTau + log2f(q / kept_sum)));      // llava_session.cpp:193
        if (report != nullptr) report[2] = __float_as_uint(q);
    }
    if (threadIdx.x == 0) {
        state[2] += 1u;
        if (pick == kNoToken) atomicOr(err, ERR_BAD_INDEX);                   // nothing kept (NaN logits): the reference returns "no token"
        if (out_token != nullptr) *out_token = pick;
        if (log_slot_base != nullptr && pick != kNoToken) {
            // the drawn token becomes the input of the next recorded step (the step that produced the logits already
            // advanced the position: slot n_tokens is where it put its greedy choice)
            if (n_tokens < log_capacity) log_slot_base[n_tokens] = pick;
            else atomicOr(err, ERR_BAD_INDEX);
        }
        if (host_token != nullptr) {
            *host_token = pick;
            __threadfence_system();
        }
    }
}

}  // namespace lv

using namespace lv;

extern "C" int lv_sample_mirostat(lv_ctx* ctx, const float* logits, uint32_t n_vocab, const uint32_t* token_log, const uint32_t* n_tokens,
                                  uint32_t* state, float forced_uniform, uint32_t* feed_token_log, uint32_t log_capacity, uint32_t* out_token,
                                  uint32_t* host_token, uint32_t* report) {
    LV_ENTER(ctx);
    LV_REQUIRE(logits && token_log && n_tokens && state && n_vocab, "bad sampler arguments");
    LV_REQUIRE(n_vocab <= uint32_t(kSampleThreads * kSamplePerThread), "vocabulary larger than 32768");
    LV_REQUIRE((reinterpret_cast<uintptr_t>(logits) & 15u) == 0, "logits must be 16-byte aligned");
    LV_CUDA(launch_pdl(ctx, sample_mirostat_kernel, dim3(1), dim3(kSampleThreads), 0, logits, n_vocab, token_log, n_tokens, state, forced_uniform,
                       feed_token_log, log_capacity, out_token, static_cast<volatile uint32_t*>(host_token), report, ctx->d_err));
    return LV_OK;
}
