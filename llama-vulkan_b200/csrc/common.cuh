// Shared device-side helpers for the sm_100a kernels: PTX wrappers for
// mbarrier and bulk (TMA) copies, bounded waits, warp reductions.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lv {

// GGML tensor type codes as they appear in ggjt files.
// T_Q4_0_V1: the q4_0 blocks of ggjt version 1 files -- f32 scale, byte j holding elements 2j (low nibble) and 2j+1 (high);
// not a GGML code: the file says "q4_0" and its version says which block layout that is.
enum : int { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_0_V1 = 258 };

constexpr int kBlockElems = 32;   // weights per quantisation block
constexpr int kQ4BlockBytes = 18; // f16 scale + 16 nibble bytes (ggjt v3)
constexpr int kQ8BlockBytes = 34; // f16 scale + 32 int8 (ggjt v3)
constexpr int kQ4V1BlockBytes = 20; // f32 scale + 16 nibble bytes (ggjt v1)

// Error word layout (one u32 per context, in device memory).  A kernel that
// gives up on a wait ORs its code in and every later wait returns at once.
enum : uint32_t { ERR_MBAR_TIMEOUT = 1u, ERR_GRID_BARRIER_TIMEOUT = 2u, ERR_PEER_TIMEOUT = 4u, ERR_BAD_INDEX = 8u };

// Upper bound, in SM clock cycles, on one wait before a kernel declares it
// lost (about a second at B200 clocks).  No wait in this library is unbounded.
constexpr long long kWaitCycleLimit = 2000000000ll;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Non-blocking form: try_wait may suspend the thread for a while when the phase is not complete, test_wait returns at once.
// For loops that poll several barriers.
__device__ __forceinline__ bool mbar_poll(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Waits for the phase with the given parity.  Gives up after kWaitCycleLimit cycles
// (or at once if another wait already failed), records the failure in *err and
// returns false; the caller must then stop touching the guarded data.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t* err) {
    if (mbar_test(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_test(bar, parity)) return true;
        if ((spin & 0xffu) == 0) {
            if (*reinterpret_cast<volatile uint32_t*>(err) != 0) return false;
            if (clock64() - t0 > kWaitCycleLimit) break;
        }
    }
    atomicOr(err, ERR_MBAR_TIMEOUT);
    return false;
}

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// Both addresses must be 16-byte aligned and `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Same with an L2 evict-first hint: weight bytes are read once per token.
__device__ __forceinline__ void bulk_g2s_stream(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar,
                                                uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// 2-D tiled TMA load: one instruction fetches a box of rows x bytes described by a tensor
// map (tile coordinates x = inner element index, y = row) and counts the box on `bar`.
// The inner coordinate times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tensor_map, int x, int y, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(smem_u32(smem_dst)), "l"(tensor_map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// 3-D tiled TMA load (coordinates x = inner element index, y, z).
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tensor_map, int x, int y, int z, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
        ::"r"(smem_u32(smem_dst)), "l"(tensor_map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// Programmatic dependent launch.  Every kernel of this library lets its successor start
// launching at once (the successor's prologue -- barrier set-up, the first weight copies --
// then overlaps this kernel's tail) and waits for its predecessor to finish before it reads
// activations or writes anything.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// System-scope release store / acquire load: flags that another GPU reads or writes over NVLink.
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Four consecutive flag words with one acquire load (16-byte aligned): each word is an acquire read of its own.
__device__ __forceinline__ uint4 ld_acquire_sys_v4(const uint32_t* p) {
    uint4 v;
    asm volatile("ld.acquire.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Device-scope release store / acquire load: flags between CTAs of one GPU.
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sums over up to 32 warps with a single barrier; `scratch` holds 64 floats of
// shared memory that must not be in use by another reduction.  Every thread adds the warp
// totals itself in warp order, so every thread gets the same, reproducible result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                      // the previous use of scratch is over
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < nwarps; ++w) t += scratch[w];
    return t;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h16)));
}

}  // namespace lv
