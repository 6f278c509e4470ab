// Shared host/device helpers for the functs_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/functs_b200.h"

namespace fb {

// ---- host side: error text + launch accounting -----------------------------------------
void set_error(const char* fmt, ...);
void count_launch(int n = 1);
// Returns FB_OK, or records the CUDA error text and returns FB_ERR_CUDA.
int check_cuda(cudaError_t e, const char* what);
inline int check_launch(const char* what) { return check_cuda(cudaGetLastError(), what); }
// Profiling hook: records the caller's event number `index` on `st` if functs_b200_set_stage_events armed one.
void record_stage_event(int index, cudaStream_t st);

#define FB_REQUIRE(cond, ...)                \
    do {                                     \
        if (!(cond)) {                       \
            ::fb::set_error(__VA_ARGS__);    \
            return FB_ERR_INVALID_ARGUMENT;  \
        }                                    \
    } while (0)

#define FB_TRY(expr)                 \
    do {                             \
        int fb_rc_ = (expr);         \
        if (fb_rc_ != FB_OK) return fb_rc_; \
    } while (0)

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grid sizes below are chosen against this

// ---- device side ------------------------------------------------------------------------
#ifdef __CUDACC__

constexpr unsigned kFullMask = 0xffffffffu;

// sigmoid as 1 / (1 + exp(-x)), every step rounded on its own (no contraction), accurate expf.
__device__ __forceinline__ float sigmoid_f32(float x) {
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
}

// Candidate key: score bits in the high word, inverted flat index in the low word, so that
// "larger key" == "larger score, then smaller index".  Requires score > 0.
__device__ __forceinline__ uint64_t make_key(float score, uint32_t flat_idx) {
    return (static_cast<uint64_t>(__float_as_uint(score)) << 32) | static_cast<uint64_t>(0xFFFFFFFFu - flat_idx);
}
__device__ __forceinline__ float key_score(uint64_t k) { return __uint_as_float(static_cast<uint32_t>(k >> 32)); }
__device__ __forceinline__ uint32_t key_index(uint64_t k) { return 0xFFFFFFFFu - static_cast<uint32_t>(k & 0xFFFFFFFFull); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier + bulk (TMA, untiled) copy helpers.  No multicast anywhere. -------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
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
// Bounded wait: gives up after `limit` polls and returns false (the caller records a status bit and
// leaves without touching the data).  Each try_wait already blocks for a hardware-defined time slice.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = 4000000u) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}
// global -> shared bulk copy of `bytes` (multiple of 16; both addresses 16-byte aligned), completion on `bar`.
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

#endif  // __CUDACC__

}  // namespace fb
