// Shared device/host helpers for the sm_100a decode kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/stark_b200.h"

namespace sb {

// ---- error word written by kernels whose bounded waits ran out -------------------------------
// Bit 0: an mbarrier wait gave up.  Bit 1: a cross-CTA flag wait gave up.  Bit 2: a peer wait gave up.
constexpr uint32_t kErrMbarTimeout = 1u;
constexpr uint32_t kErrFlagTimeout = 2u;
constexpr uint32_t kErrPeerTimeout = 4u;

// ---- bf16 / f16 bit helpers --------------------------------------------------------------------
__host__ __device__ inline float bf16_bits_to_f32(uint16_t h) {
#ifdef __CUDA_ARCH__
    return __uint_as_float((uint32_t)h << 16);
#else
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
#endif
}

// Round to nearest even, NaN kept quiet: the same bit procedure as the reference's bf16 type.
__host__ __device__ inline uint16_t f32_to_bf16_bits(float f) {
#ifdef __CUDA_ARCH__
    uint32_t u = __float_as_uint(f);
#else
    uint32_t u;
    memcpy(&u, &f, 4);
#endif
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

__device__ inline float bf16_round(float f) { return bf16_bits_to_f32(f32_to_bf16_bits(f)); }
// Two roundings in one instruction: bits 0-15 = bf16(lo), bits 16-31 = bf16(hi), round to nearest even.
// Differs from f32_to_bf16_bits only in the payload of a NaN (the hardware returns the canonical one).
__device__ inline uint32_t f32x2_to_bf16x2(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

// ---- warp / block reductions ---------------------------------------------------------------------
__device__ inline float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ inline float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- PTX wrappers -----------------------------------------------------------------------------------
__device__ inline uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ inline void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ inline void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ inline void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ inline bool mbar_test(uint64_t *bar, uint32_t parity) {
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
// Bounded wait: returns false once the iteration budget is spent (the caller records the error
// and carries on with whatever is in shared memory, so that control flow stays convergent).
__device__ inline bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, const volatile uint32_t *abort_flag) {
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        if (mbar_test(bar, parity)) return true;
        if (it > 64) {
            if (*abort_flag) return false;
            __nanosleep(64);
        }
    }
    return false;
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted on an mbarrier.
__device__ inline void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Programmatic dependent launch: wait for the producer grid / allow the consumer grid to start.
__device__ inline void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ inline void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ inline void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// (a & b) | c
__device__ inline uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ inline void mma_m16n8k16_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ inline uint4 ldg_nc_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// ---- optional in-kernel timeline (off unless a trace buffer is passed) ---------------------------
// One slot per launch of a recorded token sequence: when the first CTA entered, when the first wait on
// the previous kernel returned, when the last CTA finished its prologue, when the last CTA left, and
// when the last CTA entered / saw its wait return (how far the CTAs of a launch are spread).
struct TraceSlot {
    unsigned long long start, ready, compute, end, start_last, ready_last;
};
constexpr unsigned kTraceFields = 6;
__device__ inline unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ inline void trace_min(unsigned long long *field) {
    if (field) atomicMin(field, global_ns());
}
__device__ inline void trace_max(unsigned long long *field) {
    if (field) atomicMax(field, global_ns());
}

// ---- host-side status plumbing ---------------------------------------------------------------------
// Last CUDA error seen by this library on the calling thread (for stark_b200_last_cuda_error).
inline cudaError_t &last_cuda_error() {
    static thread_local cudaError_t e = cudaSuccess;
    return e;
}

inline stark_b200_status cuda_status(cudaError_t e) {
    if (e == cudaSuccess) return STARK_B200_OK;
    last_cuda_error() = e;
    if (e == cudaErrorMemoryAllocation) return STARK_B200_OUT_OF_MEMORY;
    return STARK_B200_DEVICE_FAILURE;
}

#define SB_CUDA(expr)                                         \
    do {                                                      \
        cudaError_t _e = (expr);                              \
        if (_e != cudaSuccess) return ::sb::cuda_status(_e);  \
    } while (0)


// cudaFuncSetAttribute applies to the current device only: a kernel that needs more than 48 KB of dynamic
// shared memory is opted in once per device (one process may drive several GPUs from several threads).
struct SmemOptIn {
    std::atomic<uint64_t> devices{0};
};
template <typename Kernel>
inline stark_b200_status ensure_dynamic_smem(Kernel kernel, int bytes, SmemOptIn &once) {
    int dev = 0;
    SB_CUDA(cudaGetDevice(&dev));
    const uint64_t bit = 1ull << (dev & 63);
    if (once.devices.load(std::memory_order_acquire) & bit) return STARK_B200_OK;
    SB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    once.devices.fetch_or(bit, std::memory_order_release);
    return STARK_B200_OK;
}

}  // namespace sb
