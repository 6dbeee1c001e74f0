// The exchange step of a prompt pass under tensor parallelism: an all-gather of column slices by plain 16-byte
// stores into the peers' mapped buffers (see tp.cuh), closed by a flag round.  No multimem, no multicast load, no
// library collective; every wait on a peer is bounded in time and reports through the device error word.
#include <algorithm>

#include "tp.cuh"

namespace sb {

namespace {

constexpr int kGatherThreads = 256;

__device__ inline uint32_t *rows_flags(uint8_t *base) { return reinterpret_cast<uint32_t *>(base); }

__global__ void __launch_bounds__(kGatherThreads) tp_rows_gather_kernel(TpRowsRegion g, TpGatherArgs a, uint32_t *arrive,
                                                                        uint32_t *error_word) {
    pdl_wait();  // the slice is the previous kernel's output
    __shared__ uint32_t last_s;
    const uint32_t per_row = a.width / 8u;
    const size_t total = per_row ? (size_t)a.rows * per_row : 0u;
    for (size_t i = (size_t)blockIdx.x * kGatherThreads + threadIdx.x; i < total; i += (size_t)gridDim.x * kGatherThreads) {
        const uint32_t row = (uint32_t)(i / per_row), c = (uint32_t)(i % per_row) * 8u;
        const uint4 v = *reinterpret_cast<const uint4 *>(a.src + (size_t)row * a.src_ld + c);
        const size_t at = a.dst_offset + ((size_t)row * a.dst_ld + a.column + c) * 2u;
#pragma unroll
        for (uint32_t r = 0; r < kMaxTpRanks; ++r)
            if (r < g.size && (r != g.rank || a.own)) *reinterpret_cast<uint4 *>(g.base[r] + at) = v;
    }
    // every CTA's stores are ordered before its arrival; the last CTA to arrive orders all of them before the flags
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) last_s = atomicAdd(arrive, 1u) == gridDim.x - 1u ? 1u : 0u;
    __syncthreads();
    if (!last_s) return;
    if (threadIdx.x == 0) *arrive = 0u;  // the next launch on this stream starts from zero
    __threadfence_system();
    if (threadIdx.x < g.size && threadIdx.x != g.rank) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(rows_flags(g.base[threadIdx.x]) + g.rank), "r"(a.ticket) : "memory");
        // A peer may already be one gather ahead (it publishes before it waits), never more: it cannot complete
        // that one without this rank's flag.  Hence "at least", on the wrapping difference.
        const uint32_t *mine = rows_flags(g.base[g.rank]) + threadIdx.x;
        const unsigned long long t0 = global_ns();
        uint32_t spins = 0;
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int32_t)(v - a.ticket) >= 0) break;
            if (++spins > 32u) {
                __nanosleep(200);
                if (global_ns() - t0 > g.wait_ns) {
                    atomicOr(error_word, kErrPeerTimeout);
                    break;
                }
            }
        }
    }
}

}  // namespace

stark_b200_status tp_rows_gather_launch(const TpRowsRegion &g, const TpGatherArgs &a, uint32_t *arrive,
                                        uint32_t *error_word, cudaStream_t stream) {
    if (g.size < 2 || g.size > kMaxTpRanks || g.rank >= g.size || !arrive) return STARK_B200_INVALID_ARGUMENT;
    // width 0: the producing kernel has stored the slice to the peers itself; only the flag round is left
    if (a.width != 0 &&
        (!a.src || a.rows == 0 || a.width % 8u || a.src_ld % 8u || a.dst_ld % 8u || a.column % 8u || (a.dst_offset & 15u) ||
         (reinterpret_cast<uintptr_t>(a.src) & 15u) || a.column + a.width > a.dst_ld))
        return STARK_B200_INVALID_ARGUMENT;
    const size_t chunks = (size_t)a.rows * (a.width / 8u);
    const uint32_t ctas = (uint32_t)std::max<size_t>(1u, std::min<size_t>(148u * 4u, (chunks + kGatherThreads - 1u) / kGatherThreads));
    tp_rows_gather_kernel<<<ctas, kGatherThreads, 0, stream>>>(g, a, arrive, error_word);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

}  // namespace sb
