// Tensor-parallel exchange steps of the decode sequence: one process per GPU, peers' buffers mapped
// through CUDA IPC, plain loads and stores over NVLink (no multimem, no library collective).
//
// At batch 1 the messages are one [hidden] f32 vector per rank (16 KB), so the exchange is bound by
// latency, not bandwidth: a one-shot all-reduce (every rank reads every rank's partial and sums in
// rank order, so all ranks compute identical bits) fused with what follows it in the reference graph
// -- rounding the linear output to bf16 and the residual add -- costs one flag round trip.
#pragma once
#include "common.cuh"
#include "ops.cuh"

namespace sb {

constexpr uint32_t kMaxTpRanks = 8;
constexpr uint32_t kTpFlagSets = 3;  // two alternating all-reduce buffers + the greedy-token gather

// Layout of one rank's exchange region (a single allocation, exported to the peers):
//   [0, 4 KB)            flags: [kTpFlagSets][kMaxTpRanks] u32, written by the peers
//   [4 KB, 8 KB)         gather slots: [kMaxTpRanks] {value bits, index}
//   [8 KB, ...)          partial[2][hidden] f32, written by this rank's matvecs, read by everyone
struct TpRegion {
    uint8_t *base[kMaxTpRanks];  // this rank's view of every rank's region (base[rank] is local)
    uint32_t rank, size, hidden;
};
__host__ __device__ inline size_t tp_region_bytes(uint32_t hidden) { return 8192u + 2u * (size_t)hidden * 4u; }
__host__ __device__ inline uint32_t *tp_flags(uint8_t *base, uint32_t set) {
    return reinterpret_cast<uint32_t *>(base) + set * kMaxTpRanks;
}
__host__ __device__ inline uint32_t *tp_gather(uint8_t *base) { return reinterpret_cast<uint32_t *>(base + 4096u); }
__host__ __device__ inline float *tp_partial(uint8_t *base, uint32_t buf, uint32_t hidden) {
    return reinterpret_cast<float *>(base + 8192u) + (size_t)buf * hidden;
}

// h[i] = bf16(bf16(sum over ranks of partial[buf][i]) + h[i]) on every rank.  `seq` is this rank's
// [kTpFlagSets] count of exchanges done per flag set (device words, advanced by the kernels); a token
// sequence alternates buf 0 / buf 1, which is what makes reuse of a buffer safe without a second
// round trip: nobody can reach the next use of a buffer before everyone has left the previous one.
stark_b200_status tp_allreduce_residual_launch(const TpRegion &region, uint32_t buf, uint32_t *seq, uint16_t *h,
                                               uint32_t *error_word, TraceSlot *trace, bool pdl, cudaStream_t stream);
// Greedy token across vocabulary shards: every rank contributes (max, first global index) of its
// shard; the result (first index of the global maximum) updates the step state identically everywhere.
stark_b200_status tp_argmax_finalize_launch(const TpRegion &region, uint32_t *seq, const float *partial_max,
                                            const uint32_t *partial_index, uint32_t count, uint32_t vocab_offset,
                                            StepState *state, uint32_t *generated, uint32_t *error_word, bool pdl,
                                            cudaStream_t stream);

}  // namespace sb
