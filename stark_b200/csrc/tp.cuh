// Tensor-parallel exchange steps of the decode sequence: one process per GPU, peers' buffers mapped
// through CUDA IPC, plain loads and stores over NVLink (no multimem, no library collective).
//
// At batch 1 the messages are one [hidden] f32 vector per rank (16 KB), so the exchange is bound by
// latency, not bandwidth.  The all-reduce after a K-split projection is therefore taken apart
// (QmvExchange in qmv.cuh): the projection's epilogue pushes its share into every rank's receive buffer
// as self-validating {value, ticket} packets, and a small kernel between the two matvecs polls the
// packets, sums the shares in rank order (so all ranks compute identical bits) and folds the bf16-rounded
// sum into the residual stream.  (The consuming matvec can also do that in its own prologue; see the
// consumer hooks.)  What else needs kernels of its own is the end of a token: the greedy pick across
// vocabulary shards, or, for a cache-only prompt row, closing the last exchange.
#pragma once
#include "common.cuh"
#include "ops.cuh"

namespace sb {

constexpr uint32_t kMaxTpRanks = kMaxExchangeRanks;
constexpr uint32_t kTpFlagSets = 1;  // the greedy-token gather

// Layout of one rank's exchange region (a single allocation, exported to the peers):
//   [0, 4 KB)      flags: [kTpFlagSets][kMaxTpRanks] u32, flag [set][r] written by rank r
//   [4 KB, 8 KB)   gather slots: [kMaxTpRanks] {value bits, index}, slot r written by rank r
//   [8 KB, ...)    recv[2][kMaxTpRanks][hidden] packets of 8 bytes, row [buf][r] written by rank r's matvec
struct TpRegion {
    uint8_t *base[kMaxTpRanks];  // this rank's view of every rank's region (base[rank] is local)
    uint32_t rank, size, hidden;
    unsigned long long wait_ns;  // how long a kernel waits for a peer before it gives up (kDefaultPeerWaitNs)
};
constexpr unsigned long long kDefaultPeerWaitNs = 4000000000ull;  // 4 s
__host__ __device__ inline size_t tp_region_bytes(uint32_t hidden) {
    return 8192u + 2u * (size_t)kMaxTpRanks * hidden * 8u;
}
__host__ __device__ inline uint32_t *tp_flags(uint8_t *base, uint32_t set) {
    return reinterpret_cast<uint32_t *>(base) + set * kMaxTpRanks;
}
__host__ __device__ inline uint32_t *tp_gather(uint8_t *base) { return reinterpret_cast<uint32_t *>(base + 4096u); }
__host__ __device__ inline unsigned long long *tp_recv(uint8_t *base, uint32_t buf, uint32_t src_rank,
                                                       uint32_t hidden) {
    return reinterpret_cast<unsigned long long *>(base + 8192u) + ((size_t)buf * kMaxTpRanks + src_rank) * hidden;
}

// Hooks for the matvec that produces exchange `index` of a token (0 .. per_token-1; buffer index & 1)
// and for the one that consumes it.  `tokens` is the device word counting finished tokens.
QmvExchange tp_producer_hooks(const TpRegion &g, uint32_t index, uint32_t per_token, const uint32_t *tokens);
QmvExchange tp_consumer_hooks(const TpRegion &g, uint32_t index, uint32_t per_token, const uint32_t *tokens,
                              uint16_t *h_out);

// The exchange as a kernel of its own between the producing and the consuming matvec (the alternative to
// the consumer hooks): h[i] = bf16(bf16(sum over ranks) + h[i]), in place, packets summed once.
stark_b200_status tp_reduce_residual_launch(const TpRegion &g, uint32_t index, uint32_t per_token,
                                            const uint32_t *tokens, uint16_t *h, uint32_t *error_word, TraceSlot *trace,
                                            bool pdl, cudaStream_t stream);

// The same step by one CTA that also leaves the following matvec's input ready (qmv.cuh `kProStaged`): the RMS norm
// with `norm_weight`, the f16 scale and the per-group sums are formed once here instead of once per consuming CTA.
stark_b200_status tp_reduce_stage_launch(const TpRegion &g, uint32_t index, uint32_t per_token, const uint32_t *tokens,
                                         uint16_t *h, const float *norm_weight, float eps, void *staged,
                                         uint32_t *error_word, TraceSlot *trace, bool pdl, cudaStream_t stream);

// End of a cache-only prompt row: waits until every rank's packets of the row's last exchange are in
// (nobody may start the next row's pushes into a buffer a slower rank still reads), then position += 1,
// token = pending[cursor++], tokens += 1.
stark_b200_status tp_ingest_advance_launch(const TpRegion &g, uint32_t last_index, uint32_t per_token,
                                           uint32_t *tokens, StepState *state, const uint32_t *pending,
                                           uint32_t *error_word, bool pdl, cudaStream_t stream);
// Greedy token across vocabulary shards: every rank contributes (max, first global index) of its
// shard; the result (first index of the global maximum) updates the step state identically everywhere;
// tokens += 1.
stark_b200_status tp_argmax_finalize_launch(const TpRegion &g, uint32_t *tokens, const float *partial_max,
                                            const uint32_t *partial_index, uint32_t count, uint32_t vocab_offset,
                                            StepState *state, uint32_t *generated, uint32_t *error_word, bool pdl,
                                            cudaStream_t stream);

// ---- prompt passes (several rows at a time) ----------------------------------------------------------------
// A prompt pass is a chain of dense contractions over up to kPrefillBatchRows rows, so its exchange is bound by
// bandwidth, not latency, and it is an all-gather, not an all-reduce: for these passes a rank also holds the o- and
// down-projection cut by OUTPUT ROWS (a second copy of 1/size of each), computes whole output elements with the
// full contraction length, and the ranks copy their column slices of the attention output, the residual stream
// and the gated activation into one another's buffers.  Every element of every row is then the same bits as on
// one GPU.  The buffers live in a second exported allocation:
//   [0, 4 KB)   flags: [kMaxTpRanks] u32, flag r written by rank r (the number of the last gather it completed)
//   then        h [rows, hidden], attn [rows, attn_width], act [rows, inter]   bf16, whole rows of all ranks
struct TpRowsRegion {
    uint8_t *base[kMaxTpRanks];
    uint32_t rank, size;
    unsigned long long wait_ns;
};
constexpr size_t kTpRowsHeaderBytes = 4096;
inline size_t tp_rows_region_bytes(size_t rows, size_t hidden, size_t attn_width, size_t inter) {
    return kTpRowsHeaderBytes + rows * (hidden + attn_width + inter) * 2u;
}
// Copies columns [column, column + width) of `rows` rows from `src` (row stride src_ld elements) to byte offset
// `dst_offset` + the same columns (row stride dst_ld) of every OTHER rank's region -- and of this rank's own when
// `own` is set -- then publishes gather number `ticket` to the peers and waits (bounded) until every peer has
// published it too.  When the launch has finished, the buffer holds the whole rows.  `arrive` is a zeroed device
// word the launches share.  width and both strides are multiples of 8 elements.  width 0: no copy, the flag round
// alone (the kernel before it stored its output to the peers as it went: GemmArgs::peer_out).
struct TpGatherArgs {
    const uint16_t *src;
    uint32_t src_ld;
    size_t dst_offset;
    uint32_t dst_ld, column, width, rows;
    bool own;
    uint32_t ticket;
};
stark_b200_status tp_rows_gather_launch(const TpRowsRegion &g, const TpGatherArgs &a, uint32_t *arrive,
                                        uint32_t *error_word, cudaStream_t stream);

}  // namespace sb
