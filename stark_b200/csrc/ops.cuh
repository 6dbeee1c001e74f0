// Launch interface of the non-matvec decode kernels: embedding row, fused QK-norm + RoPE + KV append +
// split-KV decode attention over a paged cache, greedy read-out, and small standalone operators.
#pragma once
#include "common.cuh"
#include "qmv.cuh"

namespace sb {

constexpr uint32_t kPageTokens = 64;      // tokens per KV page
constexpr uint32_t kHeadDim = 128;        // the only head size the kernels are written for
constexpr uint32_t kMaxAttnSplits = 32;   // split-KV partitions per KV head

// Device-resident step state: kernels read the position and token from here so that one recorded
// launch sequence can be replayed for every token.
struct StepState {
    uint32_t position;    // rows already in the cache = position of the row being decoded
    uint32_t token;       // input token of this step
    uint32_t next_token;  // greedy read-out of this step (UINT32_MAX if a logit is not finite)
    uint32_t cursor;      // next entry of the pending prompt list (cache-only ingest)
    uint32_t gen_cursor;  // next free slot of the generated-token list
    uint32_t gen_capacity;
    uint32_t reserved[2];
};

// Paged KV cache of one layer.  Page p of KV head h holds kPageTokens rows of kHeadDim bf16:
//   base + ((p * kv_heads + h) * kPageTokens + r) * kHeadDim
// so each (page, head) tile is one contiguous 16 KB run.  `block_table[b]` is the physical page of
// logical block b (positions b*64 .. b*64+63).
struct KvLayer {
    uint16_t *keys;
    uint16_t *values;
};

struct AttnArgs {
    const uint16_t *qkv;      // [ (q_heads + 2 kv_heads) * 128 ] bf16, rows [q; k; v]
    uint16_t *out;            // [ q_heads * 128 ] bf16
    KvLayer kv;
    const int32_t *block_table;
    const float *q_norm;      // [128] f32 or nullptr (no per-head norm)
    const float *k_norm;
    const float *rope_cos;    // [max_positions, 128] f32 table (both halves filled) or nullptr
    const float *rope_sin;
    const StepState *state;   // position read on device
    float eps;
    float scale;              // 1/sqrt(head_dim)
    uint32_t q_heads, kv_heads;
    uint32_t splits;          // CTAs per KV head
    float *scratch;           // [kv_heads * splits * gqa * (128 + 2)] partial (o, m, l)
    uint32_t *counters;       // [kv_heads] arrival counters, zero before the launch and after it
    uint32_t *error_word;
    TraceSlot *trace;
    bool pdl;
};
stark_b200_status attention_decode_launch(const AttnArgs &a, cudaStream_t stream);
size_t attention_scratch_floats(uint32_t q_heads, uint32_t kv_heads, uint32_t splits);

// h[D] = bf16(scale * code + bias) of row `state->token` of a re-tiled 4-bit table.
stark_b200_status embedding_row_launch(const QMatrix *table, const StepState *state, uint16_t *out, bool pdl,
                                       cudaStream_t stream);

// Final reduction of the per-CTA (max, first index) partials of the logits matvec; writes
// state->next_token, optionally advances the step state (position += 1, token = next_token).
stark_b200_status argmax_finalize_launch(const float *partial_max, const uint32_t *partial_index, uint32_t count,
                                         StepState *state, uint32_t *generated, bool advance, bool pdl,
                                         cudaStream_t stream);

// End of a cache-only prompt row: position += 1, token = pending[cursor++].
stark_b200_status ingest_advance_launch(StepState *state, const uint32_t *pending, bool pdl, cudaStream_t stream);

// Standalone operators (parity tests and non-fused callers).
stark_b200_status rmsnorm_launch(const uint16_t *input, const float *scales, uint16_t *output, uint16_t *shortcut,
                                 uint32_t count, float eps, bool residual_add, cudaStream_t stream);
stark_b200_status swiglu_launch(const uint16_t *fused, uint16_t *out, uint32_t gated_dim, cudaStream_t stream);
stark_b200_status argmax_bf16_launch(const uint16_t *logits, uint32_t vocab, uint32_t *out_index,
                                     cudaStream_t stream);
// log p_i = logit_i - logsumexp(logits), in f64, over the whole vocabulary.
stark_b200_status log_softmax_launch(const float *logits, double *out, uint32_t vocab, double *scratch,
                                     cudaStream_t stream);
stark_b200_status moe_route_launch(const float *logits, uint32_t *ids, float *weights, uint32_t rows,
                                   uint32_t experts, uint32_t active, bool round_weights, bool round_logits,
                                   cudaStream_t stream);

// Stochastic sampling over one row of logits (sampling.cu); `scratch` = sampling_scratch_bytes(vocab)
// bytes of device memory, `out_device` one u32.
size_t sampling_scratch_bytes(uint32_t vocab);
stark_b200_status sampling_validate(const stark_b200_sampling &s, uint32_t vocab);
stark_b200_status sampling_launch(const void *logits, uint32_t io_type, uint32_t vocab, const stark_b200_sampling &s,
                                  void *scratch, uint32_t *out_device, cudaStream_t stream);

// Routed-expert selection of the hybrid host path: top-k of the scores (value descending, index
// ascending), softmax over the selected scores (hybrid/qwen.rs:872-874, math.rs:36-66).
stark_b200_status moe_select_launch(const float *scores, uint32_t experts, uint32_t active, uint32_t *ids,
                                    float *probs, cudaStream_t stream);
// gate[i] = silu(gate[i]) * up[i], f32 (hybrid/qwen.rs:889-891, math.rs:5-16).
stark_b200_status silu_mul_f32_launch(float *gate, const float *up, uint32_t count, cudaStream_t stream);
// out[h] = sum_r probs[r] * rows[r, h], r ascending (hybrid/qwen.rs:894-899).
stark_b200_status weighted_sum_launch(const float *rows, const float *probs, float *out, uint32_t count,
                                      uint32_t width, cudaStream_t stream);
// y = W x, dense f32, one warp per row.
stark_b200_status dense_matvec_f32_launch(const float *w, const float *x, float *y, uint32_t rows, uint32_t columns,
                                          cudaStream_t stream);

}  // namespace sb
