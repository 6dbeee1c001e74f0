// Batched prompt rows: the dense contraction Y[M, N] = X[M, K] W[N, K]^T over a 4-bit affine matrix on the
// tcgen05 tensor cores (prefill_gemm.cu), the row-wise operators around it and causal attention over the
// paged cache (prefill_ops.cu), and the model-level chunk loop (prefill_model.cu).
//
// The reference prefills a prompt in chunks of 1024 rows through a tiled GEMM with a dequantizing prologue
// (crates/stark-engine/src/engine/language_model/stream/stream.rs:441-686,
// crates/stark-engine/src/backends/metal/kernel/matmul/gemm/gemm.metal:122-203); a prompt row here goes through
// the same operators, with the same rounding points, as a row of the one-token path.
#pragma once
#include "ops.cuh"
#include "qmv.cuh"

namespace sb {

// The reference ingests 1024 rows per pass (crates/stark-engine/src/engine/language_model/stream/mod.rs:22), a
// limit its memory sets.  Rows are independent of how they are grouped (every operator is row-wise and the
// attention reads the cache), so the grouping is free here: 4096 rows per pass fill whole waves of 256-row tiles
// on 148 SMs (1024 rows x 6144 features are 192 tiles = 1.3 waves) at 250 MB of working buffers for the 8B shape.
constexpr uint32_t kPrefillBatchRows = 4096;

struct GemmArgs {
    const QMatrix *w;     // kFmtAffine4, rows a multiple of 32
    const uint16_t *x;    // [x_rows, K] bf16, row stride K
    uint32_t x_rows;      // rows the buffer holds (the extent the copy engine may touch)
    uint32_t m;           // rows in use, <= x_rows
    uint16_t *out;        // [m, ld_out] bf16; kEpiResidual reads and rewrites it
    uint32_t ld_out;
    QmvEpilogue epilogue;  // kEpiStore, kEpiResidual or kEpiSwiGlu
    uint32_t *error_word;
    // Tensor parallel (more than kPrefillSmallRows rows): `peers` further destinations, each the place of `out` in
    // another rank's row buffer.  The epilogue stores every output segment there too, so that the column slice is
    // in every rank's buffer when the launch has finished (a flag round then closes the gather).
    uint16_t *peer_out[kMaxExchangeRanks] = {};
    uint32_t peers = 0;
};
constexpr uint32_t kPrefillSmallRows = 16;  // up to this many rows take the few-rows kernels
// One launch; the kernel bounds every wait and reports through the error word.
stark_b200_status prefill_gemm_launch(const GemmArgs &args, cudaStream_t stream);
// ---- row-wise operators over a chunk of M rows (prefill_ops.cu) ---------------------------------------
// h[i] = embedding row of tokens[i]
stark_b200_status embed_rows_launch(const QMatrix *table, const uint32_t *tokens, uint32_t m, uint16_t *h,
                                    cudaStream_t stream);
// out[i] = bf16(bf16(h[i] * rms_inv_i) * bf16(w))        normalization.rs:13-191 (only-normalization mode)
// in_stride / out_stride: elements between consecutive rows (0 = d), so that rows can be read from or written
// into a wider buffer (the [e ; h] rows of the draft head's fusion input)
stark_b200_status rmsnorm_rows_launch(const uint16_t *h, const float *weight, uint16_t *out, uint32_t m, uint32_t d,
                                      float eps, cudaStream_t stream, uint32_t in_stride = 0, uint32_t out_stride = 0);
// first[i] = first index of the maximum of row i of a [m, n] bf16 matrix (UINT32_MAX if a value is not finite):
// the greedy read-out of several rows at once (unified_sampling.rs:42-45, 108-113)
stark_b200_status argmax_rows_launch(const uint16_t *rows, uint32_t m, uint32_t n, uint32_t *first, cudaStream_t stream);
// Per row and head: q heads normalized and rotated in place, k heads normalized, rotated and appended to the
// cache at position first_pos + i together with the v heads.
struct RopeAppendArgs {
    uint16_t *qkv;  // [m, (q_heads + 2 kv_heads) * 128]
    KvLayer kv;
    const int32_t *block_table;
    const float *q_norm, *k_norm, *rope_cos, *rope_sin;
    uint32_t m, first_pos, q_heads, kv_heads;
    float eps;
};
stark_b200_status rope_append_rows_launch(const RopeAppendArgs &a, cudaStream_t stream);
// Causal attention of the chunk's rows over the cache rows [0, first_pos + i]; out [m, q_heads * 128] bf16.
struct PrefillAttnArgs {
    const uint16_t *qkv;  // rotated q heads of the chunk
    KvLayer kv;
    const int32_t *block_table;
    uint16_t *out;
    uint32_t m, first_pos, q_heads, kv_heads;
    float scale;
    // Optional working memory for the few-rows form (m <= 16): prefill_attention_partial_floats(q_heads, max_splits)
    // floats.  With it, the key tiles of a long cache are divided among up to max_splits CTAs per KV head and
    // merged by a second launch; without it every (row block, KV head) is one CTA.
    float *partials = nullptr;
    uint32_t max_splits = 0;
    // Pages the cache arrays hold (the extent of the tensor maps): with it, passes of more than 16 rows run on the
    // tcgen05 tensor cores (prefill_attention_tc.cu); 0 keeps them on the mma.sync kernel.
    uint32_t num_blocks = 0;
};
constexpr uint32_t kPrefillAttnMaxSplits = 64;
inline size_t prefill_attention_partial_floats(uint32_t q_heads, uint32_t max_splits) {
    return (size_t)16u * q_heads * max_splits * (4u + 128u);
}
stark_b200_status prefill_attention_launch(const PrefillAttnArgs &a, cudaStream_t stream);
// The same attention for more than 16 rows on the tcgen05 tensor cores (what prefill_attention_launch calls when the
// arguments allow it and the tunable `prefill_attn_tc` is on).
bool prefill_attention_tc_supports(const PrefillAttnArgs &a);
stark_b200_status prefill_attention_tc_launch(const PrefillAttnArgs &a, cudaStream_t stream);

}  // namespace sb
