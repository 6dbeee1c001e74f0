/*
 * stark_b200.h -- C ABI of the B200 (sm_100a) decode engine for Stark's token loop.
 *
 * The boundary follows the reference's own foreign-engine ABI
 * (vendor/glm-exl3-bridge/include/stark_glm.h:16-175, bound from Rust in
 * crates/stark-engine/src/engine/hybrid/glm_exl3_ffi.rs:1-140): opaque handles,
 * uint32_t status codes, versioned POD structs {struct_size, abi_version, ...},
 * caller-owned buffers, serial (one host thread per handle) use, explicit destroy.
 * No C++ or framework types cross it; nothing is written to stdout/stderr.
 *
 * Two groups of entry points:
 *   (1) the model surface -- the FFI image of hybrid::Model / LanguageModel
 *       (load, reset, prefill, step, full-vocabulary read-out, prefix rewind);
 *   (2) per-operator calls (quantized matvec, norms, RoPE, attention, router,
 *       log-softmax) that play the role of the reference's per-kernel
 *       `XKernel::encode` API (crates/stark-engine/build/common/traitgen.rs:56-66)
 *       for parity tests and micro-benchmarks.
 *
 * Every pointer argument carries a `location` (host or device).  Host pointers
 * are copied through the library's own staging buffers inside the call.
 */
#ifndef STARK_B200_H
#define STARK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define STARK_B200_ABI_VERSION 1u

typedef struct stark_b200_qmatrix stark_b200_qmatrix;
typedef struct stark_b200_model stark_b200_model;

/* Same numbering as stark_glm_status (stark_glm.h:18-32). */
typedef uint32_t stark_b200_status;
enum {
    STARK_B200_OK = 0,
    STARK_B200_INVALID_ARGUMENT = 1,
    STARK_B200_ABI_MISMATCH = 2,
    STARK_B200_CONTEXT_LIMIT = 3,
    STARK_B200_CANCELLED = 4,
    STARK_B200_UNSUPPORTED = 5,
    STARK_B200_OUT_OF_MEMORY = 6,
    STARK_B200_IO_FAILURE = 7,
    STARK_B200_DEVICE_FAILURE = 8,
    STARK_B200_RELOAD_REQUIRED = 9,
    STARK_B200_BUSY = 10,
    STARK_B200_INVALID_STATE = 11
};

/* Where a caller's buffer lives. */
#define STARK_B200_HOST 0u
#define STARK_B200_DEVICE 1u

/* Element types of activation vectors. */
#define STARK_B200_BF16 0u /* converted-model path: bf16 in/out, f32 accumulate */
#define STARK_B200_F32 1u  /* hybrid host path conventions: f32 in/out */

/* Plane (scale/bias) element kinds, numbered like the reference's tensor kinds
 * (crates/stark-engine/src/engine/hybrid/weights.rs:1207). */
#define STARK_B200_PLANE_F32 0u
#define STARK_B200_PLANE_F16 1u
#define STARK_B200_PLANE_BF16 30u

/* GGUF block kinds (ggml type ids; weights.rs:2565-2584). */
#define STARK_B200_GGUF_Q8_0 8u
#define STARK_B200_GGUF_Q4_K 12u

/* stark_glm_abi_version / stark_glm_status_name (stark_glm.h:82-83). */
uint32_t stark_b200_abi_version(void);
const char *stark_b200_status_name(uint32_t status);

/* Name of the last CUDA runtime error this library saw on the calling thread ("cudaSuccess" if
 * none); a diagnostic aid, the library itself never prints. */
const char *stark_b200_last_cuda_error(void);

/* Device plumbing for callers that do not bring their own allocator. */
stark_b200_status stark_b200_device_count(int32_t *out_count);
/* Free and total memory of the current device: what the memory-admission planner of a worker measures its headroom
 * against (the reference asks its host for available memory, crates/stark-generate/src/generation.rs:1161-1164,
 * because its device memory is the host's; here the cache and the working buffers live in HBM). */
stark_b200_status stark_b200_device_memory(uint64_t *out_free_bytes, uint64_t *out_total_bytes);
stark_b200_status stark_b200_set_device(int32_t device);
stark_b200_status stark_b200_device_malloc(void **out_ptr, size_t bytes);
stark_b200_status stark_b200_device_free(void *ptr);
stark_b200_status stark_b200_memcpy_h2d(void *dst_device, const void *src_host, size_t bytes, void *stream);
stark_b200_status stark_b200_memcpy_d2h(void *dst_host, const void *src_device, size_t bytes, void *stream);
stark_b200_status stark_b200_stream_synchronize(void *stream);
/* Reads and clears the device error word that kernels set when one of their bounded waits ran
 * out (0 = no error).  A non-zero word means the results of that launch are not valid. */
stark_b200_status stark_b200_take_device_error(uint32_t *out_word);

/* ------------------------------------------------------------------------------------------
 * Quantized matrices.
 *
 * An MLX-affine matrix W[rows, columns]: w = scale * q + bias, q unsigned `bits` wide, packed
 * LSB-first along columns (8 nibbles per uint32 for 4 bits), one (scale, bias) per `group`
 * consecutive columns.  Replaces the operands of MatmulB::Quantized
 * (crates/stark-engine/src/backends/common/kernel/matmul/arguments.rs:7-24) and of
 * Weights::affine_row (crates/stark-engine/src/engine/hybrid/weights.rs:1284-1309).
 * scale_layout 0: planes [rows, groups] (MLX native); 1: planes [groups, plane_pitch]
 * (the converted-model layout, backends/common/kernel/matmul/mod.rs:120-156).
 * The create call copies and re-tiles the data into device memory; the caller's buffers are
 * not referenced afterwards.
 */
typedef struct stark_b200_affine_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t rows;
    uint32_t columns;
    uint32_t bits;         /* 4 or 8 */
    uint32_t group;        /* 64 */
    uint32_t plane_kind;   /* STARK_B200_PLANE_* */
    uint32_t scale_layout; /* 0 or 1 */
    uint32_t plane_pitch;  /* round_up4(rows) for layout 1, ignored for layout 0 */
    uint32_t location;     /* STARK_B200_HOST / _DEVICE for codes, scales, biases */
    uint32_t pair_halves;  /* 1: rows r and r + rows/2 are a fused [up; gate] pair */
    uint32_t reserved;
} stark_b200_affine_desc;

stark_b200_status stark_b200_qmatrix_create_affine(const void *codes, const void *scales, const void *biases,
                                                   const stark_b200_affine_desc *desc,
                                                   stark_b200_qmatrix **out_matrix);
/* GGUF rows: `rows` rows of columns/block consecutive blocks, as decode_values reads them
 * (crates/stark-engine/src/engine/hybrid/weights.rs:2880-2895). */
stark_b200_status stark_b200_qmatrix_create_gguf(const void *blocks, uint32_t kind, uint32_t rows,
                                                 uint32_t columns, uint32_t location,
                                                 stark_b200_qmatrix **out_matrix);
/* A bank of `experts` GGUF matrices [experts, rows, columns] (ffn_{gate,up,down}_exps tensors,
 * crates/stark-engine/src/engine/hybrid/glm.rs:954-1002), read by Weights::selected_matvec
 * (weights.rs:1612-1689). */
stark_b200_status stark_b200_qmatrix_create_gguf_bank(const void *blocks, uint32_t kind, uint32_t experts,
                                                      uint32_t rows, uint32_t columns, uint32_t location,
                                                      stark_b200_qmatrix **out_matrix);
stark_b200_status stark_b200_qmatrix_destroy(stark_b200_qmatrix **matrix);
/* One row dequantized to f32 through the kernels' own decode; must equal decode_values / affine_row
 * (weights.rs:2880-3017, 1284-1309) bit for bit.  GGUF and 8-bit affine matrices only. */
stark_b200_status stark_b200_qmatrix_dequantize_row(const stark_b200_qmatrix *matrix, uint32_t expert,
                                                    uint32_t row, float *dst_host);
/* Bytes the matrix occupies in device memory (codes + planes, after re-tiling). */
stark_b200_status stark_b200_qmatrix_device_bytes(const stark_b200_qmatrix *matrix, uint64_t *out_bytes);
/* Integer codes recovered from the re-tiled device copy through the same extraction the matvec
 * kernels use; dst[row * columns + column], one byte per code.  Must equal packed_code
 * (crates/stark-engine/src/backends/cpu/kernel/matmul/reference.rs:91-104) bit for bit. */
stark_b200_status stark_b200_qmatrix_unpack_codes(const stark_b200_qmatrix *matrix, uint8_t *dst_host,
                                                  size_t count);

/* Test-only: causal attention of `m` rows of a prompt pass over a paged cache (pages of 64 tokens; cache arrays
 * [num_blocks][kv_heads][64][128] bf16, already holding the pass's own keys and values), all HOST arrays.  qkv is
 * [m][(q_heads + 2 kv_heads) * 128] bf16 with the query heads normalized and rotated; out [m][q_heads * 128] bf16.
 * variant 0: the mma.sync kernel, 1: the tcgen05 kernel (more than 16 rows).  Replaces nothing in the reference; it
 * exposes attention_single_pass.rs:11-133 over many rows for the parity tests. */
stark_b200_status stark_b200_op_prefill_attention(const void *qkv, const void *keys, const void *values,
                                                  const int32_t *block_table, uint32_t num_blocks, void *out, uint32_t m,
                                                  uint32_t first_pos, uint32_t q_heads, uint32_t kv_heads,
                                                  uint32_t variant);
/* Y[m, rows] = X[m, columns] * W^T for many rows at once (a prompt chunk) on the tensor cores: bf16 rows in
 * and out, f32 accumulation, a 4-bit affine matrix with a multiple of 32 rows (UNSUPPORTED otherwise); the
 * dequantized operand is rounded to bf16, as in the reference's own tiled GEMM.
 * Replaces MatmulKernel::encode with a quantized B and m > 8 rows
 * (crates/stark-engine/src/backends/cpu/kernel/matmul/kernel.rs:168-285; on the reference's GPU path the tiled
 * GEMM with a dequantizing prologue, backends/metal/kernel/matmul/gemm/gemm.metal:122-203).
 * epilogue: 0 y = bf16(product); 1 y = bf16(bf16(product) + y), y holding the residual rows on entry;
 * 2 SwiGLU over a pair-ordered [up; gate] matrix, y being [m, rows / 2]. */
stark_b200_status stark_b200_op_qgemm(const stark_b200_qmatrix *matrix, const void *x, void *y, uint32_t m,
                                      uint32_t epilogue, uint32_t location, void *stream);
/* y[m, rows] = x[m, columns] * W^T for m <= 8 bf16 rows with ONE pass over a 4-bit affine matrix: the verify pass
 * of a speculative round (k + 1 rows through the target; the reference's GEMV with an input-row tile,
 * crates/stark-engine/src/backends/metal/kernel/matmul/gemv/gemv.metal:59-63, driven from
 * engine/language_model/dense_mtp.rs:786-886).  norm_weight (f32[columns], nullable; columns <= 4096): every row
 * first goes through the RMS norm with the reference's rounding points (normalization.rs:13-191).  Epilogues as
 * stark_b200_op_qgemm.  With location DEVICE all three pointers are device pointers.  UNSUPPORTED when the rows do
 * not fit the kernel's shared memory beside its weight ring (m * columns * 2 bytes). */
stark_b200_status stark_b200_op_qmv_rows(const stark_b200_qmatrix *matrix, const void *x, void *y, uint32_t m,
                                         uint32_t epilogue, const float *norm_weight, float eps, uint32_t location,
                                         void *stream);
/* y[m, rows] = x[m, columns] * W^T.  Replaces MatmulKernel::encode for a quantized B with
 * m <= 8 input rows (crates/stark-engine/src/backends/cpu/kernel/matmul/kernel.rs:168-285) and
 * Weights::matvec (weights.rs:1311-1350, 2511-2553).  io_type selects bf16 or f32 vectors. */
stark_b200_status stark_b200_op_qmv(const stark_b200_qmatrix *matrix, const void *x, void *y, uint32_t m,
                                    uint32_t io_type, uint32_t location, void *stream);

/* y[i, rows] = W[expert_ids[i]] x_i for i < count: Weights::selected_matvec (weights.rs:1612-1689), the
 * grouped expert matvec (one launch; the expert of each row is read on the device).  shared_input != 0:
 * every row uses the same input x[columns]; otherwise x is [count, columns]. */
stark_b200_status stark_b200_op_qmv_experts(const stark_b200_qmatrix *bank, const uint32_t *expert_ids,
                                            uint32_t count, const void *x, uint32_t shared_input, void *y,
                                            uint32_t io_type, uint32_t location, void *stream);
/* Dense f32 matvec (the router projection of the host path). */
stark_b200_status stark_b200_op_dense_matvec_f32(const float *w, const float *x, float *y, uint32_t rows,
                                                 uint32_t columns, uint32_t location, void *stream);
/* Routed-expert feed-forward of the hybrid host path (crates/stark-engine/src/engine/hybrid/qwen.rs:872-905,
 * without the shared expert): top-k of `scores` (value descending, index ascending), softmax over the
 * selected scores, out = sum_r p_r * down_r(silu(gate_r x) * (up_r x)), all f32.  ids_out / probs_out
 * (host, `active` entries) may be NULL. */
stark_b200_status stark_b200_op_moe_ffn(const stark_b200_qmatrix *gate_bank, const stark_b200_qmatrix *up_bank,
                                        const stark_b200_qmatrix *down_bank, const float *scores, const float *x,
                                        float *out, uint32_t active, uint32_t *ids_out, float *probs_out,
                                        uint32_t location, void *stream);

/* ------------------------------------------------------------------------------------------
 * Small operators (bf16 bit patterns unless stated).  Each names the reference routine it stands
 * in for; `location` applies to every pointer of the call.
 */
/* normalization (RMS, only-normalization rounding, optional fused residual add into `shortcut`):
 * crates/stark-engine/src/backends/cpu/kernel/normalization/normalization.rs:13-191.
 * shortcut may be NULL; residual_add != 0 requires it (ShortcutMode::Add), else it is a copy. */
stark_b200_status stark_b200_op_rmsnorm(const void *input, const float *scales, void *output, void *shortcut,
                                        uint32_t count, float epsilon, uint32_t residual_add, uint32_t location,
                                        void *stream);
/* gated_act_mul on a fused [up; gate] row, SiLU:
 * crates/stark-engine/src/backends/cpu/kernel/gated_act_mul/gated_act_mul.rs:17-152. */
stark_b200_status stark_b200_op_swiglu(const void *fused, void *out, uint32_t gated_dim, uint32_t location,
                                       void *stream);
/* Fused up/gate matvec + SwiGLU on a pair_halves matrix: out[r] = up[r] * silu(gate[r]), the
 * composition of MatmulKernel::encode and GatedActMul (crates/stark-engine/src/encodable_block/mlp/dense.rs:99-115). */
stark_b200_status stark_b200_op_qmv_swiglu(const stark_b200_qmatrix *matrix, const void *x, void *out,
                                           uint32_t location, void *stream);
/* Greedy token: first index of the maximum, UINT32_MAX if any logit is not finite
 * (crates/stark-engine/src/backends/cpu/kernel/sampling/unified_sampling.rs:36-45,108-116). */
stark_b200_status stark_b200_op_argmax(const void *logits_bf16, uint32_t vocab, uint32_t *out_index,
                                       uint32_t location, void *stream);
/* Full-vocabulary log-probabilities in f64: log p_i = logit_i - logsumexp
 * (crates/stark-score/src/scoring.rs:299-336). */
stark_b200_status stark_b200_op_log_softmax(const float *logits, double *out, uint32_t vocab, uint32_t location,
                                            void *stream);
/* moe_route: softmax over experts, iterative top-k (first maximum wins), renormalise
 * (crates/stark-engine/src/backends/cpu/kernel/moe.rs:25-82). */
stark_b200_status stark_b200_op_moe_route(const float *logits, uint32_t *ids, float *weights, uint32_t rows,
                                          uint32_t experts, uint32_t active, uint32_t round_weights,
                                          uint32_t round_logits, uint32_t location, void *stream);

/* Decode attention for one new row over a KV cache of `position` earlier rows, with the
 * per-head RMS norm of Q and K, RoPE and the cache append fused in.  Replaces QKVNorm +
 * AttentionPrepare + AttentionSinglePass/TwoPass
 * (crates/stark-engine/src/backends/cpu/kernel/attention/qkv_norm.rs:8-111,
 *  attention_prepare.rs:187-316, attention_single_pass.rs:11-133).
 * Host-memory call: keys/values are [capacity, kv_heads, 128] bf16 row-major (the reference's
 * cache layout) holding `position` valid rows; row `position` is written on return.
 * qkv is the packed [q; k; v] row; out is [q_heads, 128].  q_norm/k_norm may be NULL (no norm);
 * rope_theta <= 0 disables RoPE. */
typedef struct stark_b200_attention_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t q_heads;
    uint32_t kv_heads;
    uint32_t head_dim; /* 128 */
    uint32_t position;
    uint32_t capacity;
    uint32_t splits; /* 0 = library default */
    float epsilon;
    float rope_theta;
} stark_b200_attention_desc;
stark_b200_status stark_b200_op_attention_decode(const void *qkv, void *keys, void *values, void *out,
                                                 const float *q_norm, const float *k_norm,
                                                 const stark_b200_attention_desc *desc);

/* The same decode attention for callers that must not allocate device memory: a worker that fixed
 * its memory budget when it admitted the request, or a decode loop that cannot take the
 * device-wide stall of cudaMalloc / cudaFree.  This entry point has no counterpart in the
 * reference.  It calls no allocator: the split-KV partial results and arrival counters live in a
 * 1 MiB array inside the library image (held by every GPU that loads the library until the
 * process exits).
 *   - All pointers are DEVICE pointers.  key_pages / value_pages use the library's page layout:
 *     element ((page * kv_heads + head) * 64 + row_in_page) * 128 + dim, bf16; block_table[b] is
 *     the page of positions 64 b .. 64 b + 63 and must cover position / 64.  rope_cos / rope_sin
 *     are f32 tables [positions, 128] (both halves filled) or both NULL; q_norm / k_norm may be NULL.
 *   - desc->position rows are read, row desc->position is appended.  desc->capacity and
 *     desc->rope_theta are ignored.
 *   - Limit: q_heads * splits * 520 bytes <= 1 MiB - 1 KiB and kv_heads <= 64 (splits defaults
 *     to 8); beyond that the call returns STARK_B200_CONTEXT_LIMIT and launches nothing.
 *   - The first call on each device resolves the address of the array (that device must be
 *     current); make that first call before any stream capture begins.
 *   - All calls on a device share the array.  Each call clears the counters it needs, but two calls
 *     whose kernels overlap on the GPU (different streams) race on it: serialise them. */
stark_b200_status stark_b200_op_attention_decode_static(const void *qkv, void *key_pages, void *value_pages,
                                                        const int32_t *block_table, void *out,
                                                        const float *q_norm, const float *k_norm,
                                                        const float *rope_cos, const float *rope_sin,
                                                        const stark_b200_attention_desc *desc, void *stream);

/* ------------------------------------------------------------------------------------------
 * Model surface: the FFI image of hybrid::Model / LanguageModel for a Qwen3-shaped dense decoder
 * (crates/stark-engine/src/engine/hybrid/mod.rs:347-1428,
 *  crates/stark-engine/src/engine/language_model/mod.rs:72-127).
 * A model is built empty from its shape, receives its tensors in the reference's layouts, and is
 * then finalized; after that the calls mirror stark_glm_{reset,prefill,step,readout_f32,...}
 * (stark_glm.h:128-147).  One host thread per handle.  A device fault fences the handle.
 */
typedef struct stark_b200_dense_config {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t layers;
    uint32_t hidden;
    uint32_t q_heads;
    uint32_t kv_heads;
    uint32_t head_dim; /* 128 */
    uint32_t inter;    /* SwiGLU intermediate width */
    uint32_t vocab;
    uint32_t tied;     /* 1: read-out shares the embedding table */
    uint32_t context_tokens;
    float eps;
    float rope_theta;
    uint32_t reserved; /* draft-head layers of the multi-token-prediction path: 0 (none) or 1 */
} stark_b200_dense_config;

/* Which tensor a set call addresses.  Matrices: rows [q; k; v] for QKV and [up; gate] for UPGATE
 * (crates/stark-engine/tools: tools/converter/stark_convert/adapters/dense.py:431-432). */
#define STARK_B200_MAT_EMBED 0u
#define STARK_B200_MAT_LM_HEAD 1u
#define STARK_B200_MAT_QKV 2u
#define STARK_B200_MAT_O 3u
#define STARK_B200_MAT_UPGATE 4u
#define STARK_B200_MAT_DOWN 5u
#define STARK_B200_MAT_MTP_FUSION 6u /* draft head: [hidden, 2 * hidden] over [norm_e(embedding) ; norm_h(hidden)] */
/* Tensor parallel only, optional: this rank's OUTPUT ROWS [rank * hidden / ranks, (rank + 1) * hidden / ranks) of the
 * whole o- and down-projection (all input columns), used by batched prompt passes (see tp_rows_init). */
#define STARK_B200_MAT_O_ROWS 7u
#define STARK_B200_MAT_DOWN_ROWS 8u
#define STARK_B200_VEC_FINAL_NORM 0u
#define STARK_B200_VEC_ATTN_NORM 1u
#define STARK_B200_VEC_MLP_NORM 2u
#define STARK_B200_VEC_Q_NORM 3u
#define STARK_B200_VEC_K_NORM 4u
#define STARK_B200_VEC_MTP_EMBED_NORM 5u  /* draft head: norm of the token embedding */
#define STARK_B200_VEC_MTP_HIDDEN_NORM 6u /* draft head: norm of the incoming hidden row */
#define STARK_B200_VEC_MTP_OUT_NORM 7u    /* draft head: output norm, before the shared read-out */

typedef struct stark_b200_info {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t vocab_size;
    uint32_t prefill_chunk_tokens; /* 1024: the grid prefix reuse is aligned to */
    uint64_t context_tokens;
    uint64_t position;
    uint64_t capabilities;
    uint32_t fenced;
    uint32_t launches_per_step;
    uint64_t weight_bytes; /* device bytes of all quantized matrices */
    uint64_t kv_bytes_per_token;
    uint64_t launches_issued; /* kernels of this library launched on this handle so far */
    uint32_t trace_slots;     /* entries stark_b200_read_trace returns (0: tracing is off) */
    uint32_t persistent;      /* 1: one persistent kernel per token, 0: one kernel per operator */
} stark_b200_info;

#define STARK_B200_CAP_FULL_F32_READOUT UINT64_C(1)
#define STARK_B200_CAP_SERIAL_DECODE UINT64_C(2)
#define STARK_B200_CAP_PREFIX_REWIND UINT64_C(4)
#define STARK_B200_CAP_DEVICE_GREEDY UINT64_C(8)

stark_b200_status stark_b200_model_create(const stark_b200_dense_config *config, stark_b200_model **out_model);
/* A converted-model directory (config.json + model.safetensors in the reference's own layout) loaded, re-tiled
 * and finalized in one call, for hosts that are not Python: the image of
 * stark_glm_load(path_utf8, path_len, options, &model) (vendor/glm-exl3-bridge/include/stark_glm.h:85-87) over the
 * reference's artifact loader (crates/stark-engine/src/engine/language_model/mod.rs:72-127,
 * parameters/loader.rs:80-128, 373-408).  context_tokens 0 = the model's own maximum.  IO_FAILURE: a file is
 * missing or unreadable; INVALID_ARGUMENT: malformed JSON, a tensor with the wrong type, shape or offsets, or a
 * tensor the decoder does not consume; UNSUPPORTED: a well-formed model outside the dense decode path (other layer
 * types, scaled RoPE, biases, bit widths other than 4, ...); CONTEXT_LIMIT: more context than the model allows. */
typedef struct stark_b200_load_options {
    uint32_t struct_size;
    uint32_t abi_version;
    uint64_t context_tokens;
    uint64_t flags; /* 0 */
} stark_b200_load_options;
stark_b200_status stark_b200_load(const uint8_t *path_utf8, size_t path_len, const stark_b200_load_options *options,
                                  stark_b200_model **out_model);
/* desc->pair_halves is set by the library for UPGATE; pass the matrix in the reference's layout. */
stark_b200_status stark_b200_model_set_affine(stark_b200_model *model, uint32_t layer, uint32_t which,
                                              const void *codes, const void *scales, const void *biases,
                                              const stark_b200_affine_desc *desc);
stark_b200_status stark_b200_model_set_vector(stark_b200_model *model, uint32_t layer, uint32_t which,
                                              const float *data, uint32_t count);
/* Tensor parallelism over several GPUs of one node, one process (or thread) and one handle per GPU.
 * The reference runs on a single device, so these two calls replace nothing in it; they shard the same
 * decode graph.  The config passed to model_create holds THIS RANK'S shapes: q_heads, kv_heads and
 * inter divided by the rank count (whole heads; K shards of the o- and down-projections multiples of
 * the quantization group), vocab = the rows of this rank's slice of the read-out matrix, tied = 0.
 * The embedding table is passed whole (vocab_total rows) to every rank.
 *   tp_init     allocates this rank's exchange buffers and returns their 64-byte inter-process handle;
 *   tp_connect  takes the handles of all ranks in rank order (the caller moves them between processes)
 *               and maps the peers' buffers.
 * Afterwards model_finalize, prefill, step and generate_greedy are collective: every rank makes the
 * same calls with the same tokens.  The o- and down-projections are followed by a one-shot all-reduce
 * over NVLink peer memory fused with the bf16 rounding and the residual add; the greedy token is chosen
 * across vocabulary shards on the device.  readout_f32 / readout_bf16 return this rank's slice
 * (config.vocab entries, starting at vocab_offset); readout_logprobs_f32 is UNSUPPORTED.  A peer that
 * does not arrive within the wait limit (4 s unless tp_set_wait changed it, between tp_init and finalize)
 * sets the device error word: the rank's position and exchange tickets stay at the failed exchange, the
 * next drain returns DEVICE_FAILURE and fences the handle (reset then answers RELOAD_REQUIRED; destroy
 * works).  cancel is not collective and must not be used between ranks' calls.
 *   tp_connect_unanswered  instead of tp_connect: every peer is a zeroed local buffer nobody writes, so the
 *               rank's waits run out.  It exists to exercise the bounded wait on one GPU (the reference
 *               fences a backend after a device fault the same way, glm_exl3.rs:243-256). */
stark_b200_status stark_b200_model_tp_init(stark_b200_model *model, uint32_t rank, uint32_t ranks,
                                           uint32_t vocab_offset, uint32_t vocab_total, uint8_t handle_out[64]);
stark_b200_status stark_b200_model_tp_connect(stark_b200_model *model, const uint8_t *handles, size_t handle_bytes);
stark_b200_status stark_b200_model_tp_set_wait(stark_b200_model *model, uint64_t nanoseconds);
stark_b200_status stark_b200_model_tp_connect_unanswered(stark_b200_model *model);
/* Batched prompt passes under tensor parallelism (optional; without these calls, or without the two *_ROWS matrices
 * of every layer, a rank group ingests prompt rows one token at a time).  A prompt pass is a chain of dense
 * contractions over thousands of rows, so its exchange is an all-gather bound by bandwidth: each rank computes its
 * column slice of the attention output, of the residual stream (o and down cut by output rows, contracted over
 * their full width) and of the gated activation, and the ranks store the slices into one another's row buffers
 * over NVLink; every element is the same bits as on one GPU.
 *   tp_rows_init     after tp_connect, before finalize: allocates the row buffers (4 096 rows of hidden +
 *                    attention width + intermediate width, bf16) and returns their 64-byte handle;
 *   tp_rows_connect  takes all ranks' handles in rank order, as tp_connect does. */
stark_b200_status stark_b200_model_tp_rows_init(stark_b200_model *model, uint8_t handle_out[64]);
stark_b200_status stark_b200_model_tp_rows_connect(stark_b200_model *model, const uint8_t *handles, size_t handle_bytes);
stark_b200_status stark_b200_model_finalize(stark_b200_model *model);
stark_b200_status stark_b200_destroy(stark_b200_model **model);
stark_b200_status stark_b200_reset(stark_b200_model *model);
stark_b200_status stark_b200_drain(stark_b200_model *model);
stark_b200_status stark_b200_cancel(stark_b200_model *model);
/* Feeds token_ids; logits of the last row are available afterwards (asynchronous until a read-out
 * or drain).  hybrid::Model::ingest_prefix + step (mod.rs:897-1018). */
stark_b200_status stark_b200_prefill(stark_b200_model *model, const uint32_t *token_ids, size_t count);
stark_b200_status stark_b200_step(stark_b200_model *model, uint32_t token_id);
/* Full-vocabulary logits of the last row, f32 (stark_glm_readout_f32). */
stark_b200_status stark_b200_readout_f32(stark_b200_model *model, float *dst, size_t count);
/* The same logits as bf16 bit patterns, the precision they are computed in. */
stark_b200_status stark_b200_readout_bf16(stark_b200_model *model, uint16_t *dst, size_t count);
/* Full-vocabulary log-probabilities of the last row (f64 arithmetic, scoring.rs:299-336), as f32. */
stark_b200_status stark_b200_readout_logprobs_f32(stark_b200_model *model, float *dst, size_t count);
/* Greedy token of the last row (first index of the maximum). */
stark_b200_status stark_b200_argmax(stark_b200_model *model, uint32_t *out_token);
/* Sampling parameters of the reference's unified sampler
 * (crates/stark-engine/src/backends/cpu/kernel/sampling/unified_sampling.rs:15-117; bounds as in
 * SamplingMethod::validate, crates/stark-generate/src/generation.rs:67-111).  flags: 1 stochastic
 * (Gumbel-max with Philox4x32-10 noise keyed by `seed`; derive the seed per position on the host as the
 * reference does, sampling/prng.rs:12-22), 2 temperature, 4 top_k, 8 top_p, 16 min_p.  flags = 0 is the
 * greedy pick.  top-k / top-p / min-p cut ONE prefix of the descending order (ties: lower index first),
 * exactly as the reference; the token is UINT32_MAX if any logit is not finite. */
typedef struct stark_b200_sampling {
    uint32_t struct_size;
    uint32_t flags;
    uint64_t seed;
    float temperature;
    uint32_t top_k;
    float top_p;
    float min_p;
} stark_b200_sampling;
#define STARK_B200_SAMPLE_STOCHASTIC 1u
#define STARK_B200_SAMPLE_TEMPERATURE 2u
#define STARK_B200_SAMPLE_TOP_K 4u
#define STARK_B200_SAMPLE_TOP_P 8u
#define STARK_B200_SAMPLE_MIN_P 16u
/* With STARK_B200_SAMPLE_ORDERED_F64 (requires STOCHASTIC) the draw follows the generation worker's host
 * sampler instead (crates/stark-generate/src/hybrid.rs:1103-1212): candidates in descending total order
 * (signed zeros distinct, lower id first), probabilities exp(f64((l - max) / temperature)) summed
 * sequentially in f64, the min-p / top-p prefix on those sums, and ONE SplitMix64 draw scaled by the kept
 * mass.  `seed` is the SplitMix64 state before the draw; the caller advances its copy by
 * STARK_B200_SPLITMIX64_STEP per sampled token, as `uniform` does.  Temperature defaults to 1. */
#define STARK_B200_SAMPLE_ORDERED_F64 32u
#define STARK_B200_SPLITMIX64_STEP 0x9e3779b97f4a7c15ull
/* One row of `vocab` logits (io_type BF16 or F32; host or device) -> one token (host). */
stark_b200_status stark_b200_op_sample(const void *logits, uint32_t vocab, uint32_t io_type,
                                       const stark_b200_sampling *params, uint32_t *out_token, uint32_t location,
                                       void *stream);
/* Samples from the logits of the model's last row (Sampling::encode on the last row,
 * encodable_block/sampling/mod.rs:119-249); feed the token back with stark_b200_step.  UNSUPPORTED on a
 * tensor-parallel handle (the logits are sharded). */
stark_b200_status stark_b200_sample(stark_b200_model *model, const stark_b200_sampling *params, uint32_t *out_token);
/* Greedy decode chained on the device: out_tokens[0] is the greedy token of the current logits,
 * out_tokens[i] the one after feeding out_tokens[i-1]; steps + 1 entries.  The analogue of the
 * reference's on-device token chaining (stream.rs:1041-1047). */
stark_b200_status stark_b200_generate_greedy(stark_b200_model *model, uint32_t steps, uint32_t *out_tokens);
/* Prefix reuse: drop rows at and after `position` (KVCacheState::rewind,
 * crates/stark-engine/src/encodable_block/mixer/attention/state.rs:175-195). */
stark_b200_status stark_b200_rewind(stark_b200_model *model, uint64_t position);
stark_b200_status stark_b200_get_info(stark_b200_model *model, stark_b200_info *info);
/* Per-launch timeline of the token sequences issued since the last call: for each of the
 * launches_per_step kernels, six device-clock values in ns {first CTA entered, first wait on the previous
 * kernel returned, last prologue done, last CTA left, last CTA entered, last wait returned}.  Only available when the library was started
 * with STARK_B200_TRACE=1 (UNSUPPORTED otherwise); the analogue of the reference's aggregate
 * profiler (crates/stark-engine/src/engine/hybrid/profile.rs:1-89).  count = 6 * Info.trace_slots
 * (one slot per launch, or per operator of the persistent kernel). */
stark_b200_status stark_b200_read_trace(stark_b200_model *model, uint64_t *dst, size_t count);
/* ------------------------------------------------------------------------------------------
 * Dense multi-token prediction (speculative decoding with a one-layer draft head that shares the embedding and
 * read-out of the target): LanguageModel::dense_mtp_round,
 * crates/stark-engine/src/engine/language_model/dense_mtp.rs:661-686, 786-886; head
 * crates/stark-engine/src/encodable_block/qwen_mtp.rs:262-330.  The call shape follows the reference's own native
 * round of its foreign-engine bridge (stark_glm_native_initial / stark_glm_native_round,
 * vendor/glm-exl3-bridge/include/stark_glm.h:103-110): a pending token goes in, the committed tokens and the next
 * pending token come out.
 *
 * A model created with config.reserved = 1 has a draft head: set its matrices and norms with layer = config.layers
 * (QKV, O, UPGATE, DOWN, ATTN_NORM, MLP_NORM, Q_NORM, K_NORM), STARK_B200_MAT_MTP_FUSION and the three
 * STARK_B200_VEC_MTP_* norms before finalize.  prefill then also primes the head's cache; rewind to a position
 * other than 0 is UNSUPPORTED (the head would need the hidden row before the cut).
 *   mtp_initial  after prefill: the greedy token of the prompt's last row, not yet committed.
 *   mtp_round    drafts (<= 7; the reference allows 3) proposals by the head, one (drafts + 1)-row pass of the
 *                target, acceptance, commit.  policy GREEDY: a proposal is accepted while it equals the arg-max of
 *                the target row before it, which reproduces plain greedy decoding token for token.  policy FORCED:
 *                proposal i is accepted iff bit i of accept_mask is set (a timing aid with a fixed work mix; the
 *                reference's acceptance is data dependent, crates/stark-generate/src/hybrid/mtp.rs:226-263).
 *                tokens[0 .. count) are the committed tokens (tokens[0] is the pending token passed in).
 *   mtp_round_lookup  the same round with `count` proposals supplied by the caller instead of the head: tokens
 *                copied from the request's own context (prompt lookup, crates/stark-engine/src/engine/hybrid/
 *                mtp_lookup.rs:96-121; `RoundPlan::Lookup` in mtp_policy.rs:286-301).  No head step runs; the head's
 *                cache gets the pending row written instead.
 *   policy HELD and mtp_commit: the acceptance rule of the reference is the caller's sampler
 *                (`MtpSampler::target`, crates/stark-engine/src/engine/hybrid/mod.rs:139-171; the exact rejection
 *                sampler of crates/stark-generate/src/hybrid/mtp.rs).  A round with policy HELD proposes and
 *                verifies and stops there: tokens[0 .. count) are the pending token and ALL proposals, nothing is
 *                committed.  The caller reads the rows it needs (mtp_readout_row_f32, row i follows tokens[i]),
 *                decides, and closes the round with mtp_commit(accepted, next_pending): `accepted` proposals are
 *                kept, `next_pending` is the token its sampler drew after the last kept row.  No other call that
 *                moves the model is allowed while a round is open (INVALID_STATE); reset drops it.
 *   mtp_readout_row_f32  full-vocabulary logits of row `row` of the last round's target pass, for a host-side
 *                sampler (valid until the next round).
 */
#define STARK_B200_MTP_GREEDY 0u
#define STARK_B200_MTP_FORCED 1u
#define STARK_B200_MTP_HELD 2u
typedef struct stark_b200_mtp_round_result {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t count;        /* rows committed to the target: 1 + accepted */
    uint32_t accepted;     /* accepted proposals */
    uint32_t proposed;     /* proposals made */
    uint32_t next_pending; /* sampled after the last committed row: the input of the next round */
    uint32_t tokens[8];    /* committed tokens */
    uint64_t position;     /* rows in the target's cache afterwards */
} stark_b200_mtp_round_result;
stark_b200_status stark_b200_mtp_initial(stark_b200_model *model, uint32_t *out_pending);
stark_b200_status stark_b200_mtp_round(stark_b200_model *model, uint32_t pending, uint32_t drafts, uint32_t policy,
                                       uint32_t accept_mask, stark_b200_mtp_round_result *out);
stark_b200_status stark_b200_mtp_round_lookup(stark_b200_model *model, uint32_t pending, const uint32_t *proposals,
                                              uint32_t count, uint32_t policy, uint32_t accept_mask,
                                              stark_b200_mtp_round_result *out);
stark_b200_status stark_b200_mtp_commit(stark_b200_model *model, uint32_t accepted, uint32_t next_pending,
                                        stark_b200_mtp_round_result *out);
stark_b200_status stark_b200_mtp_readout_row_f32(stark_b200_model *model, uint32_t row, float *dst, size_t count);

/* Launch-shape settings of the decode kernels (no counterpart in the reference, whose Metal pipelines
 * fix their threadgroup shapes at build time).  Names: "qmv_consumer_warps" (8 | 16), "qmv_smem_kb",
 * "qmv_ctas_per_sm", "qmv_fold" (0 | 1 | 2), "attn_bufs" (2 | 3), "attn_splits", "pdl" (0 | 1); each
 * starts from the environment variable STARK_B200_<NAME IN CAPITALS>-style switch read at first use.
 * A model uses new values once stark_b200_model_recapture has recorded its launch sequences again
 * (cache and position are kept; single-GPU models only). */
stark_b200_status stark_b200_set_tunable(const char *name, uint32_t value);
stark_b200_status stark_b200_model_recapture(stark_b200_model *model);
/* The CUDA stream (cudaStream_t) the model's work is issued on, for callers that time it with
 * their own events. */
stark_b200_status stark_b200_model_stream(stark_b200_model *model, void **out_stream);

/* ------------------------------------------------------------------------------------------
 * Recorded launch sequences.  The reference records a whole token into one command buffer
 * (crates/stark-engine/src/engine/hybrid/decode_graph.rs; one completion per token,
 * crates/stark-engine/src/engine/language_model/stream/stream.rs:1184); the analogue here is a
 * CUDA graph captured from the per-operator calls issued on `stream` between begin and end.
 * Only calls with device pointers may be recorded.  Call every operator once outside a
 * recording first: first use may allocate library state.
 */
typedef struct stark_b200_graph stark_b200_graph;
stark_b200_status stark_b200_graph_begin(void *stream);
stark_b200_status stark_b200_graph_end(void *stream, stark_b200_graph **out_graph);
stark_b200_status stark_b200_graph_launch(stark_b200_graph *graph, void *stream);
stark_b200_status stark_b200_graph_destroy(stark_b200_graph **graph);

/* ---- Routed-expert (MoE) decoder on the hybrid host path's conventions ----------------------------------
 * f32 activations and logits, GGUF blocks decoded as decode_block, f32 key/value cache; the engine surface
 * is hybrid::Model's (crates/stark-engine/src/engine/hybrid/mod.rs:347,863,897,990: load, reset, ingest,
 * step -> logits).  The step composes the reference's host operators: rms_norm (engine/hybrid/math.rs:18-34),
 * projections + per-head norm + rope + causal attention (engine/hybrid/ripple.rs:653-741), router -> top-k ->
 * softmax over the selected -> expert mixture without a shared expert (engine/hybrid/qwen.rs:872-899),
 * pre-norm residuals and the output projection (ripple.rs:474-482).  head_dim must be 128, hidden a multiple
 * of 256, expert_intermediate a multiple of 256, experts <= 1024, active_experts <= 32. */
typedef struct stark_b200_moe_model stark_b200_moe_model;
typedef struct stark_b200_moe_config {
    uint32_t struct_size;
    uint32_t vocab, hidden, layers, q_heads, kv_heads, head_dim;
    uint32_t experts, active_experts, expert_intermediate;
    uint32_t context_tokens;
    float rms_eps, rope_theta;
} stark_b200_moe_config;
/* Matrices are borrowed qmatrix handles (they must outlive the model): QKV = Q8_0 rows [q; k; v]
 * ((q_heads + 2 kv_heads) * head_dim x hidden), O = Q8_0 hidden x q_heads*head_dim, GATE_UP = one Q4_K bank
 * [2 * experts, expert_intermediate, hidden] (every expert's gate matrix, then every expert's up matrix: one
 * launch serves both), DOWN = Q4_K bank [experts, hidden, expert_intermediate], OUTPUT =
 * Q8_0 vocab x hidden (layer ignored). */
#define STARK_B200_MOE_MAT_QKV 0u
#define STARK_B200_MOE_MAT_O 1u
#define STARK_B200_MOE_MAT_GATE_UP 2u
#define STARK_B200_MOE_MAT_DOWN 3u
#define STARK_B200_MOE_MAT_OUTPUT 4u
/* Host tensors, copied: f32 vectors ATTN_NORM / FFN_NORM [hidden], Q_NORM / K_NORM [head_dim], FINAL_NORM
 * [hidden] (layer ignored), ROUTER f32 [experts, hidden]; TOKEN_TABLE = the Q8_0 blocks of the token
 * embedding [vocab, hidden] in the file's byte layout (layer ignored).  `bytes` must match exactly. */
#define STARK_B200_MOE_TENSOR_ATTN_NORM 0u
#define STARK_B200_MOE_TENSOR_FFN_NORM 1u
#define STARK_B200_MOE_TENSOR_Q_NORM 2u
#define STARK_B200_MOE_TENSOR_K_NORM 3u
#define STARK_B200_MOE_TENSOR_FINAL_NORM 4u
#define STARK_B200_MOE_TENSOR_ROUTER 5u
#define STARK_B200_MOE_TENSOR_TOKEN_TABLE 6u
stark_b200_status stark_b200_moe_model_create(const stark_b200_moe_config *config, stark_b200_moe_model **out_model);
stark_b200_status stark_b200_moe_model_set_matrix(stark_b200_moe_model *model, uint32_t kind, uint32_t layer,
                                                  const stark_b200_qmatrix *matrix);
stark_b200_status stark_b200_moe_model_set_tensor(stark_b200_moe_model *model, uint32_t kind, uint32_t layer,
                                                  const void *host_data, size_t bytes);
/* Expert parallelism over the GPUs of one node, one process per GPU (no counterpart in the reference, which runs
 * on one device).  Every rank runs the whole token except the expert feed-forward: rank r holds experts
 * [r * experts / ranks, (r + 1) * experts / ranks) -- its GATE_UP and DOWN banks are set AFTER ep_init and contain
 * only those -- and computes the selected experts it owns; the owners push their output rows to every rank over
 * NVLink peer mappings and every rank forms the mixture in selection order, so logits and tokens are the same
 * bits on every rank and for every rank count.  ep_init (before the first token) allocates this rank's exchange
 * region and returns its 64-byte CUDA IPC handle; ep_connect takes the handles of all ranks in rank order
 * (handle_bytes = 64 * ranks).  Calls that run tokens are collective: every rank makes the same calls with the
 * same tokens.  A rank whose peers do not answer within the wait (default 4 s, ep_set_wait before the first
 * token) reports DEVICE_FAILURE and resets. */
stark_b200_status stark_b200_moe_model_ep_init(stark_b200_moe_model *model, uint32_t rank, uint32_t ranks,
                                               uint8_t *handle_out);
stark_b200_status stark_b200_moe_model_ep_connect(stark_b200_moe_model *model, const uint8_t *handles, size_t handle_bytes);
stark_b200_status stark_b200_moe_model_ep_set_wait(stark_b200_moe_model *model, uint64_t nanoseconds);
stark_b200_status stark_b200_moe_model_reset(stark_b200_moe_model *model);
/* Appends `count` prompt tokens to the cache without computing logits (Model::ingest). */
stark_b200_status stark_b200_moe_model_ingest(stark_b200_moe_model *model, const uint32_t *tokens, uint32_t count);
/* Consumes one token and returns the full-vocabulary f32 logits for the next (Model::step: finite, else the
 * model is reset and DEVICE_FAILURE returned).  logits_host may be NULL. */
stark_b200_status stark_b200_moe_model_step(stark_b200_moe_model *model, uint32_t token, float *logits_host,
                                            size_t count);
/* Greedy decode chained on the device: consumes `first`, then each step's own pick; out_tokens[i] is the pick
 * after i + 1 steps (first index of the maximum logit). */
stark_b200_status stark_b200_moe_model_generate_greedy(stark_b200_moe_model *model, uint32_t first, uint32_t steps,
                                                       uint32_t *out_tokens);
/* Expert ids the last token selected, [layers][active_experts], selection order. */
stark_b200_status stark_b200_moe_model_last_experts(stark_b200_moe_model *model, uint32_t *ids_host, size_t count);
stark_b200_status stark_b200_moe_model_position(const stark_b200_moe_model *model, uint32_t *out_position);
/* Kernel launches of one token step with logits (the graph's node count). */
stark_b200_status stark_b200_moe_model_launches_per_token(const stark_b200_moe_model *model, uint32_t *out_launches);
/* The CUDA stream (cudaStream_t) the model's work is issued on, for events around it. */
stark_b200_status stark_b200_moe_model_stream(const stark_b200_moe_model *model, void **out_stream);
stark_b200_status stark_b200_moe_model_destroy(stark_b200_moe_model **model);

#ifdef __cplusplus
}
#endif

#endif /* STARK_B200_H */
