// Dense decode engine state (see model.cu).
#pragma once
#include <vector>

#include "context.cuh"
#include "mega.cuh"
#include "ops.cuh"
#include "qmv.cuh"
#include "tp.cuh"

namespace sb {

struct ModelLayer {
    QMatrix *qkv = nullptr, *o = nullptr, *upgate = nullptr, *down = nullptr;
    // tensor parallel, optional: this rank's OUTPUT ROWS of the o- and down-projection over all input columns, for
    // prompt passes (the token path uses the column cuts above)
    QMatrix *o_rows = nullptr, *down_rows = nullptr;
    float *attn_norm = nullptr, *mlp_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    uint16_t *attn_norm_b16 = nullptr, *mlp_norm_b16 = nullptr;  // the norm weights rounded to bf16, as the kernels use them
    KvLayer kv{nullptr, nullptr};
};

// Draft head of the dense multi-token-prediction path (crates/stark-engine/src/encodable_block/qwen_mtp.rs:36-330):
// rows [norm_e(embedding(token)) ; norm_h(hidden)] -> fusion [D, 2D] -> one decoder layer with a cache of its own
// -> output norm -> the target's read-out matrix.  Its layer is stored as layers[cfg.layers].
struct MtpHead {
    bool enabled = false;
    QMatrix *fusion = nullptr;
    float *embed_norm = nullptr, *hidden_norm = nullptr, *out_norm = nullptr;
    StepState *state = nullptr;        // device: position = rows in the head's cache, token = next input
    uint64_t position = 0;             // host mirror
    uint16_t *last_hidden = nullptr;   // [D] normalized hidden of the target's last committed row
    uint16_t *draft_in = nullptr;      // [D] hidden input of the next draft step (then that step's own output)
    uint16_t *joined = nullptr;        // [2D]
    uint16_t *embedded = nullptr;      // [D]
    uint16_t *stream_h = nullptr;      // [D] residual stream of the head
    uint16_t *rows_e = nullptr;        // [chunk, D] embedding rows of a priming / repair pass
    uint16_t *rows_j = nullptr;        // [chunk, 2D] joined rows
    uint16_t *rows_hidden = nullptr;   // [16, D] normalized hidden rows of a verify pass
    uint16_t *rows_logits = nullptr;   // [16, vocab] logits rows of a verify pass
    uint32_t *rows_pick = nullptr;     // [16] greedy pick of each verify row
    uint32_t *host_words = nullptr;    // pinned scratch for the round's small read-backs
    // a round whose acceptance the caller decides stays open between mtp_round (policy HELD) and mtp_commit
    uint32_t open_rows = 0, open_prefix = 0;
    bool open_head_advance = false, open_serial = false;
    cudaGraphExec_t draft_graph = nullptr;
    uint32_t verified_rows = 0;        // rows of the last verify pass (read-out window)
    bool has_pending = false;
};

struct Model {
    stark_b200_dense_config cfg{};
    int device = 0;
    cudaStream_t stream = nullptr;
    QMatrix *embed = nullptr, *lm_head = nullptr;
    std::vector<ModelLayer> layers;
    float *final_norm = nullptr;
    uint16_t *final_norm_b16 = nullptr;
    uint32_t num_blocks = 0;
    int32_t *block_table = nullptr;
    float *rope_cos = nullptr, *rope_sin = nullptr;
    StepState *state = nullptr;
    uint32_t *pending = nullptr;    // prompt tokens still to be ingested (device)
    uint32_t *generated = nullptr;  // greedy tokens of a device-chained run (device)
    TraceSlot *trace = nullptr;     // optional per-launch timeline (STARK_B200_TRACE=1)
    uint32_t trace_slots = 0;
    uint16_t *h_alt = nullptr;      // second residual-stream buffer (tensor parallel only)
    uint16_t *h = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr, *logits = nullptr;
    float *attn_scratch = nullptr;
    uint32_t *attn_counters = nullptr;
    float *partial_max = nullptr;
    uint32_t *partial_index = nullptr;
    uint32_t attn_splits = 1;
    cudaGraphExec_t step_graph = nullptr, ingest_graph = nullptr;
    // persistent-kernel path (STARK_B200_MEGA=1)
    bool use_mega = false;
    MegaOp *mega_ops = nullptr, *mega_ingest_ops = nullptr;
    uint32_t mega_num_ops = 0, mega_num_ingest_ops = 0, mega_grid = 0, mega_smem = 0, mega_splits = 1;
    unsigned long long *mega_done = nullptr;
    float *mega_scratch = nullptr;
    MegaParams mega_full{}, mega_ingest{};
    uint32_t step_launches = 0, ingest_launches = 0;
    // tensor-parallel exchange (tp.size == 0: single GPU).  cfg then holds this rank's shard shapes
    // (heads, intermediate width, read-out rows); the embedding table is whole on every rank.
    TpRegion tp{};
    uint8_t *tp_local = nullptr;   // this rank's exchange region
    uint32_t *tp_seq = nullptr;    // [0] tokens finished: the base of the exchange tickets
    void *tp_staged = nullptr;     // the input row a reduction leaves ready for the matvec after it (qmv_staged_bytes)
    uint32_t tp_vocab_offset = 0, tp_vocab_total = 0;
    bool tp_connected = false, tp_stand_ins = false;
    // prompt passes under tensor parallelism (optional second exchange region: whole rows of h, attention output
    // and gated activation, gathered from the ranks' column slices)
    TpRowsRegion tp_rows{};
    uint8_t *tp_rows_local = nullptr;
    uint32_t *tp_rows_arrive = nullptr;
    uint32_t tp_rows_ticket = 0;       // gathers launched so far (the same number on every rank)
    bool tp_rows_connected = false;
    // batched prompt ingest (prefill_model.cu): rows of one chunk, allocated at first use
    uint32_t prefill_state = 0;  // 0 not examined, 1 the batched path serves this model, 2 it does not
    uint32_t *chunk_tokens = nullptr;
    uint16_t *chunk_h = nullptr, *chunk_x = nullptr, *chunk_qkv = nullptr, *chunk_attn = nullptr, *chunk_act = nullptr;
    float *rows_attn_partials = nullptr;  // working memory of the few-rows attention (split key tiles)
    MtpHead mtp;
    void *sample_scratch = nullptr;     // device working memory of the sampler (allocated at first use)
    StepState *host_state = nullptr;    // pinned
    uint16_t *host_logits = nullptr;    // pinned
    uint64_t position = 0;              // host mirror of state->position
    uint64_t launches_issued = 0;       // kernels of this library launched so far
    bool finalized = false, fenced = false, has_logits = false;
    volatile bool cancel_requested = false;
    ~Model();
};

stark_b200_status model_create(const stark_b200_dense_config &cfg, Model **out);
stark_b200_status model_set_matrix(Model *m, uint32_t layer, uint32_t which, QMatrix *q);  // takes ownership
stark_b200_status model_set_vector(Model *m, uint32_t layer, uint32_t which, const float *data, uint32_t count);
// Tensor parallelism, between create and finalize: init allocates this rank's exchange region and
// returns its 64-byte inter-process handle; connect maps the regions of all ranks (handles in rank
// order, this rank's own entry ignored).  After that finalize and every token are collective calls.
stark_b200_status model_tp_init(Model *m, uint32_t rank, uint32_t size, uint32_t vocab_offset, uint32_t vocab_total,
                                uint8_t *handle_out);
stark_b200_status model_tp_connect(Model *m, const uint8_t *handles);
stark_b200_status model_tp_set_wait(Model *m, uint64_t nanoseconds);
stark_b200_status model_tp_connect_unanswered(Model *m);
// Optional, after tp_connect and before finalize: the exchange region of batched prompt passes (same handle
// protocol).  Without it, or without the row cuts of o and down, prompt rows go through the token path.
stark_b200_status model_tp_rows_init(Model *m, uint8_t *handle_out);
stark_b200_status model_tp_rows_connect(Model *m, const uint8_t *handles);
stark_b200_status model_finalize(Model *m);
stark_b200_status model_reset(Model *m);
stark_b200_status model_recapture(Model *m);
stark_b200_status model_rewind(Model *m, uint64_t position);
stark_b200_status model_prefill(Model *m, const uint32_t *ids, size_t count);
stark_b200_status model_step(Model *m, uint32_t token, bool chained);
bool model_batched_prefill_ready(Model *m);
stark_b200_status model_prefill_batched(Model *m, const uint32_t *ids, size_t rows, size_t ids_total);
stark_b200_status model_rows_pass(Model *m, const uint32_t *tokens_device, uint32_t mrows, uint32_t first_pos);
stark_b200_status ensure_chunk_buffers(Model *m);
stark_b200_status model_drain(Model *m);
stark_b200_status model_next_token(Model *m, uint32_t *out);
stark_b200_status model_readout_bf16(Model *m, uint16_t *dst, size_t count);
stark_b200_status model_readout_f32(Model *m, float *dst, size_t count);
stark_b200_status model_generate_greedy(Model *m, uint32_t steps, uint32_t *out_tokens);
stark_b200_status model_read_trace(Model *m, unsigned long long *dst, size_t count);

// ---- dense multi-token prediction (mtp.cu)
constexpr uint32_t kMaxMtpDrafts = 7;   // rows of a verify pass <= 8 (the reference allows 3; dense_mtp.rs:671)
stark_b200_status mtp_create(Model *m);
void mtp_destroy(Model *m);
stark_b200_status mtp_finalize(Model *m);
stark_b200_status mtp_reset(Model *m);
// after a chunk of the target's prompt rows: the head's cache rows for the pairs (next token, row's hidden);
// `pairs` <= mrows is how many rows have a next token
stark_b200_status mtp_prime_rows(Model *m, uint32_t mrows, uint32_t pairs, uint32_t first_pos);
// after the prompt's last row went through the token path: its normalized hidden becomes the head's input
stark_b200_status mtp_after_prompt(Model *m);
// a prompt continued at a position > 0: the pair (chunk_tokens[0], last hidden) becomes the head's next cache row
stark_b200_status mtp_prime_continue(Model *m);
stark_b200_status mtp_round(Model *m, uint32_t pending, uint32_t drafts, uint32_t policy, uint32_t accept_mask,
                            stark_b200_mtp_round_result *out, const uint32_t *proposals = nullptr);
stark_b200_status mtp_commit(Model *m, uint32_t accepted, uint32_t next_pending, stark_b200_mtp_round_result *out);
stark_b200_status mtp_readout_row_f32(Model *m, uint32_t row, float *dst, size_t count);

}  // namespace sb
