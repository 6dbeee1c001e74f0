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
    float *attn_norm = nullptr, *mlp_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    uint16_t *attn_norm_b16 = nullptr, *mlp_norm_b16 = nullptr;  // the norm weights rounded to bf16, as the kernels use them
    KvLayer kv{nullptr, nullptr};
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
    uint32_t tp_vocab_offset = 0, tp_vocab_total = 0;
    bool tp_connected = false, tp_stand_ins = false;
    // batched prompt ingest (prefill_model.cu): rows of one chunk, allocated at first use
    uint32_t prefill_state = 0;  // 0 not examined, 1 the batched path serves this model, 2 it does not
    uint32_t *chunk_tokens = nullptr;
    uint16_t *chunk_h = nullptr, *chunk_x = nullptr, *chunk_qkv = nullptr, *chunk_attn = nullptr, *chunk_act = nullptr;
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
stark_b200_status model_finalize(Model *m);
stark_b200_status model_reset(Model *m);
stark_b200_status model_recapture(Model *m);
stark_b200_status model_rewind(Model *m, uint64_t position);
stark_b200_status model_prefill(Model *m, const uint32_t *ids, size_t count);
stark_b200_status model_step(Model *m, uint32_t token, bool chained);
bool model_batched_prefill_ready(Model *m);
stark_b200_status model_prefill_batched(Model *m, const uint32_t *ids, size_t rows);
stark_b200_status model_drain(Model *m);
stark_b200_status model_next_token(Model *m, uint32_t *out);
stark_b200_status model_readout_bf16(Model *m, uint16_t *dst, size_t count);
stark_b200_status model_readout_f32(Model *m, float *dst, size_t count);
stark_b200_status model_generate_greedy(Model *m, uint32_t steps, uint32_t *out_tokens);
stark_b200_status model_read_trace(Model *m, unsigned long long *dst, size_t count);

}  // namespace sb
