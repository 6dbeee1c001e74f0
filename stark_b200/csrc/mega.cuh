// Persistent decode kernel: one launch runs the whole token.  Interface between model.cu (which
// builds the operator list) and mega.cu (the kernel).
#pragma once
#include "ops.cuh"
#include "qmv.cuh"

namespace sb {

enum MegaOpType : uint32_t {
    kOpEmbed = 0,        // h = embedding row of the input token                (CTA 0)
    kOpGemv = 1,         // quantized matvec with fused prologue / epilogue     (all CTAs)
    kOpAttnPartial = 2,  // split-KV partials of one layer                      (kv_heads * splits CTAs)
    kOpAttnMerge = 3,    // merge of the partials                               (kv_heads CTAs)
    kOpFinalize = 4,     // greedy token from the read-out partials, advance    (CTA 0)
    kOpIngestAdvance = 5 // end of a cache-only prompt row                      (CTA 0)
};

struct MegaOp {
    uint32_t type;
    uint32_t dep;           // operator whose completion gates this one's inputs (0xffffffff: none)
    uint32_t participants;  // CTAs that signal completion of this operator
    uint32_t reserved;
    // kOpGemv
    const uint8_t *w;
    const uint16_t *x;
    uint16_t *y;
    const float *norm_weight;
    const uint16_t *resid;
    uint32_t rows, row_tiles, groups, stage_records, stages_per_tile, pair_halves, unit_tiles;
    uint32_t prologue, epilogue, rpw, pred, pad0;
    // kOpAttn*
    uint16_t *keys, *values;
    const float *q_norm, *k_norm;
};

struct MegaParams {
    const MegaOp *ops;
    uint32_t num_ops;
    uint32_t num_stages, stage_capacity;  // weight ring geometry
    uint32_t max_columns;                 // widest matvec input (sizes the f16 input buffer)
    StepState *state;
    unsigned long long *done;  // [num_ops] completion counters, zeroed by the host before each launch
    // embedding table (re-tiled 4-bit records)
    const uint8_t *embed;
    uint32_t embed_rows, embed_columns;
    uint16_t *h;
    // attention
    const uint16_t *qkv;
    uint16_t *attn;
    const int32_t *block_table;
    const float *rope_cos, *rope_sin;
    float *attn_scratch;
    float eps, attn_scale;
    uint32_t q_heads, kv_heads, attn_splits;
    // read-out
    float *partial_max;
    uint32_t *partial_index;
    uint32_t *generated;
    const uint32_t *pending;
    uint32_t *error_word;
    TraceSlot *trace;  // [num_ops] or nullptr
};

// Shared memory the kernel needs for a ring of `num_stages` slots.
uint32_t mega_smem_bytes(uint32_t num_stages, uint32_t stage_capacity, uint32_t max_columns);
stark_b200_status mega_launch(const MegaParams &p, uint32_t grid, uint32_t smem_bytes, cudaStream_t stream);

}  // namespace sb
