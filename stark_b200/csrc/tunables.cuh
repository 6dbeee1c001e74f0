// Launch-shape settings of the decode kernels.  Each starts from its environment variable (read once,
// when first needed) and can be changed at run time through stark_b200_set_tunable; a model picks the new
// values up when its launch sequences are recorded again (stark_b200_model_recapture).
#pragma once
#include <stdint.h>

namespace sb {

struct Tunables {
    uint32_t qmv_consumer_warps;  // STARK_B200_QMV_CW      8 | 16
    uint32_t qmv_smem_kb;         // STARK_B200_QMV_SMEM_KB 0 = the shape's own budget (56: two CTAs and a three-buffer attention CTA per SM)
    uint32_t qmv_roomy_kb;        // STARK_B200_QMV_ROOMY_KB per-CTA budget of launches flagged `roomy`
    uint32_t qmv_ctas_per_sm;     // STARK_B200_QMV_CTAS    0 = the shape's own count
    uint32_t qmv_fold;            // STARK_B200_QMV_FOLD    0 | 1 | 2
    uint32_t attn_bufs;           // STARK_B200_ATTN_BUFS   2 | 3
    uint32_t attn_splits;         // STARK_B200_ATTN_SPLITS 0 = chosen from the head count
    uint32_t attn_regs;           // STARK_B200_ATTN_REGS   96 | 128 registers per attention thread
    uint32_t pdl;                 // STARK_B200_PDL         programmatic dependent launch on / off
    uint32_t prefill_batch;       // STARK_B200_PREFILL_BATCH    0: prompt rows one at a time, 1: in chunks on the tensor cores
    uint32_t gemm_stop_after;     // STARK_B200_GEMM_STOP_AFTER  bring-up aid of the tensor-core contraction (0: whole kernel)
    uint32_t prefill_min_rows;    // STARK_B200_PREFILL_MIN_ROWS fewest cache-only rows worth a batched pass
    uint32_t tp_stage;            // STARK_B200_TP_STAGE         1: the tensor-parallel reduction also prepares the next matvec's input (one CTA; measured slower)
    uint32_t prefill_attn_tc;     // STARK_B200_PREFILL_ATTN_TC  1: attention of a prompt pass (more than 16 rows) on the tcgen05 tensor cores, 0: mma.sync
    uint32_t attn_tc_stop_after;  // STARK_B200_ATTN_TC_STOP_AFTER bring-up aid of that kernel (0: whole kernel)
    uint32_t prefill_attn_warps;  // STARK_B200_PREFILL_ATTN_WARPS warps of a prompt pass's attention CTA (4 or 8): rows that share a key / value tile
    uint32_t gemm_half_tiles;     // STARK_B200_GEMM_HALF_TILES  128-row tiles in the prompt contraction: 0 never, 1 where 256-row tiles leave SMs idle, 2 always
    uint32_t tp_rows_push;        // STARK_B200_TP_ROWS_PUSH     a prompt pass's contractions store their tiles to the other ranks themselves: 1 always, 2 between two ranks only, 0 never (a copy kernel after each)
    uint32_t rows_attention;      // STARK_B200_ROWS_ATTENTION   1: a handful of rows attend in the keys-as-rows form, 0: in 16-row tiles
    uint32_t rows_matvec;         // STARK_B200_ROWS_MATVEC      1: up to 8 rows go through the several-rows matvec, 0: through the tensor-core tile kernels
};

Tunables &tunables();
// Returns false for an unknown name or a value outside the setting's range.
bool set_tunable(const char *name, uint32_t value);

}  // namespace sb
