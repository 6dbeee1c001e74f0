// Launch-shape settings of the decode kernels.  Each starts from its environment variable (read once,
// when first needed) and can be changed at run time through stark_b200_set_tunable; a model picks the new
// values up when its launch sequences are recorded again (stark_b200_model_recapture).
#pragma once
#include <stdint.h>

namespace sb {

struct Tunables {
    uint32_t qmv_consumer_warps;  // STARK_B200_QMV_CW      8 | 16
    uint32_t qmv_smem_kb;         // STARK_B200_QMV_SMEM_KB 0 = the shape's own budget
    uint32_t qmv_ctas_per_sm;     // STARK_B200_QMV_CTAS    0 = the shape's own count
    uint32_t qmv_fold;            // STARK_B200_QMV_FOLD    0 | 1 | 2
    uint32_t attn_bufs;           // STARK_B200_ATTN_BUFS   2 | 3
    uint32_t attn_splits;         // STARK_B200_ATTN_SPLITS 0 = chosen from the head count
    uint32_t attn_regs;           // STARK_B200_ATTN_REGS   96 | 128 registers per attention thread
    uint32_t pdl;                 // STARK_B200_PDL         programmatic dependent launch on / off
};

Tunables &tunables();
// Returns false for an unknown name or a value outside the setting's range.
bool set_tunable(const char *name, uint32_t value);

}  // namespace sb
