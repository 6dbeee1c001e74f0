#include "tunables.cuh"

#include <cstdlib>
#include <cstring>

namespace sb {

namespace {

struct Entry {
    const char *name, *env;
    uint32_t Tunables::*field;
    uint32_t fallback, lo, hi;
};

const Entry kEntries[] = {
    {"qmv_consumer_warps", "STARK_B200_QMV_CW", &Tunables::qmv_consumer_warps, 8u, 8u, 16u},
    {"qmv_smem_kb", "STARK_B200_QMV_SMEM_KB", &Tunables::qmv_smem_kb, 0u, 0u, 200u},
    {"qmv_roomy_kb", "STARK_B200_QMV_ROOMY_KB", &Tunables::qmv_roomy_kb, 104u, 32u, 110u},
    {"qmv_ctas_per_sm", "STARK_B200_QMV_CTAS", &Tunables::qmv_ctas_per_sm, 0u, 0u, 2u},
    {"qmv_fold", "STARK_B200_QMV_FOLD", &Tunables::qmv_fold, 0u, 0u, 2u},
    {"attn_bufs", "STARK_B200_ATTN_BUFS", &Tunables::attn_bufs, 3u, 2u, 3u},
    {"attn_splits", "STARK_B200_ATTN_SPLITS", &Tunables::attn_splits, 0u, 0u, 32u},
    {"attn_regs", "STARK_B200_ATTN_REGS", &Tunables::attn_regs, 96u, 96u, 128u},
    {"pdl", "STARK_B200_PDL", &Tunables::pdl, 1u, 0u, 1u},
    {"prefill_batch", "STARK_B200_PREFILL_BATCH", &Tunables::prefill_batch, 1u, 0u, 1u},
    {"gemm_stop_after", "STARK_B200_GEMM_STOP_AFTER", &Tunables::gemm_stop_after, 0u, 0u, 3u},
    {"prefill_min_rows", "STARK_B200_PREFILL_MIN_ROWS", &Tunables::prefill_min_rows, 16u, 1u, 1u << 20},
    {"rows_matvec", "STARK_B200_ROWS_MATVEC", &Tunables::rows_matvec, 1u, 0u, 1u},
    {"rows_attention", "STARK_B200_ROWS_ATTENTION", &Tunables::rows_attention, 1u, 0u, 1u},
    {"tp_stage", "STARK_B200_TP_STAGE", &Tunables::tp_stage, 0u, 0u, 1u},
    {"prefill_attn_tc", "STARK_B200_PREFILL_ATTN_TC", &Tunables::prefill_attn_tc, 1u, 0u, 1u},
    {"attn_tc_stop_after", "STARK_B200_ATTN_TC_STOP_AFTER", &Tunables::attn_tc_stop_after, 0u, 0u, 2u},
    {"prefill_attn_warps", "STARK_B200_PREFILL_ATTN_WARPS", &Tunables::prefill_attn_warps, 4u, 4u, 8u},
    {"gemm_half_tiles", "STARK_B200_GEMM_HALF_TILES", &Tunables::gemm_half_tiles, 1u, 0u, 2u},
    {"tp_rows_push", "STARK_B200_TP_ROWS_PUSH", &Tunables::tp_rows_push, 2u, 0u, 2u},
};

bool valid(const Entry &e, uint32_t v) {
    if (v < e.lo || v > e.hi) return false;
    if (e.field == &Tunables::qmv_consumer_warps) return v == 8u || v == 16u;
    if (e.field == &Tunables::qmv_smem_kb) return v == 0u || v >= 32u;
    return true;
}

}  // namespace

Tunables &tunables() {
    static Tunables t = [] {
        Tunables v{};
        for (const Entry &e : kEntries) {
            v.*(e.field) = e.fallback;
            if (const char *s = getenv(e.env)) {
                const long parsed = strtol(s, nullptr, 10);
                if (parsed >= 0 && valid(e, (uint32_t)parsed)) v.*(e.field) = (uint32_t)parsed;
            }
        }
        return v;
    }();
    return t;
}

bool set_tunable(const char *name, uint32_t value) {
    if (!name) return false;
    for (const Entry &e : kEntries)
        if (strcmp(name, e.name) == 0) {
            if (!valid(e, value)) return false;
            tunables().*(e.field) = value;
            return true;
        }
    return false;
}

}  // namespace sb
