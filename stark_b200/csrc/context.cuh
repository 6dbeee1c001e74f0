// Per-device library state: the device error word and grow-only staging buffers used when a
// caller passes host pointers to a per-operator entry point.
#pragma once
#include "common.cuh"

namespace sb {

struct DeviceContext {
    int device = -1;
    uint32_t *error_word = nullptr;  // device memory, zero-initialised
    void *stage_in = nullptr;
    size_t stage_in_bytes = 0;
    void *stage_out = nullptr;
    size_t stage_out_bytes = 0;
    void *scratch = nullptr;  // small per-op scratch (partials)
    size_t scratch_bytes = 0;
};

// Context of the current device, created on first use.  Returns nullptr if allocation fails.
DeviceContext *device_context();
stark_b200_status ensure_buffer(void **buf, size_t *have, size_t want);

}  // namespace sb
