// Tensor-parallel exchange kernels (see tp.cuh): flag-synchronised one-shot all-reduce fused with the
// bf16 rounding and residual add that follow the o- and down-projections, and the gather that picks
// the greedy token across vocabulary shards.  Peers' memory is reached with plain system-scope loads
// and stores; every wait on a peer is bounded in time and reports through the device error word.
#include "tp.cuh"

namespace sb {

namespace {

constexpr unsigned long long kPeerWaitNs = 4000000000ull;  // give up on a peer after 4 s

__device__ inline void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ inline uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ inline float4 ld_sys_f32x4(const float *p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ inline uint2 ld_sys_u32x2(const uint32_t *p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ inline void st_sys_u32x2(uint32_t *p, uint2 v) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// Thread r < size tells rank r that this rank's data for exchange `ticket` is in place, then waits
// until rank r has said the same.  Returns false (and records the error) when the wait ran out.
__device__ inline bool exchange_flags(const TpRegion &g, uint32_t set, uint32_t ticket, uint32_t *error_word) {
    bool ok = true;
    if (threadIdx.x < g.size) {
        const uint32_t r = threadIdx.x;
        __threadfence_system();
        st_release_sys(tp_flags(g.base[r], set) + g.rank, ticket);
        const uint32_t *mine = tp_flags(g.base[g.rank], set) + r;
        const unsigned long long t0 = global_ns();
        uint32_t spins = 0;
        while (ld_acquire_sys(mine) != ticket) {
            if (++spins > 32u) {
                __nanosleep(100);
                if (global_ns() - t0 > kPeerWaitNs) {
                    atomicOr(error_word, kErrPeerTimeout);
                    ok = false;
                    break;
                }
            }
        }
    }
    return __syncthreads_and(ok ? 1 : 0) != 0;
}

__global__ void __launch_bounds__(1024) tp_allreduce_residual_kernel(TpRegion g, uint32_t buf, uint32_t *seq,
                                                                     uint16_t *h, uint32_t *error_word,
                                                                     TraceSlot *trace) {
    pdl_launch_dependents();
    if (threadIdx.x == 0 && trace) trace_min(&trace->start);
    pdl_wait();  // this rank's partial (the matvec before this kernel) and h are final
    if (threadIdx.x == 0 && trace) trace_min(&trace->ready);
    const uint32_t ticket = seq[buf] + 1u;
    const bool ok = exchange_flags(g, buf, ticket, error_word);
    if (threadIdx.x == 0 && trace) trace_max(&trace->compute);  // every peer's share is in place
    if (ok) {
        for (uint32_t i = threadIdx.x * 4u; i < g.hidden; i += blockDim.x * 4u) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t r = 0; r < g.size; ++r) {  // rank order: every rank computes the same bits
                const float4 v = ld_sys_f32x4(tp_partial(g.base[r], buf, g.hidden) + i);
                acc.x += v.x;
                acc.y += v.y;
                acc.z += v.z;
                acc.w += v.w;
            }
            const uint2 old = *reinterpret_cast<const uint2 *>(h + i);
            const float r0 = bf16_bits_to_f32((uint16_t)(old.x & 0xffffu)), r1 = bf16_bits_to_f32((uint16_t)(old.x >> 16));
            const float r2 = bf16_bits_to_f32((uint16_t)(old.y & 0xffffu)), r3 = bf16_bits_to_f32((uint16_t)(old.y >> 16));
            uint2 o;
            o.x = (uint32_t)f32_to_bf16_bits(bf16_round(acc.x) + r0) | ((uint32_t)f32_to_bf16_bits(bf16_round(acc.y) + r1) << 16);
            o.y = (uint32_t)f32_to_bf16_bits(bf16_round(acc.z) + r2) | ((uint32_t)f32_to_bf16_bits(bf16_round(acc.w) + r3) << 16);
            *reinterpret_cast<uint2 *>(h + i) = o;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        seq[buf] = ticket;
        if (trace) trace_max(&trace->end);
    }
}

__global__ void __launch_bounds__(256) tp_argmax_finalize_kernel(TpRegion g, uint32_t *seq, const float *partial_max,
                                                                 const uint32_t *partial_index, uint32_t count,
                                                                 uint32_t vocab_offset, StepState *state,
                                                                 uint32_t *generated, uint32_t *error_word) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float vs[8];
    __shared__ uint32_t is[8];
    float best = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) {
        const float v = partial_max[i];
        const uint32_t ix = partial_index[i];
        if (v > best || (v == best && ix < bi)) {
            best = v;
            bi = ix;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) {
            best = ov;
            bi = oi;
        }
    }
    if ((threadIdx.x & 31u) == 0) {
        vs[threadIdx.x >> 5] = best;
        is[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    const uint32_t set = kTpFlagSets - 1u;
    const uint32_t ticket = seq[set] + 1u;
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < blockDim.x / 32u; ++w)
            if (vs[w] > best || (vs[w] == best && is[w] < bi)) {
                best = vs[w];
                bi = is[w];
            }
        vs[0] = best;
        is[0] = bi == 0xffffffffu ? bi : bi + vocab_offset;
    }
    __syncthreads();
    if (threadIdx.x < g.size)  // this rank's candidate into every rank's slot table
        st_sys_u32x2(tp_gather(g.base[threadIdx.x]) + 2u * g.rank, make_uint2(__float_as_uint(vs[0]), is[0]));
    const bool ok = exchange_flags(g, set, ticket, error_word);
    if (threadIdx.x == 0) {
        float top = -INFINITY;
        uint32_t ti = 0xffffffffu;
        if (ok) {
            for (uint32_t r = 0; r < g.size; ++r) {
                const uint2 c = ld_sys_u32x2(tp_gather(g.base[g.rank]) + 2u * r);
                const float v = __uint_as_float(c.x);
                if (v > top || (v == top && c.y < ti)) {
                    top = v;
                    ti = c.y;
                }
            }
        }
        // a non-finite logit was given the key +inf by the matvec epilogue: the row is invalid
        const uint32_t tok = isfinite(top) ? ti : 0xffffffffu;
        state->next_token = tok;
        if (generated && state->gen_cursor < state->gen_capacity) generated[state->gen_cursor++] = tok;
        state->position += 1u;
        state->token = tok;
        seq[set] = ticket;
    }
}

template <typename... Args>
stark_b200_status launch_one(void (*kernel)(Args...), uint32_t threads, bool pdl, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(threads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
    return STARK_B200_OK;
}

}  // namespace

stark_b200_status tp_allreduce_residual_launch(const TpRegion &region, uint32_t buf, uint32_t *seq, uint16_t *h,
                                               uint32_t *error_word, TraceSlot *trace, bool pdl, cudaStream_t stream) {
    if (region.size < 2 || region.size > kMaxTpRanks || region.rank >= region.size || buf > 1u ||
        region.hidden % 4u != 0)
        return STARK_B200_INVALID_ARGUMENT;
    return launch_one(tp_allreduce_residual_kernel, 1024u, pdl, stream, region, buf, seq, h, error_word, trace);
}

stark_b200_status tp_argmax_finalize_launch(const TpRegion &region, uint32_t *seq, const float *partial_max,
                                            const uint32_t *partial_index, uint32_t count, uint32_t vocab_offset,
                                            StepState *state, uint32_t *generated, uint32_t *error_word, bool pdl,
                                            cudaStream_t stream) {
    if (region.size < 2 || region.size > kMaxTpRanks || region.rank >= region.size) return STARK_B200_INVALID_ARGUMENT;
    return launch_one(tp_argmax_finalize_kernel, 256u, pdl, stream, region, seq, partial_max, partial_index, count,
                      vocab_offset, state, generated, error_word);
}

}  // namespace sb
