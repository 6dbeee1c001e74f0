// Tensor-parallel end-of-token kernels (see tp.cuh; the all-reduce itself lives in the matvecs): the
// gather that picks the greedy token across vocabulary shards, and the close of a cache-only prompt row.  Peers' memory is reached with plain system-scope loads
// and stores; every wait on a peer is bounded in time and reports through the device error word.
#include "tp.cuh"

namespace sb {

namespace {

__device__ inline void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ inline uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
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

// Bounded wait of thread r < size for rank r's flag of flag set `set`.  Returns false (and records the
// error) when a wait ran out.  All threads of the block must call it.
__device__ inline bool wait_flags(const TpRegion &g, uint32_t set, uint32_t ticket, uint32_t *error_word) {
    bool ok = true;
    if (threadIdx.x < g.size) {
        const uint32_t *mine = tp_flags(g.base[g.rank], set) + threadIdx.x;
        const unsigned long long t0 = global_ns();
        uint32_t spins = 0;
        while (ld_acquire_sys(mine) != ticket) {
            if (++spins > 32u) {
                __nanosleep(100);
                if (global_ns() - t0 > g.wait_ns) {
                    atomicOr(error_word, kErrPeerTimeout);
                    ok = false;
                    break;
                }
            }
        }
    }
    return __syncthreads_and(ok ? 1 : 0) != 0;
}

__global__ void __launch_bounds__(256) tp_ingest_advance_kernel(TpRegion g, uint32_t buf, uint32_t ticket_mul,
                                                                uint32_t ticket_add, uint32_t *tokens,
                                                                StepState *state, const uint32_t *pending,
                                                                uint32_t *error_word) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t ticket = *tokens * ticket_mul + ticket_add;
    const unsigned long long t0 = global_ns();
    bool ok = true;
    for (uint32_t r = 0; r < g.size && ok; ++r) {
        const unsigned long long *row = tp_recv(g.base[g.rank], buf, r, g.hidden);
        for (uint32_t i = threadIdx.x; i < g.hidden && ok; i += blockDim.x) {
            uint32_t spins = 0;
            for (;;) {
                unsigned long long q;
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(q) : "l"(row + i) : "memory");
                if ((uint32_t)(q >> 32) == ticket) break;
                if (++spins > 8u) {
                    __nanosleep(100);
                    if (global_ns() - t0 > g.wait_ns) {
                        atomicOr(error_word, kErrPeerTimeout);
                        ok = false;
                        break;
                    }
                }
            }
        }
    }
    // A rank whose wait ran out stays where it is: position, cursor and ticket base do not move on rows that
    // were never complete, so the failed exchange remains the one every rank is at.
    if (__syncthreads_and(ok ? 1 : 0) && threadIdx.x == 0) {
        state->position += 1u;
        state->token = pending[state->cursor];
        state->cursor += 1u;
        *tokens += 1u;
    }
}

// Sums the ranks' packets of one exchange ONCE and folds the result into the residual stream:
//   h[i] = bf16(bf16(sum over ranks in rank order) + h[i]).
// A handful of small CTAs.  Everything happens after the wait on the previous kernel: the ticket depends
// on the token counter, whose writer (the end of the previous token) may still be running while the first
// kernels of this token are already resident, and a poll for a stale ticket would never be answered.
constexpr int kReduceCtas = 8, kReduceThreads = 256;
__global__ void __launch_bounds__(kReduceThreads) tp_reduce_residual_kernel(TpRegion g, uint32_t buf, uint32_t ticket_mul,
                                                                            uint32_t ticket_add, const uint32_t *tokens,
                                                                            uint16_t *h, uint32_t *error_word,
                                                                            TraceSlot *trace) {
    pdl_launch_dependents();
    if (threadIdx.x == 0 && trace) trace_min(&trace->start);
    pdl_wait();
    if (threadIdx.x == 0 && trace) trace_min(&trace->ready);
    const uint32_t ticket = __ldcg(tokens) * ticket_mul + ticket_add;
    const unsigned long long t0 = global_ns();
    for (uint32_t i = (blockIdx.x * kReduceThreads + threadIdx.x) * 2u; i < g.hidden;
         i += kReduceCtas * kReduceThreads * 2u) {
        // The packets of ALL ranks are requested in one trip to memory and checked together (a poll per rank in turn
        // costs a round trip per rank even when every packet is already there: 8 of them at 8 ranks); a trip is
        // repeated until every ticket is this exchange's.  The sum is formed in rank order afterwards, so every
        // rank computes the same bits.
        unsigned long long q0[kMaxTpRanks], q1[kMaxTpRanks];
        bool ok = true;
        uint32_t spins = 0;
        for (;;) {
            bool all = true;
#pragma unroll
            for (uint32_t r = 0; r < kMaxTpRanks; ++r) {
                if (r < g.size) {
                    const unsigned long long *src = tp_recv(g.base[g.rank], buf, r, g.hidden) + i;
                    asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(q0[r]), "=l"(q1[r]) : "l"(src) : "memory");
                }
            }
#pragma unroll
            for (uint32_t r = 0; r < kMaxTpRanks; ++r)
                if (r < g.size) all = all && (uint32_t)(q0[r] >> 32) == ticket && (uint32_t)(q1[r] >> 32) == ticket;
            if (all) break;
            if (++spins > 8u) {
                __nanosleep(64);
                if (global_ns() - t0 > g.wait_ns) {
                    atomicOr(error_word, kErrPeerTimeout);
                    ok = false;
                    break;
                }
            }
        }
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
        for (uint32_t r = 0; r < kMaxTpRanks; ++r)
            if (r < g.size) {
                a0 += __uint_as_float((uint32_t)q0[r]);
                a1 += __uint_as_float((uint32_t)q1[r]);
            }
        if (ok) {
            const uint32_t old = *reinterpret_cast<const uint32_t *>(h + i);
            const uint32_t s2 = f32x2_to_bf16x2(a0, a1);  // the projection's bf16 output
            *reinterpret_cast<uint32_t *>(h + i) =
                f32x2_to_bf16x2(__uint_as_float(s2 << 16) + __uint_as_float(old << 16),
                                __uint_as_float(s2 & 0xffff0000u) + __uint_as_float(old & 0xffff0000u));
        }
    }
    if (threadIdx.x == 0 && trace) trace_max(&trace->end);
}

__global__ void __launch_bounds__(256) tp_argmax_finalize_kernel(TpRegion g, uint32_t *tokens, const float *partial_max,
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
    const uint32_t set = 0u;
    const uint32_t ticket = *tokens + 1u;
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
    if (threadIdx.x < g.size) {  // this rank's candidate into every rank's slot table, then its flag there
        st_sys_u32x2(tp_gather(g.base[threadIdx.x]) + 2u * g.rank, make_uint2(__float_as_uint(vs[0]), is[0]));
        __threadfence_system();
        st_release_sys(tp_flags(g.base[threadIdx.x], set) + g.rank, ticket);
    }
    const bool ok = wait_flags(g, set, ticket, error_word);
    if (threadIdx.x == 0 && !ok) state->next_token = 0xffffffffu;  // no token; position and ticket base stay
    if (threadIdx.x == 0 && ok) {
        float top = -INFINITY;
        uint32_t ti = 0xffffffffu;
        {
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
        *tokens = ticket;
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

QmvExchange tp_producer_hooks(const TpRegion &g, uint32_t index, uint32_t per_token, const uint32_t *tokens) {
    QmvExchange x{};
    x.ranks = g.size;
    for (uint32_t r = 0; r < g.size; ++r) x.push[r] = tp_recv(g.base[r], index & 1u, g.rank, g.hidden);
    x.tokens = tokens;
    x.ticket_mul = per_token;
    x.ticket_add = index + 1u;
    return x;
}

QmvExchange tp_consumer_hooks(const TpRegion &g, uint32_t index, uint32_t per_token, const uint32_t *tokens,
                              uint16_t *h_out) {
    QmvExchange x{};
    x.ranks = g.size;
    x.recv = tp_recv(g.base[g.rank], index & 1u, 0u, g.hidden);
    x.h_out = h_out;
    x.wait_ns = g.wait_ns;
    x.tokens = tokens;
    x.ticket_mul = per_token;
    x.ticket_add = index + 1u;
    return x;
}

stark_b200_status tp_reduce_residual_launch(const TpRegion &g, uint32_t index, uint32_t per_token,
                                            const uint32_t *tokens, uint16_t *h, uint32_t *error_word, TraceSlot *trace,
                                            bool pdl, cudaStream_t stream) {
    if (g.size < 2 || g.size > kMaxTpRanks || g.rank >= g.size || g.hidden % 2u != 0) return STARK_B200_INVALID_ARGUMENT;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(kReduceCtas);
    cfg.blockDim = dim3(kReduceThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    SB_CUDA(cudaLaunchKernelEx(&cfg, tp_reduce_residual_kernel, g, index & 1u, per_token, index + 1u, tokens, h,
                               error_word, trace));
    return STARK_B200_OK;
}

stark_b200_status tp_ingest_advance_launch(const TpRegion &g, uint32_t last_index, uint32_t per_token,
                                           uint32_t *tokens, StepState *state, const uint32_t *pending,
                                           uint32_t *error_word, bool pdl, cudaStream_t stream) {
    if (g.size < 2 || g.size > kMaxTpRanks || g.rank >= g.size) return STARK_B200_INVALID_ARGUMENT;
    return launch_one(tp_ingest_advance_kernel, 256u, pdl, stream, g, last_index & 1u, per_token, last_index + 1u,
                      tokens, state, pending, error_word);
}

stark_b200_status tp_argmax_finalize_launch(const TpRegion &region, uint32_t *tokens, const float *partial_max,
                                            const uint32_t *partial_index, uint32_t count, uint32_t vocab_offset,
                                            StepState *state, uint32_t *generated, uint32_t *error_word, bool pdl,
                                            cudaStream_t stream) {
    if (region.size < 2 || region.size > kMaxTpRanks || region.rank >= region.size) return STARK_B200_INVALID_ARGUMENT;
    return launch_one(tp_argmax_finalize_kernel, 256u, pdl, stream, region, tokens, partial_max, partial_index, count,
                      vocab_offset, state, generated, error_word);
}

}  // namespace sb
