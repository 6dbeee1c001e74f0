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

// The same reduction by ONE CTA that then also prepares the input of the matvec that follows: it holds the whole new
// residual row, so the RMS norm (normalization.rs:13-191: bf16(bf16(h * rms_inv) * bf16(w))), the power-of-two scale
// into f16 range and the per-group sums are formed here once (QmvStagedRow) and the 2 x 148 CTAs of the matvec copy
// 8 KB instead of each normalizing the row again behind this kernel.  Four elements per thread and round.
constexpr int kStageThreads = 1024, kStageRounds = 3;  // hidden <= 12288
__global__ void __launch_bounds__(kStageThreads) tp_reduce_stage_kernel(TpRegion g, uint32_t buf, uint32_t ticket_mul,
                                                                        uint32_t ticket_add, const uint32_t *tokens,
                                                                        uint16_t *h, const float *norm_weight, float eps,
                                                                        uint8_t *staged, uint32_t *error_word,
                                                                        TraceSlot *trace) {
    __shared__ float red_s[32], red_m[32];
    pdl_launch_dependents();
    if (threadIdx.x == 0 && trace) trace_min(&trace->start);
    pdl_wait();
    if (threadIdx.x == 0 && trace) trace_min(&trace->ready);
    const uint32_t ticket = __ldcg(tokens) * ticket_mul + ticket_add;
    const unsigned long long t0 = global_ns();
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    float f[kStageRounds][4];
    float sumsq = 0.0f, vmax = 0.0f;
#pragma unroll
    for (int round = 0; round < kStageRounds; ++round) {
        const uint32_t i = (round * kStageThreads + tid) * 4u;
#pragma unroll
        for (int e = 0; e < 4; ++e) f[round][e] = 0.0f;
        if (i >= g.hidden) continue;
        float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        // the packets of four ranks per trip to memory, repeated until their tickets are this exchange's; the
        // shares are added in rank order, so every rank computes the same bits
        for (uint32_t r0 = 0; r0 < g.size; r0 += 4u) {
            unsigned long long q[4][4];
            uint32_t spins = 0;
            for (;;) {
                bool all = true;
#pragma unroll
                for (uint32_t r = 0; r < 4u; ++r) {
                    if (r0 + r < g.size) {
                        const unsigned long long *src = tp_recv(g.base[g.rank], buf, r0 + r, g.hidden) + i;
                        asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(q[r][0]), "=l"(q[r][1]) : "l"(src) : "memory");
                        asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(q[r][2]), "=l"(q[r][3]) : "l"(src + 2) : "memory");
                    }
                }
#pragma unroll
                for (uint32_t r = 0; r < 4u; ++r)
                    if (r0 + r < g.size)
#pragma unroll
                        for (int e = 0; e < 4; ++e) all = all && (uint32_t)(q[r][e] >> 32) == ticket;
                if (all) break;
                if (++spins > 8u) {
                    __nanosleep(64);
                    if (global_ns() - t0 > g.wait_ns) {  // a rank is missing: report, go on with what is there
                        atomicOr(error_word, kErrPeerTimeout);
                        break;
                    }
                }
            }
#pragma unroll
            for (uint32_t r = 0; r < 4u; ++r)
                if (r0 + r < g.size)
#pragma unroll
                    for (int e = 0; e < 4; ++e) a[e] += __uint_as_float((uint32_t)q[r][e]);
        }
        const uint2 old = *reinterpret_cast<const uint2 *>(h + i);
        const uint32_t s01 = f32x2_to_bf16x2(a[0], a[1]), s23 = f32x2_to_bf16x2(a[2], a[3]);  // the projection's bf16 output
        const uint32_t h01 = f32x2_to_bf16x2(__uint_as_float(s01 << 16) + __uint_as_float(old.x << 16),
                                             __uint_as_float(s01 & 0xffff0000u) + __uint_as_float(old.x & 0xffff0000u));
        const uint32_t h23 = f32x2_to_bf16x2(__uint_as_float(s23 << 16) + __uint_as_float(old.y << 16),
                                             __uint_as_float(s23 & 0xffff0000u) + __uint_as_float(old.y & 0xffff0000u));
        *reinterpret_cast<uint2 *>(h + i) = make_uint2(h01, h23);
        f[round][0] = __uint_as_float(h01 << 16);
        f[round][1] = __uint_as_float(h01 & 0xffff0000u);
        f[round][2] = __uint_as_float(h23 << 16);
        f[round][3] = __uint_as_float(h23 & 0xffff0000u);
        const float4 w4 = *reinterpret_cast<const float4 *>(norm_weight + i);
        const float nw[4] = {bf16_round(w4.x), bf16_round(w4.y), bf16_round(w4.z), bf16_round(w4.w)};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            sumsq = fmaf(f[round][e], f[round][e], sumsq);
            vmax = fmaxf(vmax, fabsf(f[round][e] * nw[e]));
        }
    }
    // one block-wide reduction for the sum of squares and for the bound the f16 scale is chosen from
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sumsq += __shfl_xor_sync(0xffffffffu, sumsq, o);
        vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
    }
    if (lane == 0) red_s[warp] = sumsq, red_m[warp] = vmax;
    __syncthreads();
    sumsq = 0.0f, vmax = 0.0f;
#pragma unroll
    for (int w = 0; w < kStageThreads / 32; ++w) {
        sumsq += red_s[w];
        vmax = fmaxf(vmax, red_m[w]);
    }
    const float rms_inv = 1.0f / sqrtf(sumsq / (float)g.hidden + eps);
    vmax *= rms_inv * 1.015625f;  // bounds the normalized values up to their two bf16 roundings
    int shift = 14 - ((int)((__float_as_uint(vmax) >> 23) & 0xffu) - 127);
    shift = max(-100, min(100, shift));
    if (!(vmax > 0.0f) || !isfinite(vmax)) shift = 0;
    const float xscale = __uint_as_float((uint32_t)(shift + 127) << 23);
    float *sums = reinterpret_cast<float *>(staged + (size_t)g.hidden * 2u);
#pragma unroll
    for (int round = 0; round < kStageRounds; ++round) {
        const uint32_t i = (round * kStageThreads + tid) * 4u;
        float s4 = 0.0f;
        uint32_t hh[2] = {0u, 0u};
        float nw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (i < g.hidden) {  // the weights again (cached), rather than held in registers across the reduction
            const float4 w4 = *reinterpret_cast<const float4 *>(norm_weight + i);
            nw[0] = bf16_round(w4.x), nw[1] = bf16_round(w4.y), nw[2] = bf16_round(w4.z), nw[3] = bf16_round(w4.w);
        }
#pragma unroll
        for (int e = 0; e < 4; e += 2) {
            const uint32_t n2 = f32x2_to_bf16x2(f[round][e] * rms_inv, f[round][e + 1] * rms_inv);
            const uint32_t p2 = f32x2_to_bf16x2(__uint_as_float(n2 << 16) * nw[e], __uint_as_float(n2 & 0xffff0000u) * nw[e + 1]);
            const float a = __uint_as_float(p2 << 16), b = __uint_as_float(p2 & 0xffff0000u);
            s4 += a;
            s4 += b;
            asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(hh[e >> 1]) : "f"(b * xscale), "f"(a * xscale));
        }
        // a group of 64 columns is 16 consecutive threads
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) s4 += __shfl_xor_sync(0xffffffffu, s4, o);
        if (i < g.hidden) {
            *reinterpret_cast<uint2 *>(staged + (size_t)i * 2u) = make_uint2(hh[0], hh[1]);
            if ((lane & 15u) == 0) sums[i >> 6] = s4;
        }
    }
    if (tid == 0) {
        sums[g.hidden / 64u] = __uint_as_float((uint32_t)(127 - shift) << 23);  // undoes the scale
        if (trace) trace_max(&trace->end);
    }
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

stark_b200_status tp_reduce_stage_launch(const TpRegion &g, uint32_t index, uint32_t per_token, const uint32_t *tokens,
                                         uint16_t *h, const float *norm_weight, float eps, void *staged,
                                         uint32_t *error_word, TraceSlot *trace, bool pdl, cudaStream_t stream) {
    if (g.size < 2 || g.size > kMaxTpRanks || g.rank >= g.size || g.hidden % 64u != 0 ||
        g.hidden > (uint32_t)kStageThreads * kStageRounds * 4u || !norm_weight || !staged)
        return STARK_B200_INVALID_ARGUMENT;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(kStageThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    SB_CUDA(cudaLaunchKernelEx(&cfg, tp_reduce_stage_kernel, g, index & 1u, per_token, index + 1u, tokens, h, norm_weight, eps,
                               static_cast<uint8_t *>(staged), error_word, trace));
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
