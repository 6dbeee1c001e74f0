// Non-matvec kernels of the decode step (sm_100a).  All are latency-sized (one token), so they are
// written for few launches and few dependent phases rather than for throughput; the only one that
// moves real bytes is the decode attention, which streams the KV pages of one head per CTA row.
#include "ops.cuh"
#include "device_attention.cuh"
#include "tunables.cuh"

#include <algorithm>
#include <cstdlib>

namespace sb {

namespace {

// One CTA = (split, KV head), four warps: the split's partial, then the last split of the head to
// arrive merges all of them (see device_attention.cuh).
// NBUF K / V tile pairs in flight: with three, a split of up to three pages is on its way before the new
// row exists (104 KB of shared memory instead of 70 KB).
// MINB: CTAs per SM the register allocation is sized for (5: at most 96 registers, so that a CTA fits beside
// two resident 320-thread matvec CTAs at 80; 4: up to 128).
template <int NBUF, int MINB>
__global__ void __launch_bounds__(kAttnThreads, MINB) attention_decode_kernel(const AttnParams p) {
    extern __shared__ __align__(128) uint8_t attn_smem[];
    __shared__ uint32_t is_last;
    pdl_launch_dependents();
    const uint32_t tid = threadIdx.x;
    const uint32_t split = blockIdx.x, h = blockIdx.y;
    if (tid == 0 && p.trace) {
        trace_min(&p.trace->start);
        trace_max(&p.trace->start_last);
    }
    // Before the wait: the cache rows of earlier tokens and the constants of this position do not
    // depend on the kernel before this one, so their fetch overlaps it.  Inside a recorded token the
    // position is final here (its writer ran in the previous token's graph).  In an unrecorded sequence
    // every kernel launches its dependents at once, so several later kernels can be resident and waiting
    // while the writer of `position` is still running: the position is read again after the wait and
    // the fetch repeated if it moved.
    const AttnShared sm = carve_attn_shared(attn_smem, NBUF);
    AttnPrefetch pf;
    attention_prefetch<NBUF>(p, split, h, __ldcg(&p.state->position), sm, tid, pf);
    pdl_wait();
    if (tid == 0 && p.trace) {
        trace_min(&p.trace->ready);
        trace_max(&p.trace->ready_last);
    }
    const uint32_t pos = __ldcg(&p.state->position);
    if (pos != pf.pos) {  // uniform across the CTA
        cp_async_wait<0>();
        __syncthreads();
        attention_prefetch<NBUF>(p, split, h, pos, sm, tid, pf);
    }
    attention_partial<0, kAttnThreads, NBUF>(p, split, h, pos, sm, tid, pf);
    if (tid == 0) {
        const uint32_t prev = atomicAdd(&p.counters[h], 1u);
        is_last = prev == p.splits - 1u;
    }
    __syncthreads();
    if (is_last) {
        __threadfence();
        attention_merge<0, kAttnThreads>(p, h, reinterpret_cast<float *>(attn_smem), tid);
        if (tid == 0) p.counters[h] = 0;
    }
    if (tid == 0 && p.trace) trace_max(&p.trace->end);
}

// ---------------------------------------------------------------------------------------------------

__global__ void embedding_row_kernel(const uint8_t *__restrict__ data, uint32_t rows, uint32_t columns,
                                     uint32_t pair_halves, const StepState *state, uint16_t *out) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t token = state->token;
    const uint32_t groups = columns / 64u;
    for (uint32_t col = blockIdx.x * blockDim.x + threadIdx.x; col < columns; col += gridDim.x * blockDim.x) {
        if (token >= rows) {  // input_embedding_lookup.rs:64-68
            out[col] = 0;
            continue;
        }
        // locate (token, col) in the record layout described in qmv.cuh
        uint32_t tile, r;
        if (!pair_halves) {
            tile = token / 16u;
            r = token % 16u;
        } else {
            const uint32_t half = rows / 2u, inner = token % half;
            tile = 2u * (inner / 16u) + (token >= half ? 1u : 0u);
            r = inner % 16u;
        }
        const uint32_t g = r & 7u, hrow = r >> 3;
        const uint32_t kg = col / 64u, c = col % 64u;
        const uint32_t t = c / 16u, j = (c % 16u) / 4u, r2 = (c % 4u) / 2u, e = c & 1u;
        const uint8_t *rec = data + ((size_t)tile * groups + kg) * kA4RecordBytes;
        const uint32_t word = *reinterpret_cast<const uint32_t *>(rec + (g * 4u + t) * 16u + j * 4u);
        const uint32_t q = (word >> (4u * (4u * e + 2u * r2 + hrow))) & 15u;
        const uint16_t *planes = reinterpret_cast<const uint16_t *>(rec + 512u);
        const float scale = bf16_bits_to_f32(planes[2u * g + hrow]);
        const float bias = bf16_bits_to_f32(planes[16u + 2u * g + hrow]);
        // input_embedding_lookup.rs:101-105: scale * code + bias (two roundings), then bf16
        out[col] = f32_to_bf16_bits(__fadd_rn(__fmul_rn(scale, (float)q), bias));
    }
}

__global__ void argmax_finalize_kernel(const float *__restrict__ partial_max,
                                       const uint32_t *__restrict__ partial_index, uint32_t count,
                                       StepState *state, uint32_t *generated, uint32_t advance) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float vs[32];
    __shared__ uint32_t is[32];
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
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < blockDim.x / 32u; ++w)
            if (vs[w] > best || (vs[w] == best && is[w] < bi)) {
                best = vs[w];
                bi = is[w];
            }
        // unified_sampling.rs:42-45: any non-finite logit makes the row invalid
        const uint32_t tok = isfinite(best) ? bi : 0xffffffffu;
        state->next_token = tok;
        if (generated && state->gen_cursor < state->gen_capacity) generated[state->gen_cursor++] = tok;
        if (advance) {
            state->position += 1u;
            state->token = tok;
        }
    }
}

__global__ void ingest_advance_kernel(StepState *state, const uint32_t *pending) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        state->position += 1u;
        state->token = pending[state->cursor];
        state->cursor += 1u;
    }
}

// normalization.rs:13-191 (RMS, OnlyNormalization rounding), one row, one CTA.
__global__ void rmsnorm_kernel(const uint16_t *input, const float *scales, uint16_t *output, uint16_t *shortcut,
                               uint32_t count, float eps, uint32_t residual_add) {
    __shared__ float wsum[32];
    float sq = 0.0f;
    for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) {
        uint16_t v = input[i];
        if (shortcut) {
            if (residual_add) v = f32_to_bf16_bits(bf16_bits_to_f32(v) + bf16_bits_to_f32(shortcut[i]));
            shortcut[i] = v;
        }
        const float a = bf16_bits_to_f32(v);
        sq += a * a;
    }
    sq = warp_sum(sq);
    if ((threadIdx.x & 31u) == 0) wsum[threadIdx.x >> 5] = sq;
    __syncthreads();
    float total = 0.0f;
    for (uint32_t w = 0; w < blockDim.x / 32u; ++w) total += wsum[w];
    const float rms_inv = 1.0f / sqrtf(total / (float)count + eps);
    for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) {
        const float v = bf16_bits_to_f32((shortcut && residual_add) ? shortcut[i] : input[i]);
        output[i] = f32_to_bf16_bits(bf16_round(v * rms_inv) * bf16_round(scales[i]));
    }
}

// gated_act_mul.rs:66-100 on a fused [up; gate] row.
__global__ void swiglu_kernel(const uint16_t *fused, uint16_t *out, uint32_t gated_dim) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < gated_dim; i += gridDim.x * blockDim.x) {
        const float value = bf16_bits_to_f32(fused[i]);
        const float gate = bf16_bits_to_f32(fused[gated_dim + i]);
        const float activated = bf16_round(gate / (1.0f + expf(-1.0f * gate)));
        out[i] = f32_to_bf16_bits(value * activated);
    }
}

__global__ void argmax_bf16_kernel(const uint16_t *logits, uint32_t vocab, uint32_t *out_index) {
    __shared__ float vs[32];
    __shared__ uint32_t is[32];
    float best = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (uint32_t i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float lv = bf16_bits_to_f32(logits[i]);
        const float v = isfinite(lv) ? lv : INFINITY;
        if (v > best || (v == best && i < bi)) {
            best = v;
            bi = i;
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
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < blockDim.x / 32u; ++w)
            if (vs[w] > best || (vs[w] == best && is[w] < bi)) {
                best = vs[w];
                bi = is[w];
            }
        *out_index = isfinite(best) ? bi : 0xffffffffu;
    }
}

// scoring.rs:299-336: log p = logit - (max + ln sum exp(logit - max)), f64, one CTA.
__global__ void log_softmax_kernel(const float *logits, double *out, uint32_t vocab) {
    __shared__ double red[32];
    __shared__ double bcast;
    double mx = -INFINITY;
    for (uint32_t i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmax(mx, (double)logits[i]);
    for (int o = 16; o > 0; o >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < blockDim.x / 32u; ++w) mx = fmax(mx, red[w]);
        bcast = mx;
    }
    __syncthreads();
    mx = bcast;
    double sum = 0.0;
    for (uint32_t i = threadIdx.x; i < vocab; i += blockDim.x) sum += exp((double)logits[i] - mx);
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncthreads();
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < blockDim.x / 32u; ++w) sum += red[w];
        bcast = mx + log(sum);
    }
    __syncthreads();
    const double lse = bcast;
    for (uint32_t i = threadIdx.x; i < vocab; i += blockDim.x) out[i] = (double)logits[i] - lse;
}

// moe.rs:25-82, one thread per row (experts <= 1024, active <= 32).
__global__ void moe_route_kernel(const float *logits, uint32_t *ids, float *weights, uint32_t rows, uint32_t experts,
                                 uint32_t active, uint32_t round_weights, uint32_t round_logits) {
    const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const float *src = logits + (size_t)row * experts;
    uint32_t *rid = ids + (size_t)row * active;
    float *rw = weights + (size_t)row * active;
    bool valid = experts >= 1 && experts <= 1024 && active >= 1 && active <= 32 && active <= experts;
    float maximum = -INFINITY;
    for (uint32_t e = 0; e < experts; ++e) {
        const float x = round_logits ? bf16_round(src[e]) : src[e];
        if (!isfinite(x)) valid = false;
        maximum = fmaxf(maximum, x);
    }
    float denominator = 0.0f;
    for (uint32_t e = 0; e < experts; ++e) {
        const float x = round_logits ? bf16_round(src[e]) : src[e];
        denominator += expf(x - maximum);
    }
    float selected_sum = 0.0f;
    for (uint32_t rank = 0; rank < active; ++rank) {
        float best = -INFINITY;
        uint32_t selected = 0;
        for (uint32_t e = 0; e < experts; ++e) {
            const float x = round_logits ? bf16_round(src[e]) : src[e];
            bool used = false;
            for (uint32_t r = 0; r < rank; ++r) used |= rid[r] == e;
            if (!used && x > best) {
                best = x;
                selected = e;
            }
        }
        rid[rank] = valid ? selected : 0u;
        rw[rank] = expf(best - maximum) / denominator;
        selected_sum += rw[rank];
    }
    for (uint32_t rank = 0; rank < active; ++rank) {
        float w = rw[rank] / selected_sum;
        if (round_weights) w = bf16_round(w);
        if (!valid) w = NAN;
        rw[rank] = w;
    }
}

// math.rs:55-66 topk + math.rs:36-51 softmax over the selected; one warp, experts <= 1024, active <= 32.
__global__ void moe_select_kernel(const float *scores, uint32_t experts, uint32_t active, uint32_t *ids,
                                  float *probs) {
    __shared__ uint32_t chosen[32];
    __shared__ float chosen_v[32];
    const uint32_t lane = threadIdx.x;
    for (uint32_t r = 0; r < active; ++r) {
        float best = -INFINITY;
        uint32_t bi = 0xffffffffu;
        for (uint32_t e = lane; e < experts; e += 32) {
            bool used = false;
            for (uint32_t k = 0; k < r; ++k) used |= chosen[k] == e;
            const float v = scores[e];
            if (!used && (bi == 0xffffffffu || v > best)) {
                best = v;
                bi = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0xffffffffu && (bi == 0xffffffffu || ov > best || (ov == best && oi < bi))) {
                best = ov;
                bi = oi;
            }
        }
        if (lane == 0) {
            chosen[r] = bi;
            chosen_v[r] = best;
        }
        __syncwarp();
    }
    if (lane == 0) {
        float mx = -INFINITY;
        for (uint32_t r = 0; r < active; ++r) mx = fmaxf(mx, chosen_v[r]);
        float sum = 0.0f;
        for (uint32_t r = 0; r < active; ++r) {
            probs[r] = expf(chosen_v[r] - mx);
            sum += probs[r];
        }
        for (uint32_t r = 0; r < active; ++r) {
            probs[r] /= sum;
            ids[r] = chosen[r];
        }
    }
}

__device__ inline float sigmoid_stable(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    const float e = expf(x);
    return e / (1.0f + e);
}

__global__ void silu_mul_f32_kernel(float *gate, const float *up, uint32_t count) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x)
        gate[i] = __fmul_rn(__fmul_rn(gate[i], sigmoid_stable(gate[i])), up[i]);
}

__global__ void weighted_sum_kernel(const float *rows, const float *probs, float *out, uint32_t count,
                                    uint32_t width) {
    for (uint32_t h = blockIdx.x * blockDim.x + threadIdx.x; h < width; h += gridDim.x * blockDim.x) {
        float acc = 0.0f;
        for (uint32_t r = 0; r < count; ++r) acc = __fadd_rn(acc, __fmul_rn(probs[r], rows[(size_t)r * width + h]));
        out[h] = acc;
    }
}

__global__ void dense_matvec_f32_kernel(const float *w, const float *x, float *y, uint32_t rows, uint32_t columns) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    for (uint32_t r = blockIdx.x * (blockDim.x / 32u) + warp; r < rows; r += gridDim.x * (blockDim.x / 32u)) {
        float acc = 0.0f;
        for (uint32_t c = lane; c < columns; c += 32) acc = fmaf(w[(size_t)r * columns + c], x[c], acc);
        acc = warp_sum(acc);
        if (lane == 0) y[r] = acc;
    }
}

template <typename... Args>
stark_b200_status launch_pdl_smem(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, bool pdl,
                                  cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
    return STARK_B200_OK;
}

template <typename... Args>
stark_b200_status launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, bool pdl, cudaStream_t stream,
                             Args... args) {
    return launch_pdl_smem(kernel, grid, block, 0, pdl, stream, args...);
}

}  // namespace

size_t attention_scratch_floats(uint32_t q_heads, uint32_t kv_heads, uint32_t splits) {
    (void)kv_heads;
    return (size_t)q_heads * splits * (kHeadDim + 2u);
}

stark_b200_status attention_decode_launch(const AttnArgs &a, cudaStream_t stream) {
    if (!a.qkv || !a.out || !a.kv.keys || !a.kv.values || !a.block_table || !a.state || !a.scratch || !a.counters)
        return STARK_B200_INVALID_ARGUMENT;
    if (a.kv_heads == 0 || a.q_heads % a.kv_heads != 0 || a.q_heads / a.kv_heads > (uint32_t)kMaxGqa)
        return STARK_B200_UNSUPPORTED;
    if (a.splits == 0 || a.splits > kMaxAttnSplits) return STARK_B200_INVALID_ARGUMENT;
    AttnParams p{};
    p.qkv = a.qkv;
    p.out = a.out;
    p.keys = a.kv.keys;
    p.values = a.kv.values;
    p.block_table = a.block_table;
    p.q_norm = a.q_norm;
    p.k_norm = a.k_norm;
    p.rope_cos = a.rope_cos;
    p.rope_sin = a.rope_sin;
    p.state = a.state;
    p.eps = a.eps;
    p.scale = a.scale;
    p.q_heads = a.q_heads;
    p.kv_heads = a.kv_heads;
    p.gqa = a.q_heads / a.kv_heads;
    p.splits = a.splits;
    p.scratch = a.scratch;
    p.counters = a.counters;
    p.trace = a.trace;
    const uint32_t bufs = tunables().attn_bufs;  // tile pairs in flight per CTA
    const bool wide = tunables().attn_regs >= 128u;
    using Kernel = void (*)(const AttnParams);
    static const Kernel kernels[2][2] = {{attention_decode_kernel<2, 5>, attention_decode_kernel<2, 4>},
                                         {attention_decode_kernel<3, 5>, attention_decode_kernel<3, 4>}};
    static SmemOptIn once[2][2];
    const uint32_t bi = bufs == 2u ? 0u : 1u, wi = wide ? 1u : 0u;
    const uint32_t smem = attn_shared_bytes(bi ? 3u : 2u);
    if (stark_b200_status s = ensure_dynamic_smem(kernels[bi][wi], (int)smem, once[bi][wi])) return s;
    return launch_pdl_smem(kernels[bi][wi], dim3(a.splits, a.kv_heads), dim3(kAttnThreads), smem, a.pdl, stream, p);
}

stark_b200_status embedding_row_launch(const QMatrix *table, const StepState *state, uint16_t *out, bool pdl,
                                       cudaStream_t stream) {
    if (!table || table->format != kFmtAffine4) return STARK_B200_UNSUPPORTED;
    const uint32_t blocks = std::max(1u, std::min(32u, table->columns / 256u));
    return launch_pdl(embedding_row_kernel, dim3(blocks), dim3(256), pdl, stream, (const uint8_t *)table->data,
                      table->rows, table->columns, table->pair_halves, state, out);
}

stark_b200_status argmax_finalize_launch(const float *partial_max, const uint32_t *partial_index, uint32_t count,
                                         StepState *state, uint32_t *generated, bool advance, bool pdl,
                                         cudaStream_t stream) {
    return launch_pdl(argmax_finalize_kernel, dim3(1), dim3(256), pdl, stream, partial_max, partial_index, count,
                      state, generated, advance ? 1u : 0u);
}

stark_b200_status ingest_advance_launch(StepState *state, const uint32_t *pending, bool pdl, cudaStream_t stream) {
    return launch_pdl(ingest_advance_kernel, dim3(1), dim3(32), pdl, stream, state, pending);
}

stark_b200_status rmsnorm_launch(const uint16_t *input, const float *scales, uint16_t *output, uint16_t *shortcut,
                                 uint32_t count, float eps, bool residual_add, cudaStream_t stream) {
    rmsnorm_kernel<<<1, 512, 0, stream>>>(input, scales, output, shortcut, count, eps, residual_add ? 1u : 0u);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status swiglu_launch(const uint16_t *fused, uint16_t *out, uint32_t gated_dim, cudaStream_t stream) {
    swiglu_kernel<<<std::max(1u, std::min(148u, (gated_dim + 255u) / 256u)), 256, 0, stream>>>(fused, out, gated_dim);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status argmax_bf16_launch(const uint16_t *logits, uint32_t vocab, uint32_t *out_index,
                                     cudaStream_t stream) {
    argmax_bf16_kernel<<<1, 1024, 0, stream>>>(logits, vocab, out_index);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status log_softmax_launch(const float *logits, double *out, uint32_t vocab, double *scratch,
                                     cudaStream_t stream) {
    (void)scratch;
    log_softmax_kernel<<<1, 1024, 0, stream>>>(logits, out, vocab);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status moe_route_launch(const float *logits, uint32_t *ids, float *weights, uint32_t rows,
                                   uint32_t experts, uint32_t active, bool round_weights, bool round_logits,
                                   cudaStream_t stream) {
    moe_route_kernel<<<(rows + 63u) / 64u, 64, 0, stream>>>(logits, ids, weights, rows, experts, active,
                                                           round_weights ? 1u : 0u, round_logits ? 1u : 0u);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status moe_select_launch(const float *scores, uint32_t experts, uint32_t active, uint32_t *ids,
                                    float *probs, cudaStream_t stream) {
    if (experts == 0 || experts > 1024 || active == 0 || active > 32 || active > experts) return STARK_B200_INVALID_ARGUMENT;
    moe_select_kernel<<<1, 32, 0, stream>>>(scores, experts, active, ids, probs);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status silu_mul_f32_launch(float *gate, const float *up, uint32_t count, cudaStream_t stream) {
    silu_mul_f32_kernel<<<std::max(1u, std::min(148u, (count + 255u) / 256u)), 256, 0, stream>>>(gate, up, count);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status weighted_sum_launch(const float *rows, const float *probs, float *out, uint32_t count,
                                      uint32_t width, cudaStream_t stream) {
    weighted_sum_kernel<<<std::max(1u, std::min(148u, (width + 255u) / 256u)), 256, 0, stream>>>(rows, probs, out, count,
                                                                                              width);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status dense_matvec_f32_launch(const float *w, const float *x, float *y, uint32_t rows, uint32_t columns,
                                          cudaStream_t stream) {
    dense_matvec_f32_kernel<<<std::max(1u, std::min(592u, (rows + 7u) / 8u)), 256, 0, stream>>>(w, x, y, rows, columns);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

}  // namespace sb
