// Non-matvec kernels of the decode step (sm_100a).  All are latency-sized (one token), so they are
// written for few launches and few dependent phases rather than for throughput; the only one that
// moves real bytes is the decode attention, which streams the KV pages of one head per CTA row.
#include "ops.cuh"

#include <algorithm>

namespace sb {

namespace {

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kMaxGqa = 8;
constexpr uint32_t kTileRowBytes = kHeadDim * 2u + 16u;  // 272: padded so that row-strided 16 B reads are conflict-free
constexpr uint32_t kTileBytes = kPageTokens * kTileRowBytes;
constexpr uint32_t kAttnSmemBytes = 4u * kTileBytes;  // K and V, double buffered

struct AttnParams {
    const uint16_t *qkv;
    uint16_t *out;
    uint16_t *keys;
    uint16_t *values;
    const int32_t *block_table;
    const float *q_norm;
    const float *k_norm;
    const float *rope_cos;
    const float *rope_sin;
    const StepState *state;
    float eps;
    float scale;
    uint32_t q_heads, kv_heads, gqa, splits;
    float *scratch;
    uint32_t *counters;
    TraceSlot *trace;
};

__device__ inline void cp_async16(void *smem_dst, const void *gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ inline void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Per-head RMS norm + RoPE of 128-wide heads, two heads at a time (threads 0..127 and 128..255).
//   qkv_norm.rs:44-108: f32 sum of squares, rms = 1/sqrt(mean + eps), bf16(normalized) * bf16(scale) -> bf16
//   attention_prepare.rs:7-43: half-split pairing, x*cos + (+-pair)*sin with separately rounded products
// `active` may differ between the two halves; every thread of the CTA must call it.
__device__ inline float head_norm_rope(float v, bool active, bool has_norm, float norm_w, bool has_rope,
                                       float cos_d, float sin_d, float eps, float *exch /* [256] */,
                                       float *wsum /* [kAttnWarps] */) {
    const int d = threadIdx.x & 127, half = threadIdx.x >> 7;
    if (has_norm) {
        const float sq = warp_sum(active ? v * v : 0.0f);
        if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = sq;
        __syncthreads();
        const float total = wsum[half * 4] + wsum[half * 4 + 1] + wsum[half * 4 + 2] + wsum[half * 4 + 3];
        const float rms = 1.0f / sqrtf(total / (float)kHeadDim + eps);
        v = bf16_round(bf16_round(v * rms) * bf16_round(norm_w));
        __syncthreads();
    }
    if (has_rope) {
        exch[threadIdx.x] = v;
        __syncthreads();
        const float paired = exch[half * 128 + (d < 64 ? d + 64 : d - 64)];
        const float signed_paired = d < 64 ? -paired : paired;
        v = bf16_round(__fadd_rn(__fmul_rn(v, cos_d), __fmul_rn(signed_paired, sin_d)));
        __syncthreads();
    }
    return v;
}

// One CTA = (split, KV head): streams its share of the head's KV pages through shared memory
// (16 KB K tile + 16 KB V tile per page, cp.async double buffered), keeps an
// online softmax for the G query heads that share the KV head, and publishes a partial
// (o, max, sum); the last split of a head to finish merges the partials.
__global__ void __launch_bounds__(kAttnThreads, 2) attention_decode_kernel(const AttnParams p) {
    extern __shared__ __align__(128) uint8_t tiles[];  // [2][K, V][64][272]
    __shared__ __align__(16) float q_s[kMaxGqa][kHeadDim];  // q after norm + RoPE (bf16 values), f32
    __shared__ float p_s[kMaxGqa][kPageTokens];
    __shared__ float exch[kAttnThreads];
    __shared__ float wred[2][kMaxGqa][kAttnWarps];
    __shared__ uint16_t knew[kHeadDim], vnew[kHeadDim];
    __shared__ uint32_t is_last;

    pdl_launch_dependents();

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t split = blockIdx.x, h = blockIdx.y, G = p.gqa;
    const uint32_t d128 = tid & 127u, half = tid >> 7;
    if (tid == 0 && p.trace) trace_min(&p.trace->start);
    // Constants first (they do not depend on the previous kernel).
    const float qn_w = p.q_norm ? p.q_norm[d128] : 1.0f;
    const float kn_w = p.k_norm ? p.k_norm[d128] : 1.0f;

    // Every kernel of the sequence launches its dependents at once, so several later kernels can be
    // resident and waiting here while the writer of `position` (the end of the previous token) is
    // still running: the position, and therefore the page range, is read only after the wait.
    pdl_wait();
    if (tid == 0 && p.trace) trace_min(&p.trace->ready);
    // All loads that depend only on the previous kernel are issued together (one memory round trip):
    // the position, this group's query rows and this head's new key / value row.
    const uint32_t pos = p.state->position;
    float qv[kMaxGqa / 2];
#pragma unroll
    for (int i = 0; i < kMaxGqa / 2; ++i) {
        const uint32_t g = 2u * i + half;
        qv[i] = g < G ? bf16_bits_to_f32(p.qkv[(size_t)(h * G + g) * kHeadDim + d128]) : 0.0f;
    }
    const float k_in = bf16_bits_to_f32(p.qkv[(size_t)(p.q_heads + h) * kHeadDim + d128]);
    const uint16_t v_in = p.qkv[(size_t)(p.q_heads + p.kv_heads + h) * kHeadDim + d128];

    const uint32_t seq_len = pos + 1u;
    const uint32_t nblocks = (seq_len + kPageTokens - 1u) / kPageTokens;
    const uint32_t b0 = (uint32_t)(((uint64_t)split * nblocks) / p.splits);
    const uint32_t b1 = (uint32_t)(((uint64_t)(split + 1u) * nblocks) / p.splits);
    const uint32_t new_block = pos / kPageTokens;
    const bool owner = new_block >= b0 && new_block < b1;
    const uint32_t ntiles = b1 - b0;
    // second round trip: RoPE coefficients of this position and the page numbers
    const float cos_d = p.rope_cos ? p.rope_cos[(size_t)pos * kHeadDim + d128] : 1.0f;
    const float sin_d = p.rope_sin ? p.rope_sin[(size_t)pos * kHeadDim + d128] : 0.0f;

    auto issue_tile = [&](uint32_t t) {
        const uint32_t buf = t & 1u;
        const size_t page = ((size_t)p.block_table[b0 + t] * p.kv_heads + h) * kPageTokens * kHeadDim;
        const uint8_t *ksrc = reinterpret_cast<const uint8_t *>(p.keys + page);
        const uint8_t *vsrc = reinterpret_cast<const uint8_t *>(p.values + page);
        uint8_t *kd = tiles + (size_t)(buf * 2u) * kTileBytes, *vd = kd + kTileBytes;
        // 64 rows x 16 chunks of 16 B per tile; thread -> (row, chunk)
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t idx = tid + i * kAttnThreads, row = idx >> 4, ch = idx & 15u;
            cp_async16(kd + row * kTileRowBytes + ch * 16u, ksrc + row * 256u + ch * 16u);
            cp_async16(vd + row * kTileRowBytes + ch * 16u, vsrc + row * 256u + ch * 16u);
        }
        cp_async_commit();
    };
    if (ntiles > 0) issue_tile(0);

    // Queries of this KV head's group, two heads per pass: norm + RoPE (values are bf16-exact).
#pragma unroll
    for (int i = 0; i < kMaxGqa / 2; ++i) {
        if (2u * i < G) {
            const uint32_t g = 2u * i + half;
            const bool active = g < G;
            const float v = head_norm_rope(qv[i], active, p.q_norm != nullptr, qn_w, p.rope_cos != nullptr, cos_d,
                                           sin_d, p.eps, exch, wred[0][0]);
            if (active) q_s[g][d128] = v;
        }
    }
    // The split that owns the new position appends its key and value rows to the cache.
    if (owner) {
        const bool active = tid < 128;
        const float kv = head_norm_rope(active ? k_in : 0.0f, active, p.k_norm != nullptr, kn_w,
                                        p.rope_cos != nullptr, cos_d, sin_d, p.eps, exch, wred[0][0]);
        if (active) {
            const size_t row = ((size_t)p.block_table[new_block] * p.kv_heads + h) * kPageTokens + (pos % kPageTokens);
            const uint16_t kb = f32_to_bf16_bits(kv);
            p.keys[row * kHeadDim + tid] = kb;
            p.values[row * kHeadDim + tid] = v_in;
            knew[tid] = kb;
            vnew[tid] = v_in;
        }
    }
    __syncthreads();

    if (tid == 0 && p.trace) trace_max(&p.trace->compute);
    float m_run[kMaxGqa], l_run[kMaxGqa], o_acc[kMaxGqa][2];
#pragma unroll
    for (int g = 0; g < kMaxGqa; ++g) {
        m_run[g] = -INFINITY;
        l_run[g] = 0.0f;
        o_acc[g][0] = o_acc[g][1] = 0.0f;
    }
    const uint32_t key = tid >> 2, jq = tid & 3u;  // score phase: 4 threads per key, interleaved 16 B chunks
    const uint32_t dp = tid & 63u, kq = tid >> 6;  // PV phase: dim pair, key residue mod 4

    for (uint32_t t = 0; t < ntiles; ++t) {
        if (t + 1 < ntiles) {
            issue_tile(t + 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t buf = t & 1u;
        uint8_t *kt = tiles + (size_t)(buf * 2u) * kTileBytes, *vt = kt + kTileBytes;
        const uint32_t blk = b0 + t;
        if (blk == new_block) {
            // the copy may have raced the append above: patch the new row in shared memory
            if (tid < 128) {
                reinterpret_cast<uint16_t *>(kt + (pos % kPageTokens) * kTileRowBytes)[tid] = knew[tid];
                reinterpret_cast<uint16_t *>(vt + (pos % kPageTokens) * kTileRowBytes)[tid] = vnew[tid];
            }
            __syncthreads();
        }
        const uint32_t valid = min(kPageTokens, seq_len - blk * kPageTokens);  // keys of this page in range

        // ---- scores ----
        float s[kMaxGqa];
#pragma unroll
        for (int g = 0; g < kMaxGqa; ++g) s[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t c = 4u * i + jq;
            const uint4 kv = *reinterpret_cast<const uint4 *>(kt + key * kTileRowBytes + c * 16u);
            const uint32_t w[4] = {kv.x, kv.y, kv.z, kv.w};
            float kf[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                kf[2 * e] = __uint_as_float(w[e] << 16);
                kf[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
            }
#pragma unroll
            for (int g = 0; g < kMaxGqa; ++g) {
                if (g < (int)G) {
                    const float4 qa = *reinterpret_cast<const float4 *>(&q_s[g][c * 8u]);
                    const float4 qb = *reinterpret_cast<const float4 *>(&q_s[g][c * 8u + 4u]);
                    s[g] += qa.x * kf[0] + qa.y * kf[1] + qa.z * kf[2] + qa.w * kf[3] + qb.x * kf[4] +
                            qb.y * kf[5] + qb.z * kf[6] + qb.w * kf[7];
                }
            }
        }
#pragma unroll
        for (int g = 0; g < kMaxGqa; ++g) {
            if (g < (int)G) {
                s[g] += __shfl_xor_sync(0xffffffffu, s[g], 1);
                s[g] += __shfl_xor_sync(0xffffffffu, s[g], 2);
                s[g] = key < valid ? s[g] * p.scale : -INFINITY;
                float wm = s[g];
                wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, 4));
                wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, 8));
                wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, 16));
                if (lane == 0) wred[0][g][warp] = wm;
            }
        }
        __syncthreads();
        float factor[kMaxGqa];
#pragma unroll
        for (int g = 0; g < kMaxGqa; ++g) {
            factor[g] = 1.0f;
            if (g < (int)G) {
                float cm = wred[0][g][0];
#pragma unroll
                for (int i = 1; i < kAttnWarps; ++i) cm = fmaxf(cm, wred[0][g][i]);
                const float m_new = fmaxf(m_run[g], cm);
                factor[g] = m_run[g] == -INFINITY ? 0.0f : expf(m_run[g] - m_new);
                const float e = key < valid ? expf(s[g] - m_new) : 0.0f;
                if (jq == 0) p_s[g][key] = e;
                float ws = jq == 0 ? e : 0.0f;
                ws = warp_sum(ws);
                if (lane == 0) wred[1][g][warp] = ws;
                m_run[g] = m_new;
            }
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < kMaxGqa; ++g) {
            if (g < (int)G) {
                float cs = 0.0f;
#pragma unroll
                for (int i = 0; i < kAttnWarps; ++i) cs += wred[1][g][i];
                l_run[g] = l_run[g] * factor[g] + cs;
                o_acc[g][0] *= factor[g];
                o_acc[g][1] *= factor[g];
            }
        }
        // ---- o += P V: thread = (dim pair, key residue) ----
        for (uint32_t kk = kq; kk < valid; kk += 4) {
            const uint32_t vv = *reinterpret_cast<const uint32_t *>(vt + kk * kTileRowBytes + 4u * dp);
            const float v0 = __uint_as_float(vv << 16), v1 = __uint_as_float(vv & 0xffff0000u);
#pragma unroll
            for (int g = 0; g < kMaxGqa; ++g) {
                if (g < (int)G) {
                    const float pe = p_s[g][kk];
                    o_acc[g][0] = fmaf(pe, v0, o_acc[g][0]);
                    o_acc[g][1] = fmaf(pe, v1, o_acc[g][1]);
                }
            }
        }
        __syncthreads();  // the buffer of tile t is free for tile t + 2, p_s / wred for the next tile
    }

    // Combine the four key residues (reusing the tile memory), then publish this split's partial.
    float *o_red = reinterpret_cast<float *>(tiles);  // [4][G][128]
#pragma unroll
    for (int g = 0; g < kMaxGqa; ++g) {
        if (g < (int)G) {
            o_red[(kq * G + g) * kHeadDim + 2u * dp] = o_acc[g][0];
            o_red[(kq * G + g) * kHeadDim + 2u * dp + 1u] = o_acc[g][1];
        }
    }
    __syncthreads();
    const uint32_t stride = kHeadDim + 2u;
    float *mine = p.scratch + ((size_t)(h * p.splits + split) * G) * stride;
    for (uint32_t i = tid; i < G * kHeadDim; i += kAttnThreads) {
        const uint32_t g = i >> 7, d = i & 127u;
        mine[g * stride + d] = o_red[(0 * G + g) * kHeadDim + d] + o_red[(1 * G + g) * kHeadDim + d] +
                               o_red[(2 * G + g) * kHeadDim + d] + o_red[(3 * G + g) * kHeadDim + d];
    }
    if (tid == 0) {
#pragma unroll
        for (int g = 0; g < kMaxGqa; ++g) {
            if (g < (int)G) {
                mine[g * stride + kHeadDim] = m_run[g];
                mine[g * stride + kHeadDim + 1] = l_run[g];
            }
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const uint32_t prev = atomicAdd(&p.counters[h], 1u);
        is_last = prev == p.splits - 1u;
    }
    __syncthreads();
    if (!is_last) {
        if (tid == 0 && p.trace) trace_max(&p.trace->end);
        return;
    }
    __threadfence();
    // Last split of this KV head to arrive merges all partials.  Weights first (one thread per
    // (head, split)), then every thread sums its outputs with independent loads.
    const float *base = p.scratch + ((size_t)h * p.splits * G) * stride;
    float *wgt = reinterpret_cast<float *>(tiles);  // [G][splits] weights, then [G] 1/l
    __syncthreads();
    for (uint32_t g = warp; g < G; g += kAttnWarps) {
        const float ms = lane < p.splits ? __ldcg(&base[(lane * G + g) * stride + kHeadDim]) : -INFINITY;
        const float ls = lane < p.splits ? __ldcg(&base[(lane * G + g) * stride + kHeadDim + 1]) : 0.0f;
        const float mmax = warp_max(ms);
        const float w = ms == -INFINITY ? 0.0f : expf(ms - mmax);
        const float lsum = warp_sum(w * ls);
        if (lane < p.splits) wgt[g * kMaxAttnSplits + lane] = w;
        if (lane == 0) wgt[kMaxGqa * kMaxAttnSplits + g] = 1.0f / lsum;
    }
    __syncthreads();
    for (uint32_t i = tid; i < G * kHeadDim; i += kAttnThreads) {
        const uint32_t g = i >> 7, d = i & 127u;
        float osum = 0.0f;
#pragma unroll 8
        for (uint32_t sp = 0; sp < p.splits; ++sp)
            osum = fmaf(wgt[g * kMaxAttnSplits + sp], __ldcg(&base[(sp * G + g) * stride + d]), osum);
        p.out[(size_t)(h * G + g) * kHeadDim + d] = f32_to_bf16_bits(osum * wgt[kMaxGqa * kMaxAttnSplits + g]);
    }
    if (tid == 0) p.counters[h] = 0;
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
    static bool attr_set = false;
    if (!attr_set) {
        SB_CUDA(cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kAttnSmemBytes));
        attr_set = true;
    }
    return launch_pdl_smem(attention_decode_kernel, dim3(a.splits, a.kv_heads), dim3(kAttnThreads), kAttnSmemBytes,
                           a.pdl, stream, p);
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

}  // namespace sb
