// A routed-expert (MoE) decoder on the conventions of the reference's hybrid host path: f32 activations
// and logits, GGUF blocks decoded exactly as decode_block, an f32 key/value cache.  The reference ships no
// model of exactly this shape; the token step composes its operators:
//   rms_norm                                          crates/stark-engine/src/engine/hybrid/math.rs:18-34
//   q/k/v projection, per-head norm, rope, causal attention, o projection
//                                                     engine/hybrid/ripple.rs:653-741
//   router -> top-k -> softmax over the selected -> expert mixture (no shared expert)
//                                                     engine/hybrid/qwen.rs:872-899, math.rs:36-66
//   pre-norm residuals, final norm, output projection engine/hybrid/ripple.rs:474-482
// Projections and expert banks go through the quantized matvec kernels (Q8_0 / Q4_K, tensor-core MAC);
// the kernels here are the f32 glue between them.  One token = one CUDA graph; token and position live on
// the device, so greedy decode chains without the host.
#include <cmath>
#include <cstring>
#include <vector>

#include "context.cuh"
#include "ops.cuh"
#include "qmv.cuh"

#define SB_TRY(expr)                        \
    do {                                    \
        stark_b200_status _s = (expr);      \
        if (_s != STARK_B200_OK) return _s; \
    } while (0)

namespace sb {

namespace {

struct MoeState {
    uint32_t token;     // the token this step consumes (written by the host, or taken from `next`)
    uint32_t chain;     // 1: consume `next` (the greedy pick of the previous step)
    uint32_t next;      // first index of the maximum of the last logits
    uint32_t position;  // rows in the cache
    uint32_t error;     // sticky: 1 token out of range, 2 non-finite logits, 4 context exhausted, 8 a peer did not answer
};

// ---- expert parallelism -------------------------------------------------------------------------------------
// One process per GPU.  Every rank runs the whole token (attention, router, read-out: replicated, so all ranks
// hold identical activations bit for bit) except the expert feed-forward: rank r keeps experts
// [r * E/G, (r + 1) * E/G) and computes only the selected experts it owns.  The exchange step of a layer is the
// combine: the owner of selection slot i pushes that expert's output row into EVERY rank's receive buffer
// (plain 64-bit stores over NVLink peer mappings, {value, ticket} packets that are valid exactly when the ticket
// is this layer's), and the kernel that forms the mixture polls the `active` rows and adds them in selection
// order -- the same order and the same operands as on one GPU, so the result does not depend on the rank count.
// Receive buffers are per layer; a flag round at the end of every token keeps a fast rank from overwriting a
// layer's packets before a slow rank has read them.  Every wait is bounded (error bit 8).
// Region of one rank: [0, 4 KB) flags[kMaxEpRanks] written by the peers; then packets[layers][active][hidden].
constexpr uint32_t kMaxEpRanks = 8;
constexpr uint32_t kEpSkip = 0xffffffffu;  // expert id of a selection slot another rank owns
struct EpRegion {
    uint8_t *base[kMaxEpRanks];
    uint32_t rank, ranks, local_experts;
    unsigned long long wait_ns;
};
__host__ __device__ inline size_t ep_region_bytes(uint32_t layers, uint32_t active, uint32_t hidden) {
    return 4096u + (size_t)layers * active * hidden * 8u;
}
__host__ __device__ inline unsigned long long *ep_packets(uint8_t *base, uint32_t layer, uint32_t active, uint32_t hidden) {
    return reinterpret_cast<unsigned long long *>(base + 4096u) + (size_t)layer * active * hidden;
}

constexpr uint32_t kAttnSplits = 16, kAttnWarps = 8, kMoeMaxAttnSplits = 64;
constexpr uint32_t kFinishCtas = 64;  // CTAs of the arg-max over the logits

template <int THREADS>
__device__ inline float block_sum(float v, float *scratch /* [32] */) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31u) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
    for (int w = 0; w < THREADS / 32; ++w) r += scratch[w];
    return r;
}

// Token row of a Q8_0 table in the source layout (34-byte blocks of 32): d * q, as decode_block
// (engine/hybrid/weights.rs:2936-2941).
__global__ void __launch_bounds__(256) moe_embed_kernel(MoeState *st, const uint8_t *blocks, float *x, uint32_t hidden,
                                                        uint32_t vocab, uint32_t context) {
    pdl_launch_dependents();
    pdl_wait();
    uint32_t token = st->chain ? st->next : st->token;
    __syncthreads();
    if (token >= vocab || st->position >= context) {
        if (threadIdx.x == 0) st->error |= token >= vocab ? 1u : 4u;
        token = 0;
    }
    if (threadIdx.x == 0) st->token = token;
    const uint8_t *row = blocks + (size_t)token * (hidden / 32u) * 34u;
    for (uint32_t i = threadIdx.x; i < hidden; i += 256u) {
        const uint8_t *b = row + (i >> 5) * 34u;
        const float d = __half2float(__ushort_as_half((unsigned short)(b[0] | (b[1] << 8))));
        x[i] = d * (float)(int8_t)b[2u + (i & 31u)];
    }
}

// out = x * (1 / sqrt(mean(x^2) + eps)) * w   (math.rs:18-34)
__global__ void __launch_bounds__(1024) moe_rmsnorm_kernel(const float *x, const float *w, float *out, uint32_t n,
                                                           float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += 1024u) s += x[i] * x[i];
    const float mean = block_sum<1024>(s, scratch) / (float)n;
    const float scale = 1.0f / sqrtf(mean + eps);
    for (uint32_t i = threadIdx.x; i < n; i += 1024u) out[i] = x[i] * scale * w[i];
}

// One CTA of `dim` threads per head of the fused [q; k; v] projection: q and k heads get the per-head norm
// and rope (ripple.rs:696-703, 653-666); k and v heads land in the cache row of this position.
__global__ void moe_heads_kernel(const MoeState *st, float *qkv, const float *q_norm, const float *k_norm, float *keys,
                                 float *values, uint32_t q_heads, uint32_t kv_heads, uint32_t dim, float eps,
                                 float theta, uint32_t context) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    __shared__ float head[256];
    const uint32_t h = blockIdx.x, i = threadIdx.x;
    const uint32_t position = min(st->position, context - 1u);  // a full cache is refused on the host first
    const size_t kv_row = (size_t)kv_heads * dim;
    float *src = qkv + (size_t)h * dim;
    if (h >= q_heads + kv_heads) {  // v: copy
        values[position * kv_row + (size_t)(h - q_heads - kv_heads) * dim + i] = src[i];
        return;
    }
    const float v = src[i];
    float s = v * v;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((i & 31u) == 0) scratch[i >> 5] = s;
    __syncthreads();
    float sum = 0.0f;
    for (uint32_t w = 0; w < dim / 32u; ++w) sum += scratch[w];
    const float scale = 1.0f / sqrtf(sum / (float)dim + eps);
    head[i] = v * scale * (h < q_heads ? q_norm : k_norm)[i];
    __syncthreads();
    const uint32_t half = dim / 2u, pair = i < half ? i : i - half;
    const float angle = (float)position * powf(theta, -((float)(2u * pair)) / (float)dim);
    float sn, cs;
    sincosf(angle, &sn, &cs);
    const float a = head[pair], b = head[pair + half];
    const float out = i < half ? a * cs - b * sn : a * sn + b * cs;
    if (h < q_heads)
        src[i] = out;
    else
        keys[position * kv_row + (size_t)(h - q_heads) * dim + i] = out;
}

// Causal attention of one query head over one span of the cache (ripple.rs:716-735): scores q.k / sqrt(d),
// softmax, probability-weighted values.  Each warp walks every 8th row of the span with its own running
// (max, sum, accumulator); the warps' states are merged in shared memory and the span's state goes to
// `part` for the merge kernel.  dim = 128: one float4 per lane.
__global__ void __launch_bounds__(kAttnWarps * 32) moe_attention_kernel(const MoeState *st, const float *q,
                                                                        const float *keys, const float *values,
                                                                        float *part, uint32_t q_heads,
                                                                        uint32_t kv_heads, float scale,
                                                                        uint32_t context) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr uint32_t D = 128;
    __shared__ float sm[kAttnWarps], sl[kAttnWarps];
    __shared__ float4 sacc[kAttnWarps][32];
    const uint32_t h = blockIdx.x, split = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rows = min(st->position + 1u, context);
    const uint32_t span = (rows + kAttnSplits - 1u) / kAttnSplits;
    const uint32_t lo = min(rows, split * span), hi = min(rows, lo + span);
    const size_t kv_row = (size_t)kv_heads * D;
    const uint32_t begin = h / (q_heads / kv_heads) * D;
    const float4 qv = reinterpret_cast<const float4 *>(q + (size_t)h * D)[lane];
    float m = -INFINITY, l = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    // four rows per trip: their loads and reductions are independent, only the softmax update is serial
    for (uint32_t t0 = lo + warp; t0 < hi; t0 += 4u * kAttnWarps) {
        float4 kv[4], vv[4];
        float dot[4];
#pragma unroll
        for (uint32_t j = 0; j < 4u; ++j) {
            const uint32_t t = min(t0 + j * kAttnWarps, hi - 1u);  // rows past the end repeat the last one, unused
            kv[j] = reinterpret_cast<const float4 *>(keys + t * kv_row + begin)[lane];
            vv[j] = reinterpret_cast<const float4 *>(values + t * kv_row + begin)[lane];
        }
#pragma unroll
        for (uint32_t j = 0; j < 4u; ++j) dot[j] = qv.x * kv[j].x + qv.y * kv[j].y + qv.z * kv[j].z + qv.w * kv[j].w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (uint32_t j = 0; j < 4u; ++j) dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], o);
        }
#pragma unroll
        for (uint32_t j = 0; j < 4u; ++j) {
            if (t0 + j * kAttnWarps >= hi) break;
            const float s = dot[j] * scale;
            const float nm = fmaxf(m, s);
            const float c = expf(m - nm), p = expf(s - nm);  // expf(-inf) = 0 on the first row
            l = l * c + p;
            acc.x = acc.x * c + p * vv[j].x;
            acc.y = acc.y * c + p * vv[j].y;
            acc.z = acc.z * c + p * vv[j].z;
            acc.w = acc.w * c + p * vv[j].w;
            m = nm;
        }
    }
    if (lane == 0) sm[warp] = m, sl[warp] = l;
    sacc[warp][lane] = acc;
    __syncthreads();
    if (warp == 0) {
        float gm = -INFINITY;
        for (uint32_t w = 0; w < kAttnWarps; ++w) gm = fmaxf(gm, sm[w]);
        float gl = 0.0f;
        float4 g = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t w = 0; w < kAttnWarps; ++w) {
            if (sm[w] == -INFINITY) continue;
            const float c = expf(sm[w] - gm);
            const float4 a = sacc[w][lane];
            gl += sl[w] * c;
            g.x += a.x * c, g.y += a.y * c, g.z += a.z * c, g.w += a.w * c;
        }
        float *dst = part + ((size_t)h * kAttnSplits + split) * (D + 2u);
        if (lane == 0) dst[0] = gm, dst[1] = gl;
        reinterpret_cast<float2 *>(dst + 2)[lane * 2u] = make_float2(g.x, g.y);
        reinterpret_cast<float2 *>(dst + 2)[lane * 2u + 1u] = make_float2(g.z, g.w);
    }
}

// The same attention with the query heads of one KV head handled together (G = q_heads / kv_heads): a CTA
// per (KV head, span) reads each K and V row once and scores it against all G queries, instead of G CTAs
// reading the same rows.  Per warp: G running (max, sum, accumulator) states; warp g merges head g's states.
// One 128-wide head by one warp, as moe_heads_kernel does it with one thread per element: per-head norm, then rope
// on the pairs (i, i + 64).  Lane L holds elements L, 32 + L, 64 + L, 96 + L -- the four 32-element runs whose sums
// that kernel's four warps form, added in the same order -- so the values are the same bits; both halves of a
// rotation pair sit in one lane.
__device__ inline void moe_head_prepare(const float *src, const float *norm_w, float eps, float theta, uint32_t position,
                                        uint32_t lane, float out[4]) {
    constexpr uint32_t D = 128;
    float v[4], part[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        v[k] = src[32 * k + lane];
        float s = v[k] * v[k];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        part[k] = s;
    }
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) sum += part[k];
    const float scale = 1.0f / sqrtf(sum / (float)D + eps);
    float head[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) head[k] = v[k] * scale * norm_w[32 * k + lane];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const uint32_t pair = 32u * k + lane;
        const float angle = (float)position * powf(theta, -((float)(2u * pair)) / (float)D);
        float sn, cs;
        sincosf(angle, &sn, &cs);
        const float a = head[k], b = head[k + 2];
        out[k] = a * cs - b * sn;
        out[k + 2] = a * sn + b * cs;
    }
}

// `raw` (fused form): the [q; k; v] projection as the matvec left it.  Every CTA then prepares the group's query
// heads itself (norm, rope; one warp per head) and the CTA whose span holds the new position also prepares the
// key head and writes it and the value head into the cache before anybody reads that row -- the work of
// moe_heads_kernel without its launch.  raw == nullptr: `q` holds prepared heads and the cache row is there.
template <int G>
__global__ void __launch_bounds__(kAttnWarps * 32) moe_attention_grouped_kernel(const MoeState *st, const float *q,
                                                                                float *keys, float *values, float *part,
                                                                                uint32_t splits, uint32_t kv_heads,
                                                                                float scale, uint32_t context,
                                                                                const float *raw, const float *q_norm,
                                                                                const float *k_norm, float eps,
                                                                                float theta) {
    constexpr uint32_t D = 128;
    __shared__ float sm[kAttnWarps][G], sl[kAttnWarps][G];
    __shared__ float4 sacc[kAttnWarps][G][32];
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t kvh = blockIdx.x, split = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rows = min(st->position + 1u, context);
    const uint32_t span = (rows + splits - 1u) / splits;
    const uint32_t lo = min(rows, split * span), hi = min(rows, lo + span);
    const size_t kv_row = (size_t)kv_heads * D;
    const uint32_t begin = kvh * D;
    if (raw) {
        float *qs = reinterpret_cast<float *>(&sacc[0][0][0]);  // [G][128], before the accumulators need the space
        const uint32_t position = rows - 1u, q_heads = kv_heads * G;
        float o[4];
        for (uint32_t g = warp; g < (uint32_t)G; g += kAttnWarps) {
            moe_head_prepare(raw + ((size_t)kvh * G + g) * D, q_norm, eps, theta, position, lane, o);
#pragma unroll
            for (int k = 0; k < 4; ++k) qs[g * D + 32 * k + lane] = o[k];
        }
        if (hi == rows && lo < hi) {  // this span ends with the new row
            if (warp == kAttnWarps - 1u) {
                moe_head_prepare(raw + ((size_t)q_heads + kvh) * D, k_norm, eps, theta, position, lane, o);
#pragma unroll
                for (int k = 0; k < 4; ++k) keys[position * kv_row + begin + 32 * k + lane] = o[k];
            } else if (warp == kAttnWarps - 2u) {
                const float *src = raw + ((size_t)q_heads + kv_heads + kvh) * D;
#pragma unroll
                for (int k = 0; k < 4; ++k) values[position * kv_row + begin + 32 * k + lane] = src[32 * k + lane];
            }
        }
        __syncthreads();  // the heads are in shared memory, the new cache row is visible to this CTA
        q = qs;
    }
    float4 qv[G];
#pragma unroll
    for (int g = 0; g < G; ++g)
        qv[g] = reinterpret_cast<const float4 *>(q + (raw ? (size_t)g : (size_t)kvh * G + g) * D)[lane];
    if (raw) __syncthreads();  // every warp has its copy: the accumulators may take the space
    float m[G], l[G];
    float4 acc[G];
#pragma unroll
    for (int g = 0; g < G; ++g) m[g] = -INFINITY, l[g] = 0.0f, acc[g] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (uint32_t t0 = lo + warp; t0 < hi; t0 += 2u * kAttnWarps) {
        float4 kv[2], vv[2];
        float dot[2][G];
#pragma unroll
        for (uint32_t j = 0; j < 2u; ++j) {
            const uint32_t t = min(t0 + j * kAttnWarps, hi - 1u);  // a row past the end repeats the last one, unused
            kv[j] = reinterpret_cast<const float4 *>(keys + t * kv_row + begin)[lane];
            vv[j] = reinterpret_cast<const float4 *>(values + t * kv_row + begin)[lane];
        }
#pragma unroll
        for (uint32_t j = 0; j < 2u; ++j)
#pragma unroll
            for (int g = 0; g < G; ++g)
                dot[j][g] = qv[g].x * kv[j].x + qv[g].y * kv[j].y + qv[g].z * kv[j].z + qv[g].w * kv[j].w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (uint32_t j = 0; j < 2u; ++j)
#pragma unroll
                for (int g = 0; g < G; ++g) dot[j][g] += __shfl_xor_sync(0xffffffffu, dot[j][g], o);
#pragma unroll
        for (uint32_t j = 0; j < 2u; ++j) {
            if (t0 + j * kAttnWarps >= hi) break;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float s = dot[j][g] * scale;
                const float nm = fmaxf(m[g], s);
                const float c = expf(m[g] - nm), p = expf(s - nm);
                l[g] = l[g] * c + p;
                acc[g].x = acc[g].x * c + p * vv[j].x;
                acc[g].y = acc[g].y * c + p * vv[j].y;
                acc[g].z = acc[g].z * c + p * vv[j].z;
                acc[g].w = acc[g].w * c + p * vv[j].w;
                m[g] = nm;
            }
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) sm[warp][g] = m[g], sl[warp][g] = l[g];
        sacc[warp][g][lane] = acc[g];
    }
    __syncthreads();
    if (warp < (uint32_t)G) {
        const uint32_t g = warp;
        float gm = -INFINITY;
        for (uint32_t w = 0; w < kAttnWarps; ++w) gm = fmaxf(gm, sm[w][g]);
        float gl = 0.0f;
        float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t w = 0; w < kAttnWarps; ++w) {
            if (sm[w][g] == -INFINITY) continue;
            const float c = expf(sm[w][g] - gm);
            const float4 v = sacc[w][g][lane];
            gl += sl[w][g] * c;
            a.x += v.x * c, a.y += v.y * c, a.z += v.z * c, a.w += v.w * c;
        }
        float *dst = part + (((size_t)kvh * G + g) * splits + split) * (D + 2u);
        if (lane == 0) dst[0] = gm, dst[1] = gl;
        reinterpret_cast<float2 *>(dst + 2)[lane * 2u] = make_float2(a.x, a.y);
        reinterpret_cast<float2 *>(dst + 2)[lane * 2u + 1u] = make_float2(a.z, a.w);
    }
}

// Merges the spans' (max, sum, accumulator) states of one head.  The per-span weights exp(m_s - max) are
// formed once in shared memory, so that the loop over the spans is independent loads and multiply-adds.
__global__ void __launch_bounds__(128) moe_attention_merge_kernel(const float *part, float *out, uint32_t splits) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr uint32_t D = 128;
    __shared__ float sm[kMoeMaxAttnSplits], sl[kMoeMaxAttnSplits], sc[kMoeMaxAttnSplits];
    const uint32_t h = blockIdx.x, i = threadIdx.x;
    const float *src = part + (size_t)h * splits * (D + 2u);
    if (i < splits) {
        sm[i] = src[i * (D + 2u)];
        sl[i] = src[i * (D + 2u) + 1u];
    }
    __syncthreads();
    float gm = -INFINITY;
    for (uint32_t s = 0; s < splits; ++s) gm = fmaxf(gm, sm[s]);
    if (i < splits) sc[i] = sm[i] == -INFINITY ? 0.0f : expf(sm[i] - gm);  // an empty span weighs nothing
    __syncthreads();
    float l = 0.0f, a = 0.0f;
#pragma unroll 8
    for (uint32_t s = 0; s < splits; ++s) {
        const float c = sc[s];
        l += sl[s] * c;
        a += src[s * (D + 2u) + 2u + i] * c;
    }
    out[(size_t)h * D + i] = a / l;
}

// Router scores (one CTA per expert: scores[e] = w[e] . x, f32) and, in the CTA that finishes last, the
// selection: top-k of the scores (value descending, index ascending), softmax over the selected scores
// (qwen.rs:872-874, math.rs:36-66).  ids[0, active) are the experts in selection order; ids[active, 2 active)
// the same plus `experts`, which addresses the up half of a fused [gate; up] bank.
//
// With `update` the kernel also does what moe_add_norm_kernel would have done in a launch of its own before it:
// every CTA forms n = rms_norm(residual + update, norm_w) in shared memory for its own dot product (8 KB of
// redundant reads per CTA against a launch and its hand-off), and CTA 0 leaves n in `x` for the expert matvecs.
// The residual itself is NOT rewritten here (other CTAs are still reading it): the mixture kernel after the
// experts adds `update` first and the mixture second, the order of two separate adds.  The sums are formed in the
// order of moe_add_norm_kernel's 1024 threads (thread t stands for t, t + 256, t + 512 and t + 768 of them), so
// the values are the same bits.
constexpr uint32_t kRouterNormMaxHidden = 4096;
__global__ void __launch_bounds__(256) moe_router_select_kernel(const float *w, float *x, float *scores,
                                                                uint32_t hidden, uint32_t experts, uint32_t active,
                                                                uint32_t *ids, float *probs, uint32_t *arrivals,
                                                                uint32_t *ids_global, uint32_t ep_first,
                                                                uint32_t ep_local, const float *residual,
                                                                const float *update, const float *norm_w, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    __shared__ float sv[1024];
    __shared__ bool last;
    __shared__ __align__(16) float xs[kRouterNormMaxHidden];
    const uint32_t e = blockIdx.x;
    const float4 *row = reinterpret_cast<const float4 *>(w + (size_t)e * hidden);
    const float4 *xv = reinterpret_cast<const float4 *>(x);
    if (update) {
        float part[4];
#pragma unroll
        for (uint32_t k = 0; k < 4u; ++k) {
            float s = 0.0f;
            for (uint32_t i = threadIdx.x + 256u * k; i < hidden; i += 1024u) {
                const float v = residual[i] + update[i];
                xs[i] = v;
                s += v * v;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            part[k] = s;
        }
        if ((threadIdx.x & 31u) == 0) {
#pragma unroll
            for (uint32_t k = 0; k < 4u; ++k) scratch[(threadIdx.x >> 5) + 8u * k] = part[k];
        }
        __syncthreads();
        float total = 0.0f;
        for (int wi = 0; wi < 32; ++wi) total += scratch[wi];
        const float scale = 1.0f / sqrtf(total / (float)hidden + eps);
        for (uint32_t i = threadIdx.x; i < hidden; i += 256u) {  // each thread its own elements again
            const float nv = xs[i] * scale * norm_w[i];
            xs[i] = nv;
            if (e == 0) x[i] = nv;
        }
        __syncthreads();  // also frees `scratch` for the block sum below
        xv = reinterpret_cast<const float4 *>(xs);
    }
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < hidden / 4u; i += 256u) {
        const float4 a = row[i], b = xv[i];
        s += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
    }
    s = block_sum<256>(s, scratch);
    if (threadIdx.x == 0) {
        scores[e] = s;
        __threadfence();
        last = atomicAdd(arrivals, 1u) == gridDim.x - 1u;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    for (uint32_t i = threadIdx.x; i < experts; i += 256u) sv[i] = __ldcg(scores + i);
    if (threadIdx.x == 0) *arrivals = 0;  // ready for the next launch
    __syncthreads();
    if (threadIdx.x >= 32u) return;
    const uint32_t lane = threadIdx.x;
    uint32_t taken = 0;  // bit j: expert lane + 32 j is already selected
    float chosen_v = 0.0f;  // lane r keeps the r-th selected score
    uint32_t chosen = 0;
    for (uint32_t r = 0; r < active; ++r) {
        float best = -INFINITY;
        uint32_t bi = 0xffffffffu;
        for (uint32_t j = 0, i = lane; i < experts; ++j, i += 32u) {
            const float v = sv[i];
            if (!((taken >> j) & 1u) && (bi == 0xffffffffu || v > best)) best = v, bi = i;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0xffffffffu && (bi == 0xffffffffu || ov > best || (ov == best && oi < bi))) best = ov, bi = oi;
        }
        if ((bi & 31u) == lane) taken |= 1u << (bi >> 5);
        if (lane == r) chosen_v = best, chosen = bi;
    }
    // softmax over the selected, sums in selection order
    float mx = -INFINITY;
    for (uint32_t r = 0; r < active; ++r) mx = fmaxf(mx, __shfl_sync(0xffffffffu, chosen_v, r));
    const float p = lane < active ? expf(chosen_v - mx) : 0.0f;
    float sum = 0.0f;
    for (uint32_t r = 0; r < active; ++r) sum += __shfl_sync(0xffffffffu, p, r);
    if (lane < active) {
        probs[lane] = p / sum;
        if (ep_local) {
            // expert parallel: the bank holds this rank's experts only; slots of other ranks are skipped
            const bool mine = chosen >= ep_first && chosen < ep_first + ep_local;
            ids[lane] = mine ? chosen - ep_first : kEpSkip;
            ids[active + lane] = mine ? chosen - ep_first + ep_local : kEpSkip;
            ids_global[lane] = chosen;
        } else {
            ids[lane] = chosen;
            ids[active + lane] = chosen + experts;
        }
    }
}

// x += update, where update is one row (probs == nullptr) or the expert mixture sum_r probs[r] * rows[r]
// with r ascending from zero (qwen.rs:894-899); then, if w is given, out = rms_norm(x, w): the residual add
// and the norm that always follows it, in one CTA.
// `first`, if given, is a row added before that (the attention update the router kernel left to this one).
__global__ void __launch_bounds__(1024) moe_add_norm_kernel(float *x, const float *rows, const float *probs,
                                                            uint32_t active, const float *w, float *out, uint32_t n,
                                                            float eps, const float *first) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    __shared__ float sp[32];  // the mixture weights, read once
    if (probs && threadIdx.x < active) sp[threadIdx.x] = probs[threadIdx.x];
    __syncthreads();
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += 1024u) {
        float r;
        const float xi = first ? x[i] + first[i] : x[i];
        if (probs) {
            r = 0.0f;
#pragma unroll 8
            for (uint32_t e = 0; e < active; ++e) r += sp[e] * __ldg(rows + (size_t)e * n + i);
        } else {
            r = rows[i];
        }
        const float v = xi + r;
        x[i] = v;
        s += v * v;
    }
    if (!w) return;
    const float mean = block_sum<1024>(s, scratch) / (float)n;
    const float scale = 1.0f / sqrtf(mean + eps);
    for (uint32_t i = threadIdx.x; i < n; i += 1024u) out[i] = x[i] * scale * w[i];  // this thread's own writes
}

// Expert parallel: the rows of the selection slots this rank owns go to every rank (itself included).
__global__ void __launch_bounds__(256) moe_ep_push_kernel(EpRegion g, const float *rows, const uint32_t *ids, uint32_t layer,
                                                          uint32_t layers, uint32_t active, uint32_t n,
                                                          const uint32_t *ep_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t slot = blockIdx.x;
    if (ids[slot] == kEpSkip) return;
    const uint32_t ticket = __ldcg(ep_tokens) * layers + layer + 1u;
    const float *row = rows + (size_t)slot * n;
    for (uint32_t i = threadIdx.x; i < n; i += 256u) {
        const unsigned long long packet = ((unsigned long long)ticket << 32) | __float_as_uint(row[i]);
        for (uint32_t r = 0; r < g.ranks; ++r)
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(ep_packets(g.base[r], layer, active, n) + (size_t)slot * n + i),
                         "l"(packet)
                         : "memory");
    }
}

// moe_add_norm_kernel with the expert rows taken from this rank's receive buffer: x += sum_r probs[r] * row_r in
// selection order, then the norm.  A row is there when its packets carry this layer's ticket.
__global__ void __launch_bounds__(1024) moe_ep_mix_norm_kernel(float *x, const unsigned long long *packets, const float *probs,
                                                               uint32_t active, const float *w, float *out, uint32_t n,
                                                               float eps, const uint32_t *ep_tokens, uint32_t layer,
                                                               uint32_t layers, unsigned long long wait_ns, MoeState *st,
                                                               const float *first) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    __shared__ float sp[32];
    if (threadIdx.x < active) sp[threadIdx.x] = probs[threadIdx.x];
    __syncthreads();
    const uint32_t ticket = __ldcg(ep_tokens) * layers + layer + 1u;
    const unsigned long long t0 = global_ns();
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += 1024u) {
        float r = 0.0f;
        for (uint32_t e0 = 0; e0 < active; e0 += 8u) {  // eight rows per trip to memory
            unsigned long long q[8];
            uint32_t spins = 0;
            for (;;) {
                bool all = true;
#pragma unroll
                for (uint32_t j = 0; j < 8u; ++j) {
                    if (e0 + j < active) {
                        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(q[j]) : "l"(packets + (size_t)(e0 + j) * n + i) : "memory");
                    } else {
                        q[j] = (unsigned long long)ticket << 32;
                    }
                }
#pragma unroll
                for (uint32_t j = 0; j < 8u; ++j) all = all && (uint32_t)(q[j] >> 32) == ticket;
                if (all) break;
                if (++spins > 8u) {
                    __nanosleep(64);
                    if (global_ns() - t0 > wait_ns) {  // a rank is missing: report and go on with what is there
                        atomicOr(&st->error, 8u);
                        break;
                    }
                }
            }
#pragma unroll
            for (uint32_t j = 0; j < 8u; ++j)
                if (e0 + j < active) r += sp[e0 + j] * __uint_as_float((uint32_t)q[j]);
        }
        const float v = (first ? x[i] + first[i] : x[i]) + r;
        x[i] = v;
        s += v * v;
    }
    if (!w) return;
    const float mean = block_sum<1024>(s, scratch) / (float)n;
    const float scale = 1.0f / sqrtf(mean + eps);
    for (uint32_t i = threadIdx.x; i < n; i += 1024u) out[i] = x[i] * scale * w[i];
}

// End of a token under expert parallelism: every rank tells every rank that it is through with the token's
// receive buffers, waits for all of them, and only then advances the counter the tickets are made of.
__global__ void __launch_bounds__(32) moe_ep_token_barrier_kernel(EpRegion g, uint32_t *ep_tokens, MoeState *st) {
    const uint32_t lane = threadIdx.x;
    const uint32_t done = *ep_tokens + 1u;
    if (lane < g.ranks) {
        uint32_t *peer_flag = reinterpret_cast<uint32_t *>(g.base[lane]) + g.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flag), "r"(done) : "memory");
        const uint32_t *mine = reinterpret_cast<const uint32_t *>(g.base[g.rank]) + lane;
        const unsigned long long t0 = global_ns();
        for (uint32_t spins = 0;; ++spins) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
            if ((int32_t)(seen - done) >= 0) break;
            if (spins > 8u) {
                __nanosleep(128);
                if (global_ns() - t0 > g.wait_ns) {
                    atomicOr(&st->error, 8u);
                    break;
                }
            }
        }
    }
    __syncwarp();
    if (lane == 0) *ep_tokens = done;
}

// gate[i] = silu(gate[i]) * up[i]  (qwen.rs:889-891, math.rs:5-16)
__global__ void moe_silu_mul_kernel(float *gate, const float *up, uint32_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = gate[i];
    float sg;
    if (g >= 0.0f) {
        sg = 1.0f / (1.0f + expf(-g));
    } else {
        const float e = expf(g);
        sg = e / (1.0f + e);
    }
    gate[i] = g * sg * up[i];
}

// (value, first index) of the maximum over the CTA's threads, valid in thread 0.  idx = UINT32_MAX: no entry.
__device__ inline void block_first_max(float &best, uint32_t &idx, float *bv /* [32] */, uint32_t *bi /* [32] */) {
    const auto better = [](float ov, uint32_t oi, float v, uint32_t i) {
        return oi != 0xffffffffu && (i == 0xffffffffu || ov > v || (ov == v && oi < i));
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (better(ov, oi, best, idx)) best = ov, idx = oi;
    }
    __syncthreads();
    if ((threadIdx.x & 31u) == 0) bv[threadIdx.x >> 5] = best, bi[threadIdx.x >> 5] = idx;
    __syncthreads();
    if (threadIdx.x == 0)
        for (uint32_t w = 1; w < blockDim.x / 32u; ++w)
            if (better(bv[w], bi[w], best, idx)) best = bv[w], idx = bi[w];
}

// End of a token: with logits, the first index of their maximum becomes `next` (non-finite logits raise
// the error word, as Model::step refuses them, engine/hybrid/mod.rs:990); the cache grows by one row.
// Each CTA scans its share of the row and leaves (maximum, first index, non-finite seen) in `scratch`; the
// CTA that arrives last reduces those.  Without logits: one CTA, position + 1 only.
__global__ void __launch_bounds__(1024) moe_finish_kernel(MoeState *st, const float *logits, uint32_t vocab,
                                                          float *scratch, uint32_t *arrivals) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float bv[32];
    __shared__ uint32_t bi[32];
    __shared__ bool last;
    if (!logits) {
        if (blockIdx.x == 0 && threadIdx.x == 0) st->position += 1u;
        return;
    }
    const uint32_t ctas = gridDim.x;
    float best = -INFINITY;
    uint32_t idx = 0xffffffffu;
    int bad = 0;
    for (uint32_t i = blockIdx.x * 1024u + threadIdx.x; i < vocab; i += ctas * 1024u) {
        const float v = logits[i];
        bad |= !isfinite(v);
        if (idx == 0xffffffffu || v > best) best = v, idx = i;
    }
    bad = __syncthreads_or(bad);
    block_first_max(best, idx, bv, bi);
    if (threadIdx.x == 0) {
        scratch[blockIdx.x] = best;
        scratch[ctas + blockIdx.x] = __uint_as_float(idx);
        scratch[2u * ctas + blockIdx.x] = bad ? 1.0f : 0.0f;
        __threadfence();
        last = atomicAdd(arrivals, 1u) == ctas - 1u;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    best = -INFINITY, idx = 0xffffffffu, bad = 0;
    if (threadIdx.x < ctas) {
        best = __ldcg(scratch + threadIdx.x);
        idx = __float_as_uint(__ldcg(scratch + ctas + threadIdx.x));
        bad = __ldcg(scratch + 2u * ctas + threadIdx.x) != 0.0f;
    }
    bad = __syncthreads_or(bad);
    block_first_max(best, idx, bv, bi);
    if (threadIdx.x == 0) {
        st->next = idx;
        if (bad) st->error |= 2u;
        st->position += 1u;
        *arrivals = 0;  // ready for the next launch
    }
}

}  // namespace

struct MoeModel {
    stark_b200_moe_config cfg{};
    int device = -1;
    cudaStream_t stream = nullptr;
    std::vector<const QMatrix *> qkv, o, gate_up, down;
    const QMatrix *output = nullptr;
    // owned device memory
    uint8_t *token_table = nullptr;
    float *norms = nullptr;   // [layers][2 * hidden + 2 * head_dim] then final [hidden]
    float *router = nullptr;  // [layers][experts * hidden]
    float *keys = nullptr, *values = nullptr;  // [layers][context][kv_heads * head_dim]
    float *work = nullptr;    // activations, see carve()
    uint32_t *ids = nullptr;  // [layers][2 * active]: the selected experts, then the same + experts
    uint32_t *arrivals = nullptr;  // arrival counters of [0] the router CTAs, [1] the arg-max CTAs (they return to zero by themselves)
    MoeState *state = nullptr;
    std::vector<uint8_t> have;  // which tensors were set
    // activations carved out of `work`
    float *x, *n, *qkv_out, *att, *part, *update, *scores, *probs, *gate_out, *expert_out, *logits;
    cudaGraphExec_t graph[2] = {nullptr, nullptr};  // [0] cache only, [1] with logits
    bool warmed[2] = {false, false};
    uint32_t nodes = 0;
    uint32_t position = 0;  // host mirror of the device position
    bool poisoned = false;
    // STARK_B200_MOE_FUSE=1: the launches that hold only a hand-off (residual add + norm, per-head norm + rope) run
    // inside the kernel that consumes them: 8 launches a layer instead of 10, the same bits, and no faster (the
    // consumers' CTAs repeat the work behind the same wait), so it is off by default
    bool fuse = false;
    // expert parallelism (ep.ranks == 0: one GPU)
    EpRegion ep{};
    uint8_t *ep_local = nullptr;      // this rank's exchange region
    uint32_t *ep_tokens = nullptr;    // tokens finished, never reset: what the tickets are made of
    uint32_t *ids_global = nullptr;   // [layers][active] the selected experts in the model's numbering
    bool ep_connected = false;
    std::vector<void *> ep_opened;    // peers' regions opened through IPC
    uint32_t local_experts() const { return ep.ranks ? ep.local_experts : cfg.experts; }

    size_t norm_stride() const { return 2u * (size_t)cfg.hidden + 2u * cfg.head_dim; }
    float *norm(uint32_t kind, uint32_t layer) const {
        if (kind == STARK_B200_MOE_TENSOR_FINAL_NORM) return norms + (size_t)cfg.layers * norm_stride();
        float *base = norms + (size_t)layer * norm_stride();
        if (kind == STARK_B200_MOE_TENSOR_ATTN_NORM) return base;
        if (kind == STARK_B200_MOE_TENSOR_FFN_NORM) return base + cfg.hidden;
        if (kind == STARK_B200_MOE_TENSOR_Q_NORM) return base + 2u * (size_t)cfg.hidden;
        return base + 2u * (size_t)cfg.hidden + cfg.head_dim;
    }
    size_t kv_layer() const { return (size_t)cfg.context_tokens * cfg.kv_heads * cfg.head_dim; }
    size_t have_index(uint32_t group, uint32_t kind, uint32_t layer) const {
        return ((size_t)group * 8u + kind) * cfg.layers + layer;
    }
    bool complete() const {
        for (uint32_t l = 0; l < cfg.layers; ++l) {
            for (uint32_t k = 0; k <= STARK_B200_MOE_MAT_DOWN; ++k)
                if (!have[have_index(0, k, l)]) return false;
            for (uint32_t k : {STARK_B200_MOE_TENSOR_ATTN_NORM, STARK_B200_MOE_TENSOR_FFN_NORM,
                               STARK_B200_MOE_TENSOR_Q_NORM, STARK_B200_MOE_TENSOR_K_NORM, STARK_B200_MOE_TENSOR_ROUTER})
                if (!have[have_index(1, k, l)]) return false;
        }
        return have[have_index(0, STARK_B200_MOE_MAT_OUTPUT, 0)] && have[have_index(1, STARK_B200_MOE_TENSOR_FINAL_NORM, 0)] &&
               have[have_index(1, STARK_B200_MOE_TENSOR_TOKEN_TABLE, 0)];
    }
};

namespace {

template <typename... Params, typename... Args>
stark_b200_status moe_launch(void (*kernel)(Params...), dim3 grid, dim3 block, bool pdl, cudaStream_t stream,
                             Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...));
    return STARK_B200_OK;
}

// Every kernel of a token awaits its predecessor itself (programmatic dependent launch), so the next
// kernel's CTAs are placed, and the matvecs' first weight records fetched, while the previous one drains.
// STARK_B200_PDL=0 serializes the launches instead.
bool moe_pdl() {
    static const bool on = [] {
        const char *e = getenv("STARK_B200_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

// CTAs of the grouped attention kernel over all KV heads (STARK_B200_MOE_ATTN_CTAS overrides).
uint32_t moe_attention_ctas() {
    static const uint32_t n = [] {
        const char *e = getenv("STARK_B200_MOE_ATTN_CTAS");
        const int v = e ? atoi(e) : 0;
        return v >= 16 && v <= 1024 ? (uint32_t)v : 256u;
    }();
    return n;
}

stark_b200_status moe_issue(MoeModel *m, bool want_logits, cudaStream_t s) {
    const auto &c = m->cfg;
    const uint32_t H = c.hidden, D = c.head_dim, QH = c.q_heads, KV = c.kv_heads, A = c.active_experts;
    const uint32_t I = c.expert_intermediate;
    const float scale = 1.0f / sqrtf((float)D);
    const bool pdl = moe_pdl();
    SB_TRY(moe_launch(moe_embed_kernel, 1, 256, false, s, m->state, m->token_table, m->x, H, c.vocab, c.context_tokens));
    SB_TRY(moe_launch(moe_rmsnorm_kernel, 1, 1024, pdl, s, m->x, m->norm(STARK_B200_MOE_TENSOR_ATTN_NORM, 0), m->n, H,
                      c.rms_eps));
    for (uint32_t l = 0; l < c.layers; ++l) {
        float *keys = m->keys + (size_t)l * m->kv_layer(), *values = m->values + (size_t)l * m->kv_layer();
        uint32_t *ids = m->ids + (size_t)l * 2u * A;
        SB_TRY(qmv_rows_launch(m->qkv[l], m->n, 0, m->qkv_out, 1, nullptr, STARK_B200_F32, s, pdl));
        // query heads of one KV head together where the group size has an instantiation, else head by head
        const uint32_t group = QH / KV, gsplits = std::max(kAttnSplits, std::min(kMoeMaxAttnSplits, moe_attention_ctas() / KV));
        const bool grouped_form = group == 8u || group == 4u || group == 2u;
        // per-head norm, rope and the cache row: inside the grouped attention kernel (fused), or a launch of their own
        const bool fused_heads = m->fuse && grouped_form && D == 128u;
        if (!fused_heads)
            SB_TRY(moe_launch(moe_heads_kernel, QH + 2u * KV, D, pdl, s, m->state, m->qkv_out,
                              m->norm(STARK_B200_MOE_TENSOR_Q_NORM, l), m->norm(STARK_B200_MOE_TENSOR_K_NORM, l), keys, values,
                              QH, KV, D, c.rms_eps, c.rope_theta, c.context_tokens));
        uint32_t splits = kAttnSplits;
        if (grouped_form) {
            splits = gsplits;
            auto grouped = group == 8u ? moe_attention_grouped_kernel<8>
                                       : (group == 4u ? moe_attention_grouped_kernel<4> : moe_attention_grouped_kernel<2>);
            SB_TRY(moe_launch(grouped, dim3(KV, splits), kAttnWarps * 32, pdl, s, m->state, m->qkv_out, keys, values,
                              m->part, splits, KV, scale, c.context_tokens, fused_heads ? m->qkv_out : nullptr,
                              m->norm(STARK_B200_MOE_TENSOR_Q_NORM, l), m->norm(STARK_B200_MOE_TENSOR_K_NORM, l), c.rms_eps,
                              c.rope_theta));
        } else {
            SB_TRY(moe_launch(moe_attention_kernel, dim3(QH, kAttnSplits), kAttnWarps * 32, pdl, s, m->state, m->qkv_out,
                              keys, values, m->part, QH, KV, scale, c.context_tokens));
        }
        SB_TRY(moe_launch(moe_attention_merge_kernel, QH, 128, pdl, s, m->part, m->att, splits));
        SB_TRY(qmv_rows_launch(m->o[l], m->att, 0, m->update, 1, nullptr, STARK_B200_F32, s, pdl));
        // the residual add and the norm before the router: in the router's CTAs (fused), or a launch of their own
        const bool fused_norm = m->fuse && H <= kRouterNormMaxHidden;
        if (!fused_norm)
            SB_TRY(moe_launch(moe_add_norm_kernel, 1, 1024, pdl, s, m->x, m->update, nullptr, 1u,
                              m->norm(STARK_B200_MOE_TENSOR_FFN_NORM, l), m->n, H, c.rms_eps, nullptr));
        const float *pending_update = fused_norm ? m->update : nullptr;  // added to the residual by the mixture kernel
        const bool ep = m->ep.ranks > 1u;
        SB_TRY(moe_launch(moe_router_select_kernel, c.experts, 256, pdl, s, m->router + (size_t)l * c.experts * H, m->n,
                          m->scores, H, c.experts, A, ids, m->probs, m->arrivals,
                          ep ? m->ids_global + (size_t)l * A : nullptr, ep ? m->ep.rank * m->ep.local_experts : 0u,
                          ep ? m->ep.local_experts : 0u, m->x, pending_update,
                          m->norm(STARK_B200_MOE_TENSOR_FFN_NORM, l), c.rms_eps));
        SB_TRY(qmv_rows_launch(m->gate_up[l], m->n, 0, m->gate_out, 2u * A, ids, STARK_B200_F32, s, pdl));
        if (m->down[l]->format == kFmtQ4_K) {  // the gated activation is formed while the down projection stages its input
            SB_TRY(q4kt_launch(m->down[l], m->gate_out, I, m->expert_out, A, ids, STARK_B200_F32, s, pdl,
                               m->gate_out + (size_t)A * I));
        } else {
            SB_TRY(moe_launch(moe_silu_mul_kernel, (A * I + 255u) / 256u, 256, pdl, s, m->gate_out,
                              m->gate_out + (size_t)A * I, A * I));
            SB_TRY(qmv_rows_launch(m->down[l], m->gate_out, I, m->expert_out, A, ids, STARK_B200_F32, s, pdl));
        }
        // the mixture, the residual add and the next norm: the next layer's, or the final one before the logits
        const float *next = l + 1u < c.layers ? m->norm(STARK_B200_MOE_TENSOR_ATTN_NORM, l + 1u)
                                              : (want_logits ? m->norm(STARK_B200_MOE_TENSOR_FINAL_NORM, 0) : nullptr);
        if (ep) {
            SB_TRY(moe_launch(moe_ep_push_kernel, A, 256, pdl, s, m->ep, m->expert_out, ids, l, c.layers, A, H, m->ep_tokens));
            SB_TRY(moe_launch(moe_ep_mix_norm_kernel, 1, 1024, pdl, s, m->x, ep_packets(m->ep_local, l, A, H), m->probs, A,
                              next, m->n, H, c.rms_eps, m->ep_tokens, l, c.layers, m->ep.wait_ns, m->state, pending_update));
        } else {
            SB_TRY(moe_launch(moe_add_norm_kernel, 1, 1024, pdl, s, m->x, m->expert_out, m->probs, A, next, m->n, H, c.rms_eps,
                              pending_update));
        }
    }
    if (want_logits) SB_TRY(qmv_rows_launch(m->output, m->n, 0, m->logits, 1, nullptr, STARK_B200_F32, s, pdl));
    // the attention partials are free by now: scratch for the per-CTA maxima
    SB_TRY(moe_launch(moe_finish_kernel, want_logits ? kFinishCtas : 1u, 1024, pdl, s, m->state,
                      want_logits ? m->logits : nullptr, c.vocab, m->part, m->arrivals + 1));
    if (m->ep.ranks > 1u) SB_TRY(moe_launch(moe_ep_token_barrier_kernel, 1, 32, false, s, m->ep, m->ep_tokens, m->state));
    return STARK_B200_OK;
}

// One token through the graph of its kind; the first token of each kind runs eagerly (kernels opt into
// their shared-memory sizes on first use, which a capture must not contain) and the graph is captured
// from the second.
stark_b200_status moe_token(MoeModel *m, bool want_logits) {
    const int k = want_logits ? 1 : 0;
    if (!m->warmed[k]) {
        m->warmed[k] = true;
        // The first token of a kind runs eagerly and loads its kernels: between ranks that is start-up skew, not a
        // rank that left, so its waits get a minute; the recorded graphs keep the configured limit.
        const unsigned long long configured_wait = m->ep.wait_ns;
        if (m->ep.ranks > 1u) m->ep.wait_ns = std::max<unsigned long long>(configured_wait, 60000000000ull);
        const stark_b200_status st = moe_issue(m, want_logits, m->stream);
        m->ep.wait_ns = configured_wait;
        return st;
    }
    if (!m->graph[k]) {
        cudaGraph_t g = nullptr;
        SB_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
        const stark_b200_status st = moe_issue(m, want_logits, m->stream);
        const cudaError_t e = cudaStreamEndCapture(m->stream, &g);
        if (st != STARK_B200_OK || e != cudaSuccess) {
            if (g) cudaGraphDestroy(g);
            return st != STARK_B200_OK ? st : cuda_status(e);
        }
        size_t count = 0;
        cudaGraphGetNodes(g, nullptr, &count);
        if (want_logits) m->nodes = (uint32_t)count;
        const cudaError_t ie = cudaGraphInstantiate(&m->graph[k], g, 0);
        cudaGraphDestroy(g);
        SB_CUDA(ie);
    }
    SB_CUDA(cudaGraphLaunch(m->graph[k], m->stream));
    return STARK_B200_OK;
}

stark_b200_status moe_set_input(MoeModel *m, uint32_t token, uint32_t chain) {
    const uint32_t words[2] = {token, chain};
    SB_CUDA(cudaMemcpyAsync(m->state, words, sizeof(words), cudaMemcpyHostToDevice, m->stream));
    return STARK_B200_OK;
}

stark_b200_status moe_check(MoeModel *m) {  // after a synchronize: the device error word
    MoeState st{};
    SB_CUDA(cudaMemcpy(&st, m->state, sizeof(st), cudaMemcpyDeviceToHost));
    if (st.error) {
        m->poisoned = true;
        return (st.error & 1u) ? STARK_B200_INVALID_ARGUMENT
                               : ((st.error & 4u) ? STARK_B200_CONTEXT_LIMIT : STARK_B200_DEVICE_FAILURE);
    }
    return STARK_B200_OK;
}

stark_b200_status moe_reset(MoeModel *m) {
    SB_CUDA(cudaMemsetAsync(m->state, 0, sizeof(MoeState), m->stream));
    SB_CUDA(cudaStreamSynchronize(m->stream));
    m->position = 0;
    m->poisoned = false;
    return STARK_B200_OK;
}

struct DeviceScope {
    int previous = -1;
    explicit DeviceScope(int device) {
        cudaGetDevice(&previous);
        if (previous != device) cudaSetDevice(device);
    }
    ~DeviceScope() { cudaSetDevice(previous); }
};

void moe_free(MoeModel *m) {
    for (auto &g : m->graph)
        if (g) cudaGraphExecDestroy(g);
    cudaFree(m->token_table), cudaFree(m->norms), cudaFree(m->router), cudaFree(m->keys), cudaFree(m->values);
    cudaFree(m->work), cudaFree(m->ids), cudaFree(m->arrivals), cudaFree(m->state);
    for (void *p : m->ep_opened) cudaIpcCloseMemHandle(p);
    cudaFree(m->ep_local), cudaFree(m->ep_tokens), cudaFree(m->ids_global);
    if (m->stream) cudaStreamDestroy(m->stream);
    delete m;
}

}  // namespace

}  // namespace sb

using namespace sb;

extern "C" {

stark_b200_status stark_b200_moe_model_create(const stark_b200_moe_config *config, stark_b200_moe_model **out_model) {
    if (!config || !out_model) return STARK_B200_INVALID_ARGUMENT;
    if (config->struct_size != sizeof(stark_b200_moe_config)) return STARK_B200_ABI_MISMATCH;
    const auto &c = *config;
    if (c.vocab == 0 || c.layers == 0 || c.hidden == 0 || c.hidden % 256u || c.head_dim != 128u || c.q_heads == 0 ||
        c.kv_heads == 0 || c.q_heads % c.kv_heads || c.experts == 0 || c.experts > 1024u || c.active_experts == 0 ||
        c.active_experts > 32u || c.active_experts > c.experts || c.expert_intermediate == 0 ||
        c.expert_intermediate % 256u || c.context_tokens == 0 || !(c.rms_eps > 0.0f) || !std::isfinite(c.rms_eps) ||
        !(c.rope_theta > 0.0f) || !std::isfinite(c.rope_theta))
        return STARK_B200_INVALID_ARGUMENT;
    if (!device_context()) return STARK_B200_OUT_OF_MEMORY;
    MoeModel *m = new MoeModel();
    if (const char *e = getenv("STARK_B200_MOE_FUSE")) m->fuse = e[0] == '1';
    m->cfg = c;
    cudaGetDevice(&m->device);
    m->qkv.assign(c.layers, nullptr), m->o.assign(c.layers, nullptr), m->gate_up.assign(c.layers, nullptr);
    m->down.assign(c.layers, nullptr);
    m->have.assign(2u * 8u * c.layers, 0);
    const size_t QD = (size_t)c.q_heads * c.head_dim, KD = (size_t)c.kv_heads * c.head_dim;
    const size_t AI = (size_t)c.active_experts * c.expert_intermediate;
    const size_t sizes[] = {c.hidden, c.hidden, QD + 2u * KD, QD, (size_t)c.q_heads * kMoeMaxAttnSplits * (c.head_dim + 2u),
                            c.hidden, c.experts, c.active_experts, 2u * AI, (size_t)c.active_experts * c.hidden, c.vocab};
    size_t total = 0;
    for (size_t v : sizes) total += (v + 63u) / 64u * 64u;
    bool ok = cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaMalloc(&m->token_table, (size_t)c.vocab * (c.hidden / 32u) * 34u) == cudaSuccess;
    ok = ok && cudaMalloc(&m->norms, ((size_t)c.layers * m->norm_stride() + c.hidden) * 4u) == cudaSuccess;
    ok = ok && cudaMalloc(&m->router, (size_t)c.layers * c.experts * c.hidden * 4u) == cudaSuccess;
    ok = ok && cudaMalloc(&m->keys, (size_t)c.layers * m->kv_layer() * 4u) == cudaSuccess;
    ok = ok && cudaMalloc(&m->values, (size_t)c.layers * m->kv_layer() * 4u) == cudaSuccess;
    ok = ok && cudaMalloc(&m->work, total * 4u) == cudaSuccess;
    ok = ok && cudaMalloc(&m->ids, (size_t)c.layers * c.active_experts * 8u) == cudaSuccess;
    ok = ok && cudaMalloc(&m->arrivals, 8u) == cudaSuccess;
    ok = ok && cudaMalloc(&m->state, sizeof(MoeState)) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        moe_free(m);
        return STARK_B200_OUT_OF_MEMORY;
    }
    float **slots[] = {&m->x, &m->n, &m->qkv_out, &m->att, &m->part, &m->update, &m->scores, &m->probs,
                       &m->gate_out, &m->expert_out, &m->logits};
    float *at = m->work;
    for (size_t i = 0; i < sizeof(sizes) / sizeof(sizes[0]); ++i) {
        *slots[i] = at;
        at += (sizes[i] + 63u) / 64u * 64u;
    }
    cudaMemset(m->ids, 0, (size_t)c.layers * c.active_experts * 8u);
    cudaMemset(m->arrivals, 0, 8u);
    if (moe_reset(m) != STARK_B200_OK) {
        moe_free(m);
        return STARK_B200_DEVICE_FAILURE;
    }
    *out_model = reinterpret_cast<stark_b200_moe_model *>(m);
    return STARK_B200_OK;
}

stark_b200_status stark_b200_moe_model_set_matrix(stark_b200_moe_model *model, uint32_t kind, uint32_t layer,
                                                  const stark_b200_qmatrix *matrix) {
    MoeModel *m = reinterpret_cast<MoeModel *>(model);
    const QMatrix *q = reinterpret_cast<const QMatrix *>(matrix);
    if (!m || !q || kind > STARK_B200_MOE_MAT_OUTPUT) return STARK_B200_INVALID_ARGUMENT;
    if (kind == STARK_B200_MOE_MAT_OUTPUT) layer = 0;
    if (layer >= m->cfg.layers || q->device != m->device || !qmv_rows_supports(q)) return STARK_B200_INVALID_ARGUMENT;
    const auto &c = m->cfg;
    const uint32_t QD = c.q_heads * c.head_dim, KD = c.kv_heads * c.head_dim;
    const bool q8 = q->format == kFmtQ8_0 || q->format == kFmtQ8_0T;
    const bool q4 = q->format == kFmtQ4_K || q->format == kFmtQ4_KRaw;
    const uint32_t banks = q->experts > 1u ? q->experts : 1u;
    bool fits = false;
    switch (kind) {
        case STARK_B200_MOE_MAT_QKV: fits = q8 && banks == 1u && q->rows == QD + 2u * KD && q->columns == c.hidden; break;
        case STARK_B200_MOE_MAT_O: fits = q8 && banks == 1u && q->rows == c.hidden && q->columns == QD; break;
        case STARK_B200_MOE_MAT_GATE_UP:
            fits = q4 && banks == 2u * m->local_experts() && q->rows == c.expert_intermediate && q->columns == c.hidden;
            break;
        case STARK_B200_MOE_MAT_DOWN:
            fits = q4 && banks == m->local_experts() && q->rows == c.hidden && q->columns == c.expert_intermediate;
            break;
        default: fits = q8 && banks == 1u && q->rows == c.vocab && q->columns == c.hidden; break;
    }
    if (!fits) return STARK_B200_INVALID_ARGUMENT;
    switch (kind) {
        case STARK_B200_MOE_MAT_QKV: m->qkv[layer] = q; break;
        case STARK_B200_MOE_MAT_O: m->o[layer] = q; break;
        case STARK_B200_MOE_MAT_GATE_UP: m->gate_up[layer] = q; break;
        case STARK_B200_MOE_MAT_DOWN: m->down[layer] = q; break;
        default: m->output = q; break;
    }
    m->have[m->have_index(0, kind, layer)] = 1;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_moe_model_set_tensor(stark_b200_moe_model *model, uint32_t kind, uint32_t layer,
                                                  const void *host_data, size_t bytes) {
    MoeModel *m = reinterpret_cast<MoeModel *>(model);
    if (!m || !host_data || kind > STARK_B200_MOE_TENSOR_TOKEN_TABLE) return STARK_B200_INVALID_ARGUMENT;
    const auto &c = m->cfg;
    if (kind == STARK_B200_MOE_TENSOR_FINAL_NORM || kind == STARK_B200_MOE_TENSOR_TOKEN_TABLE) layer = 0;
    if (layer >= c.layers) return STARK_B200_INVALID_ARGUMENT;
    DeviceScope scope(m->device);
    void *dst;
    size_t want;
    if (kind == STARK_B200_MOE_TENSOR_TOKEN_TABLE) {
        dst = m->token_table, want = (size_t)c.vocab * (c.hidden / 32u) * 34u;
    } else if (kind == STARK_B200_MOE_TENSOR_ROUTER) {
        dst = m->router + (size_t)layer * c.experts * c.hidden, want = (size_t)c.experts * c.hidden * 4u;
    } else {
        dst = m->norm(kind, layer);
        want = (kind == STARK_B200_MOE_TENSOR_Q_NORM || kind == STARK_B200_MOE_TENSOR_K_NORM ? c.head_dim : c.hidden) * 4u;
    }
    if (bytes != want) return STARK_B200_INVALID_ARGUMENT;
    if (kind != STARK_B200_MOE_TENSOR_TOKEN_TABLE) {  // rms_norm and the router refuse non-finite weights
        const float *v = static_cast<const float *>(host_data);
        for (size_t i = 0; i < bytes / 4u; ++i)
            if (!std::isfinite(v[i])) return STARK_B200_INVALID_ARGUMENT;
    }
    SB_CUDA(cudaMemcpy(dst, host_data, bytes, cudaMemcpyHostToDevice));
    m->have[m->have_index(1, kind, layer)] = 1;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_moe_model_ep_init(stark_b200_moe_model *model, uint32_t rank, uint32_t ranks,
                                               uint8_t *handle_out) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the interface");
    MoeModel *m = reinterpret_cast<MoeModel *>(model);
    if (!m || !handle_out) return STARK_B200_INVALID_ARGUMENT;
    if (m->ep_local || m->warmed[0] || m->warmed[1]) return STARK_B200_INVALID_STATE;
    for (uint32_t l = 0; l < m->cfg.layers; ++l)  // the banks are checked against the rank's share: set them afterwards
        if (m->gate_up[l] || m->down[l]) return STARK_B200_INVALID_STATE;
    const auto &c = m->cfg;
    if (ranks < 2u || ranks > kMaxEpRanks || rank >= ranks || c.experts % ranks != 0) return STARK_B200_INVALID_ARGUMENT;
    DeviceScope scope(m->device);
    const size_t bytes = ep_region_bytes(c.layers, c.active_experts, c.hidden);
    SB_CUDA(cudaMalloc(&m->ep_local, bytes));
    SB_CUDA(cudaMemset(m->ep_local, 0, bytes));
    SB_CUDA(cudaMalloc(&m->ep_tokens, 16u));
    SB_CUDA(cudaMemset(m->ep_tokens, 0, 16u));
    SB_CUDA(cudaMalloc(&m->ids_global, (size_t)c.layers * c.active_experts * 4u));
    SB_CUDA(cudaMemset(m->ids_global, 0, (size_t)c.layers * c.active_experts * 4u));
    SB_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t handle;
    SB_CUDA(cudaIpcGetMemHandle(&handle, m->ep_local));
    memcpy(handle_out, &handle, 64);
    m->ep.rank = rank;
    m->ep.ranks = ranks;
    m->ep.local_experts = c.experts / ranks;
    m->ep.wait_ns = 4000000000ull;
    m->ep.base[rank] = m->ep_local;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_moe_model_ep_connect(stark_b200_moe_model *model, const uint8_t *handles, size_t handle_bytes) {
    MoeModel *m = reinterpret_cast<MoeModel *>(model);
    if (!m || !handles) return STARK_B200_INVALID_ARGUMENT;
    if (!m->ep_local || m->ep_connected) return STARK_B200_INVALID_STATE;
    if (handle_bytes != (size_t)m->ep.ranks * 64u) return STARK_B200_INVALID_ARGUMENT;
    DeviceScope scope(m->device);
    for (uint32_t r = 0; r < m->ep.ranks; ++r) {
        if (r == m->ep.rank) continue;
        cudaIpcMemHandle_t handle;
        memcpy(&handle, handles + (size_t)r * 64u, 64);
        void *p = nullptr;
        SB_CUDA(cudaIpcOpenMemHandle(&p, handle, cudaIpcMemLazyEnablePeerAccess));
        m->ep_opened.push_back(p);
        m->ep.base[r] = static_cast<uint8_t *>(p);
    }
    m->ep_connected = true;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_moe_model_ep_set_wait(stark_b200_moe_model *model, uint64_t nanoseconds) {
    MoeModel *m = reinterpret_cast<MoeModel *>(model);
    if (!m) return STARK_B200_INVALID_ARGUMENT;
    if (!m->ep_local || m->warmed[0] || m->warmed[1]) return STARK_B200_INVALID_STATE;
    if (nanoseconds < 1000ull || nanoseconds > 600000000000ull) return STARK_B200_INVALID_ARGUMENT;
    m->ep.wait_ns = nanoseconds;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_moe_model_reset(stark_b200_moe_model *model) {
    MoeModel *m = reinterpret_cast<MoeModel *>(model);
    if (!m) return STARK_B200_INVALID_ARGUMENT;
    DeviceScope scope(m->device);
    return moe_reset(m);
}

static stark_b200_status moe_ready(MoeModel *m, uint32_t tokens) {
    if (!m) return STARK_B200_INVALID_ARGUMENT;
    if (!m->complete() || (m->ep_local && !m->ep_connected)) return STARK_B200_INVALID_STATE;
    if (m->poisoned) return STARK_B200_RELOAD_REQUIRED;
    if ((uint64_t)m->position + tokens > m->cfg.context_tokens) return STARK_B200_CONTEXT_LIMIT;
    return STARK_B200_OK;
}

// Any failure of a token resets the model, as hybrid::Model does (engine/hybrid/mod.rs:990).
static stark_b200_status moe_fail(MoeModel *m, stark_b200_status st) {
    cudaStreamSynchronize(m->stream);
    moe_reset(m);
    return st;
}

stark_b200_status stark_b200_moe_model_ingest(stark_b200_moe_model *model, const uint32_t *tokens, uint32_t count) {
    MoeModel *m = reinterpret_cast<MoeModel *>(model);
    SB_TRY(moe_ready(m, count));
    if (count && !tokens) return STARK_B200_INVALID_ARGUMENT;
    for (uint32_t i = 0; i < count; ++i)
        if (tokens[i] >= m->cfg.vocab) return STARK_B200_INVALID_ARGUMENT;
    DeviceScope scope(m->device);
    for (uint32_t i = 0; i < count; ++i) {
        stark_b200_status st = moe_set_input(m, tokens[i], 0);
        if (st == STARK_B200_OK) st = moe_token(m, false);
        if (st != STARK_B200_OK) return moe_fail(m, st);
    }
    if (cudaStreamSynchronize(m->stream) != cudaSuccess) return moe_fail(m, STARK_B200_DEVICE_FAILURE);
    m->position += count;
    const stark_b200_status st = moe_check(m);
    return st == STARK_B200_OK ? st : moe_fail(m, st);
}

stark_b200_status stark_b200_moe_model_step(stark_b200_moe_model *model, uint32_t token, float *logits_host,
                                            size_t count) {
    MoeModel *m = reinterpret_cast<MoeModel *>(model);
    SB_TRY(moe_ready(m, 1));
    if (token >= m->cfg.vocab || (logits_host && count != m->cfg.vocab)) return STARK_B200_INVALID_ARGUMENT;
    DeviceScope scope(m->device);
    stark_b200_status st = moe_set_input(m, token, 0);
    if (st == STARK_B200_OK) st = moe_token(m, true);
    if (st != STARK_B200_OK) return moe_fail(m, st);
    if (logits_host &&
        cudaMemcpyAsync(logits_host, m->logits, (size_t)m->cfg.vocab * 4u, cudaMemcpyDeviceToHost, m->stream) != cudaSuccess)
        return moe_fail(m, STARK_B200_DEVICE_FAILURE);
    if (cudaStreamSynchronize(m->stream) != cudaSuccess) return moe_fail(m, STARK_B200_DEVICE_FAILURE);
    m->position += 1;
    st = moe_check(m);
    return st == STARK_B200_OK ? st : moe_fail(m, st);
}

stark_b200_status stark_b200_moe_model_generate_greedy(stark_b200_moe_model *model, uint32_t first, uint32_t steps,
                                                       uint32_t *out_tokens) {
    MoeModel *m = reinterpret_cast<MoeModel *>(model);
    SB_TRY(moe_ready(m, steps));
    if (steps == 0 || !out_tokens || first >= m->cfg.vocab) return STARK_B200_INVALID_ARGUMENT;
    DeviceScope scope(m->device);
    uint32_t *picks = nullptr;  // the device-side record of every step's pick
    SB_CUDA(cudaMalloc(&picks, (size_t)steps * 4u));
    stark_b200_status st = STARK_B200_OK;
    for (uint32_t i = 0; i < steps && st == STARK_B200_OK; ++i) {
        st = moe_set_input(m, first, i == 0 ? 0u : 1u);
        if (st == STARK_B200_OK) st = moe_token(m, true);
        if (st == STARK_B200_OK &&
            cudaMemcpyAsync(picks + i, &m->state->next, 4u, cudaMemcpyDeviceToDevice, m->stream) != cudaSuccess)
            st = STARK_B200_DEVICE_FAILURE;
    }
    if (st == STARK_B200_OK && cudaMemcpyAsync(out_tokens, picks, (size_t)steps * 4u, cudaMemcpyDeviceToHost, m->stream) !=
                                   cudaSuccess)
        st = STARK_B200_DEVICE_FAILURE;
    if (st == STARK_B200_OK && cudaStreamSynchronize(m->stream) != cudaSuccess) st = STARK_B200_DEVICE_FAILURE;
    cudaFree(picks);
    if (st != STARK_B200_OK) return moe_fail(m, st);
    m->position += steps;
    st = moe_check(m);
    return st == STARK_B200_OK ? st : moe_fail(m, st);
}

stark_b200_status stark_b200_moe_model_last_experts(stark_b200_moe_model *model, uint32_t *ids_host, size_t count) {
    MoeModel *m = reinterpret_cast<MoeModel *>(model);
    if (!m || !ids_host || count != (size_t)m->cfg.layers * m->cfg.active_experts) return STARK_B200_INVALID_ARGUMENT;
    DeviceScope scope(m->device);
    SB_CUDA(cudaStreamSynchronize(m->stream));
    const size_t a = m->cfg.active_experts;
    if (m->ep.ranks > 1u) {
        SB_CUDA(cudaMemcpy(ids_host, m->ids_global, count * 4u, cudaMemcpyDeviceToHost));
    } else {
        SB_CUDA(cudaMemcpy2D(ids_host, a * 4u, m->ids, 2u * a * 4u, a * 4u, m->cfg.layers, cudaMemcpyDeviceToHost));
    }
    return STARK_B200_OK;
}

stark_b200_status stark_b200_moe_model_position(const stark_b200_moe_model *model, uint32_t *out_position) {
    const MoeModel *m = reinterpret_cast<const MoeModel *>(model);
    if (!m || !out_position) return STARK_B200_INVALID_ARGUMENT;
    *out_position = m->position;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_moe_model_launches_per_token(const stark_b200_moe_model *model, uint32_t *out_launches) {
    const MoeModel *m = reinterpret_cast<const MoeModel *>(model);
    if (!m || !out_launches) return STARK_B200_INVALID_ARGUMENT;
    *out_launches = m->nodes ? m->nodes : 4u + (m->fuse ? 8u : 10u) * m->cfg.layers + (m->ep.ranks > 1u ? m->cfg.layers + 1u : 0u);
    return STARK_B200_OK;
}

stark_b200_status stark_b200_moe_model_stream(const stark_b200_moe_model *model, void **out_stream) {
    const MoeModel *m = reinterpret_cast<const MoeModel *>(model);
    if (!m || !out_stream) return STARK_B200_INVALID_ARGUMENT;
    *out_stream = m->stream;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_moe_model_destroy(stark_b200_moe_model **model) {
    if (!model || !*model) return STARK_B200_INVALID_ARGUMENT;
    MoeModel *m = reinterpret_cast<MoeModel *>(*model);
    {
        DeviceScope scope(m->device);
        cudaStreamSynchronize(m->stream);
        moe_free(m);
    }
    *model = nullptr;
    return STARK_B200_OK;
}

}  // extern "C"
