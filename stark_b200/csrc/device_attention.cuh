// Decode attention for one new row, as device functions shared by the standalone kernel (one CTA per
// (split, KV head)) and the persistent decode kernel (the same work as one operator of its list).
#pragma once
#include "device_math.cuh"

namespace sb {

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

// Shared memory the attention functions work in (carved by the caller).
struct AttnShared {
    uint8_t *tiles;                   // 4 * kTileBytes: [2][K, V][64 rows][272 B]
    uint16_t (*q_s)[kHeadDim];        // [kMaxGqa] q after norm + RoPE, bf16
    uint16_t *knew, *vnew;            // [kHeadDim] the appended key / value row
    float (*ml_s)[kMaxGqa][2];        // [kAttnWarps] per-warp (max, sum)
};
constexpr uint32_t kAttnSharedBytes =
    kAttnSmemBytes + kMaxGqa * kHeadDim * 2u + 2u * kHeadDim * 2u + kAttnWarps * kMaxGqa * 2u * 4u;

__device__ inline AttnShared carve_attn_shared(uint8_t *base /* 128-byte aligned */) {
    AttnShared s;
    s.tiles = base;
    s.q_s = reinterpret_cast<uint16_t(*)[kHeadDim]>(base + kAttnSmemBytes);
    s.knew = reinterpret_cast<uint16_t *>(base + kAttnSmemBytes + kMaxGqa * kHeadDim * 2u);
    s.vnew = s.knew + kHeadDim;
    s.ml_s = reinterpret_cast<float(*)[kMaxGqa][2]>(s.vnew + kHeadDim);
    return s;
}

// Split `split` of KV head `h`: writes the partial (o, max, sum) of the G query heads of the group to
// p.scratch.  Threads 0 .. 127 (four warps) compute; every thread of the BAR_THREADS-wide barrier group
// must call it (the others only take part in the barriers).  The page range streams through shared
// memory (16 KB K tile + 16 KB V tile per page, cp.async, double buffered, rows padded to 272 B).  Per
// 64-key tile every warp computes S = Q K^T for all keys with mma.m16n8k16 (bf16; the G query heads
// are the M rows) and the same online softmax in f32, then O += P V for its own 32 of the 128 output
// dims, with P carried as bf16 hi + lo so that the weights keep ~16 bits.  Warps only synchronise to
// hand tile buffers over.  Inputs written by other CTAs of a running kernel are read with ld.cg.
template <int BAR_ID, int BAR_THREADS>
__device__ inline void attention_partial(const AttnParams &p, uint32_t split, uint32_t h, uint32_t pos,
                                         const AttnShared &sm, uint32_t tid) {
    const uint32_t lane = tid & 31u, warp = tid >> 5, G = p.gqa;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const bool worker = tid < (uint32_t)kAttnThreads;
    const uint32_t seq_len = pos + 1u;
    const uint32_t nblocks = (seq_len + kPageTokens - 1u) / kPageTokens;
    const uint32_t b0 = (uint32_t)(((uint64_t)split * nblocks) / p.splits);
    const uint32_t b1 = (uint32_t)(((uint64_t)(split + 1u) * nblocks) / p.splits);
    const uint32_t new_block = pos / kPageTokens;
    const bool owner = new_block >= b0 && new_block < b1;
    const uint32_t ntiles = b1 - b0;
    uint8_t *tiles = sm.tiles;

    auto issue_tile = [&](uint32_t tile) {
        const uint32_t buf = tile & 1u;
        const size_t page = ((size_t)p.block_table[b0 + tile] * p.kv_heads + h) * kPageTokens * kHeadDim;
        const uint8_t *ksrc = reinterpret_cast<const uint8_t *>(p.keys + page);
        const uint8_t *vsrc = reinterpret_cast<const uint8_t *>(p.values + page);
        uint8_t *kd = tiles + (size_t)(buf * 2u) * kTileBytes, *vd = kd + kTileBytes;
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {  // 64 rows x 16 chunks of 16 B per tile
            const uint32_t idx = tid + i * kAttnThreads, row = idx >> 4, ch = idx & 15u;
            cp_async16(kd + row * kTileRowBytes + ch * 16u, ksrc + row * 256u + ch * 16u);
            cp_async16(vd + row * kTileRowBytes + ch * 16u, vsrc + row * 256u + ch * 16u);
        }
        cp_async_commit();
    };
    if (worker && ntiles > 0) issue_tile(0);

    // Norm + RoPE: one warp per head (the G query heads, then the new key row on the owner split).
    const float *cosr = p.rope_cos ? p.rope_cos + (size_t)pos * kHeadDim : nullptr;
    const float *sinr = p.rope_sin ? p.rope_sin + (size_t)pos * kHeadDim : nullptr;
    if (worker) {
        for (uint32_t hh = warp; hh < G + 1u; hh += kAttnWarps) {
            if (hh < G) {
                warp_head_norm_rope(p.qkv + (size_t)(h * G + hh) * kHeadDim, p.q_norm, cosr, sinr, p.eps, lane,
                                    sm.q_s[hh]);
            } else if (owner) {
                warp_head_norm_rope(p.qkv + (size_t)(p.q_heads + h) * kHeadDim, p.k_norm, cosr, sinr, p.eps, lane,
                                    sm.knew);
                const uint2 vv = __ldcg(reinterpret_cast<const uint2 *>(
                    p.qkv + (size_t)(p.q_heads + p.kv_heads + h) * kHeadDim + 4u * lane));
                *reinterpret_cast<uint2 *>(sm.vnew + 4u * lane) = vv;
            }
        }
    }
    named_bar_sync(BAR_ID, BAR_THREADS);
    if (owner && tid < 16) {
        // append the new key / value rows to the cache (16 B per thread each)
        const size_t row = ((size_t)p.block_table[new_block] * p.kv_heads + h) * kPageTokens + (pos % kPageTokens);
        reinterpret_cast<uint4 *>(p.keys + row * kHeadDim)[tid] = reinterpret_cast<const uint4 *>(sm.knew)[tid];
        reinterpret_cast<uint4 *>(p.values + row * kHeadDim)[tid] = reinterpret_cast<const uint4 *>(sm.vnew)[tid];
    }
    // Q as the A operand (rows = heads of the group, zero rows above G), kept in registers.
    uint32_t qa[8][2];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        qa[kk][0] = (worker && g < G) ? *reinterpret_cast<const uint32_t *>(&sm.q_s[g][kk * 16 + 2 * t]) : 0u;
        qa[kk][1] = (worker && g < G) ? *reinterpret_cast<const uint32_t *>(&sm.q_s[g][kk * 16 + 8 + 2 * t]) : 0u;
    }
    if (tid == 0 && p.trace) trace_max(&p.trace->compute);

    // Online softmax state for head row g.  Every warp scores ALL keys of a tile (so the four warps
    // hold identical statistics and never have to be merged) but accumulates only its own 32 output
    // dims: o[n][..] is dim tile 4 * warp + n; [0,1] = row g, [2,3] = row g + 8 (padding rows).
    float m_run = -INFINITY, l_run = 0.0f;
    float o[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    // ldmatrix row addresses: lanes 0-7 -> matrix 0 rows, 8-15 -> matrix 1, 16-23 -> matrix 2, 24-31 -> matrix 3
    const uint32_t lrow = lane & 7u, lmat = lane >> 3;

    for (uint32_t tile = 0; tile < ntiles; ++tile) {
        if (worker) {
            if (tile + 1 < ntiles) {
                issue_tile(tile + 1);
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
        }
        named_bar_sync(BAR_ID, BAR_THREADS);
        const uint32_t buf = tile & 1u;
        uint8_t *kt = tiles + (size_t)(buf * 2u) * kTileBytes, *vt = kt + kTileBytes;
        const uint32_t blk = b0 + tile;
        if (blk == new_block) {
            // the copy may have raced the append above: patch the new row in shared memory
            if (tid < 16) {
                reinterpret_cast<uint4 *>(kt + (pos % kPageTokens) * kTileRowBytes)[tid] =
                    reinterpret_cast<const uint4 *>(sm.knew)[tid];
                reinterpret_cast<uint4 *>(vt + (pos % kPageTokens) * kTileRowBytes)[tid] =
                    reinterpret_cast<const uint4 *>(sm.vnew)[tid];
            }
            // rows after the new one are not part of the sequence: their weights are zero, but a
            // stale NaN pattern times zero would still poison the product, so clear the V rows
            if (worker)
                for (uint32_t i = tid; i < (kPageTokens - 1u - pos % kPageTokens) * 16u; i += kAttnThreads)
                    reinterpret_cast<uint4 *>(vt + (pos % kPageTokens + 1u + (i >> 4)) * kTileRowBytes)[i & 15u] =
                        make_uint4(0u, 0u, 0u, 0u);
            named_bar_sync(BAR_ID, BAR_THREADS);
        }
        const uint32_t valid = min(kPageTokens, seq_len - blk * kPageTokens);
        if (worker) {
            // ---- S = Q K^T for all 64 keys: 8 n-tiles of 8 keys, 8 k-steps of 16 dims ----
            float s[8][4];
#pragma unroll
            for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
                for (int kp = 0; kp < 4; ++kp) {
                    // matrices: (keys 16kp+0..7, dims kk*16+0..7), (same keys, dims +8), (keys +8, dims +0), (keys +8, dims +8)
                    uint32_t kb[4];
                    ldmatrix_x4(kb, kt + (kp * 16u + (lmat >> 1) * 8u + lrow) * kTileRowBytes +
                                        (kk * 16u + (lmat & 1u) * 8u) * 2u);
                    mma_m16n8k16_bf16(s[2 * kp], qa[kk][0], 0u, qa[kk][1], 0u, kb[0], kb[1]);
                    mma_m16n8k16_bf16(s[2 * kp + 1], qa[kk][0], 0u, qa[kk][1], 0u, kb[2], kb[3]);
                }
            }
            // lane holds row g: keys 8n + {2t, 2t+1} in s[n][0], s[n][1]
            float tm = -INFINITY;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                s[n][0] = 8u * n + 2u * t < valid ? s[n][0] * p.scale : -INFINITY;
                s[n][1] = 8u * n + 2u * t + 1u < valid ? s[n][1] * p.scale : -INFINITY;
                tm = fmaxf(tm, fmaxf(s[n][0], s[n][1]));
            }
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
            const float m_new = fmaxf(m_run, tm);  // finite: every tile holds at least one key in range
            const float factor = m_run == -INFINITY ? 0.0f : expf(m_run - m_new);
            float ts = 0.0f;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                s[n][0] = expf(s[n][0] - m_new);
                s[n][1] = expf(s[n][1] - m_new);
                ts += s[n][0] + s[n][1];
            }
            ts += __shfl_xor_sync(0xffffffffu, ts, 1);
            ts += __shfl_xor_sync(0xffffffffu, ts, 2);
            l_run = l_run * factor + ts;
            m_run = m_new;
#pragma unroll
            for (int n = 0; n < 4; ++n) o[n][0] *= factor, o[n][1] *= factor;
            // ---- O += P V for this warp's 32 dims: 4 k-steps of 16 keys, two pairs of dim tiles ----
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                // P as the A operand: C fragments of key tiles 2ks, 2ks+1 = one k16 A fragment
                uint32_t ph0, pl0, ph2, pl2;
                split_bf16x2(s[2 * ks][0], s[2 * ks][1], ph0, pl0);
                split_bf16x2(s[2 * ks + 1][0], s[2 * ks + 1][1], ph2, pl2);
#pragma unroll
                for (int np = 0; np < 2; ++np) {
                    // matrices (transposed on load): (keys 0-7, dims d0+0..7), (keys 8-15, same dims),
                    //                                (keys 0-7, dims d0+8..15), (keys 8-15, dims d0+8..15)
                    const uint32_t d0 = warp * 32u + np * 16u;
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, vt + (ks * 16u + (lmat & 1u) * 8u + lrow) * kTileRowBytes +
                                              (d0 + (lmat >> 1) * 8u) * 2u);
                    mma_m16n8k16_bf16(o[2 * np], ph0, 0u, ph2, 0u, vb[0], vb[1]);
                    mma_m16n8k16_bf16(o[2 * np], pl0, 0u, pl2, 0u, vb[0], vb[1]);
                    mma_m16n8k16_bf16(o[2 * np + 1], ph0, 0u, ph2, 0u, vb[2], vb[3]);
                    mma_m16n8k16_bf16(o[2 * np + 1], pl0, 0u, pl2, 0u, vb[2], vb[3]);
                }
            }
        }
        named_bar_sync(BAR_ID, BAR_THREADS);  // the buffer of this tile is free for tile + 2
    }

    // ---- publish this split's partial: each warp its 32 dims, warp 0 the statistics ----
    const uint32_t stride = kHeadDim + 2u;
    float *mine = p.scratch + ((size_t)(h * p.splits + split) * G) * stride;
    if (worker && g < G) {
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            mine[g * stride + warp * 32u + n * 8 + 2 * t] = o[n][0];
            mine[g * stride + warp * 32u + n * 8 + 2 * t + 1] = o[n][1];
        }
        if (warp == 0 && t == 0) {
            mine[g * stride + kHeadDim] = m_run;
            mine[g * stride + kHeadDim + 1] = l_run;
        }
    }
    if (worker) __threadfence();
    named_bar_sync(BAR_ID, BAR_THREADS);
}

// Merges the `splits` partials of KV head `h` into p.out.  Threads 0 .. 127 compute; every thread of
// the barrier group must call it.  `wgt` is scratch shared memory of kMaxGqa * (kMaxAttnSplits + 1) floats.
template <int BAR_ID, int BAR_THREADS>
__device__ inline void attention_merge(const AttnParams &p, uint32_t h, float *wgt, uint32_t tid) {
    const uint32_t lane = tid & 31u, warp = tid >> 5, G = p.gqa;
    const bool worker = tid < (uint32_t)kAttnThreads;
    const uint32_t stride = kHeadDim + 2u;
    const float *base = p.scratch + ((size_t)h * p.splits * G) * stride;
    // weights first (one warp per head, one lane per split), then independent loads per output
    if (worker) {
        for (uint32_t gg = warp; gg < G; gg += kAttnWarps) {
            const float ms = lane < p.splits ? __ldcg(&base[(lane * G + gg) * stride + kHeadDim]) : -INFINITY;
            const float ls = lane < p.splits ? __ldcg(&base[(lane * G + gg) * stride + kHeadDim + 1]) : 0.0f;
            const float mmax = warp_max(ms);
            const float w = ms == -INFINITY ? 0.0f : expf(ms - mmax);
            const float lsum = warp_sum(w * ls);
            if (lane < p.splits) wgt[gg * kMaxAttnSplits + lane] = w;
            if (lane == 0) wgt[kMaxGqa * kMaxAttnSplits + gg] = 1.0f / lsum;
        }
    }
    named_bar_sync(BAR_ID, BAR_THREADS);
    if (worker) {
        for (uint32_t i = tid; i < G * kHeadDim; i += kAttnThreads) {
            const uint32_t gg = i >> 7, d = i & 127u;
            float osum = 0.0f;
#pragma unroll 8
            for (uint32_t sp = 0; sp < p.splits; ++sp)
                osum = fmaf(wgt[gg * kMaxAttnSplits + sp], __ldcg(&base[(sp * G + gg) * stride + d]), osum);
            p.out[(size_t)(h * G + gg) * kHeadDim + d] = f32_to_bf16_bits(osum * wgt[kMaxGqa * kMaxAttnSplits + gg]);
        }
    }
}

}  // namespace sb
