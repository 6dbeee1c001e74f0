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
// nbuf = K / V tile pairs in flight (2: double buffered; 3: a split of up to three pages is fetched whole
// before the new row exists).
__host__ __device__ constexpr uint32_t attn_shared_bytes(uint32_t nbuf) {
    return nbuf * 2u * kTileBytes + kMaxGqa * kHeadDim * 2u + 2u * kHeadDim * 2u + kAttnWarps * kMaxGqa * 2u * 4u;
}
constexpr uint32_t kAttnSharedBytes = attn_shared_bytes(2);

__device__ inline AttnShared carve_attn_shared(uint8_t *base /* 128-byte aligned */, uint32_t nbuf = 2) {
    AttnShared s;
    const uint32_t tile_bytes = nbuf * 2u * kTileBytes;
    s.tiles = base;
    s.q_s = reinterpret_cast<uint16_t(*)[kHeadDim]>(base + tile_bytes);
    s.knew = reinterpret_cast<uint16_t *>(base + tile_bytes + kMaxGqa * kHeadDim * 2u);
    s.vnew = s.knew + kHeadDim;
    s.ml_s = reinterpret_cast<float(*)[kMaxGqa][2]>(s.vnew + kHeadDim);
    return s;
}

// What a split can fetch before the new row exists: its first two K / V tiles (rows of earlier tokens)
// and the per-lane constants of the head norm and RoPE at the row's position.
struct AttnPrefetch {
    uint32_t pos;
    HeadConsts cq, ck;
};

__device__ inline void attn_issue_tile(const AttnParams &p, uint32_t h, uint32_t block, uint32_t buf, uint8_t *tiles,
                                       uint32_t tid) {
    const size_t page = ((size_t)p.block_table[block] * p.kv_heads + h) * kPageTokens * kHeadDim;
    const uint8_t *ksrc = reinterpret_cast<const uint8_t *>(p.keys + page);
    const uint8_t *vsrc = reinterpret_cast<const uint8_t *>(p.values + page);
    uint8_t *kd = tiles + (size_t)(buf * 2u) * kTileBytes, *vd = kd + kTileBytes;
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {  // 64 rows x 16 chunks of 16 B per tile
        const uint32_t idx = tid + i * kAttnThreads, row = idx >> 4, ch = idx & 15u;
        cp_async16(kd + row * kTileRowBytes + ch * 16u, ksrc + row * 256u + ch * 16u);
        cp_async16(vd + row * kTileRowBytes + ch * 16u, vsrc + row * 256u + ch * 16u);
    }
}

__device__ inline void attn_split_range(const AttnParams &p, uint32_t split, uint32_t pos, uint32_t &b0, uint32_t &b1) {
    const uint32_t nblocks = (pos + 1u + kPageTokens - 1u) / kPageTokens;
    b0 = (uint32_t)(((uint64_t)split * nblocks) / p.splits);
    b1 = (uint32_t)(((uint64_t)(split + 1u) * nblocks) / p.splits);
}

// Starts the copies of the split's first NBUF tiles (NBUF cp.async groups, possibly empty) and loads the
// constants.  Touches nothing the kernel before this one writes, provided `pos` is already final; the
// caller checks that after its wait and calls this again if it was not.
template <int NBUF = 2>
__device__ inline void attention_prefetch(const AttnParams &p, uint32_t split, uint32_t h, uint32_t pos,
                                          const AttnShared &sm, uint32_t tid, AttnPrefetch &pf) {
    pf.pos = pos;
    uint32_t b0, b1;
    attn_split_range(p, split, pos, b0, b1);
    if (tid < (uint32_t)kAttnThreads) {
#pragma unroll
        for (uint32_t i = 0; i < (uint32_t)NBUF; ++i) {
            if (b1 > b0 + i) attn_issue_tile(p, h, b0 + i, i, sm.tiles, tid);
            cp_async_commit();
        }
        const float *cosr = p.rope_cos ? p.rope_cos + (size_t)pos * kHeadDim : nullptr;
        const float *sinr = p.rope_sin ? p.rope_sin + (size_t)pos * kHeadDim : nullptr;
        pf.cq = load_head_consts(p.q_norm, cosr, sinr, tid & 31u);
        pf.ck = load_head_consts(p.k_norm, cosr, sinr, tid & 31u);
    }
}

// Split `split` of KV head `h`: writes the partial (o, max, sum) of the G query heads of the group to
// p.scratch.  Threads 0 .. 127 (four warps) compute; every thread of the BAR_THREADS-wide barrier group
// must call it (the others only take part in the barriers), after attention_prefetch for the same
// position.  The page range streams through shared memory (16 KB K tile + 16 KB V tile per page,
// cp.async, double buffered, rows padded to 272 B).  Per
// 64-key tile every warp computes S = Q K^T for all keys with mma.m16n8k16 (bf16; the G query heads
// are the M rows) and the same online softmax in f32, then O += P V for its own 32 of the 128 output
// dims, with P carried as bf16 hi + lo so that the weights keep ~16 bits.  Warps only synchronise to
// hand tile buffers over.  Inputs written by other CTAs of a running kernel are read with ld.cg.
template <int BAR_ID, int BAR_THREADS, int NBUF = 2>
__device__ inline void attention_partial(const AttnParams &p, uint32_t split, uint32_t h, uint32_t pos,
                                         const AttnShared &sm, uint32_t tid, const AttnPrefetch &pf) {
    const uint32_t lane = tid & 31u, warp = tid >> 5, G = p.gqa;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const bool worker = tid < (uint32_t)kAttnThreads;
    const uint32_t seq_len = pos + 1u;
    uint32_t b0, b1;
    attn_split_range(p, split, pos, b0, b1);
    const uint32_t new_block = pos / kPageTokens;
    const bool owner = new_block >= b0 && new_block < b1;
    const uint32_t ntiles = b1 - b0;
    uint8_t *tiles = sm.tiles;

    // Norm + RoPE: one warp per head (the G query heads, then the new key row on the owner split).
    // All rows a warp needs are requested before the first is used: the owner split's extra row must not
    // cost a second trip to memory, because the slowest CTA sets the kernel's duration.
    if (worker) {
        constexpr uint32_t kMaxHeadsPerWarp = (kMaxGqa + 1u + kAttnWarps - 1u) / kAttnWarps;
        uint32_t raw_lo[kMaxHeadsPerWarp], raw_hi[kMaxHeadsPerWarp];
        uint2 vv = make_uint2(0u, 0u);
#pragma unroll
        for (uint32_t i = 0; i < kMaxHeadsPerWarp; ++i) {
            const uint32_t hh = warp + i * kAttnWarps;
            const uint16_t *row = nullptr;
            if (hh < G) row = p.qkv + (size_t)(h * G + hh) * kHeadDim;
            else if (hh == G && owner) row = p.qkv + (size_t)(p.q_heads + h) * kHeadDim;
            raw_lo[i] = raw_hi[i] = 0u;
            if (row) load_head_row(row, lane, raw_lo[i], raw_hi[i]);
            if (hh == G && owner)
                vv = __ldcg(reinterpret_cast<const uint2 *>(p.qkv + (size_t)(p.q_heads + p.kv_heads + h) * kHeadDim +
                                                            4u * lane));
        }
#pragma unroll
        for (uint32_t i = 0; i < kMaxHeadsPerWarp; ++i) {
            const uint32_t hh = warp + i * kAttnWarps;
            if (hh < G) {
                head_norm_rope_regs(raw_lo[i], raw_hi[i], pf.cq, p.q_norm != nullptr, p.rope_cos != nullptr, p.eps, lane,
                                    sm.q_s[hh]);
            } else if (hh == G && owner) {
                head_norm_rope_regs(raw_lo[i], raw_hi[i], pf.ck, p.k_norm != nullptr, p.rope_cos != nullptr, p.eps, lane,
                                    sm.knew);
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
    // Q^T as the B operand (columns = heads of the group, zero columns above G), kept in registers:
    // lane (g, t) holds head g, dims kk*16 + {2t, 2t+1} and kk*16 + 8 + {2t, 2t+1}.
    uint32_t qb[8][2];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        qb[kk][0] = (worker && g < G) ? *reinterpret_cast<const uint32_t *>(&sm.q_s[g][kk * 16 + 2 * t]) : 0u;
        qb[kk][1] = (worker && g < G) ? *reinterpret_cast<const uint32_t *>(&sm.q_s[g][kk * 16 + 8 + 2 * t]) : 0u;
    }
    if (tid == 0 && p.trace) trace_max(&p.trace->compute);

    // Each warp owns 16 of a tile's 64 keys and runs its own online softmax over them; the four states
    // are merged once at the end.  Keys are the M rows and the group's heads the N columns of both
    // products, so no tensor-core work is spent on padding:
    //   S^T[key, head] = K[key, :] Q^T            8 mma per 16 keys
    //   O^T[dim, head] += V^T[dim, key] P^T       16 mma per 16 keys (P as bf16 hi + lo: ~16 bits)
    // Lane (g, t) holds, for heads 2t and 2t+1: scores of keys g and g+8, and output dims 16 mt + g,
    // 16 mt + g + 8 for mt = 0..7.
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[8][4];
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.0f;
    // ldmatrix row addresses: lanes 0-7 -> matrix 0 rows, 8-15 -> matrix 1, 16-23 -> matrix 2, 24-31 -> matrix 3
    const uint32_t lrow = lane & 7u, lmat = lane >> 3;
    const uint32_t k0 = warp * 16u;  // this warp's keys within a tile

    for (uint32_t tile = 0; tile < ntiles; ++tile) {
        // groups in flight: this tile's and the NBUF - 1 after it (one group is committed per iteration,
        // empty past the end, so the count is uniform)
        if (worker) cp_async_wait<NBUF - 1>();
        named_bar_sync(BAR_ID, BAR_THREADS);
        const uint32_t buf = tile % (uint32_t)NBUF;
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
        if (worker && k0 < valid) {  // a slab with no key in range would have no finite maximum
            float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                // matrices: (keys 0-7, dims 0-7), (keys 8-15, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15, dims 8-15)
                uint32_t ka[4];
                ldmatrix_x4(ka, kt + (k0 + (lmat & 1u) * 8u + lrow) * kTileRowBytes + (kk * 16u + (lmat >> 1) * 8u) * 2u);
                mma_m16n8k16_bf16(sc, ka[0], ka[1], ka[2], ka[3], qb[kk][0], qb[kk][1]);
            }
            // sc[0], sc[1]: key k0+g, heads 2t, 2t+1;  sc[2], sc[3]: key k0+g+8
            const bool va = k0 + g < valid, vb = k0 + g + 8u < valid;
            float e[4], factor[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float sa = va ? sc[j] * p.scale : -INFINITY, sb2 = vb ? sc[2 + j] * p.scale : -INFINITY;
                float tm = fmaxf(sa, sb2);
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 4));
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 8));
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 16));
                const float m_new = fmaxf(m_run[j], tm);  // finite: the slab holds a key in range
                factor[j] = m_run[j] == -INFINITY ? 0.0f : expf(m_run[j] - m_new);
                e[j] = expf(sa - m_new);
                e[2 + j] = expf(sb2 - m_new);
                float ts = e[j] + e[2 + j];
                ts += __shfl_xor_sync(0xffffffffu, ts, 4);
                ts += __shfl_xor_sync(0xffffffffu, ts, 8);
                ts += __shfl_xor_sync(0xffffffffu, ts, 16);
                l_run[j] = l_run[j] * factor[j] + ts;
                m_run[j] = m_new;
            }
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                o[mt][0] *= factor[0];
                o[mt][1] *= factor[1];
                o[mt][2] *= factor[0];
                o[mt][3] *= factor[1];
            }
            // P[key, heads 2t..] (the C layout) -> P^T as the B operand (lane: head g, keys 2t.. / 2t+8..)
            uint32_t ph[2], pl[2], bh[2], bl[2];
            split_bf16x2(e[0], e[1], ph[0], pl[0]);
            split_bf16x2(e[2], e[3], ph[1], pl[1]);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                bh[i] = movmatrix_trans(ph[i]);
                bl[i] = movmatrix_trans(pl[i]);
            }
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                // V^T as the A operand, transposed on load from the [key][dim] tile; matrices:
                // (keys 0-7, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15, dims 0-7), (keys 8-15, dims 8-15)
                uint32_t va4[4];
                ldmatrix_x4_trans(va4, vt + (k0 + (lmat >> 1) * 8u + lrow) * kTileRowBytes +
                                           (mt * 16u + (lmat & 1u) * 8u) * 2u);
                mma_m16n8k16_bf16(o[mt], va4[0], va4[1], va4[2], va4[3], bh[0], bh[1]);
                mma_m16n8k16_bf16(o[mt], va4[0], va4[1], va4[2], va4[3], bl[0], bl[1]);
            }
        }
        named_bar_sync(BAR_ID, BAR_THREADS);  // the buffer of this tile is free for tile + NBUF
        if (worker) {
            if (tile + (uint32_t)NBUF < ntiles) attn_issue_tile(p, h, b0 + tile + (uint32_t)NBUF, buf, tiles, tid);
            cp_async_commit();
        }
    }

    // ---- merge the four warps' states, publish this split's partial (o, max, sum) ----
    if (worker && g == 0) {
#pragma unroll
        for (int j = 0; j < 2; ++j)
            if (2u * t + j < G) {
                sm.ml_s[warp][2u * t + j][0] = m_run[j];
                sm.ml_s[warp][2u * t + j][1] = l_run[j];
            }
    }
    if (worker) cp_async_wait<0>();
    named_bar_sync(BAR_ID, BAR_THREADS);  // also: nobody reads the tiles any more
    float *o_s = reinterpret_cast<float *>(tiles);  // [kAttnWarps][G][kHeadDim] f32
    if (worker) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t head = 2u * t + j;
            if (head < G) {
                float mx = -INFINITY;
#pragma unroll
                for (int w = 0; w < kAttnWarps; ++w) mx = fmaxf(mx, sm.ml_s[w][head][0]);
                const float f = m_run[j] == -INFINITY ? 0.0f : expf(m_run[j] - mx);
                float *dst = o_s + ((size_t)warp * G + head) * kHeadDim;
#pragma unroll
                for (int mt = 0; mt < 8; ++mt) {
                    dst[mt * 16 + g] = o[mt][j] * f;
                    dst[mt * 16 + g + 8] = o[mt][2 + j] * f;
                }
            }
        }
    }
    named_bar_sync(BAR_ID, BAR_THREADS);
    const uint32_t stride = kHeadDim + 2u;
    float *mine = p.scratch + ((size_t)(h * p.splits + split) * G) * stride;
    if (worker) {
        for (uint32_t i = tid; i < G * kHeadDim; i += kAttnThreads) {
            const uint32_t head = i >> 7, d = i & 127u;
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < kAttnWarps; ++w) acc += o_s[((size_t)w * G + head) * kHeadDim + d];
            mine[head * stride + d] = acc;
        }
        if (tid < G) {
            float mx = -INFINITY, l = 0.0f;
#pragma unroll
            for (int w = 0; w < kAttnWarps; ++w) mx = fmaxf(mx, sm.ml_s[w][tid][0]);
#pragma unroll
            for (int w = 0; w < kAttnWarps; ++w) {
                const float mw = sm.ml_s[w][tid][0];
                l += mw == -INFINITY ? 0.0f : sm.ml_s[w][tid][1] * expf(mw - mx);
            }
            mine[tid * stride + kHeadDim] = mx;
            mine[tid * stride + kHeadDim + 1] = l;
        }
        __threadfence();
    }
    named_bar_sync(BAR_ID, BAR_THREADS);
}

// Merges the `splits` partials of KV head `h` into p.out: one warp per query head, lane s holding the
// statistics of split s, lane l accumulating output dims {2l, 2l+1, 64+2l, 65+2l} over the splits in
// ascending order.  Threads 0 .. 127 compute; no barrier, no shared memory (`wgt` is unused and kept
// for the callers' signature).
template <int BAR_ID, int BAR_THREADS>
__device__ inline void attention_merge(const AttnParams &p, uint32_t h, float *wgt, uint32_t tid) {
    (void)wgt;
    const uint32_t lane = tid & 31u, warp = tid >> 5, G = p.gqa;
    if (tid >= (uint32_t)kAttnThreads) return;
    const uint32_t stride = kHeadDim + 2u;
    const float *base = p.scratch + ((size_t)h * p.splits * G) * stride;
    for (uint32_t gg = warp; gg < G; gg += kAttnWarps) {
        const float ms = lane < p.splits ? __ldcg(&base[(lane * G + gg) * stride + kHeadDim]) : -INFINITY;
        const float ls = lane < p.splits ? __ldcg(&base[(lane * G + gg) * stride + kHeadDim + 1]) : 0.0f;
        const float mmax = warp_max(ms);
        const float w = ms == -INFINITY ? 0.0f : expf(ms - mmax);
        const float inv = 1.0f / warp_sum(w * ls);
        float2 a0 = make_float2(0.0f, 0.0f), a1 = make_float2(0.0f, 0.0f);
#pragma unroll 16
        for (uint32_t sp = 0; sp < p.splits; ++sp) {
            const float ws = __shfl_sync(0xffffffffu, w, sp);
            const float *row = base + (size_t)(sp * G + gg) * stride;  // 520-byte rows: 8-byte aligned
            const float2 v0 = __ldcg(reinterpret_cast<const float2 *>(row + 2u * lane));
            const float2 v1 = __ldcg(reinterpret_cast<const float2 *>(row + 64u + 2u * lane));
            a0.x = fmaf(ws, v0.x, a0.x);
            a0.y = fmaf(ws, v0.y, a0.y);
            a1.x = fmaf(ws, v1.x, a1.x);
            a1.y = fmaf(ws, v1.y, a1.y);
        }
        uint16_t *dst = p.out + (size_t)(h * G + gg) * kHeadDim;
        *reinterpret_cast<uint32_t *>(dst + 2u * lane) =
            (uint32_t)f32_to_bf16_bits(a0.x * inv) | ((uint32_t)f32_to_bf16_bits(a0.y * inv) << 16);
        *reinterpret_cast<uint32_t *>(dst + 64u + 2u * lane) =
            (uint32_t)f32_to_bf16_bits(a1.x * inv) | ((uint32_t)f32_to_bf16_bits(a1.y * inv) << 16);
    }
}

}  // namespace sb
