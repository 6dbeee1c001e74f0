// Persistent decode kernel for sm_100a: ONE launch per token, one CTA per SM.
//
// The token's operators (embedding row, then per layer qkv matvec -> attention partials -> attention
// merge -> o matvec -> up|gate matvec -> down matvec, then the read-out matvec and the greedy token)
// are a list in device memory.  Every CTA walks the list.  What this buys over one kernel per
// operator:
//   * the producer warp streams the CTA's share of EVERY weight matrix through the shared-memory
//     ring in list order and never waits for an operator boundary, so while the consumers wait for
//     the previous operator's result (or run the attention, which has no weights) the next
//     matrices are already on their way: HBM stays busy across operators;
//   * an operator boundary costs one completion counter in global memory (each CTA adds 1 when its
//     stores are done; consumers poll until all participants have) instead of a kernel launch, CTA
//     rasterisation and a cold ring (~3-5 us per operator, 183 operators per token for the 8B shape);
//   * CTAs are resident for the whole token, so nothing is cold-started.
// Cross-CTA data (activation vectors, attention partials) is always read with ld.cg: L1 is not
// coherent between SMs and the kernel never ends between operators.  Every wait is bounded and
// reports through the device error word.
#include "mega.cuh"

#include <algorithm>

#include "device_attention.cuh"

namespace sb {

namespace {

constexpr int kCW = 16;  // consumer warps
constexpr int kCT = kCW * 32;
constexpr int kProducerWarp = kCW;
constexpr int kEpilogueWarp = kCW + 1;
constexpr int kMegaThreads = (kCW + 2) * 32;
constexpr int kMaxRounds = 3;  // 8-element input chunks per consumer thread held in registers: K <= 12288
constexpr int kRedSlots = 4;
constexpr uint32_t kNoDep = 0xffffffffu;

struct MegaSmem {
    uint32_t ring, xs, xsum, red, wred, attn, bars, flags, total;
};

__host__ __device__ inline MegaSmem mega_layout(uint32_t num_stages, uint32_t stage_capacity, uint32_t max_columns) {
    MegaSmem L;
    uint32_t off = 0;
    L.ring = off;
    off += num_stages * stage_capacity;
    L.xs = off;
    off += max_columns * 2u;
    L.xsum = off;
    off += (max_columns / 64u) * 4u;
    off = (off + 127u) & ~127u;
    L.attn = off;
    off += kAttnSharedBytes;
    off = (off + 15u) & ~15u;
    L.red = off;
    off += kRedSlots * kCW * 16u * 4u;
    L.wred = off;
    off += 2u * kCW * 4u;
    L.bars = off;
    off += (8u + 8u + 2u * kRedSlots) * 8u;
    L.flags = off;
    off += 16u;
    L.total = off;
    return L;
}

__device__ inline unsigned long long ld_acquire_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// State every role needs.
struct Ctx {
    const MegaParams *p;
    uint8_t *ring;
    __half *xs;
    float *xsum, *red, *wred;
    uint64_t *full, *empty, *red_full, *red_empty;
    volatile uint32_t *abort_flag;
};

__device__ inline void fail_wait(const Ctx &c, uint32_t bit) {
    *c.abort_flag = 1;
    atomicOr(c.p->error_word, bit);
}

// Consumers: wait until every participant of operator `dep` has finished (the counters start at
// zero: the host clears them in stream order before each launch).
// Thread 0 of the consumer group polls; the named barrier publishes the result to the rest.
__device__ inline void wait_for_op(const Ctx &c, uint32_t dep, uint32_t tid) {
    if (dep == kNoDep) return;
    if (tid == 0) {
        const unsigned long long target = c.p->ops[dep].participants;  // counters are zeroed before every launch
        bool ok = false;
        for (uint32_t it = 0; it < (1u << 24); ++it) {
            if (ld_acquire_u64(&c.p->done[dep]) >= target) {
                ok = true;
                break;
            }
            if (*c.abort_flag) break;
            if (it > 32) __nanosleep(32);
        }
        if (!ok) fail_wait(c, kErrFlagTimeout);
    }
    named_bar_sync(1, kCT);
}

// All stores of this thread for operator `op` are done: make them visible, then count this CTA in.
// Call from every storing thread of the group; `leader` does the add after the group's barrier.
__device__ inline void signal_op_consumers(const Ctx &c, uint32_t op, uint32_t tid) {
    __threadfence();
    named_bar_sync(1, kCT);
    if (tid == 0) atomicAdd(&c.p->done[op], 1ull);
}

struct TileRange {
    uint32_t t0, t1;
};
__device__ inline TileRange my_tiles(const MegaOp &op) {
    const uint32_t units = op.row_tiles / op.unit_tiles;
    const uint32_t u0 = (uint32_t)(((uint64_t)blockIdx.x * units) / gridDim.x);
    const uint32_t u1 = (uint32_t)(((uint64_t)(blockIdx.x + 1) * units) / gridDim.x);
    return TileRange{u0 * op.unit_tiles, u1 * op.unit_tiles};
}

// ---------------------------------------------------------------------------------- consumer side

// Builds the f16 input vector of a matvec in shared memory (see qmv.cu for the arithmetic): optional
// RMS norm, exact power-of-two rescale into the f16 range, per-group sums for the bias term.
__device__ inline float build_input(const Ctx &c, const MegaOp &op, uint32_t tid, uint32_t lane, uint32_t warp) {
    const uint32_t columns = op.groups * 64u, chunks = columns / 8u;
    float f[kMaxRounds][8];
#pragma unroll
    for (int r = 0; r < kMaxRounds; ++r) {
        const uint32_t ch = tid + r * kCT;
        if (ch < chunks) {
            const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(op.x) + ch);
            const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                f[r][2 * i] = __uint_as_float(wv[i] << 16);
                f[r][2 * i + 1] = __uint_as_float(wv[i] & 0xffff0000u);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[r][i] = 0.0f;
        }
    }
    if (op.prologue == kProRmsNorm) {
        float sumsq = 0.0f;
#pragma unroll
        for (int r = 0; r < kMaxRounds; ++r)
#pragma unroll
            for (int i = 0; i < 8; ++i) sumsq += f[r][i] * f[r][i];
        sumsq = warp_sum(sumsq);
        if (lane == 0) c.wred[warp] = sumsq;
        named_bar_sync(1, kCT);
        sumsq = 0.0f;
#pragma unroll
        for (int i = 0; i < kCW; ++i) sumsq += c.wred[i];
        const float rms_inv = 1.0f / sqrtf(sumsq / (float)columns + c.p->eps);
        const float4 *nw = reinterpret_cast<const float4 *>(op.norm_weight);
#pragma unroll
        for (int r = 0; r < kMaxRounds; ++r) {
            const uint32_t ch = tid + r * kCT;
            if (ch < chunks) {
                const float4 n0 = nw[2 * ch], n1 = nw[2 * ch + 1];
                const float ns[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i)  // bf16(normalized) * bf16(scale), product rounded to bf16
                    f[r][i] = bf16_round(bf16_round(f[r][i] * rms_inv) * bf16_round(ns[i]));
            }
        }
    }
    float vmax = 0.0f;
#pragma unroll
    for (int r = 0; r < kMaxRounds; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) vmax = fmaxf(vmax, fabsf(f[r][i]));
    vmax = warp_max(vmax);
    if (lane == 0) c.wred[kCW + warp] = vmax;
    named_bar_sync(1, kCT);
    vmax = 0.0f;
#pragma unroll
    for (int i = 0; i < kCW; ++i) vmax = fmaxf(vmax, c.wred[kCW + i]);
    int shift = 14 - ((int)((__float_as_uint(vmax) >> 23) & 0xffu) - 127);
    shift = max(-100, min(100, shift));
    if (!(vmax > 0.0f) || !isfinite(vmax)) shift = 0;
    const float xscale = __uint_as_float((uint32_t)(shift + 127) << 23);
    const float xunscale = __uint_as_float((uint32_t)(127 - shift) << 23);
#pragma unroll
    for (int r = 0; r < kMaxRounds; ++r) {
        const uint32_t ch = tid + r * kCT;
        float s8 = 0.0f;
        __half hh[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            s8 += f[r][i];
            hh[i] = __float2half_rn(f[r][i] * xscale);
        }
        if (ch < chunks) reinterpret_cast<uint4 *>(c.xs)[ch] = *reinterpret_cast<uint4 *>(hh);
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) s8 += __shfl_xor_sync(0xffffffffu, s8, o);
        if (ch < chunks && (lane & 7u) == 0) c.xsum[ch >> 3] = s8;
    }
    named_bar_sync(1, kCT);
    return xunscale;
}

struct RingPos {
    uint32_t slot, phase;
};
struct RedPos {
    uint32_t rb, rphase;
};

template <int RPW, bool PRED>
__device__ inline void consume_gemv(const Ctx &c, const MegaOp &op, float xunscale, RingPos &rp, RedPos &rd,
                                    uint32_t lane, uint32_t warp) {
    const MegaParams &p = *c.p;
    const TileRange tr = my_tiles(op);
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint8_t *my_rec = c.ring + warp * kA4RecordBytes + lane * 16u;
    const uint8_t *my_planes = c.ring + warp * kA4RecordBytes + 512u + 4u * g;
    const __half *my_x = c.xs + warp * 64u + t * 16u;
    for (uint32_t tile = tr.t0; tile < tr.t1; ++tile) {
        float acc_s0 = 0.0f, acc_s1 = 0.0f, acc_b0 = 0.0f, acc_b1 = 0.0f;
        uint32_t kg0 = 0;
        for (uint32_t st = 0; st < op.stages_per_tile; ++st) {
            if (!mbar_wait_bounded(&c.full[rp.slot], rp.phase, c.abort_flag)) fail_wait(c, kErrMbarTimeout);
            const uint32_t soff = rp.slot * p.stage_capacity;
            uint4 wq[RPW];
            uint32_t sw[RPW], bw[RPW];
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                if (!PRED || warp + (uint32_t)kCW * i < op.stage_records) {
                    wq[i] = *reinterpret_cast<const uint4 *>(my_rec + soff + i * kCW * kA4RecordBytes);
                    sw[i] = *reinterpret_cast<const uint32_t *>(my_planes + soff + i * kCW * kA4RecordBytes);
                    bw[i] = *reinterpret_cast<const uint32_t *>(my_planes + soff + i * kCW * kA4RecordBytes + 32u);
                }
            }
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                if (!PRED || warp + (uint32_t)kCW * i < op.stage_records) {
                    const uint32_t kofs = (kg0 + (uint32_t)kCW * i) * 64u;
                    const uint4 *xp = reinterpret_cast<const uint4 *>(my_x + kofs);
                    const uint4 xa = xp[0], xb = xp[1];
                    const uint32_t ww[4] = {wq[i].x, wq[i].y, wq[i].z, wq[i].w};
                    const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t a[4];
                        dequant_a4_word<0>(ww[j], a);
                        mma_m16n8k16_f16(acc, a, xw[2 * j], xw[2 * j + 1]);
                    }
                    const float xs_g = c.xsum[kg0 + warp + (uint32_t)kCW * i];
                    acc_s0 = fmaf(__uint_as_float(sw[i] << 16), acc[0], acc_s0);
                    acc_s1 = fmaf(__uint_as_float(sw[i] & 0xffff0000u), acc[2], acc_s1);
                    acc_b0 = fmaf(__uint_as_float(bw[i] << 16), xs_g, acc_b0);
                    acc_b1 = fmaf(__uint_as_float(bw[i] & 0xffff0000u), xs_g, acc_b1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&c.empty[rp.slot]);
            kg0 += op.stage_records;
            if (++rp.slot == p.num_stages) {
                rp.slot = 0;
                rp.phase ^= 1u;
            }
        }
        if (!mbar_wait_bounded(&c.red_empty[rd.rb], rd.rphase, c.abort_flag)) fail_wait(c, kErrMbarTimeout);
        if (t == 0) {
            c.red[(rd.rb * kCW + warp) * 16u + g] = fmaf(acc_s0, xunscale, acc_b0);
            c.red[(rd.rb * kCW + warp) * 16u + g + 8u] = fmaf(acc_s1, xunscale, acc_b1);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&c.red_full[rd.rb]);
        if (++rd.rb == kRedSlots) {
            rd.rb = 0;
            rd.rphase ^= 1u;
        }
    }
}

__device__ inline void embed_row(const MegaParams &p, uint32_t tid) {
    const uint32_t token = p.state->token, rows = p.embed_rows, columns = p.embed_columns;
    const uint32_t groups = columns / 64u;
    for (uint32_t col = tid; col < columns; col += kCT) {
        if (token >= rows) {  // input_embedding_lookup.rs:64-68
            p.h[col] = 0;
            continue;
        }
        const uint32_t tile = token / 16u, r = token % 16u;
        const uint32_t g = r & 7u, hrow = r >> 3;
        const uint32_t kg = col / 64u, cc = col % 64u;
        const uint32_t t = cc / 16u, j = (cc % 16u) / 4u, r2 = (cc % 4u) / 2u, e = cc & 1u;
        const uint8_t *rec = p.embed + ((size_t)tile * groups + kg) * kA4RecordBytes;
        const uint32_t word = *reinterpret_cast<const uint32_t *>(rec + (g * 4u + t) * 16u + j * 4u);
        const uint32_t q = (word >> (4u * (4u * e + 2u * r2 + hrow))) & 15u;
        const uint16_t *planes = reinterpret_cast<const uint16_t *>(rec + 512u);
        const float scale = bf16_bits_to_f32(planes[2u * g + hrow]);
        const float bias = bf16_bits_to_f32(planes[16u + 2u * g + hrow]);
        p.h[col] = f32_to_bf16_bits(__fadd_rn(__fmul_rn(scale, (float)q), bias));
    }
}

// ---------------------------------------------------------------------------------- the kernel

__global__ void __launch_bounds__(kMegaThreads, 1) decode_token_kernel(const MegaParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const MegaSmem L = mega_layout(p.num_stages, p.stage_capacity, p.max_columns);
    Ctx c;
    c.p = &p;
    c.ring = smem + L.ring;
    c.xs = reinterpret_cast<__half *>(smem + L.xs);
    c.xsum = reinterpret_cast<float *>(smem + L.xsum);
    c.red = reinterpret_cast<float *>(smem + L.red);
    c.wred = reinterpret_cast<float *>(smem + L.wred);
    c.full = reinterpret_cast<uint64_t *>(smem + L.bars);
    c.empty = c.full + 8;
    c.red_full = c.empty + 8;
    c.red_empty = c.red_full + kRedSlots;
    c.abort_flag = reinterpret_cast<volatile uint32_t *>(smem + L.flags);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    if (tid == 0) {
        for (uint32_t s = 0; s < p.num_stages; ++s) {
            mbar_init(&c.full[s], 1);
            mbar_init(&c.empty[s], kCW);
        }
        for (uint32_t s = 0; s < kRedSlots; ++s) {
            mbar_init(&c.red_full[s], kCW);
            mbar_init(&c.red_empty[s], 1);
        }
        *c.abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == kProducerWarp) {
        // ---------------- producer: every matvec's share of weights, in list order, never waiting
        // for an operator boundary ----------------
        if (lane == 0) {
            uint32_t slot = 0, phase = 1;
            bool alive = true;
            for (uint32_t i = 0; i < p.num_ops && alive; ++i) {
                const MegaOp &op = p.ops[i];
                if (op.type != kOpGemv) continue;
                const TileRange tr = my_tiles(op);
                const uint32_t total_stages = (tr.t1 - tr.t0) * op.stages_per_tile;
                const uint32_t stage_bytes = op.stage_records * kA4RecordBytes;
                const uint8_t *src = op.w + (size_t)tr.t0 * op.groups * kA4RecordBytes;
                for (uint32_t s = 0; s < total_stages; ++s) {
                    if (!mbar_wait_bounded(&c.empty[slot], phase, c.abort_flag)) {
                        fail_wait(c, kErrMbarTimeout);
                        alive = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&c.full[slot], stage_bytes);
                    bulk_g2s(c.ring + (size_t)slot * p.stage_capacity, src, stage_bytes, &c.full[slot]);
                    src += stage_bytes;
                    if (++slot == p.num_stages) {
                        slot = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        return;
    }

    if (warp == kEpilogueWarp) {
        // ---------------- epilogue warp: reduction and output of finished row tiles; counts the CTA
        // in when its part of a matvec is stored ----------------
        uint32_t rb = 0, rphase = 0;
        for (uint32_t i = 0; i < p.num_ops; ++i) {
            const MegaOp &op = p.ops[i];
            if (op.type != kOpGemv) continue;
            const TileRange tr = my_tiles(op);
            float held = 0.0f, best = -INFINITY;
            uint32_t best_index = 0xffffffffu;
            for (uint32_t tile = tr.t0; tile < tr.t1; ++tile) {
                if (!mbar_wait_bounded(&c.red_full[rb], rphase, c.abort_flag)) fail_wait(c, kErrMbarTimeout);
                float v = 0.0f;
                if (lane < 16) {
#pragma unroll
                    for (int wv = 0; wv < kCW; ++wv) v += c.red[(rb * kCW + wv) * 16u + lane];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&c.red_empty[rb]);
                if (++rb == kRedSlots) {
                    rb = 0;
                    rphase ^= 1u;
                }
                if (lane < 16) {
                    const uint32_t row = tile_row0(tile, op.pair_halves, op.rows) + lane;
                    const bool valid = row < op.rows;
                    if (op.epilogue == kEpiStore) {
                        if (valid) op.y[row] = f32_to_bf16_bits(v);
                    } else if (op.epilogue == kEpiResidual) {
                        if (valid) {
                            const float r = bf16_bits_to_f32(__ldcg(&op.resid[row]));
                            op.y[row] = f32_to_bf16_bits(bf16_round(v) + r);
                        }
                    } else if (op.epilogue == kEpiSwiGlu) {
                        if ((tile & 1u) == 0) {
                            held = bf16_round(v);
                        } else {
                            const float gate = bf16_round(v);
                            const float activated = bf16_round(gate / (1.0f + expf(-1.0f * gate)));
                            const uint32_t orow = (tile >> 1) * 16u + lane;
                            if (orow < op.rows / 2u) op.y[orow] = f32_to_bf16_bits(held * activated);
                        }
                    } else {  // kEpiLogits
                        if (valid) {
                            const uint16_t hb = f32_to_bf16_bits(v);
                            op.y[row] = hb;
                            const float lv = bf16_bits_to_f32(hb);
                            const float key = isfinite(lv) ? lv : INFINITY;
                            if (key > best || (key == best && row < best_index)) {
                                best = key;
                                best_index = row;
                            }
                        }
                    }
                }
            }
            if (op.epilogue == kEpiLogits) {
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                    const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_index, o);
                    if (ov > best || (ov == best && oi < best_index)) {
                        best = ov;
                        best_index = oi;
                    }
                }
                if (lane == 0) {
                    p.partial_max[blockIdx.x] = best;
                    p.partial_index[blockIdx.x] = best_index;
                }
            }
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(&p.done[i], 1ull);
            if (lane == 0 && blockIdx.x == 0 && p.trace) trace_max(&p.trace[i].end);
        }
        return;
    }

    // ---------------- consumers ----------------
    const AttnShared ash = carve_attn_shared(smem + L.attn);
    const uint32_t pos = p.state->position;
    RingPos rp{0u, 0u};
    RedPos rd{0u, 1u};
    for (uint32_t i = 0; i < p.num_ops; ++i) {
        const MegaOp &op = p.ops[i];
        if (tid == 0 && blockIdx.x == 0 && p.trace) trace_min(&p.trace[i].start);
        wait_for_op(c, op.dep, tid);
        if (tid == 0 && blockIdx.x == 0 && p.trace) trace_min(&p.trace[i].ready);
        switch (op.type) {
            case kOpEmbed:
                if (blockIdx.x == 0) {
                    embed_row(p, tid);
                    signal_op_consumers(c, i, tid);
                }
                break;
            case kOpGemv: {
                const float xunscale = build_input(c, op, tid, lane, warp);
                if (tid == 0 && blockIdx.x == 0 && p.trace) trace_max(&p.trace[i].compute);
                if (op.pred) {
                    if (op.rpw == 1) consume_gemv<1, true>(c, op, xunscale, rp, rd, lane, warp);
                    else consume_gemv<2, true>(c, op, xunscale, rp, rd, lane, warp);
                } else {
                    if (op.rpw == 1) consume_gemv<1, false>(c, op, xunscale, rp, rd, lane, warp);
                    else consume_gemv<2, false>(c, op, xunscale, rp, rd, lane, warp);
                }
                break;
            }
            case kOpAttnPartial: {
                const uint32_t unit = blockIdx.x;
                if (unit < p.kv_heads * p.attn_splits) {
                    AttnParams a;
                    a.qkv = p.qkv;
                    a.out = p.attn;
                    a.keys = op.keys;
                    a.values = op.values;
                    a.block_table = p.block_table;
                    a.q_norm = op.q_norm;
                    a.k_norm = op.k_norm;
                    a.rope_cos = p.rope_cos;
                    a.rope_sin = p.rope_sin;
                    a.state = p.state;
                    a.eps = p.eps;
                    a.scale = p.attn_scale;
                    a.q_heads = p.q_heads;
                    a.kv_heads = p.kv_heads;
                    a.gqa = p.q_heads / p.kv_heads;
                    a.splits = p.attn_splits;
                    a.scratch = p.attn_scratch;
                    a.counters = nullptr;
                    a.trace = nullptr;
                    AttnPrefetch pf;
                    attention_prefetch(a, unit % p.attn_splits, unit / p.attn_splits, pos, ash, tid, pf);
                    attention_partial<1, kCT>(a, unit % p.attn_splits, unit / p.attn_splits, pos, ash, tid, pf);
                    if (tid == 0) atomicAdd(&p.done[i], 1ull);  // attention_partial ends with fence + barrier
                }
                break;
            }
            case kOpAttnMerge: {
                if (blockIdx.x < p.kv_heads) {
                    AttnParams a;
                    a.out = p.attn;
                    a.gqa = p.q_heads / p.kv_heads;
                    a.splits = p.attn_splits;
                    a.scratch = p.attn_scratch;
                    attention_merge<1, kCT>(a, blockIdx.x, reinterpret_cast<float *>(ash.tiles), tid);
                    signal_op_consumers(c, i, tid);
                }
                break;
            }
            case kOpFinalize:
                if (blockIdx.x == 0 && warp == 0) {
                    float best = -INFINITY;
                    uint32_t bi = 0xffffffffu;
                    for (uint32_t k = lane; k < gridDim.x; k += 32) {
                        const float v = __ldcg(&p.partial_max[k]);
                        const uint32_t ix = __ldcg(&p.partial_index[k]);
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
                    if (lane == 0) {
                        const uint32_t tok = isfinite(best) ? bi : 0xffffffffu;  // unified_sampling.rs:42-45
                        StepState *s = p.state;
                        s->next_token = tok;
                        if (p.generated && s->gen_cursor < s->gen_capacity) p.generated[s->gen_cursor++] = tok;
                        s->position += 1u;
                        s->token = tok;
                    }
                }
                break;
            case kOpIngestAdvance:
                if (blockIdx.x == 0 && tid == 0) {
                    StepState *s = p.state;
                    s->position += 1u;
                    s->token = p.pending[s->cursor];
                    s->cursor += 1u;
                }
                break;
            default:
                break;
        }
        if (op.type != kOpGemv && tid == 0 && blockIdx.x == 0 && p.trace) trace_max(&p.trace[i].end);
    }
}

}  // namespace

uint32_t mega_smem_bytes(uint32_t num_stages, uint32_t stage_capacity, uint32_t max_columns) {
    return mega_layout(num_stages, stage_capacity, max_columns).total;
}

stark_b200_status mega_launch(const MegaParams &p, uint32_t grid, uint32_t smem_bytes, cudaStream_t stream) {
    static SmemOptIn once;
    if (stark_b200_status s = ensure_dynamic_smem(decode_token_kernel, 227 * 1024, once)) return s;
    if (p.max_columns > (uint32_t)kMaxRounds * kCT * 8u) return STARK_B200_UNSUPPORTED;
    decode_token_kernel<<<grid, kMegaThreads, smem_bytes, stream>>>(p);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

}  // namespace sb
