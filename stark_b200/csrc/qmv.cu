// Fused-dequant quantized matvec for sm_100a.
//
// y = W x for an MLX-affine 4-bit group-64 matrix, batch 1.  The kernel is HBM-bound
// (0.5625 bytes per weight), so the design goal is one uninterrupted stream of weight bytes:
//   * weights are re-tiled once at load time into 576-byte records (see qmv.cuh) so that each CTA
//     owns one contiguous byte range;
//   * a producer warp moves that range through a shared-memory ring with 1-D bulk copies
//     (cp.async.bulk + mbarrier complete_tx), started BEFORE griddepcontrol.wait, so under
//     programmatic dependent launch the ring is already full when the previous kernel's output
//     (the input vector) becomes visible;
//   * eight consumer warps turn nibbles into exact f16 integers with lop3 + one f16 FMA per pair
//     and feed them to mma.sync.m16n8k16 (f16 x f16 -> f32).  The CUDA cores alone cannot keep up
//     with B200's ~26 B/clk/SM of HBM bandwidth at 4 bit (2 weights per byte, one FMA + one
//     conversion each); the tensor pipe does the multiply-accumulate so the ALU pipes only run the
//     extraction.  Products q*x are exact and the accumulation is f32, as in the reference;
//   * per group: acc += scale * sum(q x) and acc += bias * sum(x), which is algebraically the
//     reference's sum x (scale q + bias)
//     (crates/stark-engine/src/backends/cpu/kernel/matmul/kernel.rs:219-265);
//   * the input vector is converted to f16 after an exact power-of-two rescale by its maximum, so
//     the f16 range never clips it; bf16 inputs convert exactly.
#include "qmv.cuh"
#include "device_math.cuh"
#include "tunables.cuh"

#include <algorithm>
#include <cstdlib>
#include <new>

namespace sb {

namespace {

// Two CTA shapes, chosen per launch (CW = consumer warps; a producer warp and an epilogue warp come on top):
//   CW = 8:  320 threads at 80 registers, two CTAs per SM.  Both fill the register file, so the CTAs of the
//            next kernel of a programmatic launch chain become resident only when these exit.
//   CW = 16: 576 threads at 56 registers and about half the shared memory, ONE CTA per SM.  The next
//            kernel's CTA fits beside it, so everything a kernel does ahead of griddepcontrol.wait (barrier
//            set-up, norm weights, filling its weight ring) overlaps the kernel before it.
constexpr uint32_t kMaxColumns = 12288;  // a consumer thread keeps its chunks of the input row in registers
constexpr int kRedSlots = 4;  // depth of the partial-sum hand-off ring between consumers and the epilogue warp

struct QmvParams {
    const uint8_t *w;
    uint32_t rows;
    uint32_t row_tiles;
    uint32_t groups;           // K / 64
    uint32_t stage_records;    // records per ring stage (divides groups)
    uint32_t stages_per_tile;  // groups / stage_records
    uint32_t stage_capacity;   // bytes reserved per ring slot
    uint32_t num_stages;       // ring depth
    uint32_t pair_halves;
    uint32_t unit_tiles;  // 1, or 2 when an epilogue needs (up, gate) tile pairs
    uint32_t io_type;
    uint32_t prologue;
    uint32_t epilogue;
    const void *x;
    void *y;
    const float *norm_weight;
    const uint16_t *norm_weight_bf16;
    const void *staged;
    float eps;
    const void *resid;
    float *partial_max;
    uint32_t *partial_index;
    uint32_t *error_word;
    TraceSlot *trace;
    QmvExchange ex;
};

struct SmemLayout {
    uint32_t ring, xs, xlo, nws, xsum, xoff, red, wred, bars, flags, total;
};

__host__ __device__ inline SmemLayout smem_layout(uint32_t num_stages, uint32_t stage_capacity, uint32_t columns,
                                                  bool split, bool norm, uint32_t cw) {
    SmemLayout L;
    uint32_t off = 0;
    L.ring = off;
    off += num_stages * stage_capacity;
    L.xs = off;
    off += columns * 2u;
    L.xlo = off;
    off += split ? columns * 2u : 0u;
    L.nws = off;
    off += norm ? columns * 2u : 0u;
    L.xsum = off;
    off += (columns / 64u) * 4u;
    L.xoff = off;
    off += (columns / 64u) * 4u;
    off = (off + 15u) & ~15u;
    L.red = off;
    off += kRedSlots * cw * 16u * 4u;
    L.wred = off;
    off += 2u * cw * 4u;
    L.bars = off;
    off += (8u + 8u + 2u * kRedSlots) * 8u;  // full[8], empty[8], red_full[4], red_empty[4]
    L.flags = off;
    off += 16u;
    L.total = off;
    return L;
}

// One thread reports a failed bounded wait; every later wait in the CTA then returns at once.
__device__ inline void wait_failed(volatile uint32_t *abort_flag, uint32_t *error_word) {
    *abort_flag = 1;
    atomicOr(error_word, kErrMbarTimeout);
}

// The consumers' prologue: waits for the previous kernel, brings the input row into shared memory as
// exactly scaled f16 (plus the per-group sums the bias term needs) and returns the factor that undoes
// the scale.  ROUNDS = chunks of 8 elements a thread keeps in registers (K <= ROUNDS * 256 * CW): the
// code is straight-line per round, and a short instance matters because every launch runs it cold.
template <int CW, int ROUNDS, bool NORM, bool SPLIT, bool TPX, int FOLD>
__device__ __forceinline__ void stage_input(const QmvParams &p, uint32_t tid, uint32_t columns, __half *xs, __half *xlo,
                                            uint16_t *nws, float *xsum, float *xoff, float *wred, float &xunscale) {
    constexpr int kConsumerWarps = CW, kConsumerThreads = CW * 32;
    const uint32_t warp = tid >> 5, lane = tid & 31u;
    // Before the wait: everything that does not depend on the previous kernel.  The norm weights
    // are constants, so their bf16-rounded values (normalization.rs:157-161 rounds them before the
    // product) are staged in shared memory while the previous kernel is still running.
    const uint32_t chunks = columns / 8u;
    const bool f32_in = !NORM && p.io_type == STARK_B200_F32;
    if (NORM && p.norm_weight_bf16) {
        // Already rounded at load time: asynchronous copies, so that a CTA which starts late reaches its wait at
        // once and the weights arrive while the input row is on its way.
        for (uint32_t c = tid; c < chunks; c += kConsumerThreads)
            cp_async16(reinterpret_cast<uint4 *>(nws) + c, reinterpret_cast<const uint4 *>(p.norm_weight_bf16) + c);
        cp_async_commit();
    } else if (NORM) {
        const float4 *nw = reinterpret_cast<const float4 *>(p.norm_weight);
        for (uint32_t c = tid; c < chunks; c += kConsumerThreads) {
            const float4 n0 = nw[2 * c], n1 = nw[2 * c + 1];
            uint4 o;
            o.x = (uint32_t)f32_to_bf16_bits(n0.x) | ((uint32_t)f32_to_bf16_bits(n0.y) << 16);
            o.y = (uint32_t)f32_to_bf16_bits(n0.z) | ((uint32_t)f32_to_bf16_bits(n0.w) << 16);
            o.z = (uint32_t)f32_to_bf16_bits(n1.x) | ((uint32_t)f32_to_bf16_bits(n1.y) << 16);
            o.w = (uint32_t)f32_to_bf16_bits(n1.z) | ((uint32_t)f32_to_bf16_bits(n1.w) << 16);
            reinterpret_cast<uint4 *>(nws)[c] = o;
        }
    }
    pdl_wait();  // the input vector belongs to the previous kernel
    if (tid == 0 && p.trace) {
        trace_min(&p.trace->ready);
        trace_max(&p.trace->ready_last);
    }

    // One trip to global memory: this thread's chunks of the input row stay in registers for the
    // whole prologue (up to ROUNDS chunks of 8 elements; the launcher checks the width).
    float f[ROUNDS][8];
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {
        const uint32_t c = tid + r * kConsumerThreads;
        if (c < chunks) {
            if (f32_in) {
                const float4 *x4 = reinterpret_cast<const float4 *>(p.x);
                const float4 a = x4[2 * c], b = x4[2 * c + 1];
                f[r][0] = a.x, f[r][1] = a.y, f[r][2] = a.z, f[r][3] = a.w;
                f[r][4] = b.x, f[r][5] = b.y, f[r][6] = b.z, f[r][7] = b.w;
            } else {
                const uint4 v = reinterpret_cast<const uint4 *>(p.x)[c];
                const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    f[r][2 * i] = __uint_as_float(wv[i] << 16);
                    f[r][2 * i + 1] = __uint_as_float(wv[i] & 0xffff0000u);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[r][i] = 0.0f;
        }
    }
    if (NORM && TPX && p.ex.recv) {
        // Tensor-parallel consumer: h' = bf16(bf16(sum of the ranks' shares, rank order) + h) replaces
        // the row just loaded.  A share is there when its packet carries this exchange's ticket.  The
        // packets of two ranks are fetched per trip to memory.
        const uint32_t ticket = __ldcg(p.ex.tokens) * p.ex.ticket_mul + p.ex.ticket_add;
        const unsigned long long t0 = global_ns();
#pragma unroll
        for (int r = 0; r < ROUNDS; ++r) {
            const uint32_t c = tid + r * kConsumerThreads;
            if (c < chunks) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (uint32_t k = 0; k < p.ex.ranks; k += 2u) {
                    const bool two = k + 1u < p.ex.ranks;
                    const unsigned long long *s0 = p.ex.recv + (size_t)k * columns + 8u * c;
                    const unsigned long long *s1 = two ? s0 + columns : s0;
                    unsigned long long q0[8], q1[8];
                    uint32_t spins = 0;
                    for (;;) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];"
                                         : "=l"(q0[2 * i]), "=l"(q0[2 * i + 1])
                                         : "l"(s0 + 2 * i)
                                         : "memory");
                            asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];"
                                         : "=l"(q1[2 * i]), "=l"(q1[2 * i + 1])
                                         : "l"(s1 + 2 * i)
                                         : "memory");
                        }
                        bool all = true;
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            all = all && (uint32_t)(q0[i] >> 32) == ticket && (uint32_t)(q1[i] >> 32) == ticket;
                        if (all) break;
                        if (++spins > 8u) {
                            __nanosleep(64);
                            if (global_ns() - t0 > p.ex.wait_ns) {  // a rank is missing: give up
                                atomicOr(p.error_word, kErrPeerTimeout);
                                break;
                            }
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        acc[i] += __uint_as_float((uint32_t)q0[i]);
                        if (two) acc[i] += __uint_as_float((uint32_t)q1[i]);
                    }
                }
                uint32_t packed[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t s2 = f32x2_to_bf16x2(acc[2 * i], acc[2 * i + 1]);  // the projection's bf16 output
                    packed[i] = f32x2_to_bf16x2(__uint_as_float(s2 << 16) + f[r][2 * i],
                                                __uint_as_float(s2 & 0xffff0000u) + f[r][2 * i + 1]);
                    f[r][2 * i] = __uint_as_float(packed[i] << 16);
                    f[r][2 * i + 1] = __uint_as_float(packed[i] & 0xffff0000u);
                }
                if (blockIdx.x == 0)
                    reinterpret_cast<uint4 *>(p.ex.h_out)[c] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
        }
    }
    // One block-wide reduction gives both the sum of squares and the magnitude the scaled input can
    // reach: max |h * w| * rms_inv bounds the normalized values up to their two bf16 roundings.  Each
    // thread reads back only the norm weights it staged itself, so no barrier is needed before this.
    float sumsq = 0.0f, vmax = 0.0f;
    if (NORM) {
        cp_async_wait<0>();  // this thread's own copies of the norm weights (if any)
#pragma unroll
        for (int r = 0; r < ROUNDS; ++r) {
            const uint32_t c = tid + r * kConsumerThreads;
            if (c < chunks) {
                const uint4 nv = reinterpret_cast<const uint4 *>(nws)[c];
                const uint32_t nwv[4] = {nv.x, nv.y, nv.z, nv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float a = f[r][2 * i], b = f[r][2 * i + 1];
                    sumsq = fmaf(a, a, sumsq);
                    sumsq = fmaf(b, b, sumsq);
                    vmax = fmaxf(vmax, fabsf(a * __uint_as_float(nwv[i] << 16)));
                    vmax = fmaxf(vmax, fabsf(b * __uint_as_float(nwv[i] & 0xffff0000u)));
                }
            }
        }
        sumsq = warp_sum(sumsq);
    } else {
#pragma unroll
        for (int r = 0; r < ROUNDS; ++r)
#pragma unroll
            for (int i = 0; i < 8; ++i) vmax = fmaxf(vmax, fabsf(f[r][i]));
    }
    vmax = warp_max(vmax);
    if (lane == 0) {
        wred[warp] = sumsq;
        wred[kConsumerWarps + warp] = vmax;
    }
    named_bar_sync(1, kConsumerThreads);
    sumsq = 0.0f;
    vmax = 0.0f;
#pragma unroll
    for (int i = 0; i < kConsumerWarps; ++i) {
        sumsq += wred[i];
        vmax = fmaxf(vmax, wred[kConsumerWarps + i]);
    }
    if (NORM) {
        const float rms_inv = 1.0f / sqrtf(sumsq / (float)columns + p.eps);
        vmax *= rms_inv * 1.015625f;
#pragma unroll
        for (int r = 0; r < ROUNDS; ++r) {
            const uint32_t c = tid + r * kConsumerThreads;
            if (c < chunks) {
                const uint4 nv = reinterpret_cast<const uint4 *>(nws)[c];
                const uint32_t nwv[4] = {nv.x, nv.y, nv.z, nv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    // bf16(normalized) * bf16(scale), product rounded to bf16; the pair is rounded by one
                    // packed conversion (every CTA normalizes the whole row, so instruction count matters)
                    const uint32_t n2 = f32x2_to_bf16x2(f[r][2 * i] * rms_inv, f[r][2 * i + 1] * rms_inv);
                    const uint32_t p2 = f32x2_to_bf16x2(__uint_as_float(n2 << 16) * __uint_as_float(nwv[i] << 16),
                                                        __uint_as_float(n2 & 0xffff0000u) *
                                                            __uint_as_float(nwv[i] & 0xffff0000u));
                    f[r][2 * i] = __uint_as_float(p2 << 16);
                    f[r][2 * i + 1] = __uint_as_float(p2 & 0xffff0000u);
                }
            }
        }
    }
    // Exact power-of-two scale: the largest element lands in [2^14, 2^15).
    int shift = 14 - ((int)((__float_as_uint(vmax) >> 23) & 0xffu) - 127);
    shift = max(-100, min(100, shift));
    if (!(vmax > 0.0f) || !isfinite(vmax)) shift = 0;
    const float xscale = __uint_as_float((uint32_t)(shift + 127) << 23);
    xunscale = __uint_as_float((uint32_t)(127 - shift) << 23);

    // Scaled f16 values, per-group sums of the input (for the bias term) and, for FOLD, -64 * the
    // per-group sum of the f16 values the tensor core will see.  Pairs are converted by one packed
    // instruction.
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {
        const uint32_t c = tid + r * kConsumerThreads;
        float s8 = 0.0f, h8 = 0.0f;
        uint32_t hh[4], hl[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float a = f[r][2 * i], b = f[r][2 * i + 1];
            s8 += a;
            s8 += b;
            const float sa = a * xscale, sb2 = b * xscale;
            asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(hh[i]) : "f"(sb2), "f"(sa));
            if (SPLIT || FOLD == 1) {
                const float2 back = __half22float2(*reinterpret_cast<const __half2 *>(&hh[i]));
                h8 += back.x;
                if (SPLIT) {
                    const float la = sa - back.x, lb = sb2 - back.y;
                    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(hl[i]) : "f"(lb), "f"(la));
                    const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&hl[i]));
                    h8 += lo.x;
                    h8 += back.y;
                    h8 += lo.y;
                } else {
                    h8 += back.y;
                }
            }
        }
        if (c < chunks) {
            reinterpret_cast<uint4 *>(xs)[c] = make_uint4(hh[0], hh[1], hh[2], hh[3]);
            if (SPLIT) reinterpret_cast<uint4 *>(xlo)[c] = make_uint4(hl[0], hl[1], hl[2], hl[3]);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            s8 += __shfl_xor_sync(0xffffffffu, s8, o);
            if (SPLIT || FOLD == 1) h8 += __shfl_xor_sync(0xffffffffu, h8, o);
        }
        if (c < chunks && (lane & 7u) == 0) {
            xsum[c >> 3] = s8;
            // FOLD == 2 with a bf16 input: the scaled f16 values are the inputs times a power of two, so
            // their sum is the sum already formed
            if (FOLD) xoff[c >> 3] = (FOLD == 2 && !SPLIT) ? -64.0f * xscale * s8 : -64.0f * h8;
        }
    }
    named_bar_sync(1, kConsumerThreads);
    if (tid == 0 && p.trace) trace_max(&p.trace->compute);

}

// The prologue of a launch whose input row was staged by the kernel before it: scaled f16 values and per-group sums
// are copied as they are (16-byte asynchronous copies), the factor that undoes the scale is one load.
template <int CW>
__device__ __forceinline__ void stage_input_staged(const QmvParams &p, uint32_t tid, uint32_t columns, __half *xs,
                                                   float *xsum, float &xunscale) {
    constexpr int kConsumerThreads = CW * 32;
    pdl_wait();  // the staged row belongs to the previous kernel
    if (tid == 0 && p.trace) {
        trace_min(&p.trace->ready);
        trace_max(&p.trace->ready_last);
    }
    const uint8_t *src = static_cast<const uint8_t *>(p.staged);
    const uint32_t groups = columns / 64u;
    for (uint32_t c = tid; c < columns / 8u; c += kConsumerThreads) cp_async16(reinterpret_cast<uint4 *>(xs) + c, src + 16u * c);
    const uint8_t *sums = src + (size_t)columns * 2u;
    for (uint32_t c = tid; c < groups / 4u; c += kConsumerThreads) cp_async16(reinterpret_cast<uint4 *>(xsum) + c, sums + 16u * c);
    for (uint32_t g = (groups / 4u) * 4u + tid; g < groups; g += kConsumerThreads)
        xsum[g] = __ldcg(reinterpret_cast<const float *>(sums) + g);
    cp_async_commit();
    xunscale = __ldcg(reinterpret_cast<const float *>(sums + (size_t)groups * 4u));
    cp_async_wait<0>();
    named_bar_sync(1, kConsumerThreads);
    if (tid == 0 && p.trace) trace_max(&p.trace->compute);
}

// SPLIT: the input is f32 and is carried as two f16 terms (hi + lo) so that ~22 mantissa bits
//        survive; bf16 inputs need one term.
// RPW:   records per consumer warp per ring stage (stage = 8 * RPW records unless PRED).
// PRED:  the stage holds fewer than 8 * RPW records (group counts that are not a multiple of 8).
// TPX:   the kernel takes part in a tensor-parallel exchange (QmvExchange); kept out of the single-GPU
//        instances so that their code and register allocation stay as they are.
// FOLD:  0 = the tensor core sees the integer codes; 1, 2 = it sees codes plus an offset that is taken out of
//        the group sums afterwards (dequant_a4_word).
// CW:    consumer warps (8: two CTAs per SM, 16: one).
template <bool SPLIT, int RPW, bool PRED, int FOLD, bool TPX = false, int CW = 8>
__global__ void __maxnreg__(CW == 16 ? 56 : 80) qmv_a4_kernel(const QmvParams p) {
    constexpr int kConsumerWarps = CW, kConsumerThreads = CW * 32;
    constexpr int kProducerWarp = CW, kEpilogueWarp = CW + 1;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t columns = p.groups * 64u;
    const SmemLayout L = smem_layout(p.num_stages, p.stage_capacity, columns, SPLIT, p.prologue == kProRmsNorm, CW);
    uint8_t *ring = smem + L.ring;
    __half *xs = reinterpret_cast<__half *>(smem + L.xs);
    __half *xlo = reinterpret_cast<__half *>(smem + L.xlo);
    uint16_t *nws = reinterpret_cast<uint16_t *>(smem + L.nws);
    float *xsum = reinterpret_cast<float *>(smem + L.xsum);
    float *xoff = reinterpret_cast<float *>(smem + L.xoff);
    float *red = reinterpret_cast<float *>(smem + L.red);
    float *wred = reinterpret_cast<float *>(smem + L.wred);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.bars);
    uint64_t *empty = full + 8;
    uint64_t *red_full = empty + 8;
    uint64_t *red_empty = red_full + kRedSlots;
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + L.flags);

    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5, lane = tid & 31u;

    // This CTA's share: whole units (1 or 2 row tiles), contiguous in memory.
    const uint32_t units = p.row_tiles / p.unit_tiles;
    const uint32_t u0 = (uint32_t)(((uint64_t)blockIdx.x * units) / gridDim.x);
    const uint32_t u1 = (uint32_t)(((uint64_t)(blockIdx.x + 1) * units) / gridDim.x);
    const uint32_t t0 = u0 * p.unit_tiles, t1 = u1 * p.unit_tiles;

    if (tid == 0) {
        for (uint32_t s = 0; s < p.num_stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumerWarps);
        }
        for (uint32_t s = 0; s < kRedSlots; ++s) {
            mbar_init(&red_full[s], kConsumerWarps);
            mbar_init(&red_empty[s], 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    if (tid == 0 && p.trace) {
        trace_min(&p.trace->start);
        trace_max(&p.trace->start_last);
    }

    if (warp == kProducerWarp) {
        // ---------------- producer: stream this CTA's byte range through the ring ----------------
        // Weights do not depend on the previous kernel, so this starts before griddepcontrol.wait.
        if (lane == 0) {
            const uint32_t total_stages = (t1 - t0) * p.stages_per_tile;
            const uint32_t stage_bytes = p.stage_records * kA4RecordBytes;
            const uint8_t *src = p.w + (size_t)t0 * p.groups * kA4RecordBytes;
            uint32_t slot = 0, phase = 1;  // a fresh barrier passes a wait on parity 1
            for (uint32_t s = 0; s < total_stages; ++s) {
                if (!mbar_wait_bounded(&empty[slot], phase, abort_flag)) {
                    wait_failed(abort_flag, p.error_word);
                    break;
                }
                mbar_arrive_expect_tx(&full[slot], stage_bytes);
                bulk_g2s(ring + (size_t)slot * p.stage_capacity, src, stage_bytes, &full[slot]);
                src += stage_bytes;
                if (++slot == p.num_stages) {
                    slot = 0;
                    phase ^= 1u;
                }
            }
        }
        return;
    }

    if (warp == kEpilogueWarp) {
        pdl_wait();  // everything the epilogue reads or overwrites belongs to the previous kernel
        // ---------------- epilogue warp: cross-warp reduction and output of finished row tiles ----------
        uint32_t rb = 0, rphase = 0;
        float held = 0.0f;  // kEpiSwiGlu: the `up` value of the even tile
        const uint32_t push_ticket =
            TPX && p.epilogue == kEpiPush ? __ldcg(p.ex.tokens) * p.ex.ticket_mul + p.ex.ticket_add : 0u;
        float best = -INFINITY;
        uint32_t best_index = 0xffffffffu;
        for (uint32_t tile = t0; tile < t1; ++tile) {
            if (!mbar_wait_bounded(&red_full[rb], rphase, abort_flag)) wait_failed(abort_flag, p.error_word);
            float v = 0.0f;
            if (lane < 16) {
#pragma unroll
                for (int wv = 0; wv < kConsumerWarps; ++wv) v += red[(rb * kConsumerWarps + wv) * 16u + lane];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&red_empty[rb]);
            if (++rb == kRedSlots) {
                rb = 0;
                rphase ^= 1u;
            }
            if (lane < 16) {
                const uint32_t row = tile_row0(tile, p.pair_halves, p.rows) + lane;
                const bool valid = row < p.rows;
                if (p.epilogue == kEpiStore) {
                    if (valid) {
                        if (p.io_type == STARK_B200_F32)
                            reinterpret_cast<float *>(p.y)[row] = v;
                        else
                            reinterpret_cast<uint16_t *>(p.y)[row] = f32_to_bf16_bits(v);
                    }
                } else if (p.epilogue == kEpiResidual) {
                    if (valid) {
                        const float r = bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(p.resid)[row]);
                        reinterpret_cast<uint16_t *>(p.y)[row] = f32_to_bf16_bits(bf16_round(v) + r);
                    }
                } else if (p.epilogue == kEpiSwiGlu) {
                    if ((tile & 1u) == 0) {
                        held = bf16_round(v);
                    } else {
                        // gated_act_mul.rs:80-95: silu in f32 -> bf16, product of two bf16 -> bf16
                        const float gate = bf16_round(v);
                        const float activated = bf16_round(gate / (1.0f + expf(-1.0f * gate)));
                        const uint32_t orow = (tile >> 1) * 16u + lane;
                        if (orow < p.rows / 2u)
                            reinterpret_cast<uint16_t *>(p.y)[orow] = f32_to_bf16_bits(held * activated);
                    }
                } else if (p.epilogue == kEpiPartialF32) {
                    if (valid) reinterpret_cast<float *>(p.y)[row] = v;
                } else if (TPX && p.epilogue == kEpiPush) {
                    if (valid) {
                        const unsigned long long packet = ((unsigned long long)push_ticket << 32) | __float_as_uint(v);
                        for (uint32_t r = 0; r < p.ex.ranks; ++r)
                            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p.ex.push[r] + row), "l"(packet)
                                         : "memory");
                    }
                } else {  // kEpiLogits
                    if (valid) {
                        const uint16_t hb = f32_to_bf16_bits(v);
                        reinterpret_cast<uint16_t *>(p.y)[row] = hb;
                        const float lv = bf16_bits_to_f32(hb);
                        // a non-finite logit must surface: it sorts as the maximum so the host sees it
                        const float key = isfinite(lv) ? lv : INFINITY;
                        if (key > best || (key == best && row < best_index)) {
                            best = key;
                            best_index = row;
                        }
                    }
                }
            }
        }
        if (lane == 0 && p.trace) trace_max(&p.trace->end);
        if (p.epilogue == kEpiLogits) {
            // first index of the maximum over this CTA's rows (lanes >= 16 hold -inf)
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
        return;
    }

    // ---------------- consumers ----------------
    float xunscale;
    const bool norm = p.prologue == kProRmsNorm;
    // Two instances of the prologue: rows of up to 4096 values, and up to kMaxColumns.
    constexpr int kShortRounds = 4096 / (kConsumerThreads * 8), kLongRounds = (int)kMaxColumns / (kConsumerThreads * 8);
    if (p.prologue == kProStaged) {
        stage_input_staged<CW>(p, tid, columns, xs, xsum, xunscale);
    } else if (columns <= 4096u) {
        if (norm) stage_input<CW, kShortRounds, true, SPLIT, TPX, FOLD>(p, tid, columns, xs, xlo, nws, xsum, xoff, wred, xunscale);
        else stage_input<CW, kShortRounds, false, SPLIT, false, FOLD>(p, tid, columns, xs, xlo, nws, xsum, xoff, wred, xunscale);
    } else {
        if (norm) stage_input<CW, kLongRounds, true, SPLIT, TPX, FOLD>(p, tid, columns, xs, xlo, nws, xsum, xoff, wred, xunscale);
        else stage_input<CW, kLongRounds, false, SPLIT, false, FOLD>(p, tid, columns, xs, xlo, nws, xsum, xoff, wred, xunscale);
    }

    // Main loop: no block-wide barrier from here on.
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint8_t *my_rec = ring + warp * kA4RecordBytes + lane * 16u;
    const uint8_t *my_planes = ring + warp * kA4RecordBytes + 512u + 4u * g;
    const __half *my_x = xs + warp * 64u + t * 16u;
    const __half *my_xlo = xlo + warp * 64u + t * 16u;
    uint32_t slot = 0, phase = 0;
    uint32_t rb = 0, rphase = 1;
    for (uint32_t tile = t0; tile < t1; ++tile) {
        float acc_s0 = 0.0f, acc_s1 = 0.0f, acc_b0 = 0.0f, acc_b1 = 0.0f;
        uint32_t kg0 = 0;  // first group of the current stage
        for (uint32_t st = 0; st < p.stages_per_tile; ++st) {
            if (!mbar_wait_bounded(&full[slot], phase, abort_flag)) wait_failed(abort_flag, p.error_word);
            const uint32_t soff = slot * p.stage_capacity;
            // All of this warp's records of the stage are loaded first; the records are independent,
            // so several tensor-pipe chains are in flight per warp.
            uint4 wq[RPW];
            uint32_t sw[RPW], bw[RPW];
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                if (!PRED || warp + (uint32_t)CW * i < p.stage_records) {
                    wq[i] = *reinterpret_cast<const uint4 *>(my_rec + soff + i * CW * kA4RecordBytes);
                    sw[i] = *reinterpret_cast<const uint32_t *>(my_planes + soff + i * CW * kA4RecordBytes);
                    bw[i] = *reinterpret_cast<const uint32_t *>(my_planes + soff + i * CW * kA4RecordBytes + 32u);
                }
            }
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                if (!PRED || warp + (uint32_t)CW * i < p.stage_records) {
                    const uint32_t kofs = (kg0 + (uint32_t)CW * i) * 64u;  // my_x already includes warp * 64
                    const uint4 *xp = reinterpret_cast<const uint4 *>(my_x + kofs);
                    const uint4 xa = xp[0], xb = xp[1];
                    const uint32_t ww[4] = {wq[i].x, wq[i].y, wq[i].z, wq[i].w};
                    const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t a[4];
                        dequant_a4_word<FOLD>(ww[j], a);
                        mma_m16n8k16_f16(c, a, xw[2 * j], xw[2 * j + 1]);
                        if (SPLIT) {
                            const uint2 lw = *reinterpret_cast<const uint2 *>(my_xlo + kofs + 4 * j);
                            mma_m16n8k16_f16(c, a, lw.x, lw.y);
                        }
                    }
                    const uint32_t kg = kg0 + warp + (uint32_t)CW * i;
                    const float xs_g = xsum[kg];
                    float d0 = c[0], d1 = c[2];
                    if (FOLD == 1) {
                        const float xo = xoff[kg];      // -64 * sum of the f16 inputs of this group
                        d0 = fmaf(16.0f, xo, d0);       // c - 1024 sum
                        d1 = fmaf(d1, 0.0625f, xo);     // c / 16 - 64 sum
                    } else if (FOLD == 2) {
                        const float xo = xoff[kg];
                        d0 += xo;                       // c - 64 sum, both row halves
                        d1 += xo;
                    }
                    acc_s0 = fmaf(__uint_as_float(sw[i] << 16), d0, acc_s0);
                    acc_s1 = fmaf(__uint_as_float(sw[i] & 0xffff0000u), d1, acc_s1);
                    acc_b0 = fmaf(__uint_as_float(bw[i] << 16), xs_g, acc_b0);
                    acc_b1 = fmaf(__uint_as_float(bw[i] & 0xffff0000u), xs_g, acc_b1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
            kg0 += p.stage_records;
            if (++slot == p.num_stages) {
                slot = 0;
                phase ^= 1u;
            }
        }
        // Hand the 16 partial sums of this warp to the epilogue warp.
        if (!mbar_wait_bounded(&red_empty[rb], rphase, abort_flag)) wait_failed(abort_flag, p.error_word);
        if (t == 0) {
            red[(rb * kConsumerWarps + warp) * 16u + g] = fmaf(acc_s0, xunscale, acc_b0);
            red[(rb * kConsumerWarps + warp) * 16u + g + 8u] = fmaf(acc_s1, xunscale, acc_b1);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&red_full[rb]);
        if (++rb == kRedSlots) {
            rb = 0;
            rphase ^= 1u;
        }
    }
}

// ------------------------------------------------------------------------------------------ re-tiling

__global__ void retile_a4_codes_kernel(const uint8_t *__restrict__ codes, uint8_t *__restrict__ out, uint32_t rows,
                                       uint32_t columns, uint32_t row_tiles, uint32_t pair_halves) {
    const uint32_t groups = columns / 64u;
    const uint64_t total = (uint64_t)row_tiles * groups * 128u;  // words
    const size_t row_bytes = columns / 2u;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total;
         i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t j = (uint32_t)(i & 3u), lane = (uint32_t)((i >> 2) & 31u);
        const uint64_t recno = i >> 7;
        const uint32_t kg = (uint32_t)(recno % groups), tile = (uint32_t)(recno / groups);
        const uint32_t g = lane >> 2, t = lane & 3u;
        const uint32_t row0 = tile_row0(tile, pair_halves, rows);
        uint32_t word = 0;
#pragma unroll
        for (uint32_t pnib = 0; pnib < 8; ++pnib) {
            const uint32_t e = pnib >> 2, r = (pnib >> 1) & 1u, h = pnib & 1u;
            const uint32_t row = row0 + g + 8u * h;
            const uint32_t col = 64u * kg + 16u * t + 4u * j + 2u * r + e;
            uint32_t q = 0;
            // packed_code for bits = 4: column 2j is the low nibble of byte j (reference.rs:91-104)
            if (row < rows) q = (codes[(size_t)row * row_bytes + (col >> 1)] >> (4u * (col & 1u))) & 15u;
            word |= q << (4u * pnib);
        }
        *reinterpret_cast<uint32_t *>(out + recno * kA4RecordBytes + lane * 16u + j * 4u) = word;
    }
}

__global__ void retile_a4_planes_kernel(const uint16_t *__restrict__ scales, const uint16_t *__restrict__ biases,
                                        uint8_t *__restrict__ out, uint32_t rows, uint32_t columns,
                                        uint32_t row_tiles, uint32_t pair_halves, uint32_t scale_layout,
                                        uint32_t plane_pitch) {
    const uint32_t groups = columns / 64u;
    const uint64_t total = (uint64_t)row_tiles * groups * 16u;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total;
         i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t idx = (uint32_t)(i & 15u);
        const uint64_t recno = i >> 4;
        const uint32_t kg = (uint32_t)(recno % groups), tile = (uint32_t)(recno / groups);
        const uint32_t row = tile_row0(tile, pair_halves, rows) + (idx >> 1) + 8u * (idx & 1u);
        uint16_t sv = 0, bv = 0;
        if (row < rows) {
            const size_t at = scale_layout == 0 ? (size_t)row * groups + kg : (size_t)kg * plane_pitch + row;
            sv = scales[at];
            bv = biases[at];
        }
        uint16_t *rec = reinterpret_cast<uint16_t *>(out + recno * kA4RecordBytes + 512u);
        rec[idx] = sv;
        rec[16u + idx] = bv;
    }
}

// Integer codes back out of the records through dequant_a4_word (the matvec's own extraction).
__global__ void unpack_a4_kernel(const uint8_t *__restrict__ data, uint8_t *__restrict__ dst, uint32_t rows,
                                 uint32_t columns, uint32_t row_tiles, uint32_t pair_halves) {
    const uint32_t groups = columns / 64u;
    const uint64_t total = (uint64_t)row_tiles * groups * 128u;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total;
         i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t j = (uint32_t)(i & 3u), lane = (uint32_t)((i >> 2) & 31u);
        const uint64_t recno = i >> 7;
        const uint32_t kg = (uint32_t)(recno % groups), tile = (uint32_t)(recno / groups);
        const uint32_t g = lane >> 2, t = lane & 3u;
        const uint32_t row0 = tile_row0(tile, pair_halves, rows);
        const uint32_t word = *reinterpret_cast<const uint32_t *>(data + recno * kA4RecordBytes + lane * 16u + j * 4u);
        uint32_t a[4];
        dequant_a4_word<0>(word, a);
        // a[0]: row g, k-pair r=0; a[1]: row g+8, r=0; a[2]: row g, r=1; a[3]: row g+8, r=1
#pragma unroll
        for (int reg = 0; reg < 4; ++reg) {
            const uint32_t h = reg & 1u, r = (uint32_t)reg >> 1;
            const __half2 v = *reinterpret_cast<const __half2 *>(&a[reg]);
            const float lo = __low2float(v), hi = __high2float(v);
            const uint32_t row = row0 + g + 8u * h;
            const uint32_t col = 64u * kg + 16u * t + 4u * j + 2u * r;
            if (row < rows) {
                dst[(size_t)row * columns + col] = (uint8_t)(int)lo;
                dst[(size_t)row * columns + col + 1u] = (uint8_t)(int)hi;
            }
        }
    }
}

// Records per ring stage: a multiple of the consumer warps when the group count allows it (no per-record
// predicates), otherwise the largest divisor of the group count that fits.
void pick_stage(uint32_t groups, uint32_t cw, uint32_t *records, uint32_t *rpw, bool *pred) {
    for (uint32_t r : {32u, 16u, 8u}) {
        if (r >= cw && groups % r == 0) {
            *records = r;
            *rpw = r / cw;
            *pred = false;
            return;
        }
    }
    uint32_t best = 1;
    for (uint32_t r = std::min(groups, kMaxStageRecords); r >= 1; --r)
        if (groups % r == 0) {
            best = r;
            break;
        }
    *records = best;
    *rpw = (best + cw - 1u) / cw;
    if (*rpw == 3) *rpw = 4;
    *pred = true;
}

int sm_count_cached() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

using KernelFn = void (*)(const QmvParams);
struct KernelChoice {
    KernelFn fn;
    SmemOptIn *opted;
};

// One table per CTA shape.  FOLD and the tensor-parallel hooks only exist for bf16 I/O (SPLIT == false).
template <int CW>
KernelChoice pick_kernel(bool split, int fold, bool pred, uint32_t rpw, bool tpx) {
    const uint32_t ri = rpw == 1 ? 0u : (rpw == 2 ? 1u : 2u);
    const uint32_t pi = pred ? 1u : 0u;
#define SB_QMV_RPW(SP, PR, FO, TP) \
    { qmv_a4_kernel<SP, 1, PR, FO, TP, CW>, qmv_a4_kernel<SP, 2, PR, FO, TP, CW>, qmv_a4_kernel<SP, (CW == 16 ? 2 : 4), PR, FO, TP, CW> }
#define SB_QMV_PRED(SP, FO, TP) { SB_QMV_RPW(SP, false, FO, TP), SB_QMV_RPW(SP, true, FO, TP) }
    static const KernelFn plain[3][2][3] = {SB_QMV_PRED(false, 0, false), SB_QMV_PRED(false, 1, false),
                                            SB_QMV_PRED(false, 2, false)};
    static const KernelFn splitk[2][3] = SB_QMV_PRED(true, 0, false);
    static const KernelFn tpxk[3][2][3] = {SB_QMV_PRED(false, 0, true), SB_QMV_PRED(false, 1, true),
                                           SB_QMV_PRED(false, 2, true)};
#undef SB_QMV_PRED
#undef SB_QMV_RPW
    static SmemOptIn once_plain[3][2][3], once_split[2][3], once_tpx[3][2][3];
    if (split) return {splitk[pi][ri], &once_split[pi][ri]};
    if (tpx) return {tpxk[fold][pi][ri], &once_tpx[fold][pi][ri]};
    return {plain[fold][pi][ri], &once_plain[fold][pi][ri]};
}

}  // namespace

void qmv_pick_stage(uint32_t groups, uint32_t *records, uint32_t *rpw, bool *pred) {
    pick_stage(groups, 8u, records, rpw, pred);
}

stark_b200_status qmv_launch(const QmvArgs &a, cudaStream_t stream) {
    const QMatrix *m = a.matrix;
    if (!m || !a.x || !a.y || a.m != 1) return STARK_B200_INVALID_ARGUMENT;
    if (m->format != kFmtAffine4) return STARK_B200_UNSUPPORTED;
    if (a.epilogue == kEpiSwiGlu && !m->pair_halves) return STARK_B200_INVALID_ARGUMENT;
    if (a.io_type == STARK_B200_F32 && (a.prologue != kProPlain || a.epilogue != kEpiStore))
        return STARK_B200_UNSUPPORTED;
    if (m->columns > kMaxColumns) return STARK_B200_UNSUPPORTED;

    const bool split = a.io_type == STARK_B200_F32;
    const Tunables &tune = tunables();
    const uint32_t cw = tune.qmv_consumer_warps;
    QmvParams p{};
    p.w = m->data;
    p.rows = m->rows;
    p.row_tiles = m->row_tiles;
    p.groups = m->groups;
    uint32_t rpw = 1;
    bool pred = false;
    pick_stage(m->groups, cw, &p.stage_records, &rpw, &pred);
    p.stages_per_tile = m->groups / p.stage_records;
    p.stage_capacity = (p.stage_records * kA4RecordBytes + 127u) & ~127u;
    p.pair_halves = m->pair_halves;
    p.unit_tiles = a.epilogue == kEpiSwiGlu ? 2u : 1u;
    p.io_type = a.io_type;
    p.prologue = a.prologue;
    p.epilogue = a.epilogue;
    p.x = a.x;
    p.y = a.y;
    p.norm_weight = a.norm_weight;
    p.norm_weight_bf16 = a.norm_weight_bf16;
    p.staged = a.staged;
    p.eps = a.eps;
    p.resid = a.resid;
    p.partial_max = a.partial_max;
    p.partial_index = a.partial_index;
    p.error_word = a.error_word;
    p.trace = a.trace;
    if (a.exchange) p.ex = *a.exchange;
    if ((a.epilogue == kEpiPush) != (p.ex.ranks != 0 && p.ex.push[0] != nullptr)) return STARK_B200_INVALID_ARGUMENT;
    if (p.ex.recv && a.prologue != kProRmsNorm) return STARK_B200_INVALID_ARGUMENT;

    if (a.prologue == kProStaged && (!a.staged || split || (reinterpret_cast<uintptr_t>(a.staged) & 15u)))
        return STARK_B200_INVALID_ARGUMENT;
    // a staged row carries no offset sums: the plain extraction only
    const int fold = (split || a.prologue == kProStaged) ? 0 : (int)tune.qmv_fold;
    // Ring depth: what fits the per-CTA budget.  With two CTAs per SM the register file is full; with one,
    // the CTA of the next kernel of a programmatic launch chain sits beside it and fills its own ring
    // while this one drains.
    const uint32_t ctas_per_sm = tune.qmv_ctas_per_sm ? tune.qmv_ctas_per_sm : (cw == 16u ? 1u : 2u);
    // 56 KB: two CTAs leave room for a three-buffer attention CTA that fetches its cache tiles meanwhile (the qkv
    // projection before attention, the o projection that starts beside it); 104 KB where nothing of the kind
    // follows, which buys a deeper ring (measured on the read-out: 61 -> 57 us).
    const uint32_t own_budget = cw == 16u ? 112u : (a.roomy ? tune.qmv_roomy_kb : 56u);
    const uint32_t budget = (tune.qmv_smem_kb ? tune.qmv_smem_kb : own_budget) * 1024u;
    uint32_t stages = 8;
    const bool norm = a.prologue == kProRmsNorm;
    while (stages > 2 && smem_layout(stages, p.stage_capacity, m->columns, split, norm, cw).total > budget) --stages;
    p.num_stages = stages;
    const uint32_t smem = smem_layout(stages, p.stage_capacity, m->columns, split, norm, cw).total;
    if (smem > 220u * 1024u) return STARK_B200_UNSUPPORTED;

    const uint32_t units = p.row_tiles / p.unit_tiles;
    const uint32_t grid = std::max(1u, std::min(units, (uint32_t)sm_count_cached() * ctas_per_sm));
    if (a.out_grid) *a.out_grid = grid;

    const bool tpx = p.ex.ranks != 0;
    if (tpx && split) return STARK_B200_UNSUPPORTED;
    const KernelChoice k = cw == 16u ? pick_kernel<16>(split, fold, pred, rpw, tpx) : pick_kernel<8>(split, fold, pred, rpw, tpx);
    if (stark_b200_status s = ensure_dynamic_smem(k.fn, 220 * 1024, *k.opted)) return s;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((cw + 2u) * 32u);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 1 : 0;
    SB_CUDA(cudaLaunchKernelEx(&cfg, k.fn, p));
    return STARK_B200_OK;
}

stark_b200_status qmatrix_from_affine_device(const uint8_t *codes, const void *scales, const void *biases,
                                             const stark_b200_affine_desc &d, cudaStream_t stream, QMatrix **out) {
    if (d.bits != 4 || d.group != 64 || d.plane_kind != STARK_B200_PLANE_BF16) return STARK_B200_UNSUPPORTED;
    if (d.rows == 0 || d.columns == 0 || d.columns % 64u != 0) return STARK_B200_INVALID_ARGUMENT;
    if (d.pair_halves && (d.rows % 32u != 0)) return STARK_B200_INVALID_ARGUMENT;
    if (d.scale_layout == 1 && d.plane_pitch < d.rows) return STARK_B200_INVALID_ARGUMENT;
    QMatrix *m = new (std::nothrow) QMatrix();
    if (!m) return STARK_B200_OUT_OF_MEMORY;
    m->format = kFmtAffine4;
    m->rows = d.rows;
    m->columns = d.columns;
    m->row_tiles = (d.rows + 15u) / 16u;
    m->groups = d.columns / 64u;
    m->pair_halves = d.pair_halves;
    m->record_bytes = kA4RecordBytes;
    m->bytes = (size_t)m->row_tiles * m->groups * kA4RecordBytes;
    cudaGetDevice(&m->device);
    cudaError_t e = cudaMalloc(&m->data, m->bytes);
    if (e != cudaSuccess) {
        delete m;
        return cuda_status(e);
    }
    const uint64_t words = (uint64_t)m->row_tiles * m->groups * 128u;
    const uint32_t blocks = (uint32_t)std::min<uint64_t>((words + 255u) / 256u, 148u * 16u);
    retile_a4_codes_kernel<<<blocks, 256, 0, stream>>>(codes, m->data, m->rows, m->columns, m->row_tiles,
                                                       m->pair_halves);
    const uint64_t planes = (uint64_t)m->row_tiles * m->groups * 16u;
    const uint32_t pblocks = (uint32_t)std::min<uint64_t>((planes + 255u) / 256u, 148u * 16u);
    retile_a4_planes_kernel<<<pblocks, 256, 0, stream>>>(
        reinterpret_cast<const uint16_t *>(scales), reinterpret_cast<const uint16_t *>(biases), m->data, m->rows,
        m->columns, m->row_tiles, m->pair_halves, d.scale_layout, d.plane_pitch);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        cudaFree(m->data);
        delete m;
        return cuda_status(e);
    }
    *out = m;
    return STARK_B200_OK;
}

stark_b200_status qmatrix_unpack_codes_device(const QMatrix *m, uint8_t *dst, cudaStream_t stream) {
    if (m->format != kFmtAffine4) return STARK_B200_UNSUPPORTED;
    const uint64_t words = (uint64_t)m->row_tiles * m->groups * 128u;
    const uint32_t blocks = (uint32_t)std::min<uint64_t>((words + 255u) / 256u, 148u * 16u);
    unpack_a4_kernel<<<blocks, 256, 0, stream>>>(m->data, dst, m->rows, m->columns, m->row_tiles, m->pair_halves);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

void qmatrix_free(QMatrix *m) {
    if (!m) return;
    if (m->data) cudaFree(m->data);
    delete m;
}

}  // namespace sb
