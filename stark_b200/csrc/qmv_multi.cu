// y[r, :] = W x[r, :] for a handful of input rows (1..8) over a 4-bit affine group-64 matrix: the matrix streams
// from HBM ONCE for all rows.  This is the verify pass of a speculative round (k proposals + the pending token =
// k + 1 rows through the target; the reference runs it as a GEMV with an input-row tile of 2-4,
// crates/stark-engine/src/backends/metal/kernel/matmul/gemv/gemv.metal:59-63), where the work is the weight
// stream exactly as in one-token decoding, not a dense contraction.
//
// Same machinery as the one-row kernel (qmv.cu): one producer thread streams the CTA's contiguous share of the
// re-tiled records through a shared-memory ring with bulk copies, consumer warps multiply record by record on
// mma.sync.m16n8k16, an epilogue warp sums the warps' partials per 16-row tile and writes.  What differs:
//   * the eight columns of the tensor-core tile are eight different input rows (the one-row kernel feeds the same
//     row to all eight), so the rows cost no extra tensor-core or memory work;
//   * operands are bf16, the activations' own type: codes enter as the exact bf16 integers 128 + q (one lop3 per
//     pair), inputs as they are, products are exact in the f32 accumulator, and 128 * sum(x) leaves with the bias
//     term: acc += scale * c + (bias - 128 scale) * sum_group(x).  No input scaling is needed;
//   * ONE CTA of 16 consumer warps per SM: the rows of the input live in shared memory (R * K * 2 bytes).
// Prologues: plain (bf16 rows copied as they are) or RMS norm of each row with the reference's rounding points
// (normalization.rs:13-191); epilogues: store, residual add, SwiGLU over pair-ordered [up; gate] tiles.
// Every wait is bounded and reports through the device error word.
#include <algorithm>

#include "device_math.cuh"
#include "prefill.cuh"
#include "qmv.cuh"

namespace sb {

namespace {

constexpr int kCW = 16;
constexpr int kConsumerThreads = kCW * 32;
constexpr int kProducerWarp = kCW, kEpilogueWarp = kCW + 1;
constexpr int kThreads = (kCW + 2) * 32;
constexpr uint32_t kRed = 2;            // depth of the hand-off ring between consumers and the epilogue warp
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kRowPad = 16;        // bytes: rows 16 B apart modulo 128 B, so the fragment loads are conflict-free
constexpr uint32_t kNormMaxColumns = 4096;  // one 8-element chunk per consumer thread and row

struct MultiParams {
    const uint8_t *w;
    uint32_t rows, row_tiles, groups, stage_records, stages_per_tile, stage_capacity, num_stages, pair_halves, unit_tiles;
    uint32_t m;                // input rows
    const uint16_t *x;
    uint32_t x_stride;
    uint16_t *y;
    uint32_t y_stride;
    const float *norm_weight;  // non-null: RMS norm prologue
    float eps;
    uint32_t epilogue;
    uint32_t *error_word;
};

struct MultiSmem {
    uint32_t ring, xs, xsum, red, wred, bars, flags, total, x_row_bytes;
};

__host__ __device__ inline MultiSmem multi_layout(uint32_t num_stages, uint32_t stage_capacity, uint32_t columns,
                                                  uint32_t m) {
    MultiSmem L;
    uint32_t off = 0;
    L.ring = off;
    off += num_stages * stage_capacity;
    L.x_row_bytes = columns * 2u + kRowPad;
    L.xs = off;
    off += m * L.x_row_bytes;
    off = (off + 15u) & ~15u;
    L.xsum = off;
    off += 8u * (columns / 64u) * 4u;  // [group][8 rows]: the two rows a lane needs are one 8-byte load
    off = (off + 15u) & ~15u;
    L.red = off;
    off += kRed * kCW * 128u * 4u;
    L.wred = off;
    off += 8u * kCW * 4u;
    L.bars = off;
    off += (2u * kMaxStages + 2u * kRed) * 8u;
    L.flags = off;
    off += 16u;
    L.total = off;
    return L;
}

__device__ inline void multi_wait_failed(volatile uint32_t *abort_flag, uint32_t *error_word) {
    *abort_flag = 1;
    atomicOr(error_word, kErrMbarTimeout);
}

template <bool NORM>
__global__ void __launch_bounds__(kThreads, 1) qmv_multi_a4_kernel(const MultiParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t columns = p.groups * 64u;
    const MultiSmem L = multi_layout(p.num_stages, p.stage_capacity, columns, p.m);
    uint8_t *ring = smem + L.ring;
    uint8_t *xs = smem + L.xs;
    float *xsum = reinterpret_cast<float *>(smem + L.xsum);
    float *red = reinterpret_cast<float *>(smem + L.red);
    float *wred = reinterpret_cast<float *>(smem + L.wred);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.bars);
    uint64_t *empty = full + kMaxStages;
    uint64_t *red_full = empty + kMaxStages;
    uint64_t *red_empty = red_full + kRed;
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + L.flags);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t units = p.row_tiles / p.unit_tiles;
    const uint32_t u0 = (uint32_t)(((uint64_t)blockIdx.x * units) / gridDim.x);
    const uint32_t u1 = (uint32_t)(((uint64_t)(blockIdx.x + 1) * units) / gridDim.x);
    const uint32_t t0 = u0 * p.unit_tiles, t1 = u1 * p.unit_tiles;

    if (tid == 0) {
        for (uint32_t s = 0; s < p.num_stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kCW);
        }
        for (uint32_t s = 0; s < kRed; ++s) {
            mbar_init(&red_full[s], kCW);
            mbar_init(&red_empty[s], 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kProducerWarp) {
        // the weights do not depend on the previous kernel: the stream starts at once
        if (lane == 0) {
            const uint32_t total_stages = (t1 - t0) * p.stages_per_tile;
            const uint32_t stage_bytes = p.stage_records * kA4RecordBytes;
            const uint8_t *src = p.w + (size_t)t0 * p.groups * kA4RecordBytes;
            uint32_t slot = 0, phase = 1;
            for (uint32_t s = 0; s < total_stages; ++s) {
                if (!mbar_wait_bounded(&empty[slot], phase, abort_flag)) {
                    multi_wait_failed(abort_flag, p.error_word);
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
        pdl_wait();
        // lane -> matrix row (lane & 15) of the tile and input rows 4 * (lane >> 4) .. + 3
        const uint32_t wrow = lane & 15u, xr0 = 4u * (lane >> 4);
        uint32_t rb = 0, rphase = 0;
        float held[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // SwiGLU: the `up` values of the even tile
        for (uint32_t tile = t0; tile < t1; ++tile) {
            if (!mbar_wait_bounded(&red_full[rb], rphase, abort_flag)) multi_wait_failed(abort_flag, p.error_word);
            float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int wv = 0; wv < kCW; ++wv) {
                const float4 q = *reinterpret_cast<const float4 *>(red + ((rb * kCW + wv) * 16u + wrow) * 8u + xr0);
                v[0] += q.x;
                v[1] += q.y;
                v[2] += q.z;
                v[3] += q.w;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&red_empty[rb]);
            if (++rb == kRed) {
                rb = 0;
                rphase ^= 1u;
            }
            const uint32_t row = tile_row0(tile, p.pair_halves, p.rows) + wrow;
            const bool valid = row < p.rows;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t xr = xr0 + i;
                if (xr >= p.m) continue;
                uint16_t *yrow = p.y + (size_t)xr * p.y_stride;
                if (p.epilogue == kEpiStore) {
                    if (valid) yrow[row] = f32_to_bf16_bits(v[i]);
                } else if (p.epilogue == kEpiResidual) {
                    if (valid) yrow[row] = f32_to_bf16_bits(bf16_round(v[i]) + bf16_bits_to_f32(yrow[row]));
                } else {  // kEpiSwiGlu: gated_act_mul.rs:80-95
                    if ((tile & 1u) == 0) {
                        held[i] = bf16_round(v[i]);
                    } else {
                        const float gate = bf16_round(v[i]);
                        const float activated = bf16_round(gate / (1.0f + expf(-1.0f * gate)));
                        const uint32_t orow = (tile >> 1) * 16u + wrow;
                        if (orow < p.rows / 2u) yrow[orow] = f32_to_bf16_bits(held[i] * activated);
                    }
                }
            }
        }
        return;
    }

    // ------------------------------------------------------------------ consumers: the rows into shared memory
    const uint32_t chunks = columns / 8u;  // 16-byte chunks per row
    if (NORM) {
        // one chunk per thread and row (columns <= 4096); weights rounded to bf16 before the wait
        float nw[8];
        const bool mine = tid < chunks;
        if (mine) {
            const float4 a = reinterpret_cast<const float4 *>(p.norm_weight)[2 * tid];
            const float4 b = reinterpret_cast<const float4 *>(p.norm_weight)[2 * tid + 1];
            const float raw[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) nw[i] = bf16_round(raw[i]);
        }
        pdl_wait();
        float f[8][8];
        float sumsq[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            sumsq[r] = 0.0f;
            if (r < (int)p.m && mine) {
                const uint4 v = reinterpret_cast<const uint4 *>(p.x + (size_t)r * p.x_stride)[tid];
                const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    f[r][2 * i] = __uint_as_float(wv[i] << 16);
                    f[r][2 * i + 1] = __uint_as_float(wv[i] & 0xffff0000u);
                    sumsq[r] = fmaf(f[r][2 * i], f[r][2 * i], sumsq[r]);
                    sumsq[r] = fmaf(f[r][2 * i + 1], f[r][2 * i + 1], sumsq[r]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) f[r][i] = 0.0f;
            }
            sumsq[r] = warp_sum(sumsq[r]);
        }
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < 8; ++r) wred[r * kCW + warp] = sumsq[r];
        }
        named_bar_sync(1, kConsumerThreads);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r >= (int)p.m) break;
            float total = 0.0f;
#pragma unroll
            for (int i = 0; i < kCW; ++i) total += wred[r * kCW + i];
            const float rms_inv = 1.0f / sqrtf(total / (float)columns + p.eps);
            uint32_t packed[4];
            float s8 = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // bf16(normalized) * bf16(weight), product rounded to bf16
                const uint32_t n2 = f32x2_to_bf16x2(f[r][2 * i] * rms_inv, f[r][2 * i + 1] * rms_inv);
                packed[i] = f32x2_to_bf16x2(__uint_as_float(n2 << 16) * nw[2 * i], __uint_as_float(n2 & 0xffff0000u) * nw[2 * i + 1]);
                s8 += __uint_as_float(packed[i] << 16);
                s8 += __uint_as_float(packed[i] & 0xffff0000u);
            }
            if (mine) *reinterpret_cast<uint4 *>(xs + (size_t)r * L.x_row_bytes + tid * 16u) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) s8 += __shfl_xor_sync(0xffffffffu, s8, o);
            if (mine && (lane & 7u) == 0) xsum[(tid >> 3) * 8u + r] = s8;
        }
    } else {
        pdl_wait();
        // Every 16-byte chunk of every row goes global -> shared memory as an asynchronous copy, all of them in
        // flight at once (one trip to L2 instead of one per batch of registers); the per-group sums are then formed
        // from shared memory: chunk c of row r by the lane that copied it, 8 consecutive lanes per group.
        const uint32_t total = p.m * chunks;
        for (uint32_t idx = tid; idx < total; idx += kConsumerThreads) {
            const uint32_t r = idx / chunks, c = idx - r * chunks;
            cp_async16(xs + (size_t)r * L.x_row_bytes + c * 16u, reinterpret_cast<const uint4 *>(p.x + (size_t)r * p.x_stride) + c);
        }
        cp_async_commit();
        cp_async_wait<0>();
        for (uint32_t base = 0; base < total; base += kConsumerThreads) {
            const uint32_t idx = base + tid;
            float s8 = 0.0f;
            uint32_t r = 0, c = 0;
            if (idx < total) {
                r = idx / chunks;
                c = idx - r * chunks;
                const uint4 v = *reinterpret_cast<const uint4 *>(xs + (size_t)r * L.x_row_bytes + c * 16u);  // this thread's own copy
                const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    s8 += __uint_as_float(wv[i] << 16);
                    s8 += __uint_as_float(wv[i] & 0xffff0000u);
                }
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) s8 += __shfl_xor_sync(0xffffffffu, s8, o);
            if (idx < total && (lane & 7u) == 0) xsum[(c >> 3) * 8u + r] = s8;
        }
    }
    named_bar_sync(1, kConsumerThreads);

    // ------------------------------------------------------------------ main loop
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t xrow = g < p.m ? g : 0u;  // columns of the tensor-core tile beyond the last row repeat row 0
    const uint8_t *my_x = xs + (size_t)xrow * L.x_row_bytes + t * 32u;
    const float *my_xsum = xsum + 2u * t;  // rows 2t and 2t + 1 of a group (rows past the last one hold stale values
                                           // whose results nobody reads)
    uint32_t slot = 0, phase = 0, rb = 0, rphase = 1;
    for (uint32_t tile = t0; tile < t1; ++tile) {
        float acc[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};  // [matrix row g, g + 8][input row 2t, 2t + 1]
        uint32_t kg0 = 0;
        for (uint32_t st = 0; st < p.stages_per_tile; ++st) {
            if (!mbar_wait_bounded(&full[slot], phase, abort_flag)) multi_wait_failed(abort_flag, p.error_word);
            const uint8_t *stage = ring + (size_t)slot * p.stage_capacity;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t rec_index = warp + (uint32_t)kCW * i;
                if (rec_index < p.stage_records) {
                    const uint8_t *rec = stage + rec_index * kA4RecordBytes;
                    const uint4 wq = *reinterpret_cast<const uint4 *>(rec + lane * 16u);
                    const uint32_t sw = *reinterpret_cast<const uint32_t *>(rec + 512u + 4u * g);
                    const uint32_t bw = *reinterpret_cast<const uint32_t *>(rec + 544u + 4u * g);
                    const uint32_t kg = kg0 + rec_index;
                    const uint4 *xp = reinterpret_cast<const uint4 *>(my_x + kg * 128u);
                    const uint4 xa = xp[0], xb = xp[1];
                    const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
                    const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                    float c[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t magic = 0x43004300u, mask = 0x000f000fu;  // bf16 pair (128 + q, 128 + q')
                        const uint32_t a0 = lop3_and_or(ww[j], mask, magic);
                        const uint32_t a1 = lop3_and_or(ww[j] >> 4, mask, magic);
                        const uint32_t a2 = lop3_and_or(ww[j] >> 8, mask, magic);
                        const uint32_t a3 = lop3_and_or(ww[j] >> 12, mask, magic);
                        if (j == 0) {  // the record's first product starts from zero: no accumulator to clear
                            asm volatile(
                                "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                                "{%10,%10,%10,%10};"
                                : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(xw[0]), "r"(xw[1]), "f"(0.0f));
                        } else {
                            mma_m16n8k16_bf16(c, a0, a1, a2, a3, xw[2 * j], xw[2 * j + 1]);
                        }
                    }
                    const float s0 = __uint_as_float(sw << 16), s1 = __uint_as_float(sw & 0xffff0000u);
                    const float b0 = fmaf(-128.0f, s0, __uint_as_float(bw << 16));
                    const float b1 = fmaf(-128.0f, s1, __uint_as_float(bw & 0xffff0000u));
                    const float2 xs2 = *reinterpret_cast<const float2 *>(my_xsum + kg * 8u);
                    const float xa_sum = xs2.x, xb_sum = xs2.y;
                    acc[0][0] = fmaf(b0, xa_sum, fmaf(s0, c[0], acc[0][0]));
                    acc[0][1] = fmaf(b0, xb_sum, fmaf(s0, c[1], acc[0][1]));
                    acc[1][0] = fmaf(b1, xa_sum, fmaf(s1, c[2], acc[1][0]));
                    acc[1][1] = fmaf(b1, xb_sum, fmaf(s1, c[3], acc[1][1]));
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
        if (!mbar_wait_bounded(&red_empty[rb], rphase, abort_flag)) multi_wait_failed(abort_flag, p.error_word);
        float *dst = red + (rb * kCW + warp) * 128u;
        *reinterpret_cast<float2 *>(dst + g * 8u + 2u * t) = make_float2(acc[0][0], acc[0][1]);
        *reinterpret_cast<float2 *>(dst + (g + 8u) * 8u + 2u * t) = make_float2(acc[1][0], acc[1][1]);
        __syncwarp();
        if (lane == 0) mbar_arrive(&red_full[rb]);
        if (++rb == kRed) {
            rb = 0;
            rphase ^= 1u;
        }
    }
}

int multi_sm_count() {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    return n;
}

// Records per ring stage: the largest divisor of `groups` that two passes of the 16 consumer warps cover.
uint32_t multi_stage_records(uint32_t groups) {
    for (uint32_t r = std::min(groups, 2u * (uint32_t)kCW); r > 1u; --r)
        if (groups % r == 0) return r;
    return 1u;
}

bool multi_geometry(const QMatrix *w, uint32_t m, MultiParams *p, uint32_t *smem_bytes) {
    p->stage_records = multi_stage_records(w->groups);
    p->stages_per_tile = w->groups / p->stage_records;
    p->stage_capacity = (p->stage_records * kA4RecordBytes + 127u) & ~127u;
    uint32_t stages = kMaxStages;
    while (stages > 2u && multi_layout(stages, p->stage_capacity, w->columns, m).total > 220u * 1024u) --stages;
    p->num_stages = stages;
    *smem_bytes = multi_layout(stages, p->stage_capacity, w->columns, m).total;
    return *smem_bytes <= 220u * 1024u;
}

}  // namespace

bool qmv_multi_supports(const QMatrix *w, uint32_t m, bool norm) {
    if (!w || w->format != kFmtAffine4 || m == 0 || m > kQmvMultiMaxRows || w->columns % 64u != 0) return false;
    if (norm && w->columns > kNormMaxColumns) return false;
    MultiParams p{};
    uint32_t smem = 0;
    return multi_geometry(w, m, &p, &smem);
}

stark_b200_status qmv_multi_launch(const QmvMultiArgs &a, cudaStream_t stream) {
    const QMatrix *w = a.matrix;
    if (!w || !a.x || !a.y || a.m == 0) return STARK_B200_INVALID_ARGUMENT;
    const bool norm = a.norm_weight != nullptr;
    if (!qmv_multi_supports(w, a.m, norm)) return STARK_B200_UNSUPPORTED;
    if (a.epilogue != kEpiStore && a.epilogue != kEpiResidual && a.epilogue != kEpiSwiGlu) return STARK_B200_UNSUPPORTED;
    if ((a.epilogue == kEpiSwiGlu) != (w->pair_halves != 0)) return STARK_B200_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(a.x) & 15u) || (a.x_stride % 8u) != 0) return STARK_B200_INVALID_ARGUMENT;
    MultiParams p{};
    uint32_t smem = 0;
    multi_geometry(w, a.m, &p, &smem);
    p.w = w->data;
    p.rows = w->rows;
    p.row_tiles = w->row_tiles;
    p.groups = w->groups;
    p.pair_halves = w->pair_halves;
    p.unit_tiles = a.epilogue == kEpiSwiGlu ? 2u : 1u;
    p.m = a.m;
    p.x = a.x;
    p.x_stride = a.x_stride ? a.x_stride : w->columns;
    p.y = a.y;
    p.y_stride = a.y_stride;
    p.norm_weight = a.norm_weight;
    p.eps = a.eps;
    p.epilogue = a.epilogue;
    p.error_word = a.error_word;
    const uint32_t units = p.row_tiles / p.unit_tiles;
    const uint32_t grid = std::max(1u, std::min(units, (uint32_t)multi_sm_count()));
    static SmemOptIn once_norm, once_plain;
    void (*fn)(MultiParams) = norm ? qmv_multi_a4_kernel<true> : qmv_multi_a4_kernel<false>;
    if (stark_b200_status s = ensure_dynamic_smem(fn, 220 * 1024, norm ? once_norm : once_plain)) return s;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 1 : 0;
    SB_CUDA(cudaLaunchKernelEx(&cfg, fn, p));
    return STARK_B200_OK;
}

}  // namespace sb
