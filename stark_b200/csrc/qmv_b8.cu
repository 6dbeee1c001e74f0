// 8-bit formats on the tensor cores: GGUF Q8_0 (int8 codes, one f16 scale per 32 columns) and MLX affine
// 8-bit (unsigned codes, bf16 scale and bias per 64 columns), re-tiled once at load into super-records of
// 16 rows x 256 columns, 4352 bytes -- exactly the bytes of the source (16 x 8 x 34, or 16 x 256 codes +
// 16 x 4 x 4 plane bytes), so the formats keep their 1.0625 bytes per weight:
//   [0, 4096)     8 sub-records of 512 B, one per 32-column sub-block jb.  Lane L (g = L>>2, t = L&3) owns 16
//                 bytes = 4 words; word 2*j + r (mma step j, k-half r) holds the codes of
//                   rows row0+g, row0+g, row0+g+8, row0+g+8 at columns 256*sb + 32*jb + 8*t + 4*j + 2*r + {0,1,0,1}
//                 so that two byte permutes turn a word into two A-fragment registers of mma.m16n8k16.
//   [4096, 4352)  Q8_0: f16 d[jb][row] (8 x 16);  affine: {bf16 scale, bf16 bias}[group][row] (4 x 16).
// Codes become exact f16 integers without a conversion instruction: byte | 0x6400 is 1024 + byte.  The
// rest follows the Q4_K kernel (qmv_q4k.cu): warp teams per row tile, cp.async pipeline per warp, the
// input as f16 head + remainder in the even / odd B columns, scales applied per sub-block by lane
// jb mod 4 == t.  Decode of a row stays bit-identical to the reference (weights.rs:2936-2941 for Q8_0,
// 1284-1309 for affine rows).
#include <algorithm>
#include <cmath>

#include "device_math.cuh"
#include "qmv.cuh"

namespace sb {

namespace {

constexpr uint32_t kB8SuperBytes = 4352;

__device__ inline float f16_bits_f32(uint32_t h) { return __half2float(__ushort_as_half((uint16_t)h)); }

// one word of four codes -> two A-fragment registers (rows g and g + 8), exact integers in f16
template <bool AFFINE>
__device__ inline void bytes_to_f16(uint32_t w, uint32_t &row_g, uint32_t &row_g8) {
    if (!AFFINE) w ^= 0x80808080u;  // int8 -> int8 + 128
    const __half2 off = __half2half2(__ushort_as_half(AFFINE ? 0x6400 : 0x6480));  // 1024, or 1024 + 128
    const uint32_t a = __byte_perm(w, 0x64646464u, 0x4140), b = __byte_perm(w, 0x64646464u, 0x4342);
    const __half2 ra = __hsub2(*reinterpret_cast<const __half2 *>(&a), off);
    const __half2 rb = __hsub2(*reinterpret_cast<const __half2 *>(&b), off);
    row_g = *reinterpret_cast<const uint32_t *>(&ra);
    row_g8 = *reinterpret_cast<const uint32_t *>(&rb);
}

struct B8Params {
    const uint8_t *data;
    uint32_t rows, columns, row_tiles, supers;  // supers = columns / 256
    size_t expert_bytes;
    const uint32_t *expert_ids;
    uint32_t experts;
    const void *x;
    size_t x_stride;
    void *y;
    uint32_t io_type;
    uint32_t team_major;
};

// WARPS x STAGES super-records of shared memory per CTA: how many warps hide the decode latency against how
// many copies each keeps in flight.
// KS warps (a team) share a row tile, each taking every KS-th super-block, and add their partial rows
// through shared memory: small matrices have too few row tiles to fill the GPU with one warp per tile.
template <bool AFFINE, int kQ4Warps, int kQ4Stages, int KS>
__global__ void __launch_bounds__(kQ4Warps * 32) qmv_b8t_kernel(const B8Params p) {
    constexpr int kQ4Threads = kQ4Warps * 32;
    constexpr int kTeams = kQ4Warps / KS;
    __shared__ float team_rows[kQ4Warps][16];
    extern __shared__ __align__(16) uint8_t b8_smem[];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, b = blockIdx.y;
    const uint32_t g = lane >> 2, t = lane & 3u, K = p.columns;
    __half *xhi = reinterpret_cast<__half *>(b8_smem);
    __half *xlo = xhi + K + 32;  // 64 bytes on: the head and remainder reads of a warp hit different banks
    float *xsum = reinterpret_cast<float *>(xlo + K + 32);  // per 32 columns, of the unscaled input
    float *red = xsum + K / 32u;                       // [kQ4Warps] block maxima
    uint8_t *stage = reinterpret_cast<uint8_t *>(red + kQ4Warps) + (size_t)warp * kQ4Stages * kB8SuperBytes;

    // The first copies of this warp's records go out before the input row is staged: they do not depend on it,
    // nor (without expert ids) on the kernel before this one, whose completion is only awaited after them.
    pdl_launch_dependents();
    if (p.expert_ids) pdl_wait();
    uint32_t expert = 0;
    if (p.expert_ids) {
        expert = p.expert_ids[b];
        if (expert == 0xffffffffu) return;  // expert parallel: another rank owns this selection slot (whole CTA, before any barrier)
        if (expert >= p.experts) expert = 0;  // moe_gather_rows: an invalid id falls back to expert 0 (moe.rs:84-101)
    }
    const uint8_t *base = p.data + (size_t)expert * p.expert_bytes;
    const uint32_t team = warp / KS, member = warp % KS;
    // teams, not warps; team-major numbering spreads few row tiles over many CTAs (one busy team in each)
    const uint32_t nw = gridDim.x * kTeams;
    const uint32_t gw = p.team_major ? team * gridDim.x + blockIdx.x : blockIdx.x * kTeams + team;
    const uint32_t my_tiles = gw < p.row_tiles ? (p.row_tiles - gw + nw - 1u) / nw : 0u;
    const uint32_t items = my_tiles * (p.supers / KS);  // the launcher makes KS divide the super-block count

    uint32_t in_tile = gw, in_sb = member, in_item = 0;
    auto issue = [&]() {
        if (in_item < items) {
            const uint8_t *src = base + ((size_t)in_tile * p.supers + in_sb) * kB8SuperBytes;
            uint8_t *dst = stage + (in_item % kQ4Stages) * kB8SuperBytes;
            for (uint32_t off = lane * 16u; off < kB8SuperBytes; off += 512u) cp_async16(dst + off, src + off);
            ++in_item;
            if ((in_sb += KS) >= p.supers) {
                in_sb = member;
                in_tile += nw;
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < kQ4Stages - 1; ++i) issue();

    if (!p.expert_ids) pdl_wait();
    // ---- input row: exact power-of-two scale into f16 range, head + remainder, per-32 sums ----
    float vmax = 0.0f;
    for (uint32_t i = tid; i < K; i += kQ4Threads) {
        const float v = p.io_type == STARK_B200_F32
                            ? reinterpret_cast<const float *>(p.x)[(size_t)b * p.x_stride + i]
                            : bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(p.x)[(size_t)b * p.x_stride + i]);
        vmax = fmaxf(vmax, fabsf(v));
    }
    vmax = warp_max(vmax);
    if (lane == 0) red[warp] = vmax;
    __syncthreads();
    vmax = 0.0f;
#pragma unroll
    for (int w = 0; w < kQ4Warps; ++w) vmax = fmaxf(vmax, red[w]);
    int shift = 14 - ((int)((__float_as_uint(vmax) >> 23) & 0xffu) - 127);
    shift = max(-100, min(100, shift));
    if (!(vmax > 0.0f) || !isfinite(vmax)) shift = 0;
    const float xscale = __uint_as_float((uint32_t)(shift + 127) << 23);
    const float xunscale = __uint_as_float((uint32_t)(127 - shift) << 23);
    for (uint32_t i = tid; i < K; i += kQ4Threads) {  // K is a multiple of 256: every warp sums whole blocks
        const float v = p.io_type == STARK_B200_F32
                            ? reinterpret_cast<const float *>(p.x)[(size_t)b * p.x_stride + i]
                            : bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(p.x)[(size_t)b * p.x_stride + i]);
        const float sv = v * xscale;
        const __half h = __float2half_rn(sv);
        xhi[i] = h;
        xlo[i] = __float2half_rn(sv - __half2float(h));
        const float s = warp_sum(v);  // lanes of a warp hold 32 consecutive columns
        if (lane == 0) xsum[i >> 5] = s;
    }
    __syncthreads();


    const __half *xsel = (g & 1u) ? xlo : xhi;  // B column n = g: even columns the head, odd the remainder
    float acc_s0 = 0.0f, acc_s1 = 0.0f, acc_m0 = 0.0f, acc_m1 = 0.0f;
    uint32_t tile = gw, sb = member;
    for (uint32_t item = 0; item < items; ++item) {
        issue();
        cp_async_wait<kQ4Stages - 1>();
        __syncwarp();
        const uint8_t *rec = stage + (item % kQ4Stages) * kB8SuperBytes;
        // this lane scales sub-blocks t and t + 4 of rows g and g + 8
        float sc0[2], sc1[2], bi0[2] = {0.0f, 0.0f}, bi1[2] = {0.0f, 0.0f};
        const uint16_t *meta = reinterpret_cast<const uint16_t *>(rec + 4096u);
#pragma unroll
        for (uint32_t u = 0; u < 2; ++u) {
            const uint32_t jb = t + 4u * u;
            if (AFFINE) {
                const uint32_t e0 = ((jb >> 1) * 16u + g) * 2u, e1 = ((jb >> 1) * 16u + g + 8u) * 2u;
                sc0[u] = bf16_bits_to_f32(meta[e0]);
                bi0[u] = bf16_bits_to_f32(meta[e0 + 1u]);
                sc1[u] = bf16_bits_to_f32(meta[e1]);
                bi1[u] = bf16_bits_to_f32(meta[e1 + 1u]);
            } else {
                sc0[u] = f16_bits_f32(meta[jb * 16u + g]);
                sc1[u] = f16_bits_f32(meta[jb * 16u + g + 8u]);
            }
        }
        const __half *xk = xsel + (size_t)sb * 256u + 8u * t;
        float s0[2] = {0.0f, 0.0f}, s1[2] = {0.0f, 0.0f};  // sum(q x) of this lane's two sub-blocks, rows g and g + 8
#pragma unroll
        for (uint32_t jb = 0; jb < 8; ++jb) {
            const uint4 w = *reinterpret_cast<const uint4 *>(rec + jb * 512u + lane * 16u);
            const uint4 xv = *reinterpret_cast<const uint4 *>(xk + 32u * jb);
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t a[4];
            bytes_to_f16<AFFINE>(w.x, a[0], a[1]);
            bytes_to_f16<AFFINE>(w.y, a[2], a[3]);
            mma_m16n8k16_f16(c, a, xv.x, xv.y);
            bytes_to_f16<AFFINE>(w.z, a[0], a[1]);
            bytes_to_f16<AFFINE>(w.w, a[2], a[3]);
            mma_m16n8k16_f16(c, a, xv.z, xv.w);
            const bool mine = (jb & 3u) == t;
            s0[jb >> 2] = mine ? c[0] + c[1] : s0[jb >> 2];
            s1[jb >> 2] = mine ? c[2] + c[3] : s1[jb >> 2];
        }
        acc_s0 = fmaf(sc0[0], s0[0], fmaf(sc0[1], s0[1], acc_s0));
        acc_s1 = fmaf(sc1[0], s1[0], fmaf(sc1[1], s1[1], acc_s1));
        if (AFFINE) {
            const float xa = xsum[sb * 8u + t], xb = xsum[sb * 8u + t + 4u];
            acc_m0 = fmaf(bi0[0], xa, fmaf(bi0[1], xb, acc_m0));
            acc_m1 = fmaf(bi1[0], xa, fmaf(bi1[1], xb, acc_m1));
        }
        __syncwarp();  // the stage may be refilled by the next iteration's copy
        if ((sb += KS) >= p.supers) {
            sb = member;
            float v0 = fmaf(acc_s0, xunscale, acc_m0), v1 = fmaf(acc_s1, xunscale, acc_m1);  // bias terms add
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            acc_s0 = acc_s1 = acc_m0 = acc_m1 = 0.0f;
            if (KS > 1) {
                // the team's members finish a tile together (same item count): add their rows in member order
                if (t == 0) {
                    team_rows[warp][g] = v0;
                    team_rows[warp][g + 8u] = v1;
                }
                named_bar_sync(1 + (int)team, KS * 32);
                if (member == 0) {
                    v0 = 0.0f, v1 = 0.0f;
#pragma unroll
                    for (int r = 0; r < KS; ++r) {
                        v0 += team_rows[team * KS + r][g];
                        v1 += team_rows[team * KS + r][g + 8u];
                    }
                }
                named_bar_sync(1 + (int)team, KS * 32);  // the rows may be overwritten by the next tile
            }
            if (t == 0 && member == 0) {
                const uint32_t r0 = tile * 16u + g, r1 = r0 + 8u;
                if (p.io_type == STARK_B200_F32) {
                    float *y = reinterpret_cast<float *>(p.y) + (size_t)b * p.rows;
                    if (r0 < p.rows) y[r0] = v0;
                    if (r1 < p.rows) y[r1] = v1;
                } else {
                    uint16_t *y = reinterpret_cast<uint16_t *>(p.y) + (size_t)b * p.rows;
                    if (r0 < p.rows) y[r0] = f32_to_bf16_bits(v0);
                    if (r1 < p.rows) y[r1] = f32_to_bf16_bits(v1);
                }
            }
            tile += nw;
        }
    }
}

struct B8Source {
    const uint8_t *codes;      // Q8_0: blocks [experts][rows][columns/32][34]; affine: codes [experts][rows][columns]
    const uint16_t *scales;    // affine only: [experts][rows][columns/64] bf16
    const uint16_t *biases;
};

template <bool AFFINE>
__global__ void retile_b8_kernel(const B8Source src, uint8_t *__restrict__ dst, uint32_t experts, uint32_t rows,
                                 uint32_t columns, uint32_t row_tiles) {
    const uint32_t supers = columns / 256u;
    const uint64_t words_per_super = kB8SuperBytes / 4u;  // 1024 code words + 64 meta words
    const uint64_t total = (uint64_t)experts * row_tiles * supers * words_per_super;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t wi = (uint32_t)(i % words_per_super);
        const uint64_t rec = i / words_per_super;
        const uint32_t sb = (uint32_t)(rec % supers);
        const uint32_t tile = (uint32_t)((rec / supers) % row_tiles);
        const uint32_t expert = (uint32_t)(rec / supers / row_tiles);
        uint32_t word = 0;
        if (wi < 1024u) {
            const uint32_t jb = wi >> 7, lane = (wi >> 2) & 31u, q = wi & 3u, j = q >> 1, r = q & 1u;
            const uint32_t g = lane >> 2, t = lane & 3u;
#pragma unroll
            for (uint32_t bi = 0; bi < 4; ++bi) {
                const uint32_t row = tile * 16u + g + 8u * (bi >> 1);
                const uint32_t col = 256u * sb + 32u * jb + 8u * t + 4u * j + 2u * r + (bi & 1u);
                uint32_t code = AFFINE ? 0u : 0u;
                if (row < rows) {
                    if (AFFINE) code = src.codes[((size_t)expert * rows + row) * columns + col];
                    else code = src.codes[(((size_t)expert * rows + row) * (columns / 32u) + (col >> 5)) * 34u + 2u + (col & 31u)];
                }
                word |= code << (8u * bi);
            }
        } else {
            const uint32_t m = wi - 1024u;
            if (AFFINE) {
                const uint32_t gi = m >> 4, r16 = m & 15u, row = tile * 16u + r16;
                if (row < rows) {
                    const size_t e = ((size_t)expert * rows + row) * (columns / 64u) + sb * 4u + gi;
                    word = (uint32_t)src.scales[e] | ((uint32_t)src.biases[e] << 16);
                }
            } else {
#pragma unroll
                for (uint32_t h = 0; h < 2; ++h) {
                    const uint32_t entry = 2u * m + h, jb = entry >> 4, r16 = entry & 15u, row = tile * 16u + r16;
                    if (row < rows) {
                        const uint8_t *blk = src.codes + (((size_t)expert * rows + row) * (columns / 32u) + sb * 8u + jb) * 34u;
                        word |= ((uint32_t)blk[0] | ((uint32_t)blk[1] << 8)) << (16u * h);
                    }
                }
            }
        }
        reinterpret_cast<uint32_t *>(dst)[i] = word;
    }
}

// One row back to f32 values and / or codes, bit-identical to the reference's decode of the source.
template <bool AFFINE>
__global__ void dequant_b8t_kernel(const uint8_t *__restrict__ data, uint32_t supers, uint32_t columns, uint32_t row,
                                   float *out, uint8_t *codes_out) {
    const uint32_t tile = row >> 4, r16 = row & 15u, g = r16 & 7u, hrow = r16 >> 3;
    for (uint32_t col = blockIdx.x * blockDim.x + threadIdx.x; col < columns; col += gridDim.x * blockDim.x) {
        const uint32_t sb = col >> 8, jb = (col >> 5) & 7u, l = col & 31u;
        const uint32_t t = l >> 3, j = (l >> 2) & 1u, r = (l >> 1) & 1u, e = l & 1u;
        const uint8_t *rec = data + ((size_t)tile * supers + sb) * kB8SuperBytes;
        const uint32_t code = rec[jb * 512u + (g * 4u + t) * 16u + (2u * j + r) * 4u + 2u * hrow + e];
        const uint16_t *meta = reinterpret_cast<const uint16_t *>(rec + 4096u);
        float v;
        if (AFFINE) {
            const uint32_t m = ((jb >> 1) * 16u + r16) * 2u;
            v = __fadd_rn(__fmul_rn(bf16_bits_to_f32(meta[m]), (float)code), bf16_bits_to_f32(meta[m + 1u]));
        } else {
            v = __fmul_rn(f16_bits_f32(meta[jb * 16u + r16]), (float)(int8_t)code);
        }
        if (out) out[col] = v;
        if (codes_out) codes_out[col] = (uint8_t)code;
    }
}

template <bool AFFINE>
stark_b200_status launch_b8(const QMatrix *m, const B8Params &p, uint32_t batch, cudaStream_t stream, bool pdl) {
    const uint32_t supers = m->columns / 256u;
    uint32_t ks = 1;
    double best = 0.0;
    for (uint32_t cand = 1; cand <= 4u; cand *= 2u) {  // team size: least waste in the last wave of warps
        if (supers % cand != 0) break;
        const double slots = 148.0 * 12.0, units = (double)m->row_tiles * cand * batch;
        const double waves = std::ceil(units / slots);
        const double score = units / (waves * slots) * (cand == 1 ? 1.0 : (cand == 2 ? 0.98 : 0.96));
        if (score > best) {
            best = score;
            ks = cand;
        }
    }
    // 12 warps x 3 records in flight, or (STARK_B200_B8_WARPS=20) 20 warps x 2: more warps to hide the
    // conversion and shared-memory latencies against fewer copies per warp.
    static const bool wide = [] {
        const char *e = getenv("STARK_B200_B8_WARPS");
        return e && atoi(e) == 20;
    }();
    const uint32_t warps = wide ? 20u : 12u, stages = wide ? 2u : 3u;
    const size_t smem = (size_t)m->columns * 4u + 128u + (size_t)(m->columns / 32u) * 4u + 4u * warps +
                        (size_t)warps * stages * kB8SuperBytes;
    const int slot = (wide ? 3 : 0) + (ks == 4u ? 2 : (ks == 2u ? 1 : 0));
    void (*const kernels[6])(B8Params) = {qmv_b8t_kernel<AFFINE, 12, 3, 1>, qmv_b8t_kernel<AFFINE, 12, 3, 2>,
                                          qmv_b8t_kernel<AFFINE, 12, 3, 4>, qmv_b8t_kernel<AFFINE, 20, 2, 1>,
                                          qmv_b8t_kernel<AFFINE, 20, 2, 2>, qmv_b8t_kernel<AFFINE, 20, 2, 4>};
    auto kernel = kernels[slot];
    static SmemOptIn once[6];
    if (stark_b200_status s = ensure_dynamic_smem(kernel, 220 * 1024, once[slot])) return s;
    if (smem > 220u * 1024u) return STARK_B200_UNSUPPORTED;
    const uint32_t teams = warps / ks;
    uint32_t blocks = std::max(1u, std::min((m->row_tiles + teams - 1u) / teams, (148u + batch - 1u) / batch));
    B8Params q = p;
    // A matrix whose row tiles fill fewer than half the SMs (a 2048-row projection: 43 CTAs) is bound by what
    // one SM can pull: one team per CTA on up to 148 CTAs instead.
    if (batch == 1u && blocks * 2u <= 148u && m->row_tiles > blocks) {
        q.team_major = 1u;
        blocks = std::min(m->row_tiles, 148u);
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks, batch);
    cfg.blockDim = dim3(warps * 32u);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, q));
    return STARK_B200_OK;
}

}  // namespace

size_t b8t_bytes(uint32_t experts, uint32_t rows, uint32_t columns) {
    return (size_t)experts * ((rows + 15u) / 16u) * (columns / 256u) * kB8SuperBytes;
}

// `codes` (and for the affine format `scales`, `biases`) are device copies of the source tensors.
stark_b200_status b8t_retile(const uint8_t *codes, const uint16_t *scales, const uint16_t *biases, QMatrix *m,
                             cudaStream_t stream) {
    const bool affine = m->format == kFmtAffine8T;
    const uint32_t experts = m->experts ? m->experts : 1u;
    const uint64_t words = (uint64_t)experts * m->row_tiles * (m->columns / 256u) * (kB8SuperBytes / 4u);
    const uint32_t grid = (uint32_t)std::min<uint64_t>((words + 255u) / 256u, 148u * 16u);
    B8Source src{codes, scales, biases};
    if (affine) retile_b8_kernel<true><<<grid, 256, 0, stream>>>(src, m->data, experts, m->rows, m->columns, m->row_tiles);
    else retile_b8_kernel<false><<<grid, 256, 0, stream>>>(src, m->data, experts, m->rows, m->columns, m->row_tiles);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status b8t_launch(const QMatrix *m, const void *x, size_t x_stride, void *y, uint32_t batch,
                             const uint32_t *expert_ids, uint32_t io_type, cudaStream_t stream, bool pdl) {
    if (m->columns % 256u != 0 || m->columns > 12288u) return STARK_B200_UNSUPPORTED;
    B8Params p{};
    p.data = m->data;
    p.rows = m->rows;
    p.columns = m->columns;
    p.row_tiles = m->row_tiles;
    p.supers = m->columns / 256u;
    p.experts = m->experts ? m->experts : 1u;
    p.expert_bytes = (size_t)m->row_tiles * p.supers * kB8SuperBytes;
    p.expert_ids = expert_ids;
    p.x = x;
    p.x_stride = x_stride;
    p.y = y;
    p.io_type = io_type;
    return m->format == kFmtAffine8T ? launch_b8<true>(m, p, batch, stream, pdl) : launch_b8<false>(m, p, batch, stream, pdl);
}

stark_b200_status b8t_dequantize(const QMatrix *m, uint32_t expert, uint32_t row, float *out_device,
                                 uint8_t *codes_device, cudaStream_t stream) {
    const uint32_t supers = m->columns / 256u;
    const uint8_t *data = m->data + (size_t)expert * m->row_tiles * supers * kB8SuperBytes;
    const uint32_t blocks = std::max(1u, std::min(64u, (m->columns + 255u) / 256u));
    if (m->format == kFmtAffine8T)
        dequant_b8t_kernel<true><<<blocks, 256, 0, stream>>>(data, supers, m->columns, row, out_device, codes_device);
    else
        dequant_b8t_kernel<false><<<blocks, 256, 0, stream>>>(data, supers, m->columns, row, out_device, codes_device);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

}  // namespace sb
