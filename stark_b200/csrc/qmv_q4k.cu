// GGUF Q4_K matvec on the tensor cores.  The matrix is re-tiled once at load into *super-records* of
// 16 rows x 256 columns (one Q4_K super-block per row), 2304 bytes -- exactly the 16 x 144 bytes of the
// source blocks, so the format keeps its 0.5625 bytes per weight:
//   [0, 2048)     8 sub-records of 256 B, one per 32-column sub-block jb.  Lane L (g = L>>2, t = L&3) owns
//                 8 bytes = words j = 0, 1; nibble p of word j holds the 4-bit code of
//                   W[row0 + g + 8*(p&1)][256*sb + 32*jb + 8*t + 4*j + 2*((p>>1)&1) + (p>>2)],
//                 the A-fragment order of mma.m16n8k16 after the lop3 extraction (dequant_a4_word), with
//                 the sub-block's 32 columns dealt 8 per t so that one sub-block is exactly two mma steps.
//   [2048, 2304)  16 rows x 16 B: the first 16 bytes of each row's source block (f16 d, f16 dmin, 12
//                 bytes of packed 6-bit scales and minima), untouched.
// Super-records are ordered [expert][row tile][super-block].
//
// A warp owns whole row tiles and streams their super-records global -> shared with 16-byte cp.async
// copies, four in flight.  Per sub-block it issues two mma steps with the codes as exact f16 integers in A
// and the input vector in B -- even columns the f16 head of x, odd columns the f16 remainder, so
// c[0] + c[1] is the dot product with ~22 bits of x -- then the lane responsible for that sub-block (jb mod
// 4 == t) applies d*sc and dmin*m.  The value of a weight is (d*sc)*q - dmin*m as in the reference's
// decode (crates/stark-engine/src/engine/hybrid/weights.rs:2993-3017, 2908-2920); the dot product
// regroups it as d*sc * sum(q x) - dmin*m * sum(x), inside the reference's 2e-5 * sum|w x| bound.
#include <algorithm>
#include <cmath>

#include "device_math.cuh"
#include "qmv.cuh"

namespace sb {

namespace {

constexpr uint32_t kSuperBytes = 2304;

__device__ inline float f16_bits_f32(uint32_t h) { return __half2float(__ushort_as_half((uint16_t)h)); }

// (scale, minimum) of sub-block j from the 12 packed bytes held in words y, z, w of the row header
// (weights.rs:2908-2920), branch-free.
__device__ inline void q4k_pair(const uint4 &hdr, uint32_t j, uint32_t &sc, uint32_t &mn) {
    const uint32_t s = 8u * (j & 3u);
    const uint32_t lo = (hdr.y >> s) & 255u, mid = (hdr.z >> s) & 255u, hi = (hdr.w >> s) & 255u;
    const bool upper = j >= 4u;
    sc = upper ? ((hi & 15u) | ((lo >> 6) << 4)) : (lo & 63u);
    mn = upper ? ((hi >> 4) | ((mid >> 6) << 4)) : (mid & 63u);
}

// d*sc and dmin*m of sub-blocks t and t + 4 of one row: both take their bytes from the same lane of the
// three scale words, so the extraction is shared.
__device__ inline void q4k_scales_pair(const uint4 &hdr, uint32_t t, float (&dsc)[2], float (&dm)[2]) {
    const uint32_t s = 8u * t;
    const uint32_t lo = (hdr.y >> s) & 255u, mid = (hdr.z >> s) & 255u, hi = (hdr.w >> s) & 255u;
    const float d = f16_bits_f32(hdr.x & 0xffffu), dmin = f16_bits_f32(hdr.x >> 16);
    dsc[0] = d * (float)(lo & 63u);
    dm[0] = dmin * (float)(mid & 63u);
    dsc[1] = d * (float)((hi & 15u) | ((lo >> 6) << 4));
    dm[1] = dmin * (float)((hi >> 4) | ((mid >> 6) << 4));
}

struct Q4ktParams {
    const uint8_t *data;
    uint32_t rows, columns, row_tiles, supers;  // supers = columns / 256
    size_t expert_bytes;
    const uint32_t *expert_ids;
    uint32_t experts;
    const void *x;
    size_t x_stride;
    void *y;
    uint32_t io_type;
    const float *x_mul;  // f32 input only: the input is silu(x[i]) * x_mul[i] (the gated activation), nullptr = x
};

// Element i of launch row b's input.  With x_mul the input is the gated activation of the routed-expert
// feed-forward, silu(x) * x_mul with the reference's two-branch sigmoid (engine/hybrid/math.rs:5-16,
// qwen.rs:889-891), formed here instead of in a kernel of its own.
__device__ inline float load_input(const Q4ktParams &p, uint32_t b, uint32_t i) {
    const size_t at = (size_t)b * p.x_stride + i;
    if (p.io_type != STARK_B200_F32) return bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(p.x)[at]);
    const float g = reinterpret_cast<const float *>(p.x)[at];
    if (!p.x_mul) return g;
    float sg;
    if (g >= 0.0f) {
        sg = 1.0f / (1.0f + expf(-g));
    } else {
        const float e = expf(g);
        sg = e / (1.0f + e);
    }
    return g * sg * p.x_mul[at];
}

// WARPS x STAGES super-records of shared memory per CTA: how many warps hide the decode latency against how
// many copies each keeps in flight.
// KS warps (a team) share a row tile, each taking every KS-th super-block, and add their partial rows
// through shared memory: small matrices have too few row tiles to fill the GPU with one warp per tile.
template <int kQ4Warps, int kQ4Stages, int KS>
__global__ void __launch_bounds__(kQ4Warps * 32) qmv_q4kt_kernel(const Q4ktParams p) {
    constexpr int kQ4Threads = kQ4Warps * 32;
    constexpr int kTeams = kQ4Warps / KS;
    __shared__ float team_rows[kQ4Warps][16];
    extern __shared__ __align__(16) uint8_t q4_smem[];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, b = blockIdx.y;
    const uint32_t g = lane >> 2, t = lane & 3u, K = p.columns;
    __half *xhi = reinterpret_cast<__half *>(q4_smem);
    __half *xlo = xhi + K + 32;  // 64 bytes on: the head and remainder reads of a warp hit different banks
    float *xsum = reinterpret_cast<float *>(xlo + K + 32);  // per 32 columns, of the unscaled input
    float *red = xsum + K / 32u;                       // [kQ4Warps] block maxima
    uint8_t *stage = reinterpret_cast<uint8_t *>(red + kQ4Warps) + (size_t)warp * kQ4Stages * kSuperBytes;

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
    const uint32_t gw = blockIdx.x * kTeams + team, nw = gridDim.x * kTeams;  // teams, not warps
    const uint32_t my_tiles = gw < p.row_tiles ? (p.row_tiles - gw + nw - 1u) / nw : 0u;
    const uint32_t items = my_tiles * (p.supers / KS);  // the launcher makes KS divide the super-block count

    uint32_t in_tile = gw, in_sb = member, in_item = 0;
    auto issue = [&]() {
        if (in_item < items) {
            const uint8_t *src = base + ((size_t)in_tile * p.supers + in_sb) * kSuperBytes;
            uint8_t *dst = stage + (in_item % kQ4Stages) * kSuperBytes;
            for (uint32_t off = lane * 16u; off < kSuperBytes; off += 512u) cp_async16(dst + off, src + off);
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
        const float v = load_input(p, b, i);
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
        const float v = load_input(p, b, i);
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
        const uint8_t *rec = stage + (item % kQ4Stages) * kSuperBytes;
        // this lane scales sub-blocks t and t + 4 of rows g and g + 8
        const uint4 h0 = *reinterpret_cast<const uint4 *>(rec + 2048u + 16u * g);
        const uint4 h1 = *reinterpret_cast<const uint4 *>(rec + 2048u + 16u * (g + 8u));
        float dsc0[2], dm0[2], dsc1[2], dm1[2];
        q4k_scales_pair(h0, t, dsc0, dm0);
        q4k_scales_pair(h1, t, dsc1, dm1);
        const __half *xk = xsel + (size_t)sb * 256u + 8u * t;
        float s0[2] = {0.0f, 0.0f}, s1[2] = {0.0f, 0.0f};  // sum(q x) of this lane's two sub-blocks, rows g and g + 8
#pragma unroll
        for (uint32_t jb = 0; jb < 8; ++jb) {
            const uint2 w = *reinterpret_cast<const uint2 *>(rec + jb * 256u + lane * 8u);
            const uint4 xv = *reinterpret_cast<const uint4 *>(xk + 32u * jb);
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t a[4];
            dequant_a4_word<0>(w.x, a);
            mma_m16n8k16_f16(c, a, xv.x, xv.y);
            dequant_a4_word<0>(w.y, a);
            mma_m16n8k16_f16(c, a, xv.z, xv.w);
            const bool mine = (jb & 3u) == t;
            s0[jb >> 2] = mine ? c[0] + c[1] : s0[jb >> 2];
            s1[jb >> 2] = mine ? c[2] + c[3] : s1[jb >> 2];
        }
        const float xa = xsum[sb * 8u + t], xb = xsum[sb * 8u + t + 4u];
        acc_s0 = fmaf(dsc0[0], s0[0], fmaf(dsc0[1], s0[1], acc_s0));
        acc_s1 = fmaf(dsc1[0], s1[0], fmaf(dsc1[1], s1[1], acc_s1));
        acc_m0 = fmaf(dm0[0], xa, fmaf(dm0[1], xb, acc_m0));
        acc_m1 = fmaf(dm1[0], xa, fmaf(dm1[1], xb, acc_m1));
        __syncwarp();  // the stage may be refilled by the next iteration's copy
        if ((sb += KS) >= p.supers) {
            sb = member;
            float v0 = fmaf(acc_s0, xunscale, -acc_m0), v1 = fmaf(acc_s1, xunscale, -acc_m1);
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

// Source blocks [experts][rows][supers][144] -> super-records.
__global__ void retile_q4k_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, uint32_t experts,
                                  uint32_t rows, uint32_t supers, uint32_t row_tiles) {
    const uint64_t words_per_super = kSuperBytes / 4u;  // 512 nibble words + 64 header words
    const uint64_t total = (uint64_t)experts * row_tiles * supers * words_per_super;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t wi = (uint32_t)(i % words_per_super);
        const uint64_t rec = i / words_per_super;
        const uint32_t sb = (uint32_t)(rec % supers);
        const uint32_t tile = (uint32_t)((rec / supers) % row_tiles);
        const uint32_t expert = (uint32_t)(rec / supers / row_tiles);
        const uint8_t *mat = src + (size_t)expert * rows * supers * 144u;
        uint32_t word = 0;
        if (wi < 512u) {
            const uint32_t jb = wi >> 6, lane = (wi >> 1) & 31u, j = wi & 1u, g = lane >> 2, t = lane & 3u;
#pragma unroll
            for (uint32_t pn = 0; pn < 8; ++pn) {
                const uint32_t row = tile * 16u + g + 8u * (pn & 1u);
                const uint32_t l = 8u * t + 4u * j + 2u * ((pn >> 1) & 1u) + (pn >> 2);
                uint32_t q = 0;
                if (row < rows) {
                    const uint8_t *blk = mat + ((size_t)row * supers + sb) * 144u;
                    q = (blk[16u + (jb >> 1) * 32u + l] >> (4u * (jb & 1u))) & 15u;
                }
                word |= q << (4u * pn);
            }
        } else {
            const uint32_t hw = wi - 512u, r16 = hw >> 2, part = hw & 3u, row = tile * 16u + r16;
            if (row < rows) word = *reinterpret_cast<const uint32_t *>(mat + ((size_t)row * supers + sb) * 144u + 4u * part);
        }
        reinterpret_cast<uint32_t *>(dst)[i] = word;
    }
}

// One row back to f32 values and / or 4-bit codes, bit-identical to the reference's decode of the
// source block (value = (d*sc)*q - dmin*m with separately rounded products).
__global__ void dequant_q4kt_kernel(const uint8_t *__restrict__ data, uint32_t supers, uint32_t columns, uint32_t row,
                                    float *out, uint8_t *codes_out) {
    const uint32_t tile = row >> 4, r16 = row & 15u, g = r16 & 7u, hrow = r16 >> 3;
    for (uint32_t col = blockIdx.x * blockDim.x + threadIdx.x; col < columns; col += gridDim.x * blockDim.x) {
        const uint32_t sb = col >> 8, jb = (col >> 5) & 7u, l = col & 31u;
        const uint32_t t = l >> 3, j = (l >> 2) & 1u, r = (l >> 1) & 1u, e = l & 1u, pn = 4u * e + 2u * r + hrow;
        const uint8_t *rec = data + ((size_t)tile * supers + sb) * kSuperBytes;
        const uint32_t word = *reinterpret_cast<const uint32_t *>(rec + jb * 256u + (g * 4u + t) * 8u + j * 4u);
        const uint32_t q = (word >> (4u * pn)) & 15u;
        const uint4 hdr = *reinterpret_cast<const uint4 *>(rec + 2048u + 16u * r16);
        uint32_t sc, mn;
        q4k_pair(hdr, jb, sc, mn);
        const float dsc = __fmul_rn(f16_bits_f32(hdr.x & 0xffffu), (float)sc);
        const float dm = __fmul_rn(f16_bits_f32(hdr.x >> 16), (float)mn);
        if (out) out[col] = __fsub_rn(__fmul_rn(dsc, (float)q), dm);
        if (codes_out) codes_out[col] = (uint8_t)q;
    }
}

}  // namespace

size_t q4kt_bytes(uint32_t experts, uint32_t rows, uint32_t columns) {
    return (size_t)experts * ((rows + 15u) / 16u) * (columns / 256u) * kSuperBytes;
}

// `blocks` = device copy of the source bytes; `m->data` must hold q4kt_bytes().
stark_b200_status q4kt_retile(const uint8_t *blocks, QMatrix *m, cudaStream_t stream) {
    const uint32_t supers = m->columns / 256u, experts = m->experts ? m->experts : 1u;
    const uint64_t words = (uint64_t)experts * m->row_tiles * supers * (kSuperBytes / 4u);
    const uint32_t grid = (uint32_t)std::min<uint64_t>((words + 255u) / 256u, 148u * 16u);
    retile_q4k_kernel<<<grid, 256, 0, stream>>>(blocks, m->data, experts, m->rows, supers, m->row_tiles);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status q4kt_launch(const QMatrix *m, const void *x, size_t x_stride, void *y, uint32_t batch,
                              const uint32_t *expert_ids, uint32_t io_type, cudaStream_t stream, bool pdl,
                              const float *x_mul) {
    if (m->columns % 256u != 0 || m->columns > 12288u) return STARK_B200_UNSUPPORTED;
    if (x_mul && io_type != STARK_B200_F32) return STARK_B200_INVALID_ARGUMENT;
    Q4ktParams p{};
    p.data = m->data;
    p.rows = m->rows;
    p.columns = m->columns;
    p.row_tiles = m->row_tiles;
    p.supers = m->columns / 256u;
    p.experts = m->experts ? m->experts : 1u;
    p.expert_bytes = (size_t)m->row_tiles * p.supers * kSuperBytes;
    p.expert_ids = expert_ids;
    p.x = x;
    p.x_stride = x_stride;
    p.y = y;
    p.io_type = io_type;
    p.x_mul = x_mul;
    // 12 warps x 3 copies in flight each; teams of 1, 2 or 4 warps per row tile so that a GPU's worth of warps
    // (~24 per SM) has work even when the matrix has few row tiles.  STARK_B200_Q4K_TEAM overrides.
    const uint32_t supers = m->columns / 256u;
    // team size: the one that wastes the least of the last wave of warps (a team costs one barrier pair per tile)
    uint32_t ks = 1;
    double best = 0.0;
    for (uint32_t cand = 1; cand <= 4u; cand *= 2u) {
        if (supers % cand != 0) break;
        const double slots = 148.0 * 2.0 * 12.0, units = (double)m->row_tiles * cand * batch;
        const double waves = std::ceil(units / slots);
        const double score = units / (waves * slots) * (cand == 1 ? 1.0 : (cand == 2 ? 0.98 : 0.96));
        if (score > best) {
            best = score;
            ks = cand;
        }
    }
    static const int forced = [] {
        const char *e = getenv("STARK_B200_Q4K_TEAM");
        return e ? atoi(e) : 0;
    }();
    if ((forced == 1 || forced == 2 || forced == 4) && supers % (uint32_t)forced == 0) ks = (uint32_t)forced;
    constexpr uint32_t warps = 12, stages = 3;
    const size_t smem = (size_t)m->columns * 4u + 128u + (size_t)(m->columns / 32u) * 4u + 4u * warps +
                        (size_t)warps * stages * kSuperBytes;
    auto kernel = ks == 4u ? qmv_q4kt_kernel<12, 3, 4> : (ks == 2u ? qmv_q4kt_kernel<12, 3, 2> : qmv_q4kt_kernel<12, 3, 1>);
    static SmemOptIn once[3];
    if (stark_b200_status s = ensure_dynamic_smem(kernel, 160 * 1024, once[ks == 4u ? 2 : (ks == 2u ? 1 : 0)])) return s;
    if (smem > 160u * 1024u) return STARK_B200_UNSUPPORTED;
    const uint32_t per_sm = (uint32_t)std::max<size_t>(1, std::min<size_t>(3, (220u * 1024u) / smem));
    const uint32_t teams = warps / ks;
    const uint32_t blocks =
        std::max(1u, std::min((m->row_tiles + teams - 1u) / teams, (148u * per_sm + batch - 1u) / batch));
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
    SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    return STARK_B200_OK;
}

stark_b200_status q4kt_dequantize(const QMatrix *m, uint32_t expert, uint32_t row, float *out_device,
                                  uint8_t *codes_device, cudaStream_t stream) {
    const uint32_t supers = m->columns / 256u;
    const uint8_t *data = m->data + (size_t)expert * m->row_tiles * supers * kSuperBytes;
    const uint32_t blocks = std::max(1u, std::min(64u, (m->columns + 255u) / 256u));
    dequant_q4kt_kernel<<<blocks, 256, 0, stream>>>(data, supers, m->columns, row, out_device, codes_device);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

}  // namespace sb
