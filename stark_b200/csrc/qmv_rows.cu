// Row-wise fused-dequant matvec for the formats that keep the reference's byte layout in device
// memory: MLX affine 8-bit (group 64, bf16 planes), GGUF Q8_0 and GGUF Q4_K.  One warp per output row,
// the input vector staged in shared memory as f32, f32 accumulation, f32 or bf16 output.  Also the
// grouped form: a bank of `experts` matrices with the expert of each launch row read on the device.
//
// Decode arithmetic follows the reference's decode_block to the operation
// (crates/stark-engine/src/engine/hybrid/weights.rs:2936-2941 for Q8_0, 2993-3017 and 2908-2920 for
// Q4_K; 1284-1309 for affine rows): products and differences are formed with explicit
// round-to-nearest multiplies so that the compiler cannot contract them, which makes a dequantized row
// bit-identical to the CPU decode.
#include <algorithm>

#include "device_math.cuh"
#include "qmv.cuh"

namespace sb {

namespace {

constexpr int kRowThreads = 256;
constexpr int kRowWarps = kRowThreads / 32;

__device__ inline float f16_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// scale_min: weights.rs:2908-2920
__device__ inline void q4k_scale_min(const uint8_t *scales, int index, uint32_t &sc, uint32_t &mn) {
    if (index < 4) {
        sc = scales[index] & 63u;
        mn = scales[index + 4] & 63u;
    } else {
        sc = (scales[index + 4] & 15u) | ((uint32_t)(scales[index - 4] >> 6) << 4);
        mn = (uint32_t)(scales[index + 4] >> 4) | ((uint32_t)(scales[index] >> 6) << 4);
    }
}

// One Q4_K sub-block (32 values): value = d*sc*q - dmin*m, evaluated left to right like the reference.
struct Q4kSub {
    float dsc, dm;  // d * sc and dmin * m
    uint4 qa, qb;   // the 32 bytes that hold this sub-block's nibbles
    uint32_t shift; // 0 (low nibbles) or 4 (high nibbles)
};
__device__ inline Q4kSub q4k_load_sub(const uint8_t *block, uint32_t j) {
    Q4kSub s;
    const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(block));
    const float dmin = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(block + 2));
    uint32_t sc, mn;
    q4k_scale_min(block + 4, (int)j, sc, mn);
    s.dsc = __fmul_rn(d, (float)sc);
    s.dm = __fmul_rn(dmin, (float)mn);
    const uint4 *q = reinterpret_cast<const uint4 *>(block + 16u + (j >> 1) * 32u);
    s.qa = q[0];
    s.qb = q[1];
    s.shift = (j & 1u) * 4u;
    return s;
}
__device__ inline uint32_t q4k_code(const Q4kSub &s, uint32_t l) {
    const uint32_t words[8] = {s.qa.x, s.qa.y, s.qa.z, s.qa.w, s.qb.x, s.qb.y, s.qb.z, s.qb.w};
    return (words[l >> 2] >> (8u * (l & 3u) + s.shift)) & 15u;
}
__device__ inline float q4k_value(const Q4kSub &s, uint32_t code) {
    return __fsub_rn(__fmul_rn(s.dsc, (float)code), s.dm);
}

struct RowParams {
    const uint8_t *data;      // matrix (or bank) bytes in the reference layout
    const uint16_t *scales;   // affine 8-bit planes [rows, groups] bf16
    const uint16_t *biases;
    uint32_t format, rows, columns;
    size_t row_bytes;
    size_t expert_bytes;      // bank stride (0 for a single matrix)
    size_t expert_plane_elems;
    const uint32_t *expert_ids;  // [launch rows] or nullptr
    uint32_t experts;
    const void *x;            // [batch, columns]
    size_t x_stride;          // elements between the inputs of consecutive launch rows (0: shared input)
    void *y;                  // [batch, rows]
    uint32_t io_type;
};

template <uint32_t FORMAT>
__device__ inline float row_dot(const RowParams &p, const uint8_t *row, const uint16_t *srow, const uint16_t *brow,
                                const float *xs, uint32_t lane) {
    float acc = 0.0f;
    if (FORMAT == kFmtQ4_KRaw) {
        const uint32_t subs = p.columns / 32u;
        for (uint32_t si = lane; si < subs; si += 32) {
            const Q4kSub s = q4k_load_sub(row + (size_t)(si >> 3) * 144u, si & 7u);
            const float *xb = xs + si * 32u;
#pragma unroll
            for (uint32_t l = 0; l < 32; ++l) acc = fmaf(q4k_value(s, q4k_code(s, l)), xb[l], acc);
        }
    } else if (FORMAT == kFmtQ8_0) {
        const uint32_t blocks = p.columns / 32u;
        for (uint32_t b = lane; b < blocks; b += 32) {
            const uint16_t *blk = reinterpret_cast<const uint16_t *>(row + (size_t)b * 34u);
            const float d = f16_bits_to_f32(blk[0]);
            const float *xb = xs + b * 32u;
#pragma unroll
            for (uint32_t i = 0; i < 16; ++i) {
                const uint16_t two = blk[1 + i];
                acc = fmaf(__fmul_rn(d, (float)(int8_t)(two & 0xffu)), xb[2 * i], acc);
                acc = fmaf(__fmul_rn(d, (float)(int8_t)(two >> 8)), xb[2 * i + 1], acc);
            }
        }
    } else {  // kFmtAffine8
        const uint32_t chunks = p.columns / 16u;
        for (uint32_t c = lane; c < chunks; c += 32) {
            const uint4 q = *reinterpret_cast<const uint4 *>(row + (size_t)c * 16u);
            const uint32_t words[4] = {q.x, q.y, q.z, q.w};
            const float scale = bf16_bits_to_f32(srow[c >> 2]);
            const float bias = bf16_bits_to_f32(brow[c >> 2]);
            const float *xb = xs + c * 16u;
#pragma unroll
            for (uint32_t i = 0; i < 16; ++i) {
                const float code = (float)((words[i >> 2] >> (8u * (i & 3u))) & 255u);
                acc = fmaf(__fadd_rn(__fmul_rn(scale, code), bias), xb[i], acc);
            }
        }
    }
    return warp_sum(acc);
}

// Fallback for widths whose rows do not start on 16-byte boundaries (one lane per 32-value block straight
// from global memory; slow).  grid = (row blocks, batch).  Launch row `blockIdx.y` multiplies matrix
// `expert_ids[blockIdx.y]` of the bank (or the only matrix) with its input row.
template <uint32_t FORMAT>
__global__ void __launch_bounds__(kRowThreads) qmv_rows_generic_kernel(const RowParams p) {
    extern __shared__ __align__(16) float xs[];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t b = blockIdx.y;
    if (p.io_type == STARK_B200_F32) {
        const float *x = reinterpret_cast<const float *>(p.x) + (size_t)b * p.x_stride;
        for (uint32_t i = tid; i < p.columns; i += kRowThreads) xs[i] = x[i];
    } else {
        const uint16_t *x = reinterpret_cast<const uint16_t *>(p.x) + (size_t)b * p.x_stride;
        for (uint32_t i = tid; i < p.columns; i += kRowThreads) xs[i] = bf16_bits_to_f32(x[i]);
    }
    __syncthreads();
    uint32_t expert = 0;
    if (p.expert_ids) {
        expert = p.expert_ids[b];
        if (expert == 0xffffffffu) return;  // expert parallel: another rank owns this selection slot (whole CTA; no barrier follows)
        if (expert >= p.experts) expert = 0;  // moe_gather_rows: an invalid id falls back to expert 0 (moe.rs:84-101)
    }
    const uint8_t *base = p.data + (size_t)expert * p.expert_bytes;
    const uint16_t *sbase = p.scales ? p.scales + (size_t)expert * p.expert_plane_elems : nullptr;
    const uint16_t *bbase = p.biases ? p.biases + (size_t)expert * p.expert_plane_elems : nullptr;
    const uint32_t groups = p.columns / 64u;
    for (uint32_t row = blockIdx.x * kRowWarps + warp; row < p.rows; row += gridDim.x * kRowWarps) {
        const float v = row_dot<FORMAT>(p, base + (size_t)row * p.row_bytes, sbase ? sbase + (size_t)row * groups : nullptr,
                                        bbase ? bbase + (size_t)row * groups : nullptr, xs, lane);
        if (lane == 0) {
            if (p.io_type == STARK_B200_F32)
                reinterpret_cast<float *>(p.y)[(size_t)b * p.rows + row] = v;
            else
                reinterpret_cast<uint16_t *>(p.y)[(size_t)b * p.rows + row] = f32_to_bf16_bits(v);
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// Streaming kernel.  A warp owns whole rows; a row is cut into chunks of 1024 values (Q8_0: 1088 bytes,
// Q4_K: 576, affine 8-bit: 1024) that travel global -> shared memory as 16-byte cp.async copies, four
// chunks deep per warp, so the DRAM side sees long contiguous reads regardless of the block layout.
// Each lane then decodes one 32-value block of the chunk from shared memory.  Codes become f32 without
// an integer conversion (byte | 0x4B000000 is 2^23 + byte), the block's scale is applied once to the
// block's sum of code * x, and the offset terms (Q4_K minimum, affine bias) use sums of x over 32
// values prepared once per CTA.  The input vector sits in shared memory as f32, stored so that the 32
// lanes' 128-bit reads of their own blocks hit distinct banks (float4 index XOR block index).
constexpr uint32_t kChunkValues = 1024;

template <uint32_t FORMAT>
__host__ __device__ constexpr uint32_t chunk_bytes() {
    return FORMAT == kFmtQ8_0 ? 1088u : (FORMAT == kFmtQ4_KRaw ? 576u : 1024u);
}

__device__ inline float byte_to_f32(uint32_t word, uint32_t selector) {
    // selector 0x7540 + j: byte j of `word` under the exponent of 2^23
    return __uint_as_float(__byte_perm(word, 0x4B000000u, selector)) - 8388608.0f;
}
__device__ inline float dot4_bytes(uint32_t w, const float4 &x, float acc) {
    acc = fmaf(byte_to_f32(w, 0x7540u), x.x, acc);
    acc = fmaf(byte_to_f32(w, 0x7541u), x.y, acc);
    acc = fmaf(byte_to_f32(w, 0x7542u), x.z, acc);
    acc = fmaf(byte_to_f32(w, 0x7543u), x.w, acc);
    return acc;
}

// NB = 32-value blocks a lane decodes per item (an item is NB * 1024 values of one row): the larger the
// item, the less the per-item bookkeeping weighs; STAGES = items in flight per warp.
template <uint32_t FORMAT, uint32_t NB, uint32_t STAGES>
__global__ void __launch_bounds__(kRowThreads) qmv_rows_kernel(const RowParams p) {
    extern __shared__ __align__(16) uint8_t rows_smem[];
    constexpr uint32_t CB1 = chunk_bytes<FORMAT>();
    constexpr uint32_t CB = CB1 * NB;
    constexpr uint32_t kRowStages = STAGES;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t b = blockIdx.y;
    const uint32_t padded = (p.columns + kChunkValues - 1u) / kChunkValues * kChunkValues;
    float4 *xs4 = reinterpret_cast<float4 *>(rows_smem);
    float *xsum = reinterpret_cast<float *>(rows_smem + (size_t)padded * 4u);
    uint8_t *stage = rows_smem + (size_t)padded * 4u + (size_t)(padded / 32u) * 4u + (size_t)warp * kRowStages * CB;

    // input vector: f32, float4 (block, i4) of every chunk stored at block * 8 + (i4 ^ (block & 7))
    for (uint32_t q = tid; q < padded / 4u; q += kRowThreads) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q * 4u < p.columns) {
            if (p.io_type == STARK_B200_F32) {
                v = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.x) + (size_t)b * p.x_stride)[q];
            } else {
                const uint2 h = reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(p.x) + (size_t)b * p.x_stride)[q];
                v = make_float4(__uint_as_float(h.x << 16), __uint_as_float(h.x & 0xffff0000u),
                                __uint_as_float(h.y << 16), __uint_as_float(h.y & 0xffff0000u));
            }
        }
        const uint32_t block = q >> 3, i4 = q & 7u;
        xs4[block * 8u + (i4 ^ (block & 7u))] = v;
        float s4 = (v.x + v.y) + (v.z + v.w);
        s4 += __shfl_xor_sync(0xffffffffu, s4, 1);
        s4 += __shfl_xor_sync(0xffffffffu, s4, 2);
        s4 += __shfl_xor_sync(0xffffffffu, s4, 4);
        if (i4 == 0) xsum[block] = s4;
    }
    __syncthreads();

    uint32_t expert = 0;
    if (p.expert_ids) {
        expert = p.expert_ids[b];
        if (expert == 0xffffffffu) return;  // expert parallel: another rank owns this selection slot (whole CTA; no barrier follows)
        if (expert >= p.experts) expert = 0;  // moe_gather_rows: an invalid id falls back to expert 0 (moe.rs:84-101)
    }
    const uint8_t *base = p.data + (size_t)expert * p.expert_bytes;
    const uint16_t *sbase = p.scales ? p.scales + (size_t)expert * p.expert_plane_elems : nullptr;
    const uint16_t *bbase = p.biases ? p.biases + (size_t)expert * p.expert_plane_elems : nullptr;
    const uint32_t groups = p.columns / 64u;
    const uint32_t cpr = (p.columns + kChunkValues * NB - 1u) / (kChunkValues * NB);  // items per row
    const uint32_t gw = blockIdx.x * kRowWarps + warp, nw = gridDim.x * kRowWarps;
    const uint32_t my_rows = gw < p.rows ? (p.rows - gw + nw - 1u) / nw : 0u;
    const uint32_t items = my_rows * cpr;

    // (row, chunk) of the next item to copy and of the next item to compute advance as counters: no
    // division in the loop
    uint32_t in_row = gw, in_c = 0, in_item = 0;
    auto issue = [&]() {
        if (in_item < items) {
            const uint32_t bytes = min((uint32_t)CB, (uint32_t)(p.row_bytes - (size_t)in_c * CB));
            const uint8_t *src = base + (size_t)in_row * p.row_bytes + (size_t)in_c * CB;
            uint8_t *dst = stage + (in_item & (kRowStages - 1)) * CB;
            for (uint32_t off = lane * 16u; off < bytes; off += 512u) cp_async16(dst + off, src + off);
            ++in_item;
            if (++in_c == cpr) {
                in_c = 0;
                in_row += nw;
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < kRowStages - 1; ++i) issue();

    float acc = 0.0f;
    uint32_t row = gw, c = 0;
    for (uint32_t item = 0; item < items; ++item) {
        issue();
        cp_async_wait<kRowStages - 1>();
        __syncwarp();
#pragma unroll
        for (uint32_t nb = 0; nb < NB; ++nb) {
        const uint8_t *chunk = stage + (item & (kRowStages - 1)) * CB + nb * CB1;
        const uint32_t block = (c * NB + nb) * 32u + lane;  // one of this lane's 32-value blocks of the row
        if (block * 32u < p.columns) {
            const float4 *xb = xs4 + (size_t)block * 8u;
            const uint32_t sw = lane & 7u;               // block & 7 == lane & 7
            if (FORMAT == kFmtQ8_0) {
                const uint8_t *blk = chunk + 34u * lane;
                const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(blk));
                // The 32 codes start 2 bytes into the 34-byte block, i.e. on a 4-byte boundary for odd
                // lanes and 2 bytes past one for even lanes: read aligned words and funnel-shift.
                const uint32_t qoff = 34u * lane + 2u, sh = (qoff & 2u) * 8u;
                const uint32_t *wp = reinterpret_cast<const uint32_t *>(chunk + (qoff & ~3u));
                uint32_t wv[9];
#pragma unroll
                for (uint32_t k = 0; k < 8; ++k) wv[k] = wp[k];
                wv[8] = sh ? wp[8] : 0u;  // only even lanes need the ninth word (it exists: it is the next block)
                float t = 0.0f;
#pragma unroll
                for (uint32_t i4 = 0; i4 < 8; ++i4) {
                    const uint32_t w = __funnelshift_r(wv[i4], wv[i4 + 1], sh) ^ 0x80808080u;  // int8 + 128
                    t = dot4_bytes(w, xb[i4 ^ sw], t);
                }
                // sum (q + 128) x - 128 sum x
                acc = fmaf(d, fmaf(-128.0f, xsum[block], t), acc);
            } else if (FORMAT == kFmtQ4_KRaw) {
                const uint8_t *blk = chunk + 144u * (lane >> 3);
                const uint32_t j = lane & 7u;
                const uint32_t dd = *reinterpret_cast<const uint32_t *>(blk);
                const float d = f16_bits_to_f32((uint16_t)(dd & 0xffffu)), dmin = f16_bits_to_f32((uint16_t)(dd >> 16));
                uint32_t sc, mn;
                q4k_scale_min(blk + 4, (int)j, sc, mn);
                const uint4 *q = reinterpret_cast<const uint4 *>(blk + 16u + (j >> 1) * 32u);
                const uint4 qa = q[0], qb = q[1];
                const uint32_t words[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                const uint32_t shift = (j & 1u) * 4u;
                float t = 0.0f;
#pragma unroll
                for (uint32_t i4 = 0; i4 < 8; ++i4) t = dot4_bytes((words[i4] >> shift) & 0x0f0f0f0fu, xb[i4 ^ sw], t);
                acc = fmaf(d * (float)sc, t, acc);
                acc = fmaf(-(dmin * (float)mn), xsum[block], acc);
            } else {  // kFmtAffine8
                const uint4 *q = reinterpret_cast<const uint4 *>(chunk + 32u * lane);
                const uint4 qa = q[0], qb = q[1];
                const uint32_t words[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                const float scale = bf16_bits_to_f32(sbase[(size_t)row * groups + (block >> 1)]);
                const float bias = bf16_bits_to_f32(bbase[(size_t)row * groups + (block >> 1)]);
                float t = 0.0f;
#pragma unroll
                for (uint32_t i4 = 0; i4 < 8; ++i4) t = dot4_bytes(words[i4], xb[i4 ^ sw], t);
                acc = fmaf(scale, t, acc);
                acc = fmaf(bias, xsum[block], acc);
            }
        }
        }
        __syncwarp();  // the stage may be refilled by the next iteration's copy
        if (++c == cpr) {
            c = 0;
            const float v = warp_sum(acc);
            acc = 0.0f;
            if (lane == 0) {
                if (p.io_type == STARK_B200_F32)
                    reinterpret_cast<float *>(p.y)[(size_t)b * p.rows + row] = v;
                else
                    reinterpret_cast<uint16_t *>(p.y)[(size_t)b * p.rows + row] = f32_to_bf16_bits(v);
            }
            row += nw;
        }
    }
}

template <uint32_t FORMAT>
size_t rows_smem_bytes(uint32_t columns, uint32_t nb, uint32_t stages) {
    const uint32_t padded = (columns + kChunkValues - 1u) / kChunkValues * kChunkValues;
    return (size_t)padded * 4u + (size_t)(padded / 32u) * 4u + (size_t)kRowWarps * stages * nb * chunk_bytes<FORMAT>();
}

// Dequantizes one row to f32 (bit-exact image of decode_values / affine_row), one thread per element.
template <uint32_t FORMAT>
__global__ void dequant_row_kernel(const RowParams p, uint32_t row, float *out, uint8_t *codes_out) {
    const uint8_t *r = p.data + (size_t)row * p.row_bytes;
    const uint32_t groups = p.columns / 64u;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < p.columns; i += gridDim.x * blockDim.x) {
        float v;
        uint32_t code;
        if (FORMAT == kFmtQ4_KRaw) {
            const Q4kSub s = q4k_load_sub(r + (size_t)(i >> 8) * 144u, (i >> 5) & 7u);
            code = q4k_code(s, i & 31u);
            v = q4k_value(s, code);
        } else if (FORMAT == kFmtQ8_0) {
            const uint8_t *blk = r + (size_t)(i >> 5) * 34u;
            const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(blk));
            code = blk[2 + (i & 31u)];
            v = __fmul_rn(d, (float)(int8_t)code);
        } else {
            code = r[i];
            const float scale = bf16_bits_to_f32(p.scales[(size_t)row * groups + (i >> 6)]);
            const float bias = bf16_bits_to_f32(p.biases[(size_t)row * groups + (i >> 6)]);
            v = __fadd_rn(__fmul_rn(scale, (float)code), bias);
        }
        if (out) out[i] = v;
        if (codes_out) codes_out[i] = (uint8_t)code;
    }
}

size_t format_row_bytes(QFormat f, uint32_t columns) {
    switch (f) {
        case kFmtQ4_KRaw: return (size_t)(columns / 256u) * 144u;
        case kFmtQ8_0: return (size_t)(columns / 32u) * 34u;
        case kFmtAffine8: return columns;
        default: return 0;
    }
}

RowParams row_params(const QMatrix *m) {
    RowParams p{};
    p.data = m->data;
    p.format = m->format;
    p.rows = m->rows;
    p.columns = m->columns;
    p.row_bytes = format_row_bytes(m->format, m->columns);
    p.experts = m->experts ? m->experts : 1u;
    p.expert_bytes = p.row_bytes * m->rows;
    if (m->format == kFmtAffine8) {
        // planes follow the codes of the whole bank: [experts, rows, groups] scales, then biases
        const size_t codes = p.expert_bytes * p.experts;
        const size_t plane = (size_t)p.experts * m->rows * (m->columns / 64u);
        p.scales = reinterpret_cast<const uint16_t *>(m->data + codes);
        p.biases = p.scales + plane;
        p.expert_plane_elems = (size_t)m->rows * (m->columns / 64u);
    }
    return p;
}

template <uint32_t FORMAT>
stark_b200_status launch_rows(const QMatrix *m, const RowParams &p, uint32_t batch, cudaStream_t s) {
    // the streaming kernel copies 16 bytes at a time: every row must start on a 16-byte boundary
    if (p.row_bytes % 16u == 0) {
        // whole rows per item where they are long enough: 4096 values x 2 in flight, else 2048 x 4, else 1024 x 4
        const uint32_t nb = m->columns >= 4096u ? 4u : (m->columns >= 2048u ? 2u : 1u);
        const uint32_t stages = nb == 4u ? 2u : 4u;
        const size_t smem = rows_smem_bytes<FORMAT>(m->columns, nb, stages);
        auto kernel = nb == 4u ? qmv_rows_kernel<FORMAT, 4, 2> : (nb == 2u ? qmv_rows_kernel<FORMAT, 2, 4> : qmv_rows_kernel<FORMAT, 1, 4>);
        static SmemOptIn once[3];
        if (stark_b200_status s = ensure_dynamic_smem(kernel, 160 * 1024, once[nb == 4u ? 2 : (nb == 2u ? 1 : 0)])) return s;
        if (smem > 160u * 1024u) return STARK_B200_UNSUPPORTED;
        const uint32_t per_sm = (uint32_t)std::max<size_t>(1, std::min<size_t>(4, (220u * 1024u) / smem));
        const uint32_t row_blocks =
            std::max(1u, std::min((m->rows + kRowWarps - 1u) / kRowWarps, (148u * per_sm + batch - 1u) / batch));
        kernel<<<dim3(row_blocks, batch), kRowThreads, smem, s>>>(p);
    } else {
        const size_t smem = (size_t)m->columns * 4u;
        static SmemOptIn once;
        if (stark_b200_status s = ensure_dynamic_smem(qmv_rows_generic_kernel<FORMAT>, 64 * 1024, once)) return s;
        const uint32_t row_blocks =
            std::max(1u, std::min((m->rows + kRowWarps - 1u) / kRowWarps, 148u * 4u / std::max(1u, batch) + 1u));
        qmv_rows_generic_kernel<FORMAT><<<dim3(row_blocks, batch), kRowThreads, smem, s>>>(p);
    }
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

}  // namespace

bool qmv_rows_supports(const QMatrix *m) {
    return m && (m->format == kFmtQ4_K || m->format == kFmtQ4_KRaw || m->format == kFmtQ8_0 ||
                 m->format == kFmtAffine8 || m->format == kFmtQ8_0T || m->format == kFmtAffine8T);
}

stark_b200_status qmv_rows_launch(const QMatrix *m, const void *x, size_t x_stride, void *y, uint32_t batch,
                                  const uint32_t *expert_ids, uint32_t io_type, cudaStream_t stream, bool pdl) {
    if (!qmv_rows_supports(m) || !x || !y || batch == 0) return STARK_B200_INVALID_ARGUMENT;
    if (m->format == kFmtQ4_K) return q4kt_launch(m, x, x_stride, y, batch, expert_ids, io_type, stream, pdl);
    if (m->format == kFmtQ8_0T || m->format == kFmtAffine8T)
        return b8t_launch(m, x, x_stride, y, batch, expert_ids, io_type, stream, pdl);
    if (m->columns > 12288u) return STARK_B200_UNSUPPORTED;
    RowParams p = row_params(m);
    p.x = x;
    p.x_stride = x_stride;
    p.y = y;
    p.io_type = io_type;
    p.expert_ids = expert_ids;
    if (m->format == kFmtQ4_KRaw) return launch_rows<kFmtQ4_KRaw>(m, p, batch, stream);
    if (m->format == kFmtQ8_0) return launch_rows<kFmtQ8_0>(m, p, batch, stream);
    return launch_rows<kFmtAffine8>(m, p, batch, stream);
}

stark_b200_status qmv_rows_dequantize(const QMatrix *m, uint32_t expert, uint32_t row, float *out_device,
                                      uint8_t *codes_device, cudaStream_t stream) {
    if (!qmv_rows_supports(m) || row >= m->rows || expert >= (m->experts ? m->experts : 1u)) return STARK_B200_INVALID_ARGUMENT;
    if (m->format == kFmtQ4_K) return q4kt_dequantize(m, expert, row, out_device, codes_device, stream);
    if (m->format == kFmtQ8_0T || m->format == kFmtAffine8T)
        return b8t_dequantize(m, expert, row, out_device, codes_device, stream);
    RowParams p = row_params(m);
    p.data += (size_t)expert * p.expert_bytes;
    if (p.scales) {
        p.scales += (size_t)expert * p.expert_plane_elems;
        p.biases += (size_t)expert * p.expert_plane_elems;
    }
    const uint32_t blocks = std::max(1u, std::min(64u, (m->columns + 255u) / 256u));
    if (m->format == kFmtQ4_KRaw) dequant_row_kernel<kFmtQ4_KRaw><<<blocks, 256, 0, stream>>>(p, row, out_device, codes_device);
    else if (m->format == kFmtQ8_0) dequant_row_kernel<kFmtQ8_0><<<blocks, 256, 0, stream>>>(p, row, out_device, codes_device);
    else dequant_row_kernel<kFmtAffine8><<<blocks, 256, 0, stream>>>(p, row, out_device, codes_device);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

}  // namespace sb
