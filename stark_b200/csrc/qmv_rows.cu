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
    if (FORMAT == kFmtQ4_K) {
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

// grid = (row blocks, batch).  Launch row `blockIdx.y` multiplies matrix `expert_ids[blockIdx.y]` of the
// bank (or the only matrix) with its input row.
template <uint32_t FORMAT>
__global__ void __launch_bounds__(kRowThreads) qmv_rows_kernel(const RowParams p) {
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

// Dequantizes one row to f32 (bit-exact image of decode_values / affine_row), one thread per element.
template <uint32_t FORMAT>
__global__ void dequant_row_kernel(const RowParams p, uint32_t row, float *out, uint8_t *codes_out) {
    const uint8_t *r = p.data + (size_t)row * p.row_bytes;
    const uint32_t groups = p.columns / 64u;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < p.columns; i += gridDim.x * blockDim.x) {
        float v;
        uint32_t code;
        if (FORMAT == kFmtQ4_K) {
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
        case kFmtQ4_K: return (size_t)(columns / 256u) * 144u;
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

template <typename... Args>
void dispatch_rows(QFormat f, dim3 grid, size_t smem, cudaStream_t s, const RowParams &p) {
    if (f == kFmtQ4_K) qmv_rows_kernel<kFmtQ4_K><<<grid, kRowThreads, smem, s>>>(p);
    else if (f == kFmtQ8_0) qmv_rows_kernel<kFmtQ8_0><<<grid, kRowThreads, smem, s>>>(p);
    else qmv_rows_kernel<kFmtAffine8><<<grid, kRowThreads, smem, s>>>(p);
}

}  // namespace

bool qmv_rows_supports(const QMatrix *m) {
    return m && (m->format == kFmtQ4_K || m->format == kFmtQ8_0 || m->format == kFmtAffine8);
}

stark_b200_status qmv_rows_launch(const QMatrix *m, const void *x, size_t x_stride, void *y, uint32_t batch,
                                  const uint32_t *expert_ids, uint32_t io_type, cudaStream_t stream) {
    if (!qmv_rows_supports(m) || !x || !y || batch == 0) return STARK_B200_INVALID_ARGUMENT;
    if (m->columns > 12288u) return STARK_B200_UNSUPPORTED;
    RowParams p = row_params(m);
    p.x = x;
    p.x_stride = x_stride;
    p.y = y;
    p.io_type = io_type;
    p.expert_ids = expert_ids;
    const size_t smem = (size_t)m->columns * 4u;
    static bool attr_set = false;
    if (!attr_set) {
        SB_CUDA(cudaFuncSetAttribute(qmv_rows_kernel<kFmtQ4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        SB_CUDA(cudaFuncSetAttribute(qmv_rows_kernel<kFmtQ8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        SB_CUDA(cudaFuncSetAttribute(qmv_rows_kernel<kFmtAffine8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        attr_set = true;
    }
    const uint32_t row_blocks = std::max(1u, std::min((m->rows + kRowWarps - 1u) / kRowWarps, 148u * 4u / std::max(1u, batch) + 1u));
    dispatch_rows(m->format, dim3(row_blocks, batch), smem, stream, p);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status qmv_rows_dequantize(const QMatrix *m, uint32_t expert, uint32_t row, float *out_device,
                                      uint8_t *codes_device, cudaStream_t stream) {
    if (!qmv_rows_supports(m) || row >= m->rows || expert >= (m->experts ? m->experts : 1u)) return STARK_B200_INVALID_ARGUMENT;
    RowParams p = row_params(m);
    p.data += (size_t)expert * p.expert_bytes;
    if (p.scales) {
        p.scales += (size_t)expert * p.expert_plane_elems;
        p.biases += (size_t)expert * p.expert_plane_elems;
    }
    const uint32_t blocks = std::max(1u, std::min(64u, (m->columns + 255u) / 256u));
    if (m->format == kFmtQ4_K) dequant_row_kernel<kFmtQ4_K><<<blocks, 256, 0, stream>>>(p, row, out_device, codes_device);
    else if (m->format == kFmtQ8_0) dequant_row_kernel<kFmtQ8_0><<<blocks, 256, 0, stream>>>(p, row, out_device, codes_device);
    else dequant_row_kernel<kFmtAffine8><<<blocks, 256, 0, stream>>>(p, row, out_device, codes_device);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

}  // namespace sb
