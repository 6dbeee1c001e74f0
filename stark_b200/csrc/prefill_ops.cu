// Row-wise operators of the batched prompt path and causal attention over the paged cache (sm_100a).
// Each reproduces, for every row of a chunk, what the one-token kernels do for their single row -- same
// formulas, same rounding points -- so that a prompt row costs the same arithmetic whichever path takes it.
#include <algorithm>

#include "device_math.cuh"
#include "prefill.cuh"
#include "tunables.cuh"

namespace sb {

namespace {

// A launch that may begin while the kernel before it is still running (programmatic stream serialization): the
// kernels launched through this call griddepcontrol.wait before they touch anything that kernel writes.
template <typename... Params, typename... Args>
cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}


// ------------------------------------------------------------------------------------------ embedding rows
// input_embedding_lookup.rs:17-160: row `token` of the quantized table, scale * code + bias with two roundings,
// then bf16.  Same record arithmetic as embedding_row_kernel (ops.cu), one row per blockIdx.y.
__global__ void embed_rows_kernel(const uint8_t *__restrict__ data, uint32_t rows, uint32_t columns,
                                  uint32_t pair_halves, const uint32_t *__restrict__ tokens, uint16_t *out) {
    const uint32_t token = tokens[blockIdx.y];
    uint16_t *dst = out + (size_t)blockIdx.y * columns;
    const uint32_t groups = columns / 64u;
    for (uint32_t col = blockIdx.x * blockDim.x + threadIdx.x; col < columns; col += gridDim.x * blockDim.x) {
        if (token >= rows) {  // input_embedding_lookup.rs:64-68
            dst[col] = 0;
            continue;
        }
        uint32_t tile, r;
        if (!pair_halves) {
            tile = token / 16u;
            r = token % 16u;
        } else {
            const uint32_t half = rows / 2u, inner = token % half;
            tile = 2u * (inner / 16u) + (token >= half ? 1u : 0u);
            r = inner % 16u;
        }
        const uint32_t g = r & 7u, hrow = r >> 3;
        const uint32_t kg = col / 64u, c = col % 64u;
        const uint32_t t = c / 16u, j = (c % 16u) / 4u, r2 = (c % 4u) / 2u, e = c & 1u;
        const uint8_t *rec = data + ((size_t)tile * groups + kg) * kA4RecordBytes;
        const uint32_t word = *reinterpret_cast<const uint32_t *>(rec + (g * 4u + t) * 16u + j * 4u);
        const uint32_t q = (word >> (4u * (4u * e + 2u * r2 + hrow))) & 15u;
        const uint16_t *planes = reinterpret_cast<const uint16_t *>(rec + 512u);
        const float scale = bf16_bits_to_f32(planes[2u * g + hrow]);
        const float bias = bf16_bits_to_f32(planes[16u + 2u * g + hrow]);
        dst[col] = f32_to_bf16_bits(__fadd_rn(__fmul_rn(scale, (float)q), bias));
    }
}

// ------------------------------------------------------------------------------------------ RMS norm rows
// normalization.rs:13-191, only-normalization mode: f32 sum of squares, rms_inv = 1 / sqrt(mean + eps),
// bf16(x * rms_inv) * bf16(weight) rounded to bf16.  One CTA per row, the row held in registers.
constexpr int kNormThreads = 256;
constexpr int kNormMaxChunks = 6;  // 8 elements each: rows of up to 12288
__global__ void __launch_bounds__(kNormThreads) rmsnorm_rows_kernel(const uint16_t *__restrict__ h,
                                                                    const float *__restrict__ weight,
                                                                    uint16_t *__restrict__ out, uint32_t d, float eps,
                                                                    uint32_t in_stride, uint32_t out_stride) {
    __shared__ float red[kNormThreads / 32];
    const uint32_t tid = threadIdx.x, chunks = d / 8u;
    const uint4 *src = reinterpret_cast<const uint4 *>(h + (size_t)blockIdx.x * in_stride);
    uint4 v[kNormMaxChunks];
    float sumsq = 0.0f;
#pragma unroll
    for (int r = 0; r < kNormMaxChunks; ++r) {
        const uint32_t c = tid + r * kNormThreads;
        v[r] = c < chunks ? src[c] : make_uint4(0u, 0u, 0u, 0u);
        const uint32_t w4[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float a = __uint_as_float(w4[i] << 16), b = __uint_as_float(w4[i] & 0xffff0000u);
            sumsq = fmaf(a, a, sumsq);
            sumsq = fmaf(b, b, sumsq);
        }
    }
    sumsq = warp_sum(sumsq);
    if ((tid & 31u) == 0) red[tid >> 5] = sumsq;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormThreads / 32; ++i) total += red[i];
    const float rms_inv = 1.0f / sqrtf(total / (float)d + eps);
    uint4 *dst = reinterpret_cast<uint4 *>(out + (size_t)blockIdx.x * out_stride);
#pragma unroll
    for (int r = 0; r < kNormMaxChunks; ++r) {
        const uint32_t c = tid + r * kNormThreads;
        if (c >= chunks) continue;
        const float4 w0 = reinterpret_cast<const float4 *>(weight)[2 * c], w1 = reinterpret_cast<const float4 *>(weight)[2 * c + 1];
        const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        const uint32_t w4[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t n2 = f32x2_to_bf16x2(__uint_as_float(w4[i] << 16) * rms_inv,
                                                __uint_as_float(w4[i] & 0xffff0000u) * rms_inv);
            o[i] = f32x2_to_bf16x2(__uint_as_float(n2 << 16) * bf16_round(wf[2 * i]),
                                   __uint_as_float(n2 & 0xffff0000u) * bf16_round(wf[2 * i + 1]));
        }
        dst[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ------------------------------------------------------------------------------------------ row arg-max
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const uint16_t *__restrict__ rows, uint32_t n, uint32_t *first) {
    __shared__ float vs[32];
    __shared__ uint32_t is[32];
    const uint16_t *row = rows + (size_t)blockIdx.x * n;
    float best = -INFINITY;
    uint32_t bi = 0xffffffffu;
    auto consider = [&](uint32_t bits, uint32_t i) {
        const float v = bf16_bits_to_f32((uint16_t)bits);
        const float key = isfinite(v) ? v : INFINITY;  // a non-finite logit must surface
        if (key > best || (key == best && i < bi)) {
            best = key;
            bi = i;
        }
    };
    // eight values per 16-byte load where the row allows it (the loads of several iterations are in flight at
    // once: they do not depend on the comparisons), the rest one by one
    const bool wide = ((reinterpret_cast<uintptr_t>(row) | ((size_t)n * 2u)) & 15u) == 0;
    const uint32_t chunks = wide ? n / 8u : 0u;
#pragma unroll 4
    for (uint32_t c = threadIdx.x; c < chunks; c += blockDim.x) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(row) + c);
        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (uint32_t e = 0; e < 4; ++e) {
            consider(w4[e] & 0xffffu, c * 8u + 2u * e);
            consider(w4[e] >> 16, c * 8u + 2u * e + 1u);
        }
    }
    for (uint32_t i = chunks * 8u + threadIdx.x; i < n; i += blockDim.x) consider(row[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) {
            best = ov;
            bi = oi;
        }
    }
    if ((threadIdx.x & 31u) == 0) {
        vs[threadIdx.x >> 5] = best;
        is[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < blockDim.x / 32u; ++w)
            if (vs[w] > best || (vs[w] == best && is[w] < bi)) {
                best = vs[w];
                bi = is[w];
            }
        first[blockIdx.x] = isfinite(best) ? bi : 0xffffffffu;
    }
}

// ------------------------------------------------------------------------------------------ head norm + RoPE + append
// One warp per (row, head): q heads in place, k heads into the cache row of the token's position, v heads copied
// (qkv_norm.rs:8-111, attention_prepare.rs:7-43,187-316; the helper is the one the decode attention uses).
struct RopeParams {
    uint16_t *qkv;
    uint16_t *keys, *values;
    const int32_t *block_table;
    const float *q_norm, *k_norm, *rope_cos, *rope_sin;
    uint32_t first_pos, q_heads, kv_heads;
    float eps;
};
__global__ void __launch_bounds__(128) rope_append_rows_kernel(const RopeParams p) {
    __shared__ __align__(16) uint16_t head_s[4][kHeadDim];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t head = blockIdx.x * 4u + warp, row = blockIdx.y;
    const uint32_t heads = p.q_heads + 2u * p.kv_heads;
    pdl_launch_dependents();
    pdl_wait();  // the rows come from the projection before this launch
    if (head >= heads) return;
    const uint32_t pos = p.first_pos + row;
    uint16_t *src = p.qkv + ((size_t)row * heads + head) * kHeadDim;
    if (head < p.q_heads) {
        warp_head_norm_rope(src, p.q_norm, p.rope_cos ? p.rope_cos + (size_t)pos * kHeadDim : nullptr,
                            p.rope_sin ? p.rope_sin + (size_t)pos * kHeadDim : nullptr, p.eps, lane, head_s[warp]);
        __syncwarp();
        reinterpret_cast<uint2 *>(src)[lane] = reinterpret_cast<const uint2 *>(head_s[warp])[lane];
        return;
    }
    const bool is_key = head < p.q_heads + p.kv_heads;
    const uint32_t kvh = is_key ? head - p.q_heads : head - p.q_heads - p.kv_heads;
    const size_t cache_row = ((size_t)p.block_table[pos / kPageTokens] * p.kv_heads + kvh) * kPageTokens + pos % kPageTokens;
    if (is_key) {
        warp_head_norm_rope(src, p.k_norm, p.rope_cos ? p.rope_cos + (size_t)pos * kHeadDim : nullptr,
                            p.rope_sin ? p.rope_sin + (size_t)pos * kHeadDim : nullptr, p.eps, lane, head_s[warp]);
        __syncwarp();
        reinterpret_cast<uint2 *>(p.keys + cache_row * kHeadDim)[lane] = reinterpret_cast<const uint2 *>(head_s[warp])[lane];
    } else {
        reinterpret_cast<uint2 *>(p.values + cache_row * kHeadDim)[lane] = reinterpret_cast<const uint2 *>(src)[lane];
    }
}

// ------------------------------------------------------------------------------------------ causal attention
// attention_single_pass.rs:11-133 for every row of the chunk: scores q.k in f32 scaled by 1/sqrt(d), online
// softmax in f32, output rounded to bf16.  A CTA takes one KV head and a block of rows; warp w works on query
// head (w mod G) of the group and row block (w div G), 16 rows each, so every K / V page (one 64-key tile,
// 16 KB each, contiguous in the paged cache) is fetched once for the whole group.  Tensor cores through
// mma.sync.m16n8k16 (bf16): S = Q K^T with the rows as M, then O += P V with P carried as bf16 hi + lo so that
// the weights keep ~16 bits, as in the decode kernel.
struct PrefillAttnParams {
    const uint16_t *qkv;
    const uint16_t *keys, *values;
    const int32_t *block_table;
    uint16_t *out;
    uint32_t m, first_pos, q_heads, kv_heads, gqa, row_blocks;  // row_blocks = 16-row blocks per CTA
    float scale;
    float *partials;  // SPLIT: [m][q_heads][splits][kPartialFloats] = running maximum, denominator, unnormalized output
    uint32_t splits;
};
constexpr uint32_t kPartialFloats = 4u + kHeadDim;

// SPLIT: a handful of rows over a long cache (the rows a speculative round verifies).  The key tiles are divided
// among gridDim.z CTAs per (row block, KV head); each leaves its running maximum, denominator and unnormalized
// output, which prefill_attention_merge_kernel combines -- the same scheme as the one-row decode kernel.
// PLO: the probabilities enter the second product as bf16 hi + lo (about 16 bits, as in the one-row kernel).
// Carrying them as one bf16 saves a third of the tensor-core work and was measured: the prompt of the 8B shape
// went from 91.4 to 86.9 ms, and the teacher-forced agreement with the oracle after a chunked prompt fell from
// 60/60 to 58/60 picks inside the near-tie window, below the 0.99 bar.  Parity comes first: PLO stays on.
template <int WARPS, bool SPLIT, bool PLO = true>
__global__ void __launch_bounds__(WARPS * 32) prefill_attention_kernel(const PrefillAttnParams p) {
    extern __shared__ __align__(128) uint8_t pa_smem[];  // [2][K, V][64 rows][272 B]
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t kvh = blockIdx.y;
    pdl_launch_dependents();
    pdl_wait();  // query rows and the appended cache rows come from the launch before this one
    const uint32_t rows_per_cta = 16u * p.row_blocks;
    // causal: a block of late rows reads the most keys, so the late blocks are issued first and the short ones fill
    // the tail of the launch
    const uint32_t row0_cta = (SPLIT ? blockIdx.x : gridDim.x - 1u - blockIdx.x) * rows_per_cta;
    const uint32_t head = kvh * p.gqa + warp % p.gqa;
    const uint32_t row0 = row0_cta + 16u * (warp / p.gqa);  // this warp's 16 rows
    const uint32_t heads = p.q_heads + 2u * p.kv_heads;
    const uint32_t last_row = min(p.m, row0_cta + rows_per_cta) - 1u;
    const uint32_t all_tiles = (p.first_pos + last_row) / kPageTokens + 1u;
    const uint32_t tile_begin = SPLIT ? (uint32_t)((uint64_t)all_tiles * blockIdx.z / p.splits) : 0u;
    const uint32_t ntiles = SPLIT ? (uint32_t)((uint64_t)all_tiles * (blockIdx.z + 1u) / p.splits) : all_tiles;

    auto issue_tile = [&](uint32_t tile, uint32_t buf) {
        const size_t page = ((size_t)p.block_table[tile] * p.kv_heads + kvh) * kPageTokens * kHeadDim;
        const uint8_t *ksrc = reinterpret_cast<const uint8_t *>(p.keys + page);
        const uint8_t *vsrc = reinterpret_cast<const uint8_t *>(p.values + page);
        uint8_t *kd = pa_smem + (size_t)(buf * 2u) * kTileBytes, *vd = kd + kTileBytes;
        for (uint32_t idx = tid; idx < kPageTokens * 16u; idx += WARPS * 32u) {
            const uint32_t r = idx >> 4, ch = idx & 15u;
            cp_async16(kd + r * kTileRowBytes + ch * 16u, ksrc + r * 256u + ch * 16u);
            cp_async16(vd + r * kTileRowBytes + ch * 16u, vsrc + r * 256u + ch * 16u);
        }
    };
    if (tile_begin < ntiles) issue_tile(tile_begin, 0);
    cp_async_commit();
    if (tile_begin + 1u < ntiles) issue_tile(tile_begin + 1u, 1);
    cp_async_commit();

    // Q as the A operand: rows row0 + g and row0 + g + 8, dims 16 kk + {2t, 2t+1} and + 8
    uint32_t qa[8][4];
    const uint32_t ra = row0 + g, rb = row0 + g + 8u;
    const uint16_t *qa_row = p.qkv + ((size_t)min(ra, p.m - 1u) * heads + head) * kHeadDim;
    const uint16_t *qb_row = p.qkv + ((size_t)min(rb, p.m - 1u) * heads + head) * kHeadDim;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        qa[kk][0] = *reinterpret_cast<const uint32_t *>(qa_row + kk * 16 + 2 * t);
        qa[kk][1] = *reinterpret_cast<const uint32_t *>(qb_row + kk * 16 + 2 * t);
        qa[kk][2] = *reinterpret_cast<const uint32_t *>(qa_row + kk * 16 + 8 + 2 * t);
        qa[kk][3] = *reinterpret_cast<const uint32_t *>(qb_row + kk * 16 + 8 + 2 * t);
    }
    const uint32_t pos_a = p.first_pos + ra, pos_b = p.first_pos + rb;  // last key each row may see

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[16][4];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
    const uint32_t lrow = lane & 7u, lmat = lane >> 3;

    for (uint32_t tile = tile_begin; tile < ntiles; ++tile) {
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t buf = (tile - tile_begin) & 1u;
        const uint8_t *kt = pa_smem + (size_t)(buf * 2u) * kTileBytes, *vt = kt + kTileBytes;
        const uint32_t key0 = tile * kPageTokens;
        if (key0 <= p.first_pos + min(row0 + 15u, p.m - 1u) && row0 < p.m) {  // some row of the warp sees this tile
            // ---- S = Q K^T: 8 key blocks of 8 keys; K as the B operand (n = key, k = dim) straight from [key][dim]
            float s[8][4];
#pragma unroll
            for (int nb = 0; nb < 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
                for (int nb2 = 0; nb2 < 4; ++nb2) {
                    // matrices: (keys 16 nb2 + 0-7, dims 16 kk + 0-7), (same keys, dims + 8), (keys + 8, dims 0-7), (keys + 8, dims + 8)
                    uint32_t kb[4];
                    ldmatrix_x4(kb, kt + (16u * nb2 + (lmat >> 1) * 8u + lrow) * kTileRowBytes + (kk * 16u + (lmat & 1u) * 8u) * 2u);
                    mma_m16n8k16_bf16(s[2 * nb2], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], kb[0], kb[1]);
                    mma_m16n8k16_bf16(s[2 * nb2 + 1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], kb[2], kb[3]);
                }
            }
            // s[nb][0..1]: row a, keys key0 + 8 nb + 2t, +1;  s[nb][2..3]: row b
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t key = key0 + 8u * nb + 2u * t + e;
                    s[nb][e] = key <= pos_a ? s[nb][e] * p.scale : -INFINITY;
                    s[nb][2 + e] = key <= pos_b ? s[nb][2 + e] * p.scale : -INFINITY;
                    tmax[0] = fmaxf(tmax[0], s[nb][e]);
                    tmax[1] = fmaxf(tmax[1], s[nb][2 + e]);
                }
            }
            float factor[2], m_new[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 1));
                tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 2));
                m_new[j] = fmaxf(m_run[j], tmax[j]);
                // a row past the end of the chunk, or one that sees no key of this tile, keeps -inf
                factor[j] = (m_run[j] == -INFINITY) ? 0.0f : expf(m_run[j] - m_new[j]);
            }
            float tsum[2] = {0.0f, 0.0f};
            uint32_t ph[8][2], pl[8][2];
#pragma unroll
            for (int nb = 0; nb < 8; ++nb) {
                float e4[4];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    e4[e] = m_new[0] == -INFINITY ? 0.0f : expf(s[nb][e] - m_new[0]);
                    e4[2 + e] = m_new[1] == -INFINITY ? 0.0f : expf(s[nb][2 + e] - m_new[1]);
                }
                tsum[0] += e4[0] + e4[1];
                tsum[1] += e4[2] + e4[3];
                if (PLO) {
                    split_bf16x2(e4[0], e4[1], ph[nb][0], pl[nb][0]);  // row a, keys 8 nb + 2t, +1
                    split_bf16x2(e4[2], e4[3], ph[nb][1], pl[nb][1]);  // row b
                } else {
                    ph[nb][0] = f32x2_to_bf16x2(e4[0], e4[1]);
                    ph[nb][1] = f32x2_to_bf16x2(e4[2], e4[3]);
                }
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                tsum[j] += __shfl_xor_sync(0xffffffffu, tsum[j], 1);
                tsum[j] += __shfl_xor_sync(0xffffffffu, tsum[j], 2);
                l_run[j] = l_run[j] * factor[j] + tsum[j];
                m_run[j] = m_new[j];
            }
#pragma unroll
            for (int nt = 0; nt < 16; ++nt) {
                o[nt][0] *= factor[0];
                o[nt][1] *= factor[0];
                o[nt][2] *= factor[1];
                o[nt][3] *= factor[1];
            }
            // ---- O += P V: P (the C layout of two adjacent key blocks) is the A operand of a 16-key step;
            // V as the B operand (n = dim, k = key) is the transpose of the [key][dim] tile: ldmatrix.trans
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {  // 16 keys per step
                const uint32_t a_h[4] = {ph[2 * ks][0], ph[2 * ks][1], ph[2 * ks + 1][0], ph[2 * ks + 1][1]};
                const uint32_t a_l[4] = {pl[2 * ks][0], pl[2 * ks][1], pl[2 * ks + 1][0], pl[2 * ks + 1][1]};
#pragma unroll
                for (int nt2 = 0; nt2 < 8; ++nt2) {
                    // matrices: (keys 16 ks + 0-7, dims 16 nt2 + 0-7), (keys + 8, same dims), (keys 0-7, dims + 8), (keys + 8, dims + 8)
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, vt + (16u * ks + (lmat & 1u) * 8u + lrow) * kTileRowBytes + (nt2 * 16u + (lmat >> 1) * 8u) * 2u);
                    mma_m16n8k16_bf16(o[2 * nt2], a_h[0], a_h[1], a_h[2], a_h[3], vb[0], vb[1]);
                    if (PLO) mma_m16n8k16_bf16(o[2 * nt2], a_l[0], a_l[1], a_l[2], a_l[3], vb[0], vb[1]);
                    mma_m16n8k16_bf16(o[2 * nt2 + 1], a_h[0], a_h[1], a_h[2], a_h[3], vb[2], vb[3]);
                    if (PLO) mma_m16n8k16_bf16(o[2 * nt2 + 1], a_l[0], a_l[1], a_l[2], a_l[3], vb[2], vb[3]);
                }
            }
        }
        __syncthreads();  // the buffer of this tile is free for tile + 2
        if (tile + 2u < ntiles) issue_tile(tile + 2u, buf);
        cp_async_commit();
    }
    cp_async_wait<0>();

    // o[nt][0..1]: row a, dims 8 nt + 2t, +1;  o[nt][2..3]: row b
    if (SPLIT) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t r = j ? rb : ra;
            if (r >= p.m) continue;
            float *dst = p.partials + (((size_t)r * p.q_heads + head) * p.splits + blockIdx.z) * kPartialFloats;
            if (t == 0) {
                dst[0] = m_run[j];
                dst[1] = l_run[j];
            }
#pragma unroll
            for (int nt = 0; nt < 16; ++nt)
                *reinterpret_cast<float2 *>(dst + 4 + 8 * nt + 2 * t) = make_float2(o[nt][2 * j], o[nt][2 * j + 1]);
        }
        return;
    }
    const float inv_a = l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f, inv_b = l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f;
    if (ra < p.m) {
        uint16_t *dst = p.out + ((size_t)ra * p.q_heads + head) * kHeadDim;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt)
            *reinterpret_cast<uint32_t *>(dst + 8 * nt + 2 * t) = f32x2_to_bf16x2(o[nt][0] * inv_a, o[nt][1] * inv_a);
    }
    if (rb < p.m) {
        uint16_t *dst = p.out + ((size_t)rb * p.q_heads + head) * kHeadDim;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt)
            *reinterpret_cast<uint32_t *>(dst + 8 * nt + 2 * t) = f32x2_to_bf16x2(o[nt][2] * inv_b, o[nt][3] * inv_b);
    }
}

// A handful of rows (the verify pass of a speculative round) in the one-row kernel's form: the KEYS are the M rows of
// both tensor-core products and the columns are (row, head of the group) pairs, 8 per column tile, so that no
// tensor-core work is spent on padding rows (the 16-row tile kernel above runs 5 rows as 16):
//   S^T[key, col] = K[key, :] Q_col^T          8 NT mma per 16 keys, the K fragments shared by the column tiles
//   O^T[dim, col] += V^T[dim, key] P^T         16 NT mma per 16 keys (P as bf16 hi + lo), the V fragments shared
// One CTA per (KV head, split of the key tiles); each of its four warps owns 16 keys of a 64-key tile with its own
// online softmax per column, merged once at the end; the causal limit is per column (row r sees keys up to
// first_pos + r).  Query rows are already normalized and rotated, the new keys and values already in the cache
// (rope_append_rows_kernel).  Partials go where prefill_attention_merge_kernel expects them.
template <int NT>
__global__ void __launch_bounds__(128) rows_attention_kernel(const PrefillAttnParams p) {
    extern __shared__ __align__(128) uint8_t ra_smem[];  // [2][K, V][64 rows][272 B], reused for the warps' outputs
    __shared__ float ml_s[4][NT * 8][2];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t kvh = blockIdx.y, G = p.gqa, ncols = p.m * G;
    pdl_launch_dependents();
    pdl_wait();  // query rows and the appended cache rows come from the launch before this one
    const uint32_t heads = p.q_heads + 2u * p.kv_heads;
    const uint32_t all_tiles = (p.first_pos + p.m - 1u) / kPageTokens + 1u;
    const uint32_t tile_begin = (uint32_t)((uint64_t)all_tiles * blockIdx.z / p.splits);
    const uint32_t tile_end = (uint32_t)((uint64_t)all_tiles * (blockIdx.z + 1u) / p.splits);

    auto issue_tile = [&](uint32_t tile, uint32_t buf) {
        const size_t page = ((size_t)p.block_table[tile] * p.kv_heads + kvh) * kPageTokens * kHeadDim;
        const uint8_t *ksrc = reinterpret_cast<const uint8_t *>(p.keys + page);
        const uint8_t *vsrc = reinterpret_cast<const uint8_t *>(p.values + page);
        uint8_t *kd = ra_smem + (size_t)(buf * 2u) * kTileBytes, *vd = kd + kTileBytes;
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {  // 64 rows x 16 chunks of 16 B per tile
            const uint32_t idx = tid + i * 128u, r = idx >> 4, ch = idx & 15u;
            cp_async16(kd + r * kTileRowBytes + ch * 16u, ksrc + r * 256u + ch * 16u);
            cp_async16(vd + r * kTileRowBytes + ch * 16u, vsrc + r * 256u + ch * 16u);
        }
    };
    if (tile_begin < tile_end) issue_tile(tile_begin, 0);
    cp_async_commit();
    if (tile_begin + 1u < tile_end) issue_tile(tile_begin + 1u, 1);
    cp_async_commit();

    // Q^T as the B operand: lane (g, t) holds column 8 j + g, dims 16 kk + {2t, 2t+1} and + 8
    uint32_t qb[NT][8][2];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const uint32_t col = 8u * j + g;
        const uint16_t *q = col < ncols ? p.qkv + ((size_t)(col / G) * heads + kvh * G + col % G) * kHeadDim : nullptr;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            qb[j][kk][0] = q ? *reinterpret_cast<const uint32_t *>(q + kk * 16 + 2 * t) : 0u;
            qb[j][kk][1] = q ? *reinterpret_cast<const uint32_t *>(q + kk * 16 + 8 + 2 * t) : 0u;
        }
    }
    // last key each of this lane's columns (8 j + 2t, + 1 in the accumulator layout) may see; -1: no such column
    int32_t limit[NT][2];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const uint32_t col = 8u * j + 2u * t + e;
            limit[j][e] = col < ncols ? (int32_t)(p.first_pos + col / G) : -1;
        }
    float m_run[NT][2], l_run[NT][2], o[NT][8][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        m_run[j][0] = m_run[j][1] = -INFINITY;
        l_run[j][0] = l_run[j][1] = 0.0f;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) o[j][mt][0] = o[j][mt][1] = o[j][mt][2] = o[j][mt][3] = 0.0f;
    }
    const uint32_t lrow = lane & 7u, lmat = lane >> 3;
    const uint32_t k0 = warp * 16u;
    const int32_t last_key = (int32_t)(p.first_pos + p.m - 1u);

    for (uint32_t tile = tile_begin; tile < tile_end; ++tile) {
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t buf = (tile - tile_begin) & 1u;
        const uint8_t *kt = ra_smem + (size_t)(buf * 2u) * kTileBytes, *vt = kt + kTileBytes;
        const int32_t key_a = (int32_t)(tile * kPageTokens + k0 + g), key_b = key_a + 8;
        if ((int32_t)(tile * kPageTokens + k0) <= last_key) {  // some column sees a key of this warp's slab
            float sc[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                uint32_t ka[4];
                ldmatrix_x4(ka, kt + (k0 + (lmat & 1u) * 8u + lrow) * kTileRowBytes + (kk * 16u + (lmat >> 1) * 8u) * 2u);
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_m16n8k16_bf16(sc[j], ka[0], ka[1], ka[2], ka[3], qb[j][kk][0], qb[j][kk][1]);
            }
            uint32_t bh[NT][2], bl[NT][2];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                float e4[4], factor[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float sa = key_a <= limit[j][e] ? sc[j][e] * p.scale : -INFINITY;
                    const float sb = key_b <= limit[j][e] ? sc[j][2 + e] * p.scale : -INFINITY;
                    float tm = fmaxf(sa, sb);
                    tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 4));
                    tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 8));
                    tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 16));
                    const float m_new = fmaxf(m_run[j][e], tm);
                    const bool none = m_new == -INFINITY;  // the column sees no key so far
                    factor[e] = m_run[j][e] == -INFINITY ? 0.0f : expf(m_run[j][e] - m_new);
                    e4[e] = none ? 0.0f : expf(sa - m_new);
                    e4[2 + e] = none ? 0.0f : expf(sb - m_new);
                    float ts = e4[e] + e4[2 + e];
                    ts += __shfl_xor_sync(0xffffffffu, ts, 4);
                    ts += __shfl_xor_sync(0xffffffffu, ts, 8);
                    ts += __shfl_xor_sync(0xffffffffu, ts, 16);
                    l_run[j][e] = l_run[j][e] * factor[e] + ts;
                    m_run[j][e] = m_new;
                }
#pragma unroll
                for (int mt = 0; mt < 8; ++mt) {
                    o[j][mt][0] *= factor[0];
                    o[j][mt][1] *= factor[1];
                    o[j][mt][2] *= factor[0];
                    o[j][mt][3] *= factor[1];
                }
                uint32_t ph[2], pl[2];
                split_bf16x2(e4[0], e4[1], ph[0], pl[0]);
                split_bf16x2(e4[2], e4[3], ph[1], pl[1]);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    bh[j][i] = movmatrix_trans(ph[i]);
                    bl[j][i] = movmatrix_trans(pl[i]);
                }
            }
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                uint32_t va4[4];
                ldmatrix_x4_trans(va4, vt + (k0 + (lmat >> 1) * 8u + lrow) * kTileRowBytes + (mt * 16u + (lmat & 1u) * 8u) * 2u);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    mma_m16n8k16_bf16(o[j][mt], va4[0], va4[1], va4[2], va4[3], bh[j][0], bh[j][1]);
                    mma_m16n8k16_bf16(o[j][mt], va4[0], va4[1], va4[2], va4[3], bl[j][0], bl[j][1]);
                }
            }
        }
        __syncthreads();  // the buffer of this tile is free for tile + 2
        if (tile + 2u < tile_end) issue_tile(tile + 2u, buf);
        cp_async_commit();
    }
    cp_async_wait<0>();

    // ---- merge the four warps' states, publish this split's partial (max, sum, unnormalized output) per column
    if (g == 0) {
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                ml_s[warp][8 * j + 2 * t + e][0] = m_run[j][e];
                ml_s[warp][8 * j + 2 * t + e][1] = l_run[j][e];
            }
    }
    __syncthreads();  // also: nobody reads the tiles any more
    float *o_s = reinterpret_cast<float *>(ra_smem);  // [4 warps][NT * 8 columns][128] f32
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const uint32_t col = 8u * j + 2u * t + e;
            float mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) mx = fmaxf(mx, ml_s[w][col][0]);
            const float f = m_run[j][e] == -INFINITY ? 0.0f : expf(m_run[j][e] - mx);
            float *dst = o_s + ((size_t)warp * (NT * 8) + col) * kHeadDim;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                dst[mt * 16 + g] = o[j][mt][e] * f;
                dst[mt * 16 + g + 8] = o[j][mt][2 + e] * f;
            }
        }
    __syncthreads();
    for (uint32_t i = tid; i < ncols * kHeadDim; i += 128u) {
        const uint32_t col = i >> 7, d = i & 127u;
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) acc += o_s[((size_t)w * (NT * 8) + col) * kHeadDim + d];
        float *dst = p.partials + (((size_t)(col / G) * p.q_heads + kvh * G + col % G) * p.splits + blockIdx.z) * kPartialFloats;
        dst[4 + d] = acc;
    }
    if (tid < ncols) {
        float mx = -INFINITY, l = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) mx = fmaxf(mx, ml_s[w][tid][0]);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = ml_s[w][tid][0];
            l += mw == -INFINITY ? 0.0f : ml_s[w][tid][1] * expf(mw - mx);
        }
        float *dst = p.partials + (((size_t)(tid / G) * p.q_heads + kvh * G + tid % G) * p.splits + blockIdx.z) * kPartialFloats;
        dst[0] = mx;
        dst[1] = l;
    }
}

// out[row][head][d] = sum_s w_s o_s[d] / sum_s w_s l_s with w_s = exp(m_s - max m): one CTA per (row, head)
__global__ void __launch_bounds__(kHeadDim) prefill_attention_merge_kernel(const float *partials, uint16_t *out,
                                                                           uint32_t q_heads, uint32_t splits) {
    const uint32_t row = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
    pdl_launch_dependents();  // a matvec that follows may start filling its weight ring; it awaits this grid itself
    pdl_wait();               // the partials come from the launch before this one
    const float *src = partials + ((size_t)row * q_heads + head) * splits * kPartialFloats;
    float top = -INFINITY;
    for (uint32_t s = 0; s < splits; ++s) top = fmaxf(top, src[(size_t)s * kPartialFloats]);
    float denom = 0.0f, acc = 0.0f;
    for (uint32_t s = 0; s < splits; ++s) {
        const float *ps = src + (size_t)s * kPartialFloats;
        const float w = ps[0] == -INFINITY ? 0.0f : expf(ps[0] - top);
        denom += w * ps[1];
        acc += w * ps[4 + d];
    }
    const float v = denom > 0.0f ? acc / denom : 0.0f;
    out[((size_t)row * q_heads + head) * kHeadDim + d] = f32_to_bf16_bits(v);
}

}  // namespace

stark_b200_status embed_rows_launch(const QMatrix *table, const uint32_t *tokens, uint32_t m, uint16_t *h,
                                    cudaStream_t stream) {
    if (!table || table->format != kFmtAffine4 || !tokens || !h || m == 0) return STARK_B200_INVALID_ARGUMENT;
    const dim3 grid(std::max(1u, std::min(16u, table->columns / 256u)), m);
    embed_rows_kernel<<<grid, 256, 0, stream>>>(table->data, table->rows, table->columns, table->pair_halves, tokens, h);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status rmsnorm_rows_launch(const uint16_t *h, const float *weight, uint16_t *out, uint32_t m, uint32_t d,
                                      float eps, cudaStream_t stream, uint32_t in_stride, uint32_t out_stride) {
    if (!h || !weight || !out || m == 0 || d % 8u != 0 || d > (uint32_t)kNormThreads * kNormMaxChunks * 8u ||
        in_stride % 8u != 0 || out_stride % 8u != 0)
        return STARK_B200_INVALID_ARGUMENT;
    rmsnorm_rows_kernel<<<m, kNormThreads, 0, stream>>>(h, weight, out, d, eps, in_stride ? in_stride : d,
                                                        out_stride ? out_stride : d);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status argmax_rows_launch(const uint16_t *rows, uint32_t m, uint32_t n, uint32_t *first, cudaStream_t stream) {
    if (!rows || !first || m == 0 || n == 0) return STARK_B200_INVALID_ARGUMENT;
    argmax_rows_kernel<<<m, 1024, 0, stream>>>(rows, n, first);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

stark_b200_status rope_append_rows_launch(const RopeAppendArgs &a, cudaStream_t stream) {
    if (!a.qkv || !a.kv.keys || !a.kv.values || !a.block_table || a.m == 0) return STARK_B200_INVALID_ARGUMENT;
    RopeParams p{a.qkv, a.kv.keys, a.kv.values, a.block_table, a.q_norm, a.k_norm, a.rope_cos, a.rope_sin,
                 a.first_pos, a.q_heads, a.kv_heads, a.eps};
    const uint32_t heads = a.q_heads + 2u * a.kv_heads;
    SB_CUDA(launch_dependent(rope_append_rows_kernel, dim3((heads + 3u) / 4u, a.m), dim3(128), 0, stream, p));
    return STARK_B200_OK;
}

stark_b200_status prefill_attention_launch(const PrefillAttnArgs &a, cudaStream_t stream) {
    if (!a.qkv || !a.kv.keys || !a.kv.values || !a.block_table || !a.out || a.m == 0) return STARK_B200_INVALID_ARGUMENT;
    if (a.kv_heads == 0 || a.q_heads % a.kv_heads != 0) return STARK_B200_UNSUPPORTED;
    const uint32_t gqa = a.q_heads / a.kv_heads;
    if (a.m > 16u && tunables().prefill_attn_tc && prefill_attention_tc_supports(a)) return prefill_attention_tc_launch(a, stream);
    if (gqa != 1u && gqa != 2u && gqa != 4u && gqa != 8u) return STARK_B200_UNSUPPORTED;
    PrefillAttnParams p{};
    p.qkv = a.qkv;
    p.keys = a.kv.keys;
    p.values = a.kv.values;
    p.block_table = a.block_table;
    p.out = a.out;
    p.m = a.m;
    p.first_pos = a.first_pos;
    p.q_heads = a.q_heads;
    p.kv_heads = a.kv_heads;
    p.gqa = gqa;
    p.scale = a.scale;
    const uint32_t smem = 4u * kTileBytes;
    static SmemOptIn once4, once8, once4s, once8s;
    // few rows over a long cache: divide the key tiles among CTAs so that the whole GPU reads the cache
    uint32_t splits = 0;
    if (a.partials && a.max_splits > 1u && a.m <= 16u) {
        const uint32_t tiles = (a.first_pos + a.m - 1u) / kPageTokens + 1u;
        // two CTAs per SM (70 KB of shared memory each): about 300 CTAs share the cache's key tiles
        splits = std::min(std::min(tiles, a.max_splits), std::max(1u, 296u / a.kv_heads));
        if (splits < 2u) splits = 0;
    }
    p.partials = a.partials;
    p.splits = splits;
    const uint32_t column_tiles = (a.m * gqa + 7u) / 8u;
    if (splits && column_tiles <= 4u && tunables().rows_attention) {
        // a handful of (row, head) columns: the keys-as-rows form
        static SmemOptIn once_rows[4];
        void (*fn)(PrefillAttnParams) = column_tiles == 1u ? rows_attention_kernel<1>
                                        : column_tiles == 2u ? rows_attention_kernel<2>
                                        : column_tiles == 3u ? rows_attention_kernel<3> : rows_attention_kernel<4>;
        if (stark_b200_status s = ensure_dynamic_smem(fn, (int)smem, once_rows[column_tiles - 1u])) return s;
        SB_CUDA(launch_dependent(fn, dim3(1, a.kv_heads, splits), dim3(128), smem, stream, p));
    } else if (gqa == 8u || (!splits && a.m > 16u && tunables().prefill_attn_warps == 8u)) {
        p.row_blocks = 8u / gqa;  // 8 warps a CTA: a key / value tile serves 8 / gqa blocks of 16 rows
        if (splits) {
            if (stark_b200_status s = ensure_dynamic_smem(prefill_attention_kernel<8, true>, (int)smem, once8s)) return s;
            SB_CUDA(launch_dependent(prefill_attention_kernel<8, true>, dim3(1, a.kv_heads, splits), dim3(256), smem, stream, p));
        } else {
            if (stark_b200_status s = ensure_dynamic_smem(prefill_attention_kernel<8, false>, (int)smem, once8)) return s;
            const uint32_t rows_per_cta = 16u * p.row_blocks;
            prefill_attention_kernel<8, false><<<dim3((a.m + rows_per_cta - 1u) / rows_per_cta, a.kv_heads), 256, smem, stream>>>(p);
        }
    } else {
        p.row_blocks = 4u / gqa;
        const uint32_t rows_per_cta = 16u * p.row_blocks;
        if (splits) {
            if (stark_b200_status s = ensure_dynamic_smem(prefill_attention_kernel<4, true>, (int)smem, once4s)) return s;
            SB_CUDA(launch_dependent(prefill_attention_kernel<4, true>, dim3(1, a.kv_heads, splits), dim3(128), smem, stream, p));
        } else {
            if (stark_b200_status s = ensure_dynamic_smem(prefill_attention_kernel<4, false>, (int)smem, once4)) return s;
            prefill_attention_kernel<4, false><<<dim3((a.m + rows_per_cta - 1u) / rows_per_cta, a.kv_heads), 128, smem, stream>>>(p);
        }
    }
    SB_CUDA(cudaGetLastError());
    if (splits) {
        SB_CUDA(launch_dependent(prefill_attention_merge_kernel, dim3(a.m, a.q_heads), dim3(kHeadDim), 0, stream, a.partials,
                                 a.out, a.q_heads, splits));
    }
    return STARK_B200_OK;
}

}  // namespace sb
