// Causal attention of a prompt pass on the sm_100a tensor cores (tcgen05.mma, accumulators in tensor memory):
// the same arithmetic as prefill_attention_kernel (attention_single_pass.rs:11-133: scores q.k in f32 scaled by
// 1/sqrt(d), softmax in f32, probabilities into the second product as bf16 hi + lo, output rounded to bf16), in the
// shape the tensor core wants.
//
// One CTA owns 128 rows of one query head and walks the keys in steps of 128 (two pages of the cache) TWICE:
//   pass 1   S = Q K^T per step, only to find every row's maximum;
//   pass 2   S again, P = exp2(S - max) (already final: no accumulator is ever rescaled), O += P V.
// The second look at the keys costs a quarter more tensor-core work and removes the read-modify-write of the output
// accumulator that an online softmax needs whenever a maximum moves.  Roles:
//   warps 0-7   softmax: thread = row (tensor-memory lane) x half of the step's keys; tcgen05.ld of S in 32-column
//               pieces, mask by the row's causal limit, maximum (pass 1) or exp2 / row sum / bf16 hi + lo written as
//               the K-major, 128-byte swizzled A operand of the second product (pass 2); at the end the read-out of O
//   warp 8      one thread: TMA loads -- Q once, then per step the K tile (and in pass 2 the V tile) as four
//               [64 keys x 64 dims] boxes straight from the paged cache
//   warp 9      owns tensor memory (S twice, so that step j + 1 is multiplied while step j is exponentiated, and O);
//               one thread issues the MMAs: S = Q K^T with both operands K-major, O += P V with V as an MN-major
//               operand (its rows are keys, the contraction index), and commits them to the barriers
// Every wait is bounded; a wait that runs out sets the error word, the CTA drains and frees its tensor memory.
#include <cuda.h>

#include <algorithm>

#include "context.cuh"
#include "device_math.cuh"
#include "prefill.cuh"
#include "tc05.cuh"
#include "tunables.cuh"

namespace sb {

namespace {

constexpr uint32_t kBox = 64u * 128u;       // [64 rows][64 elements] bf16 in 128-byte swizzled lines: 8 KB
constexpr uint32_t kBlock = 2u * kBox;      // 128 rows x 64 elements: 16 KB
constexpr uint32_t kOperand = 2u * kBlock;  // 128 x 128: 32 KB
constexpr uint32_t kSoftmaxWarps = 8, kTcThreads = (kSoftmaxWarps + 2u) * 32u;
// shared memory: Q | K, two stages | V, two stages | P hi | P lo | barriers (256 B) | exchange words [2][128] f32
constexpr uint32_t kQOff = 0, kKOff = kOperand, kVOff = 3u * kOperand, kPOff = 5u * kOperand, kBarOff = 7u * kOperand;
constexpr uint32_t kTcSmem = 7u * kOperand + 2048u /* barriers, exchange words */ + 1024u /* alignment */;
constexpr uint32_t kTcTmemColumns = 512;  // S twice (2 x 128) and O (128); allocations are powers of two
// D f32, A and B bf16, M 128, N 128; the second product takes B (V) MN-major
constexpr uint32_t kIdescS = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kIdescPV = kIdescS | (1u << 16);

__device__ inline float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct TcAttnParams {
    uint16_t *out;
    const int32_t *block_table;
    uint32_t m, first_pos, q_heads, kv_heads, gqa, num_blocks;
    float scale_log2;  // log2(e) / sqrt(d)
    uint32_t *error_word;
    uint32_t stop_after;  // 0 whole kernel; 1 set-up and tensor memory only; 2 pass 1 only (no MN-major operand)
};

__global__ void __launch_bounds__(kTcThreads, 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                            const __grid_constant__ CUtensorMap v_map, const TcAttnParams p) {
    extern __shared__ uint8_t tc_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023u) & ~(uintptr_t)1023u);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kBarOff);
    uint64_t *q_full = bars, *k_full = bars + 1, *k_empty = bars + 3, *v_full = bars + 5, *v_empty = bars + 7;
    uint64_t *s_full = bars + 9, *s_free = bars + 11, *p_full = bars + 13, *p_free = bars + 14, *o_full = bars + 15;
    uint64_t *a_full = bars + 16, *a_empty = bars + 20;  // pass 1: the K and V stages together are a ring of four K tiles
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 24);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    float *exchange = reinterpret_cast<float *>(smem + kBarOff + 256u);  // what the two warps of a row tell each other

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t head = blockIdx.x, kvh = head / p.gqa;
    // causal: late row blocks read the most keys, so they are issued first
    const uint32_t row0 = (gridDim.y - 1u - blockIdx.y) * 128u;
    const uint32_t last_row = min(p.m, row0 + 128u) - 1u;
    const uint32_t steps = (p.first_pos + last_row) / 128u + 1u;
    const uint32_t passes = p.stop_after == 2u ? 1u : 2u;

    if (tid == 0) {
        mbar_init(q_full, 1);
        for (uint32_t s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&s_free[s], kSoftmaxWarps);
        }
        for (uint32_t s = 0; s < 4; ++s) {
            mbar_init(&a_full[s], 1);
            mbar_init(&a_empty[s], 1);
        }
        mbar_init(p_full, kSoftmaxWarps);
        mbar_init(p_free, 1);
        mbar_init(o_full, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == kSoftmaxWarps + 1u) tmem_alloc(tmem_slot, kTcTmemColumns);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    auto give_up = [&]() {
        *abort_flag = 1;
        atomicOr(p.error_word, kErrMbarTimeout);
    };

    if (p.stop_after == 1u) {
        // nothing between allocation and release
    } else if (warp == kSoftmaxWarps) {
        // ------------------------------------------------ tiles by TMA
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, kOperand);
            tma_load_2d(smem + kQOff, &q_map, head * 128u, row0, q_full);
            tma_load_2d(smem + kQOff + kBlock, &q_map, head * 128u + 64u, row0, q_full);
            // a page past the allocated ones is read out of bounds: the copy engine fills zeros
            auto page_row = [&](uint32_t page) -> uint32_t {
                return page < p.num_blocks ? ((uint32_t)p.block_table[page] * p.kv_heads + kvh) * kPageTokens
                                           : p.num_blocks * p.kv_heads * kPageTokens;
            };
            auto load_tile = [&](uint8_t *dst, const CUtensorMap *map, uint32_t y0, uint32_t y1, uint64_t *bar) {
                mbar_arrive_expect_tx(bar, kOperand);
                tma_load_2d(dst, map, 0u, y0, bar);
                tma_load_2d(dst + kBox, map, 0u, y1, bar);
                tma_load_2d(dst + kBlock, map, 64u, y0, bar);
                tma_load_2d(dst + kBlock + kBox, map, 64u, y1, bar);
            };
            uint32_t ks = 0, kph = 1, vs = 0, vph = 1;  // a fresh barrier passes a wait on parity 1
            bool ok = true;
            {   // pass 1: K tiles only, four in flight
                uint32_t as = 0, aph = 1;
                for (uint32_t j = 0; j < steps && ok; ++j) {
                    if (!(ok = mbar_wait_bounded(&a_empty[as], aph, abort_flag))) break;
                    load_tile(smem + kKOff + as * kOperand, &k_map, page_row(2u * j), page_row(2u * j + 1u), &a_full[as]);
                    if (++as == 4u) as = 0, aph ^= 1u;
                }
                // pass 2 loads into the same memory: every stage's last pass-1 tile must have been multiplied
                for (uint32_t s = 0; s < 4u && ok && passes == 2u; ++s) {
                    const uint32_t uses = steps > s ? (steps - s + 3u) / 4u : 0u;
                    if (uses) ok = mbar_wait_bounded(&a_empty[s], (uses - 1u) & 1u, abort_flag);
                }
            }
            for (uint32_t pass = 1; pass < passes && ok; ++pass) {
                for (uint32_t j = 0; j < steps && ok; ++j) {
                    const uint32_t y0 = page_row(2u * j), y1 = page_row(2u * j + 1u);
                    if (!(ok = mbar_wait_bounded(&k_empty[ks], kph, abort_flag))) break;
                    load_tile(smem + kKOff + ks * kOperand, &k_map, y0, y1, &k_full[ks]);
                    if (++ks == 2u) ks = 0, kph ^= 1u;
                    if (pass == 1u) {
                        if (!(ok = mbar_wait_bounded(&v_empty[vs], vph, abort_flag))) break;
                        load_tile(smem + kVOff + vs * kOperand, &v_map, y0, y1, &v_full[vs]);
                        if (++vs == 2u) vs = 0, vph ^= 1u;
                    }
                }
            }
            if (!ok) give_up();
        }
    } else if (warp == kSoftmaxWarps + 1u) {
        // ------------------------------------------------ tensor-core issue
        if (lane == 0) {
            bool ok = mbar_wait_bounded(q_full, 0, abort_flag);
            uint32_t ks = 0, kph = 0, vs = 0, vph = 0, g = 0;  // g counts score tiles: buffer g & 1
            const uint32_t q_addr = smem_u32(smem + kQOff);
            const uint32_t ring = 4u;  // pass 1; pass 2 below passes 2
            auto scores = [&](uint64_t *full, uint64_t *empty, uint32_t slots) {
                const uint32_t b = g & 1u, use = g >> 1;
                ok = ok && mbar_wait_bounded(&full[ks], kph, abort_flag) &&
                     mbar_wait_bounded(&s_free[b], (use & 1u) ^ 1u, abort_flag);  // the softmax warps are done with use - 1
                if (!ok) return;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(smem + kKOff + ks * kOperand);
#pragma unroll
                for (uint32_t i = 0; i < 8u; ++i) {  // 16 dims a step; 64 dims a block
                    const uint32_t at = (i >> 2) * kBlock + (i & 3u) * 32u;
                    umma_f16(tmem_base + b * 128u, smem_desc_sw128(q_addr + at), smem_desc_sw128(k_addr + at), kIdescS,
                             i != 0u ? 1u : 0u);
                }
                umma_commit(&empty[ks]);
                umma_commit(&s_full[b]);
                if (++ks == slots) ks = 0, kph ^= 1u;
                ++g;
            };
            for (uint32_t j = 0; j < steps && ok; ++j) scores(a_full, a_empty, ring);
            ks = 0, kph = 0;
            if (passes == 2u) {
                const uint32_t ph_addr = smem_u32(smem + kPOff), pl_addr = ph_addr + kOperand;
                for (uint32_t j = 0; j <= steps && ok; ++j) {
                    if (j < steps) scores(k_full, k_empty, 2u);  // step j is multiplied while step j - 1 is exponentiated
                    if (j == 0u || !ok) continue;
                    const uint32_t t = j - 1u;
                    ok = mbar_wait_bounded(p_full, t & 1u, abort_flag) && mbar_wait_bounded(&v_full[vs], vph, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t v_addr = smem_u32(smem + kVOff + vs * kOperand);
#pragma unroll
                    for (uint32_t i = 0; i < 8u; ++i) {  // 16 keys a step
                        const uint64_t vdesc = smem_desc_sw128_mn(v_addr + i * 2048u, kBlock);
                        const uint32_t at = (i >> 2) * kBlock + (i & 3u) * 32u;
                        umma_f16(tmem_base + 256u, smem_desc_sw128(ph_addr + at), vdesc, kIdescPV, (t | i) != 0u ? 1u : 0u);
                        umma_f16(tmem_base + 256u, smem_desc_sw128(pl_addr + at), vdesc, kIdescPV, 1u);
                    }
                    umma_commit(&v_empty[vs]);
                    umma_commit(p_free);
                    if (++vs == 2u) vs = 0, vph ^= 1u;
                }
            }
            if (!ok) give_up();
            umma_commit(o_full);  // also on the give-up path: the softmax warps wait on it
        }
    } else {
        // ------------------------------------------------ softmax: thread = row (tensor-memory lane) x half of the keys
        // Warps w and w + 4 share the 32 rows of lane group w & 3 (a warp reaches only the lanes of its index modulo
        // 4) and take the step's keys 0-63 and 64-127: twice the warps that issue exponentials and conversions.
        const uint32_t sub = warp & 3u, half = warp >> 2;
        const uint32_t r = 32u * sub + lane, row = row0 + r;
        const uint32_t pos = p.first_pos + min(row, p.m - 1u);  // last key this row may see
        const uint32_t lanes = (32u * sub) << 16, col0 = 64u * half;
        float mrow = -INFINITY;
        uint32_t g = 0;
        bool ok = true;
        for (uint32_t j = 0; j < steps && ok; ++j, ++g) {
            const uint32_t b = g & 1u;
            if (!(ok = mbar_wait_bounded(&s_full[b], (g >> 1) & 1u, abort_flag))) break;
            tc_fence_after();
            uint32_t v[2][32];
#pragma unroll
            for (uint32_t c = 0; c < 2u; ++c) tmem_ld_32x32_issue(tmem_base + lanes + b * 128u + col0 + 32u * c, v[c]);
#pragma unroll
            for (uint32_t c = 0; c < 2u; ++c) {
                tmem_ld_wait_32(v[c]);
                const uint32_t key0 = j * 128u + col0 + 32u * c;
                float mx = -INFINITY;
                if (key0 + 31u <= pos) {  // the row sees the whole piece
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(v[c][i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (key0 + i <= pos) mx = fmaxf(mx, __uint_as_float(v[c][i]));
                }
                mrow = fmaxf(mrow, mx * p.scale_log2);  // the scale is positive: it commutes with the maximum
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[b]);
        }
        // the row's maximum over both halves of the keys
        exchange[half * 128u + r] = mrow;
        named_bar_sync(1, kSoftmaxWarps * 32u);
        mrow = fmaxf(mrow, exchange[(half ^ 1u) * 128u + r]);
        named_bar_sync(1, kSoftmaxWarps * 32u);  // everybody has read: the words are free for the row sums
        float l = 0.0f;
        if (passes == 2u) {
            uint8_t *p_hi = smem + kPOff + half * kBlock + r * 128u, *p_lo = p_hi + kOperand;  // key block `half` of the row
            for (uint32_t j = 0; j < steps && ok; ++j, ++g) {
                const uint32_t b = g & 1u;
                if (!(ok = mbar_wait_bounded(&s_full[b], (g >> 1) & 1u, abort_flag))) break;
                tc_fence_after();
                uint32_t v[2][32];
                tmem_ld_32x32_issue(tmem_base + lanes + b * 128u + col0, v[0]);
                tmem_ld_32x32_issue(tmem_base + lanes + b * 128u + col0 + 32u, v[1]);
#pragma unroll
                for (uint32_t c = 0; c < 2u; ++c) {
                    if (!ok) break;
                    uint32_t hi[16], lo[16];
                    tmem_ld_wait_32(v[c]);
                    const uint32_t key0 = j * 128u + col0 + 32u * c;
                    const bool whole = key0 + 31u <= pos;
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        // exp2 of a non-positive argument: the hardware approximation is good to two units of an f32's
                        // last place, far inside what the bf16 pair keeps
                        float e0 = ex2_approx(fmaf(__uint_as_float(v[c][i]), p.scale_log2, -mrow));
                        float e1 = ex2_approx(fmaf(__uint_as_float(v[c][i + 1]), p.scale_log2, -mrow));
                        if (!whole) {
                            if (key0 + i > pos) e0 = 0.0f;
                            if (key0 + i + 1 > pos) e1 = 0.0f;
                        }
                        l += e0;
                        l += e1;
                        split_bf16x2(e0, e1, hi[i >> 1], lo[i >> 1]);
                    }
                    // the previous step's second product must have read P before it is overwritten
                    if (c == 0u && !(ok = mbar_wait_bounded(p_free, (j & 1u) ^ 1u, abort_flag))) break;
                    // 32 keys = four 16-byte chunks of the row's 128-byte line
#pragma unroll
                    for (uint32_t q = 0; q < 4u; ++q) {
                        const uint32_t at = ((c * 4u + q) ^ (r & 7u)) << 4;
                        *reinterpret_cast<uint4 *>(p_hi + at) = make_uint4(hi[4 * q], hi[4 * q + 1], hi[4 * q + 2], hi[4 * q + 3]);
                        *reinterpret_cast<uint4 *>(p_lo + at) = make_uint4(lo[4 * q], lo[4 * q + 1], lo[4 * q + 2], lo[4 * q + 3]);
                    }
                }
                proxy_fence_async();  // the tensor core reads shared memory through the async proxy
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&s_free[b]);
                    mbar_arrive(p_full);
                }
            }
            // the row's sum over both halves, in key order
            exchange[half * 128u + r] = l;
            named_bar_sync(1, kSoftmaxWarps * 32u);
            l = exchange[r] + exchange[128u + r];
            // ---- read-out of O: this warp's 64 of the 128 dims
            const bool o_ok = mbar_wait_bounded(o_full, 0, abort_flag);
            if (!o_ok && lane == 0) atomicOr(p.error_word, kErrMbarTimeout);
            tc_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            uint16_t *dst = p.out + ((size_t)row * p.q_heads + head) * kHeadDim + col0;
            uint32_t v[2][32];
#pragma unroll
            for (uint32_t c = 0; c < 2u; ++c) tmem_ld_32x32_issue(tmem_base + lanes + 256u + col0 + 32u * c, v[c]);
#pragma unroll
            for (uint32_t c = 0; c < 2u; ++c) {
                tmem_ld_wait_32(v[c]);
                if (row < p.m && o_ok && ok) {
                    uint32_t packed[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        packed[i >> 1] = f32x2_to_bf16x2(__uint_as_float(v[c][i]) * inv, __uint_as_float(v[c][i + 1]) * inv);
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        reinterpret_cast<uint4 *>(dst + 32u * c)[q] =
                            make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                }
            }
        }
        if (!ok && lane == 0) give_up();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kSoftmaxWarps + 1u) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTcTmemColumns);
    }
}

}  // namespace

bool prefill_attention_tc_supports(const PrefillAttnArgs &a) {
    return a.num_blocks != 0 && a.m > 16u && a.kv_heads != 0 && a.q_heads % a.kv_heads == 0 &&
           (reinterpret_cast<uintptr_t>(a.qkv) & 15u) == 0 && encode_tiled() != nullptr;
}

stark_b200_status prefill_attention_tc_launch(const PrefillAttnArgs &a, cudaStream_t stream) {
    if (!a.qkv || !a.kv.keys || !a.kv.values || !a.block_table || !a.out || a.m == 0) return STARK_B200_INVALID_ARGUMENT;
    if (!prefill_attention_tc_supports(a)) return STARK_B200_UNSUPPORTED;
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    EncodeTiledFn encode = encode_tiled();
    const uint32_t heads = a.q_heads + 2u * a.kv_heads;
    CUtensorMap q_map, k_map, v_map;
    const cuuint32_t elem[2] = {1u, 1u};
    {
        // the query heads of the pass's rows: [m][heads * 128], the q heads first in every row
        const cuuint64_t dims[2] = {(cuuint64_t)a.q_heads * kHeadDim, a.m};
        const cuuint64_t strides[1] = {(cuuint64_t)heads * kHeadDim * 2u};
        const cuuint32_t box[2] = {64u, 128u};
        if (encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(a.qkv), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return STARK_B200_DEVICE_FAILURE;
    }
    {
        // the paged cache of the layer as rows of one head's 128 dims: [(page, kv head, token)][128]
        const cuuint64_t dims[2] = {kHeadDim, (cuuint64_t)a.num_blocks * a.kv_heads * kPageTokens};
        const cuuint64_t strides[1] = {(cuuint64_t)kHeadDim * 2u};
        const cuuint32_t box[2] = {64u, kPageTokens};
        for (int which = 0; which < 2; ++which)
            if (encode(which ? &v_map : &k_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, which ? a.kv.values : a.kv.keys, dims,
                       strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return STARK_B200_DEVICE_FAILURE;
    }
    TcAttnParams p{};
    p.out = a.out;
    p.block_table = a.block_table;
    p.m = a.m;
    p.first_pos = a.first_pos;
    p.q_heads = a.q_heads;
    p.kv_heads = a.kv_heads;
    p.gqa = a.q_heads / a.kv_heads;
    p.num_blocks = a.num_blocks;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.error_word = ctx->error_word;
    p.stop_after = tunables().attn_tc_stop_after;
    static SmemOptIn once;
    if (stark_b200_status s = ensure_dynamic_smem(prefill_attention_tc_kernel, (int)kTcSmem, once)) return s;
    prefill_attention_tc_kernel<<<dim3(a.q_heads, (a.m + 127u) / 128u), kTcThreads, kTcSmem, stream>>>(q_map, k_map, v_map, p);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

}  // namespace sb
