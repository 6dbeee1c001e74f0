// Y[M, N] = X[M, K] W[N, K]^T for a 4-bit affine group-64 matrix, many rows at a time: the prompt-chunk
// contraction of the token loop on the sm_100a tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// One CTA owns a tile of 256 rows x 256 output features and walks K in steps of one quantization group (64):
//   warp 0      one thread: TMA loads of the two 128-row activation boxes of the step (bf16, 128-byte swizzle)
//   warp 1      allocates tensor memory (all 512 columns: two 128 x 256 f32 accumulators); one thread issues
//               2 x 4 tcgen05.mma (128 x 256 x 16) per step and commits them to the barrier that frees the stage
//   warps 2-9   the dequantizing prologue: warp d turns two records (16 features x 64 columns, 576 bytes each,
//               read straight from the re-tiled matrix the matvec kernels stream) into bf16 rows of the B operand --
//               codes become exact bf16 integers (shift, lop3 and one bf16 subtract per pair), then
//               bf16(scale * q + bias) in one bf16 FMA per pair -- written in the swizzled K-major layout the
//               tensor core reads.  The same warps run the epilogue: tcgen05.ld of the accumulators, bf16 rounding,
//               residual add or SwiGLU, 64-byte row segments to global memory.
// Rounding points are those of the one-row path (f32 accumulation, one bf16 rounding of the product, then the
// epilogue's own roundings); the operand W is rounded to bf16, the activations' type, as the reference's own
// tiled GEMM does, where the one-row path keeps scale * q + bias in f32: inside the per-operator tolerance.
// The tile is as wide as tensor memory allows because the activation tile is what the step re-reads from L2 (once
// per feature tile) and what the tensor core re-reads from shared memory: at 256 features a step moves 41 KB from
// L2 and 160 KB through shared memory for 1024 tensor-core cycles (156 B/cycle of the 128 B/cycle an SM has, the
// binding limit), at 128 features 37 KB and 112 KB for 512 cycles.
// Every wait is bounded; a wait that runs out sets the error word, the CTA drains and frees its tensor memory.
#include <cuda.h>

#include <algorithm>

#include "device_math.cuh"
#include "prefill.cuh"
#include "tc05.cuh"
#include "tunables.cuh"

namespace sb {

namespace {

constexpr uint32_t kBM = 256, kBN = 256, kBK = 64;
constexpr uint32_t kStages = 3;
constexpr uint32_t kABox = 128u * 128u;            // one 128-row x 64-column bf16 box: 16 KB
constexpr uint32_t kAStage = 2u * kABox;           // 32 KB
constexpr uint32_t kBStage = kBN * 128u;           // 32 KB
constexpr uint32_t kStageBytes = kAStage + kBStage;
constexpr uint32_t kDequantWarps = 8;
constexpr uint32_t kGemmThreads = (2u + kDequantWarps) * 32u;
constexpr uint32_t kTmemColumns = 512;             // two 128 x 256 f32 accumulators: all of tensor memory
constexpr uint32_t kGemmSmem = kStages * kStageBytes + 1024u /* alignment */ + 256u /* barriers */;

struct GemmParams {
    const uint8_t *w;
    uint32_t row_tiles, groups, rows;
    uint32_t m;
    uint16_t *out;
    uint32_t ld_out;
    uint32_t epilogue;
    uint32_t *error_word;
    // tensor parallel: the same place in the other ranks' row buffers (peer mappings); the epilogue stores every
    // output segment there as well, tile by tile, so the all-gather of the column slices rides under the contraction
    uint16_t *peer_out[kMaxExchangeRanks];
    uint32_t peers;
    uint32_t stop_after;  // 0: the whole kernel.  1: set-up and tensor-memory allocation only; 2: + operand staging
                          // (no tensor-core work); 3: + tcgen05.mma (accumulators not read).  A bring-up aid: a
                          // fault in one kind of instruction is located by the first stage that shows it.
};

// Instruction descriptor: D f32, A bf16 (activations), B bf16 (dequantized weights), both K-major, M 128, N 256.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kBN >> 3) << 17) | ((128u >> 4) << 24);

struct RecordRegs {
    uint4 q;
    uint32_t scales, biases;  // bf16 pairs: rows g and g + 8
};

__device__ inline RecordRegs load_record(const uint8_t *w, uint32_t tile, uint32_t row_tiles, uint32_t groups,
                                         uint32_t kg, uint32_t lane) {
    RecordRegs r;
    if (tile < row_tiles) {
        const uint8_t *rec = w + ((size_t)tile * groups + kg) * kA4RecordBytes;
        r.q = ldg_nc_v4(rec + lane * 16u);
        r.scales = __ldg(reinterpret_cast<const uint32_t *>(rec + 512u + 4u * (lane >> 2)));
        r.biases = __ldg(reinterpret_cast<const uint32_t *>(rec + 544u + 4u * (lane >> 2)));
    } else {  // past the last row tile: zero rows
        r.q = make_uint4(0u, 0u, 0u, 0u);
        r.scales = 0u;
        r.biases = 0u;
    }
    return r;
}

// One record word -> the eight codes as exact bf16 integers, in the fragment order of dequant_a4_word:
// (w >> 4s) & 0x000f000f | 0x43004300 is the bf16 pair (128 + q, 128 + q') -- 0x4300 is 128.0 and the last
// mantissa bit of a bf16 in [128, 256) weighs 1 -- and 128 is then subtracted exactly.
__device__ inline void codes_to_bf16(uint32_t w, __nv_bfloat162 (&q)[4]) {
    const uint32_t magic = 0x43004300u;
    const __nv_bfloat162 k128 = __float2bfloat162_rn(128.0f);
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const uint32_t v = lop3_and_or(w >> (4 * s), 0x000f000fu, magic);
        q[s] = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&v), k128);
    }
}
__device__ inline __nv_bfloat162 bf16_pair(uint32_t bits16) {
    const uint32_t v = bits16 | (bits16 << 16);
    return *reinterpret_cast<const __nv_bfloat162 *>(&v);
}

// One record (16 features x 64 columns) into rows [16 d, 16 d + 16) of the B stage: lane (g, t) owns columns
// 16 t .. 16 t + 15 of rows g and g + 8, i.e. two 16-byte chunks in each of the two rows.
__device__ inline void dequant_record_to_smem(const RecordRegs &r, uint8_t *b_stage, uint32_t d, uint32_t lane) {
    const uint32_t g = lane >> 2, t = lane & 3u;
    const __nv_bfloat162 s0 = bf16_pair(r.scales & 0xffffu), s1 = bf16_pair(r.scales >> 16);
    const __nv_bfloat162 b0 = bf16_pair(r.biases & 0xffffu), b1 = bf16_pair(r.biases >> 16);
    const uint32_t ww[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
    uint32_t lo_row[8], hi_row[8];  // 16 bf16 values per row
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 a[4];
        codes_to_bf16(ww[j], a);  // a[0], a[2]: row g, columns 4j + {0,1}, {2,3}; a[1], a[3]: row g + 8
        // bf16(scale * q + bias): one fused multiply-add, one rounding -- the dequantized operand in the
        // activations' type, as the reference's tiled GEMM stages it (gemm.metal:122-203, `threadgroup BT b_shared`)
        const __nv_bfloat162 v0 = __hfma2(a[0], s0, b0);
        const __nv_bfloat162 v2 = __hfma2(a[2], s0, b0);
        const __nv_bfloat162 v1 = __hfma2(a[1], s1, b1);
        const __nv_bfloat162 v3 = __hfma2(a[3], s1, b1);
        lo_row[2 * j] = *reinterpret_cast<const uint32_t *>(&v0);
        lo_row[2 * j + 1] = *reinterpret_cast<const uint32_t *>(&v2);
        hi_row[2 * j] = *reinterpret_cast<const uint32_t *>(&v1);
        hi_row[2 * j + 1] = *reinterpret_cast<const uint32_t *>(&v3);
    }
    // row R of the stage starts at R * 128; its 16-byte chunk c sits at chunk position c ^ (R & 7)
    const uint32_t r_lo = 16u * d + g, r_hi = r_lo + 8u;  // both have (R & 7) == g
    uint8_t *p_lo = b_stage + r_lo * 128u, *p_hi = b_stage + r_hi * 128u;
    const uint32_t c0 = ((2u * t) ^ g) * 16u, c1 = ((2u * t + 1u) ^ g) * 16u;
    *reinterpret_cast<uint4 *>(p_lo + c0) = make_uint4(lo_row[0], lo_row[1], lo_row[2], lo_row[3]);
    *reinterpret_cast<uint4 *>(p_lo + c1) = make_uint4(lo_row[4], lo_row[5], lo_row[6], lo_row[7]);
    *reinterpret_cast<uint4 *>(p_hi + c0) = make_uint4(hi_row[0], hi_row[1], hi_row[2], hi_row[3]);
    *reinterpret_cast<uint4 *>(p_hi + c1) = make_uint4(hi_row[4], hi_row[5], hi_row[6], hi_row[7]);
}

// HALVES = 2: a CTA owns 256 rows (two 128-row accumulators over one dequantized weight tile).  HALVES = 1: 128
// rows -- twice the CTAs, each amortizing its dequantization over half the rows -- for contractions too narrow to
// fill the SMs with 256-row tiles (a 1 024-feature slice of o or down under tensor parallelism, a 1 024-row pass).
template <uint32_t HALVES>
__global__ void __launch_bounds__(kGemmThreads, 1)
prefill_gemm_a4_kernel(const __grid_constant__ CUtensorMap x_map, const GemmParams p) {
    extern __shared__ uint8_t gemm_smem_raw[];
    // operand stages need 1024-byte alignment (swizzle atom = 8 rows x 128 bytes)
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023u) & ~(uintptr_t)1023u);
    uint8_t *stages = smem;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * kStageBytes);
    uint64_t *full_a = bars, *full_b = bars + kStages, *empty = bars + 2 * kStages, *acc_full = bars + 3 * kStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * kStages + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t n_tile0 = blockIdx.x * (kBN / 16u);  // first 16-row storage tile of this CTA
    const uint32_t m0 = blockIdx.y * (128u * HALVES);

    if (tid == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(&full_a[s], 1);
            mbar_init(&full_b[s], kDequantWarps);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemColumns);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t stop = p.stop_after;

    if (stop == 1u) {
        // nothing between allocation and release
    } else if (warp == 0) {
        // ------------------------------------------------ activation tiles by TMA
        if (lane == 0) {
            uint32_t slot = 0, phase = 1;  // a fresh barrier passes a wait on parity 1
            for (uint32_t kg = 0; kg < p.groups; ++kg) {
                if (!mbar_wait_bounded(&empty[slot], phase, abort_flag)) {
                    *abort_flag = 1;
                    atomicOr(p.error_word, kErrMbarTimeout);
                    break;
                }
                uint8_t *a_stage = stages + slot * kStageBytes;
                mbar_arrive_expect_tx(&full_a[slot], HALVES * kABox);
                tma_load_2d(a_stage, &x_map, kg * kBK, m0, &full_a[slot]);
                if (HALVES == 2u) tma_load_2d(a_stage + kABox, &x_map, kg * kBK, m0 + 128u, &full_a[slot]);
                if (++slot == kStages) {
                    slot = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ tensor-core issue
        if (lane == 0) {
            uint32_t slot = 0, phase = 0;
            bool ok = true;
            for (uint32_t kg = 0; kg < p.groups && ok; ++kg) {
                ok = mbar_wait_bounded(&full_a[slot], phase, abort_flag) && mbar_wait_bounded(&full_b[slot], phase, abort_flag);
                if (!ok) {
                    *abort_flag = 1;
                    atomicOr(p.error_word, kErrMbarTimeout);
                    break;
                }
                if (stop == 2u) {  // staging only: hand the stage back without touching the tensor core
                    mbar_arrive(&empty[slot]);
                    if (++slot == kStages) {
                        slot = 0;
                        phase ^= 1u;
                    }
                    continue;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(stages + slot * kStageBytes);
                const uint32_t b_addr = a_addr + kAStage;
#pragma unroll
                for (uint32_t half = 0; half < HALVES; ++half) {
#pragma unroll
                    for (uint32_t k4 = 0; k4 < kBK / 16u; ++k4) {
                        const uint64_t adesc = smem_desc_sw128(a_addr + half * kABox + k4 * 32u);
                        const uint64_t bdesc = smem_desc_sw128(b_addr + k4 * 32u);
                        umma_f16(tmem_base + half * kBN, adesc, bdesc, kIdesc, (kg | k4) != 0u ? 1u : 0u);
                    }
                }
                umma_commit(&empty[slot]);  // arrives when the MMAs reading this stage are done
                if (++slot == kStages) {
                    slot = 0;
                    phase ^= 1u;
                }
            }
            if (stop == 2u) mbar_arrive(acc_full);
            else umma_commit(acc_full);  // also on the give-up path: the epilogue warps wait on it
        }
    } else {
        // ------------------------------------------------ dequantizing prologue (one record per warp per step)
        const uint32_t d = warp - 2u;
        const uint32_t tile = n_tile0 + d;  // and tile + 8: rows 16 d .. and 128 + 16 d .. of the B stage
        uint32_t slot = 0, phase = 1;
        constexpr uint32_t kAhead = 4;  // steps requested ahead of use (global latency >> one step)
        RecordRegs ring[kAhead][2];
#pragma unroll
        for (uint32_t i = 0; i < kAhead; ++i) {
            ring[i][0] = load_record(p.w, i < p.groups ? tile : 0xffffffffu, p.row_tiles, p.groups, i, lane);
            ring[i][1] = load_record(p.w, i < p.groups ? tile + 8u : 0xffffffffu, p.row_tiles, p.groups, i, lane);
        }
        bool ok = true;
        for (uint32_t kb = 0; kb < p.groups && ok; kb += kAhead) {
#pragma unroll
            for (uint32_t i = 0; i < kAhead; ++i) {
                const uint32_t kg = kb + i;
                if (kg >= p.groups) break;
                const RecordRegs cur0 = ring[i][0], cur1 = ring[i][1];
                const uint32_t next = kg + kAhead;
                ring[i][0] = load_record(p.w, next < p.groups ? tile : 0xffffffffu, p.row_tiles, p.groups,
                                         next < p.groups ? next : 0u, lane);
                ring[i][1] = load_record(p.w, next < p.groups ? tile + 8u : 0xffffffffu, p.row_tiles, p.groups,
                                         next < p.groups ? next : 0u, lane);
                if (!mbar_wait_bounded(&empty[slot], phase, abort_flag)) {
                    if (lane == 0) {
                        *abort_flag = 1;
                        atomicOr(p.error_word, kErrMbarTimeout);
                    }
                    ok = false;
                    break;
                }
                dequant_record_to_smem(cur0, stages + slot * kStageBytes + kAStage, d, lane);
                dequant_record_to_smem(cur1, stages + slot * kStageBytes + kAStage, d + 8u, lane);
                proxy_fence_async();  // the tensor core reads shared memory through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_b[slot]);
                if (++slot == kStages) {
                    slot = 0;
                    phase ^= 1u;
                }
            }
        }

        // ------------------------------------------------ epilogue: warp -> (sub-partition, accumulator half)
        // (with one accumulator the two warps of a sub-partition share its columns instead)
        const uint32_t sub = warp & 3u, half = HALVES == 2u ? d >> 2 : 0u;
        const uint32_t c_first = HALVES == 2u ? 0u : (d >> 2) * (kBN / 64u), c_count = kBN / 32u / (3u - HALVES);
        const bool acc_ok = mbar_wait_bounded(acc_full, 0, abort_flag);
        if (!acc_ok && lane == 0) atomicOr(p.error_word, kErrMbarTimeout);
        tc_fence_after();
        // every tensor-core read of the operand stages has completed: their first bytes serve as 4 KB of scratch per warp
        uint8_t *scratch = stages + d * 4096u;
        const uint32_t row = m0 + half * 128u + sub * 32u + lane;  // this thread's row of the output
        const bool row_ok = row < p.m;
#pragma unroll 1
        for (uint32_t c = c_first; c < (stop == 0u ? c_first + c_count : 0u); ++c) {
            uint32_t acc[32];
            tmem_ld_32x32(tmem_base + ((sub * 32u) << 16) + half * kBN + c * 32u, acc);
            // columns of the accumulator are storage rows of the matrix: feature = 16 * tile + r
            const uint32_t f0 = n_tile0 * 16u + c * 32u;
            if (p.epilogue == kEpiSwiGlu) {
                // storage tiles alternate up / gate (pair_halves): columns 0-15 up rows, 16-31 the gate rows
                // of the same logical rows.  gated_act_mul.rs:80-95: silu in f32 -> bf16, product -> bf16
                uint32_t packed[8];
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    float o2[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float up = bf16_round(__uint_as_float(acc[i + e]));
                        const float gate = bf16_round(__uint_as_float(acc[16 + i + e]));
                        const float activated = bf16_round(gate / (1.0f + expf(-1.0f * gate)));
                        o2[e] = up * activated;
                    }
                    packed[i >> 1] = f32x2_to_bf16x2(o2[0], o2[1]);
                }
                const uint32_t o0 = (f0 / 32u) * 16u;  // logical row of the pair
                if (row_ok && o0 + 16u <= p.rows / 2u) {
                    uint4 *dst = reinterpret_cast<uint4 *>(p.out + (size_t)row * p.ld_out + o0);
                    dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
                if (p.peers && acc_ok) {
                    // The same 32 x 16 block to the other ranks.  A lane holds 32 bytes of ITS row: stored from here, one
                    // instruction would touch 32 rows with 16 bytes each, and over NVLink every such fragment is a packet
                    // of its own.  Through the warp's scratch rows (48-byte pitch: conflict-free) the lanes regroup
                    // so that two neighbours write one row's 32 contiguous bytes.
                    uint4 *mine = reinterpret_cast<uint4 *>(scratch + lane * 48u);
                    mine[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    mine[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    __syncwarp();
#pragma unroll
                    for (uint32_t j = 0; j < 2u; ++j) {
                        const uint32_t r = 16u * j + (lane >> 1), q = lane & 1u;
                        const uint4 v = *reinterpret_cast<const uint4 *>(scratch + r * 48u + q * 16u);
                        const uint32_t prow = row - lane + r;
                        if (prow < p.m && o0 + 16u <= p.rows / 2u) {
                            const size_t at = (size_t)prow * p.ld_out + o0 + q * 8u;
#pragma unroll
                            for (uint32_t k = 0; k + 1u < kMaxExchangeRanks; ++k) {
                                if (k >= p.peers) break;
                                *reinterpret_cast<uint4 *>(p.peer_out[k] + at) = v;
                            }
                        }
                    }
                    __syncwarp();
                }
            } else {
                const bool cols_ok = f0 + 32u <= p.rows;
                uint16_t *dst16 = p.out + (size_t)row * p.ld_out + f0;
                uint32_t packed[16];
                if (p.epilogue == kEpiResidual && row_ok && cols_ok) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(dst16);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const uint4 rv = src[q4];
                        const uint32_t rr[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int i = q4 * 8 + e * 2;
                            const uint32_t y2 = f32x2_to_bf16x2(__uint_as_float(acc[i]), __uint_as_float(acc[i + 1]));
                            packed[q4 * 4 + e] = f32x2_to_bf16x2(__uint_as_float(y2 << 16) + __uint_as_float(rr[e] << 16),
                                                                 __uint_as_float(y2 & 0xffff0000u) +
                                                                     __uint_as_float(rr[e] & 0xffff0000u));
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        packed[i >> 1] = f32x2_to_bf16x2(__uint_as_float(acc[i]), __uint_as_float(acc[i + 1]));
                }
                if (row_ok && cols_ok) {
                    uint4 *dst = reinterpret_cast<uint4 *>(dst16);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        dst[q4] = make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
                }
                if (p.peers && acc_ok) {
                    // to the other ranks, regrouped through the warp's scratch rows (80-byte pitch) so that four
                    // neighbouring lanes write one row's 64 contiguous bytes (see the gated branch)
                    uint4 *mine = reinterpret_cast<uint4 *>(scratch + lane * 80u);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        mine[q4] = make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
                    __syncwarp();
#pragma unroll
                    for (uint32_t j = 0; j < 4u; ++j) {
                        const uint32_t r = 8u * j + (lane >> 2), q = lane & 3u;
                        const uint4 v = *reinterpret_cast<const uint4 *>(scratch + r * 80u + q * 16u);
                        const uint32_t prow = row - lane + r;
                        if (prow < p.m && cols_ok) {
                            const size_t at = (size_t)prow * p.ld_out + f0 + q * 8u;
#pragma unroll
                            for (uint32_t k = 0; k + 1u < kMaxExchangeRanks; ++k) {
                                if (k >= p.peers) break;
                                *reinterpret_cast<uint4 *>(p.peer_out[k] + at) = v;
                            }
                        }
                    }
                    __syncwarp();
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

// ---------------------------------------------------------------------------------------- few rows
// The same contraction for a handful of rows (the k + 1 rows a speculative round verifies): the operand roles are
// swapped so that the 128 output features of a CTA are the M rows of the tensor-core tile and at most 16
// activation rows its N columns.  The tensor-core work then shrinks with the row count (128 x 16 x 16 per
// instruction instead of 128 x 128 x 16) and the kernel runs at the pace of its dequantizing prologue, i.e. of
// the weight stream.  Accumulators: lane = feature, column = row.
constexpr uint32_t kSmallRows = 16;
static_assert(kSmallRows == kPrefillSmallRows, "the model-level pass decides by this bound who stores to the peers");
constexpr uint32_t kSmallXStage = kSmallRows * 128u;            // 2 KB: 16 rows x 64 columns bf16
constexpr uint32_t kSmallWStage = 128u * 128u;                  // 16 KB: 128 features x 64 columns bf16
constexpr uint32_t kSmallStageBytes = kSmallWStage + kSmallXStage;   // 18 KB, a multiple of 1024
constexpr uint32_t kSmallStages = 6;
constexpr uint32_t kSmallSmem = kSmallStages * kSmallStageBytes + 1024u + 256u;
constexpr uint32_t kSmallTmemColumns = 32;
constexpr uint32_t kIdescSmall = (1u << 4) | (1u << 7) | (1u << 10) | ((kSmallRows >> 3) << 17) | ((128u >> 4) << 24);

__global__ void __launch_bounds__(kGemmThreads, 1)
prefill_gemm_a4_small_kernel(const __grid_constant__ CUtensorMap x_map, const GemmParams p) {
    extern __shared__ uint8_t gemm_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023u) & ~(uintptr_t)1023u);
    uint8_t *stages = smem;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kSmallStages * kSmallStageBytes);
    uint64_t *full_x = bars, *full_w = bars + kSmallStages, *empty = bars + 2 * kSmallStages, *acc_full = bars + 3 * kSmallStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * kSmallStages + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t n_tile0 = blockIdx.x * 8u;  // 128 features = 8 storage tiles per CTA
    const uint32_t t0 = blockIdx.y * kSmallRows;  // first activation row of this CTA

    if (tid == 0) {
        for (uint32_t s = 0; s < kSmallStages; ++s) {
            mbar_init(&full_x[s], 1);
            mbar_init(&full_w[s], kDequantWarps);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, kSmallTmemColumns);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t slot = 0, phase = 1;
            for (uint32_t kg = 0; kg < p.groups; ++kg) {
                if (!mbar_wait_bounded(&empty[slot], phase, abort_flag)) {
                    *abort_flag = 1;
                    atomicOr(p.error_word, kErrMbarTimeout);
                    break;
                }
                mbar_arrive_expect_tx(&full_x[slot], kSmallXStage);
                tma_load_2d(stages + slot * kSmallStageBytes + kSmallWStage, &x_map, kg * kBK, t0, &full_x[slot]);
                if (++slot == kSmallStages) {
                    slot = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t slot = 0, phase = 0;
            for (uint32_t kg = 0; kg < p.groups; ++kg) {
                if (!(mbar_wait_bounded(&full_x[slot], phase, abort_flag) && mbar_wait_bounded(&full_w[slot], phase, abort_flag))) {
                    *abort_flag = 1;
                    atomicOr(p.error_word, kErrMbarTimeout);
                    break;
                }
                tc_fence_after();
                const uint32_t w_addr = smem_u32(stages + slot * kSmallStageBytes);
                const uint32_t x_addr = w_addr + kSmallWStage;
#pragma unroll
                for (uint32_t k4 = 0; k4 < kBK / 16u; ++k4)
                    umma_f16(tmem_base, smem_desc_sw128(w_addr + k4 * 32u), smem_desc_sw128(x_addr + k4 * 32u), kIdescSmall,
                             (kg | k4) != 0u ? 1u : 0u);
                umma_commit(&empty[slot]);
                if (++slot == kSmallStages) {
                    slot = 0;
                    phase ^= 1u;
                }
            }
            umma_commit(acc_full);
        }
    } else {
        const uint32_t d = warp - 2u;
        const uint32_t tile = n_tile0 + d;
        uint32_t slot = 0, phase = 1;
        constexpr uint32_t kAhead = 4;
        RecordRegs ring[kAhead];
#pragma unroll
        for (uint32_t i = 0; i < kAhead; ++i)
            ring[i] = load_record(p.w, i < p.groups ? tile : 0xffffffffu, p.row_tiles, p.groups, i, lane);
        bool ok = true;
        for (uint32_t kb = 0; kb < p.groups && ok; kb += kAhead) {
#pragma unroll
            for (uint32_t i = 0; i < kAhead; ++i) {
                const uint32_t kg = kb + i;
                if (kg >= p.groups) break;
                const RecordRegs cur = ring[i];
                const uint32_t next = kg + kAhead;
                ring[i] = load_record(p.w, next < p.groups ? tile : 0xffffffffu, p.row_tiles, p.groups,
                                      next < p.groups ? next : 0u, lane);
                if (!mbar_wait_bounded(&empty[slot], phase, abort_flag)) {
                    if (lane == 0) {
                        *abort_flag = 1;
                        atomicOr(p.error_word, kErrMbarTimeout);
                    }
                    ok = false;
                    break;
                }
                dequant_record_to_smem(cur, stages + slot * kSmallStageBytes, d, lane);
                proxy_fence_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_w[slot]);
                if (++slot == kSmallStages) {
                    slot = 0;
                    phase ^= 1u;
                }
            }
        }
        if (d < 4u) {
            // ---- epilogue: four warps cover the 128 lanes of the accumulator; lane = feature, column = row
            const uint32_t sub = warp & 3u;
            if (!mbar_wait_bounded(acc_full, 0, abort_flag) && lane == 0) atomicOr(p.error_word, kErrMbarTimeout);
            tc_fence_after();
            uint32_t acc[16];
            tmem_ld_32x16(tmem_base + ((sub * 32u) << 16), acc);
            const uint32_t feature = n_tile0 * 16u + sub * 32u + lane;  // storage row of the matrix
#pragma unroll
            for (uint32_t j = 0; j < kSmallRows; ++j) {
                const uint32_t row = t0 + j;
                const float v = __uint_as_float(acc[j]);
                if (p.epilogue == kEpiSwiGlu) {
                    // lanes 0-15 hold an `up` tile, lanes 16-31 the `gate` tile of the same logical rows
                    const float gate_raw = __shfl_down_sync(0xffffffffu, v, 16);
                    if (lane < 16u && row < p.m) {
                        const float up = bf16_round(v), gate = bf16_round(gate_raw);
                        const float activated = bf16_round(gate / (1.0f + expf(-1.0f * gate)));
                        const uint32_t logical = (feature / 32u) * 16u + lane;
                        if (logical < p.rows / 2u)
                            p.out[(size_t)row * p.ld_out + logical] = f32_to_bf16_bits(up * activated);
                    }
                } else if (row < p.m && feature < p.rows) {
                    uint16_t *dst = p.out + (size_t)row * p.ld_out + feature;
                    const float y = bf16_round(v);
                    *dst = p.epilogue == kEpiResidual ? f32_to_bf16_bits(y + bf16_bits_to_f32(*dst)) : f32_to_bf16_bits(y);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kSmallTmemColumns);
    }
}

// ---------------------------------------------------------------------------------------- host side

}  // namespace

stark_b200_status prefill_gemm_launch(const GemmArgs &a, cudaStream_t stream) {
    const QMatrix *w = a.w;
    if (!w || !a.x || !a.out || a.m == 0 || a.m > a.x_rows) return STARK_B200_INVALID_ARGUMENT;
    if (w->format != kFmtAffine4) return STARK_B200_UNSUPPORTED;
    if (a.epilogue != kEpiStore && a.epilogue != kEpiResidual && a.epilogue != kEpiSwiGlu) return STARK_B200_UNSUPPORTED;
    // a pair-ordered [up; gate] matrix stores its rows interleaved: only the SwiGLU epilogue puts them back
    if ((a.epilogue == kEpiSwiGlu) != (w->pair_halves != 0)) return STARK_B200_INVALID_ARGUMENT;
    if (w->rows % 32u != 0) return STARK_B200_UNSUPPORTED;  // the epilogue writes whole 32-feature segments
    if ((reinterpret_cast<uintptr_t>(a.x) & 15u) || (reinterpret_cast<uintptr_t>(a.out) & 15u) || (a.ld_out % 8u) != 0)
        return STARK_B200_INVALID_ARGUMENT;
    // A handful of rows is a weight stream, not a contraction: the several-rows matvec reads the matrix once at the
    // pace of the one-token path.
    if (a.peers > kMaxExchangeRanks) return STARK_B200_INVALID_ARGUMENT;
    for (uint32_t r = 0; r < a.peers; ++r)
        if (!a.peer_out[r] || (reinterpret_cast<uintptr_t>(a.peer_out[r]) & 15u)) return STARK_B200_INVALID_ARGUMENT;
    if (a.peers && a.m <= kSmallRows) return STARK_B200_UNSUPPORTED;  // only the 256-row tile kernel stores to peers
    if (tunables().rows_matvec && qmv_multi_supports(w, a.m, false)) {
        QmvMultiArgs q{};
        q.matrix = w;
        q.x = a.x;
        q.x_stride = w->columns;
        q.m = a.m;
        q.y = a.out;
        q.y_stride = a.ld_out;
        q.epilogue = a.epilogue;
        q.error_word = a.error_word;
        q.pdl = true;  // the kernel awaits its predecessor itself, after its weight ring has begun to fill
        return qmv_multi_launch(q, stream);
    }
    EncodeTiledFn encode = encode_tiled();
    if (!encode) return STARK_B200_UNSUPPORTED;

    // Up to 16 rows take the few-rows kernel (rows as the N side of the tile); more take 256-row tiles.
    const bool small = a.m <= kSmallRows;
    CUtensorMap map;
    const cuuint64_t dims[2] = {w->columns, a.x_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)w->columns * 2u};
    const cuuint32_t box[2] = {kBK, small ? kSmallRows : 128u};
    const cuuint32_t elem[2] = {1u, 1u};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(a.x), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return STARK_B200_DEVICE_FAILURE;

    GemmParams p{};
    p.w = w->data;
    p.row_tiles = w->row_tiles;
    p.groups = w->groups;
    p.rows = w->rows;
    p.m = a.m;
    p.out = a.out;
    p.ld_out = a.ld_out;
    p.epilogue = a.epilogue;
    p.error_word = a.error_word;
    p.peers = a.peers;
    for (uint32_t r = 0; r < a.peers; ++r) p.peer_out[r] = a.peer_out[r];
    p.stop_after = tunables().gemm_stop_after;
    static SmemOptIn once, once_small;
    const uint32_t width = small ? 128u : kBN;
    const uint32_t feature_tiles = (w->row_tiles * 16u + width - 1u) / width;
    if (small) {
        if (stark_b200_status s = ensure_dynamic_smem(prefill_gemm_a4_small_kernel, (int)kSmallSmem, once_small)) return s;
        prefill_gemm_a4_small_kernel<<<dim3(feature_tiles, (a.m + kSmallRows - 1u) / kSmallRows), kGemmThreads, kSmallSmem,
                                       stream>>>(map, p);
    } else {
        // Tile height by waves over the SMs: a 128-row tile takes 0.87 of a 256-row tile's time (measured: it
        // dequantizes the same weight tile for half the rows), so it pays only where 256-row tiles leave more than
        // half of the SMs idle.
        const uint32_t sms = 148u, full = feature_tiles * ((a.m + kBM - 1u) / kBM), halved = feature_tiles * ((a.m + 127u) / 128u);
        const float cost_full = (float)((full + sms - 1u) / sms), cost_half = 0.87f * (float)((halved + sms - 1u) / sms);
        const uint32_t mode = tunables().gemm_half_tiles;  // 0 never, 1 by the rule above, 2 always
        if (mode == 2u || (mode == 1u && cost_half < cost_full)) {
            static SmemOptIn once_half;
            if (stark_b200_status s = ensure_dynamic_smem(prefill_gemm_a4_kernel<1>, (int)kGemmSmem, once_half)) return s;
            prefill_gemm_a4_kernel<1><<<dim3(feature_tiles, (a.m + 127u) / 128u), kGemmThreads, kGemmSmem, stream>>>(map, p);
        } else {
            if (stark_b200_status s = ensure_dynamic_smem(prefill_gemm_a4_kernel<2>, (int)kGemmSmem, once)) return s;
            prefill_gemm_a4_kernel<2><<<dim3(feature_tiles, (a.m + kBM - 1u) / kBM), kGemmThreads, kGemmSmem, stream>>>(map, p);
        }
    }
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

}  // namespace sb
