// Device helpers shared by the matvec, attention and persistent decode kernels.
#pragma once
#include "common.cuh"
#include "ops.cuh"

namespace sb {

constexpr int kAttnThreads = 128;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kMaxGqa = 8;
constexpr uint32_t kTileRowBytes = kHeadDim * 2u + 16u;  // 272: rows 16 B apart modulo 128 B, so ldmatrix is conflict-free
constexpr uint32_t kTileBytes = kPageTokens * kTileRowBytes;
constexpr uint32_t kAttnSmemBytes = 4u * kTileBytes;  // K and V, double buffered


// 4-bit -> f16 conversion of one record word into an m16n8k16 A fragment.
//   (w & 0x000f000f) | 0x64006400 is the f16 pair (1024 + q, 1024 + q');
//   (w & 0x00f000f0) | 0x64006400 is (1024 + 16 q, ...);
//   (w & 0x00f000f0) | 0x54005400 is (64 + q, ...): 0x5400 is 64.0 and bit 4 of an f16 in [64, 128) weighs 1.
// FOLD == 0: the offsets are removed here, exactly (x - 1024; x/16 - 64 in one FMA), so the tensor core
//   sees the integers q: 9 instructions per 8 codes.
// FOLD == 1: the first two patterns go to the tensor core as they are and the offsets are removed from
//   the f32 group sums afterwards (row g: c - 1024 sum(x); row g+8: c/16 - 64 sum(x)): 5 instructions.
//   The accumulation then carries 1024 x + q x, which costs about 7 bits of the f32 accumulator.
// FOLD == 2: every nibble is shifted to bits 4..7 of its half and becomes 64 + q; both row halves carry
//   64 x + q x and the group sums lose 64 sum(x): 7 instructions, about 3 bits of the accumulator --
//   less than what a sequential f32 sum over a row of a few thousand products loses anyway.
template <int FOLD>
__device__ inline void dequant_a4_word(uint32_t w, uint32_t (&a)[4]) {
    if (FOLD == 2) {
        const uint32_t magic64 = 0x54005400u, mask = 0x00f000f0u;
        a[0] = lop3_and_or(w << 4, mask, magic64);
        a[1] = lop3_and_or(w, mask, magic64);
        a[2] = lop3_and_or(w >> 4, mask, magic64);
        a[3] = lop3_and_or(w >> 8, mask, magic64);
        return;
    }
    const uint32_t magic = 0x64006400u;
    const uint32_t lo0 = lop3_and_or(w, 0x000f000fu, magic);
    const uint32_t hi0 = lop3_and_or(w, 0x00f000f0u, magic);
    const uint32_t w8 = w >> 8;
    const uint32_t lo1 = lop3_and_or(w8, 0x000f000fu, magic);
    const uint32_t hi1 = lop3_and_or(w8, 0x00f000f0u, magic);
    if (FOLD == 1) {
        a[0] = lo0;
        a[1] = hi0;
        a[2] = lo1;
        a[3] = hi1;
    } else {
        const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
        const __half2 k16th = __half2half2(__ushort_as_half(0x2c00));   // 1/16
        const __half2 kneg64 = __half2half2(__ushort_as_half(0xd400));  // -64
        __half2 r0 = __hsub2(*reinterpret_cast<const __half2 *>(&lo0), k1024);
        __half2 r1 = __hfma2(*reinterpret_cast<const __half2 *>(&hi0), k16th, kneg64);
        __half2 r2 = __hsub2(*reinterpret_cast<const __half2 *>(&lo1), k1024);
        __half2 r3 = __hfma2(*reinterpret_cast<const __half2 *>(&hi1), k16th, kneg64);
        a[0] = *reinterpret_cast<uint32_t *>(&r0);
        a[1] = *reinterpret_cast<uint32_t *>(&r1);
        a[2] = *reinterpret_cast<uint32_t *>(&r2);
        a[3] = *reinterpret_cast<uint32_t *>(&r3);
    }
}


__device__ inline void cp_async16(void *smem_dst, const void *gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ inline void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ inline void ldmatrix_x4(uint32_t (&r)[4], const void *smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}
__device__ inline void ldmatrix_x4_trans(uint32_t (&r)[4], const void *smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}
__device__ inline void mma_m16n8k16_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Transposes an 8x8 matrix of 16-bit elements held one row-pair per lane (lane (g, t): row g, columns
// 2t, 2t+1); afterwards the lane holds row g of the transpose.
__device__ inline uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
// f32 pair -> packed bf16 (hi) and the packed bf16 of the remainders (lo): hi + lo carries ~16 bits.
__device__ inline void split_bf16x2(float x, float y, uint32_t &hi, uint32_t &lo) {
    hi = f32x2_to_bf16x2(x, y);
    lo = f32x2_to_bf16x2(x - __uint_as_float(hi << 16), y - __uint_as_float(hi & 0xffff0000u));
}

// Per-head RMS norm + RoPE of one 128-wide head by ONE warp; lane l holds dims {2l, 2l+1, 64+2l, 65+2l},
// so the half-split RoPE pairs (d, d+64) sit in the same lane and no shared memory is needed.
//   qkv_norm.rs:44-108: f32 sum of squares, rms = 1/sqrt(mean + eps), bf16(normalized) * bf16(scale) -> bf16
//   attention_prepare.rs:7-43: x*cos + (+-pair)*sin with separately rounded products, then bf16
// The constants of a lane (norm weights already rounded to bf16, cos / sin of the row's position) can be
// fetched before the row itself exists.
struct HeadConsts {
    float nw[4], cs[4], sn[4];
};
__device__ inline HeadConsts load_head_consts(const float *norm_w, const float *cosr, const float *sinr,
                                              uint32_t lane) {
    HeadConsts c;
    const uint32_t d[4] = {2u * lane, 2u * lane + 1u, 64u + 2u * lane, 65u + 2u * lane};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        c.nw[i] = norm_w ? bf16_round(norm_w[d[i]]) : 1.0f;
        c.cs[i] = cosr ? cosr[d[i]] : 1.0f;
        c.sn[i] = sinr ? sinr[d[i]] : 0.0f;
    }
    return c;
}
// The lane's four values of a head row (two packed bf16 pairs).
__device__ inline void load_head_row(const uint16_t *head, uint32_t lane, uint32_t &lo2, uint32_t &hi2) {
    // ld.cg: the row may have been written by another CTA of a kernel that is still running
    lo2 = __ldcg(reinterpret_cast<const uint32_t *>(head + 2u * lane));
    hi2 = __ldcg(reinterpret_cast<const uint32_t *>(head + 64u + 2u * lane));
}
__device__ inline void head_norm_rope_regs(uint32_t lo2, uint32_t hi2, const HeadConsts &c, bool has_norm, bool has_rope,
                                           float eps, uint32_t lane, uint16_t *out /* smem [128] */) {
    float v[4] = {__uint_as_float(lo2 << 16), __uint_as_float(lo2 & 0xffff0000u), __uint_as_float(hi2 << 16),
                  __uint_as_float(hi2 & 0xffff0000u)};
    // The roundings go through the packed hardware conversion (round to nearest even, like the reference's
    // bf16 type; only the payload of a NaN differs): this code sits on the critical path of every layer.
    if (has_norm) {
        const float total = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
        const float rms = 1.0f / sqrtf(total / (float)kHeadDim + eps);
#pragma unroll
        for (int i = 0; i < 4; i += 2) {
            const uint32_t n2 = f32x2_to_bf16x2(v[i] * rms, v[i + 1] * rms);
            const uint32_t p2 = f32x2_to_bf16x2(__uint_as_float(n2 << 16) * c.nw[i],
                                                __uint_as_float(n2 & 0xffff0000u) * c.nw[i + 1]);
            v[i] = __uint_as_float(p2 << 16);
            v[i + 1] = __uint_as_float(p2 & 0xffff0000u);
        }
    }
    uint32_t lo_pair, hi_pair;
    if (has_rope) {
        // first half: x*cos - pair*sin ; second half: x*cos + pair*sin (products rounded separately)
        lo_pair = f32x2_to_bf16x2(__fadd_rn(__fmul_rn(v[0], c.cs[0]), __fmul_rn(-v[2], c.sn[0])),
                                  __fadd_rn(__fmul_rn(v[1], c.cs[1]), __fmul_rn(-v[3], c.sn[1])));
        hi_pair = f32x2_to_bf16x2(__fadd_rn(__fmul_rn(v[2], c.cs[2]), __fmul_rn(v[0], c.sn[2])),
                                  __fadd_rn(__fmul_rn(v[3], c.cs[3]), __fmul_rn(v[1], c.sn[3])));
    } else {
        lo_pair = f32x2_to_bf16x2(v[0], v[1]);
        hi_pair = f32x2_to_bf16x2(v[2], v[3]);
    }
    *reinterpret_cast<uint32_t *>(out + 2u * lane) = lo_pair;
    *reinterpret_cast<uint32_t *>(out + 64u + 2u * lane) = hi_pair;
}
__device__ inline void warp_head_norm_rope(const uint16_t *head, const HeadConsts &c, bool has_norm, bool has_rope,
                                           float eps, uint32_t lane, uint16_t *out /* smem [128] */) {
    uint32_t lo2, hi2;
    load_head_row(head, lane, lo2, hi2);
    head_norm_rope_regs(lo2, hi2, c, has_norm, has_rope, eps, lane, out);
}
__device__ inline void warp_head_norm_rope(const uint16_t *head, const float *norm_w, const float *cosr,
                                           const float *sinr, float eps, uint32_t lane, uint16_t *out) {
    const HeadConsts c = load_head_consts(norm_w, cosr, sinr, lane);
    warp_head_norm_rope(head, c, norm_w != nullptr, cosr != nullptr, eps, lane, out);
}


}  // namespace sb
