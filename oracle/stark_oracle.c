/*
 * stark_oracle.c -- CPU restatement of the reference token-loop arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against (tests, the smoke check, and the `cpu_baseline` / `--impl reference`
 * legs of the benchmark).  Nothing in the shipped library links, loads or calls
 * it, and the shipped library has no CPU fallback.
 *
 * The reference (jshahbazi/stark) is Rust; it cannot be compiled where this
 * repository is built, so each function below restates one reference routine
 * and names it (paths are relative to the reference's repository root).  The
 * restatement is pinned by the reference's own known answers:
 *   - packed_code vectors            crates/stark-engine/src/backends/cpu/kernel/matmul/reference.rs:195-219
 *   - exact packed tails             .../matmul/reference.rs:240-285
 *   - GGUF block SHA-256 table       crates/stark-engine/src/engine/hybrid/weights.rs:3183-3221
 *   - MLX plane layout closed forms  crates/stark-engine/src/engine/hybrid/weights.rs:4044-4083
 *   - softmax / top-k / rms KATs     crates/stark-engine/src/engine/hybrid/math.rs:72-99
 * Parts that depend on the platform libm (sinf/cosf/expf/powf in RoPE tables,
 * SiLU and softmax) follow the reference's formulas and operation order, but a
 * last-bit difference between libm implementations cannot be excluded there.
 *
 * Build with -ffp-contract=off: Rust never contracts a*b+c into an FMA.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define SO_OK 0
#define SO_INVALID 1

/* ------------------------------------------------------------------ scalars */

/* half::bf16::to_f32 */
static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* half::bf16::from_f32: round to nearest even, NaN kept quiet. */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t round_bit = 0x00008000u;
    if ((u & round_bit) != 0 && (u & (3u * round_bit - 1u)) != 0) return (uint16_t)((u >> 16) + 1u);
    return (uint16_t)(u >> 16);
}

static inline float bf16_round(float f) { return bf16_to_f32(f32_to_bf16(f)); }

/* half::f16::to_f32 */
static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {
            int e = -1;
            do {
                e++;
                man <<= 1;
            } while ((man & 0x400u) == 0);
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

uint16_t so_f32_to_bf16(float f) { return f32_to_bf16(f); }
float so_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
float so_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

/* ------------------------------------------------------- integer unpacking */

/* packed_code: crates/stark-engine/src/backends/cpu/kernel/matmul/reference.rs:91-104.
 * Code `index` starts at bit index*bits, LSB first inside little-endian bytes. */
uint8_t so_packed_code(const uint8_t *codes, size_t bits, size_t index) {
    size_t bit = index * bits;
    size_t offset = bit / 8;
    size_t shift = bit % 8;
    uint16_t value = codes[offset];
    if (shift + bits > 8) value |= (uint16_t)codes[offset + 1] << 8;
    return (uint8_t)((value >> shift) & ((1u << bits) - 1u));
}

void so_unpack_codes(const uint8_t *codes, size_t bits, size_t count, uint8_t *out) {
    for (size_t i = 0; i < count; i++) out[i] = so_packed_code(codes, bits, i);
}

/* ------------------------------------------------------ MLX-affine matvec */

/* Path A: MatmulCpuKernel quantized branch,
 * crates/stark-engine/src/backends/cpu/kernel/matmul/kernel.rs:168-285.
 *   acc(f32) += f32(a[m,k]) * (scale*f32(q) + bias), k ascending; output RNE to bf16.
 * scale_layout 0: planes [N, G]  (MLX native, output_stride = G, group_stride = 1)
 * scale_layout 1: planes [G, npad] (GroupOutput layout, crates/stark-engine/src/backends/common/kernel/matmul/mod.rs:120-156)
 * correction 0: explicit bias plane; 1: symmetric (bias = -scale*2^(bits-1)).
 * signed_codes: code ^= 1 << (bits-1) before widening (kernel.rs:233-235). */
int so_affine_matvec_bf16(const uint8_t *codes, const uint16_t *scales, const uint16_t *biases, const uint16_t *a,
                          uint16_t *d, uint32_t m, uint32_t n, uint32_t k, uint32_t bits, uint32_t group,
                          uint32_t scale_layout, uint32_t npad, uint32_t correction, uint32_t signed_codes,
                          int threads) {
    if (!(bits == 4 || bits == 8) || group == 0 || k % group != 0) return SO_INVALID;
    const size_t groups = k / group;
    const size_t out_stride = scale_layout == 0 ? groups : 1;
    const size_t grp_stride = scale_layout == 0 ? 1 : npad;
    const float midpoint = (float)(1u << (bits - 1));
    (void)threads;
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
    for (int64_t col = 0; col < (int64_t)n; col++) {
        for (uint32_t row = 0; row < m; row++) {
            float acc = 0.0f;
            for (uint32_t inner = 0; inner < k; inner++) {
                float a_value = bf16_to_f32(a[(size_t)row * k + inner]);
                uint8_t code = so_packed_code(codes, bits, (size_t)col * k + inner);
                if (signed_codes) code ^= (uint8_t)(1u << (bits - 1));
                float q = (float)code;
                size_t meta = (size_t)col * out_stride + (inner / group) * grp_stride;
                float scale = bf16_to_f32(scales[meta]);
                float bias_term = correction == 0 ? bf16_to_f32(biases[meta]) : -scale * midpoint;
                float b_value = scale * q + bias_term;
                acc += a_value * b_value;
            }
            d[(size_t)row * n + col] = f32_to_bf16(1.0f * acc);
        }
    }
    return SO_OK;
}

/* Path B: Weights::affine_row + matrix_slice host branch,
 * crates/stark-engine/src/engine/hybrid/weights.rs:1284-1309, 2534-2552.
 * Decode a whole row to f32 (scale*q+bias), then sum(w*x) sequentially in f32.
 * plane_kind: 0 = f32, 1 = f16, 30 = bf16 (weights.rs:1207). */
static inline float plane_scalar(uint32_t kind, const void *base, size_t index) {
    if (kind == 0) return ((const float *)base)[index];
    if (kind == 1) return f16_to_f32(((const uint16_t *)base)[index]);
    return bf16_to_f32(((const uint16_t *)base)[index]);
}

int so_affine_matvec_f32(const uint8_t *codes, const void *scales, const void *biases, uint32_t plane_kind,
                         const float *x, float *y, uint32_t rows, uint32_t columns, uint32_t bits, uint32_t group,
                         int threads) {
    if (!(bits == 4 || bits == 8) || !(group == 32 || group == 64 || group == 128) || columns % group != 0)
        return SO_INVALID;
    for (uint32_t i = 0; i < columns; i++)
        if (!isfinite(x[i])) return SO_INVALID;
    const size_t group_count = columns / group;
    const size_t packed_row = (size_t)columns * bits / 8;
    (void)threads;
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
    for (int64_t row = 0; row < (int64_t)rows; row++) {
        const uint8_t *row_codes = codes + (size_t)row * packed_row;
        float total = 0.0f;
        for (uint32_t column = 0; column < columns; column++) {
            size_t index = (size_t)row * group_count + column / group;
            float scale = plane_scalar(plane_kind, scales, index);
            float bias = plane_scalar(plane_kind, biases, index);
            uint8_t q = (uint8_t)((row_codes[(size_t)column * bits / 8] >> ((size_t)column * bits % 8)) &
                                  (uint8_t)((1u << bits) - 1u));
            float w = scale * (float)q + bias;
            total += w * x[column];
        }
        y[row] = total;
    }
    return SO_OK;
}

/* Dequantize one affine row (for the plane-layout known answers). */
int so_affine_row_f32(const uint8_t *codes, const void *scales, const void *biases, uint32_t plane_kind, float *out,
                      uint32_t row, uint32_t columns, uint32_t bits, uint32_t group) {
    if (!(bits == 4 || bits == 8) || columns % group != 0) return SO_INVALID;
    const size_t group_count = columns / group;
    const uint8_t *row_codes = codes + (size_t)row * columns * bits / 8;
    for (uint32_t column = 0; column < columns; column++) {
        size_t index = (size_t)row * group_count + column / group;
        uint8_t q = (uint8_t)((row_codes[(size_t)column * bits / 8] >> ((size_t)column * bits % 8)) &
                              (uint8_t)((1u << bits) - 1u));
        out[column] = plane_scalar(plane_kind, scales, index) * (float)q + plane_scalar(plane_kind, biases, index);
    }
    return SO_OK;
}

/* ------------------------------------------------------------ GGUF blocks */

/* block_layout: crates/stark-engine/src/engine/hybrid/weights.rs:2565-2584 (kinds 8 and 12 only). */
int so_block_layout(uint32_t kind, uint32_t *elements, uint32_t *bytes) {
    if (kind == 8) {
        *elements = 32;
        *bytes = 34;
        return SO_OK;
    }
    if (kind == 12) {
        *elements = 256;
        *bytes = 144;
        return SO_OK;
    }
    return SO_INVALID;
}

/* scale_min: weights.rs:2908-2920 */
static inline void scale_min(const uint8_t *scales, int index, uint8_t *sc, uint8_t *mn) {
    if (index < 4) {
        *sc = scales[index] & 63;
        *mn = scales[index + 4] & 63;
    } else {
        *sc = (uint8_t)((scales[index + 4] & 15) | ((scales[index - 4] >> 6) << 4));
        *mn = (uint8_t)((scales[index + 4] >> 4) | ((scales[index] >> 6) << 4));
    }
}

/* decode_block kinds 8 (Q8_0) and 12 (Q4_K): weights.rs:2936-2941, 2993-3017. */
int so_decode_block(uint32_t kind, const uint8_t *bytes, float *output) {
    if (kind == 8) {
        float d = f16_to_f32((uint16_t)(bytes[0] | (bytes[1] << 8)));
        for (int i = 0; i < 32; i++) output[i] = d * (float)(int8_t)bytes[2 + i];
        return SO_OK;
    }
    if (kind == 12) {
        float d = f16_to_f32((uint16_t)(bytes[0] | (bytes[1] << 8)));
        float minimum = f16_to_f32((uint16_t)(bytes[2] | (bytes[3] << 8)));
        const uint8_t *scales = bytes + 4;
        for (int part = 0; part < 4; part++) {
            for (int half = 0; half < 2; half++) {
                uint8_t sc, mn;
                scale_min(scales, part * 2 + half, &sc, &mn);
                int at = part * 64 + half * 32;
                for (int l = 0; l < 32; l++) {
                    uint8_t ql = (bytes[16 + part * 32 + l] >> (half * 4)) & 15;
                    output[at + l] = d * (float)sc * (float)ql - minimum * (float)mn;
                }
            }
        }
        return SO_OK;
    }
    return SO_INVALID;
}

/* Integer fields of a Q4_K block, for the bit-exact unpack test:
 * codes[256], sub-block scales[8], mins[8]. */
int so_q4k_unpack(const uint8_t *bytes, uint8_t *codes, uint8_t *scales6, uint8_t *mins6) {
    for (int part = 0; part < 4; part++)
        for (int half = 0; half < 2; half++) {
            scale_min(bytes + 4, part * 2 + half, &scales6[part * 2 + half], &mins6[part * 2 + half]);
            for (int l = 0; l < 32; l++)
                codes[part * 64 + half * 32 + l] = (bytes[16 + part * 32 + l] >> (half * 4)) & 15;
        }
    return SO_OK;
}

/* decode_values + host matvec: weights.rs:2880-2895, 2534-2552.  GGUF rows are
 * `columns/block` consecutive blocks; y[row] = sum(w*x) sequentially in f32. */
int so_gguf_matvec_f32(uint32_t kind, const uint8_t *bytes, const float *x, float *y, uint32_t rows,
                       uint32_t columns, int threads) {
    uint32_t be, bb;
    if (so_block_layout(kind, &be, &bb) != SO_OK || columns % be != 0) return SO_INVALID;
    for (uint32_t i = 0; i < columns; i++)
        if (!isfinite(x[i])) return SO_INVALID;
    const size_t row_bytes = (size_t)(columns / be) * bb;
    (void)threads;
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
    for (int64_t row = 0; row < (int64_t)rows; row++) {
        float values[256];
        float total = 0.0f;
        const uint8_t *src = bytes + (size_t)row * row_bytes;
        for (uint32_t b = 0; b < columns / be; b++) {
            so_decode_block(kind, src + (size_t)b * bb, values);
            for (uint32_t i = 0; i < be; i++) total += values[i] * x[b * be + i];
        }
        y[row] = total;
    }
    return SO_OK;
}

int so_gguf_decode_row(uint32_t kind, const uint8_t *bytes, float *out, uint32_t columns) {
    uint32_t be, bb;
    if (so_block_layout(kind, &be, &bb) != SO_OK || columns % be != 0) return SO_INVALID;
    for (uint32_t b = 0; b < columns / be; b++) so_decode_block(kind, bytes + (size_t)b * bb, out + (size_t)b * be);
    return SO_OK;
}

/* ------------------------------------------------------------- small ops */

/* normalization (RMS, bf16 in/out, f32 scales, OnlyNormalization rounding):
 * crates/stark-engine/src/backends/cpu/kernel/normalization/normalization.rs:13-191.
 * residual_add != 0: val = bf16(input + shortcut), shortcut = val (ShortcutMode::Add);
 * residual_add == 0 and shortcut != NULL: shortcut = input (ShortcutMode::Copy). */
void so_rmsnorm_bf16(const uint16_t *input, const float *scales, uint16_t *output, uint16_t *shortcut,
                     uint32_t batch, uint32_t count, float epsilon, int residual_add) {
    for (uint32_t b = 0; b < batch; b++) {
        const uint16_t *in = input + (size_t)b * count;
        uint16_t *out = output + (size_t)b * count;
        uint16_t *sc = shortcut ? shortcut + (size_t)b * count : NULL;
        float sum_sq = 0.0f;
        for (uint32_t i = 0; i < count; i++) {
            uint16_t val = in[i];
            if (sc) {
                if (residual_add) val = f32_to_bf16(bf16_to_f32(val) + bf16_to_f32(sc[i]));
                sc[i] = val;
            }
            float a = bf16_to_f32(val);
            sum_sq = sum_sq + a * a;
        }
        float variance = sum_sq / (float)count - 0.0f * 0.0f;
        float rms_inv = 1.0f / sqrtf(variance + epsilon);
        for (uint32_t i = 0; i < count; i++) {
            float v = (sc && residual_add) ? bf16_to_f32(sc[i]) : bf16_to_f32(in[i]);
            float normalized = (v - 0.0f) * rms_inv;
            float lo = bf16_round(normalized);
            float s = bf16_round(scales[i] + 0.0f);
            out[i] = f32_to_bf16(lo * s);
        }
    }
}

/* hybrid::math::rms_norm (f32 path): crates/stark-engine/src/engine/hybrid/math.rs:18-34 */
int so_rmsnorm_f32(const float *x, const float *weight, float *out, uint32_t count, float eps) {
    if (count == 0 || !(eps > 0.0f) || !isfinite(eps)) return SO_INVALID;
    float sum = 0.0f;
    for (uint32_t i = 0; i < count; i++) {
        if (!isfinite(x[i]) || !isfinite(weight[i])) return SO_INVALID;
        sum += x[i] * x[i];
    }
    float mean = sum / (float)count;
    float scale = 1.0f / sqrtf(mean + eps);
    for (uint32_t i = 0; i < count; i++) out[i] = x[i] * scale * weight[i];
    return SO_OK;
}

/* qkv_norm (per-head RMS norm, in place, bf16, f32 scales):
 * crates/stark-engine/src/backends/cpu/kernel/attention/qkv_norm.rs:8-111 */
void so_head_norm_bf16(uint16_t *row, const float *scales, uint32_t head_offset, uint32_t head_count,
                       uint32_t head_dim, float epsilon) {
    for (uint32_t head = 0; head < head_count; head++) {
        uint16_t *h = row + (size_t)(head_offset + head) * head_dim;
        float total = 0.0f;
        for (uint32_t i = 0; i < head_dim; i++) {
            float v = bf16_to_f32(h[i]);
            total = total + v * v;
        }
        float mean_square = total / (float)head_dim;
        float rms = 1.0f / sqrtf(mean_square + epsilon);
        for (uint32_t i = 0; i < head_dim; i++) {
            float normalized = bf16_to_f32(h[i]) * rms;
            h[i] = f32_to_bf16(bf16_round(normalized) * bf16_round(scales[i] + 0.0f));
        }
    }
}

/* RoPE coefficient for (position, pair): precalculate_cpu_tables, UnscaledRoPEConfig,
 * crates/stark-engine/src/encodable_block/mixer/attention/rope.rs:346-440 */
void so_rope_coeffs(uint32_t position, uint32_t head_dim, float base, float *cosines, float *sines) {
    uint32_t half = head_dim / 2;
    for (uint32_t pair = 0; pair < half; pair++) {
        uint32_t channel = pair * 2;
        float inv = 1.0f / powf(base, (float)channel / (float)head_dim);
        float embedding = (float)position * inv;
        float s = sinf(embedding) * 1.0f;
        float c = cosf(embedding) * 1.0f;
        sines[pair] = s;
        sines[pair + half] = s;
        cosines[pair] = c;
        cosines[pair + half] = c;
    }
}

/* apply_rope, half-split pairing, f32 math, bf16 store:
 * crates/stark-engine/src/backends/cpu/kernel/attention/attention_prepare.rs:7-43 */
void so_rope_head_bf16(const uint16_t *head, uint16_t *out, const float *cosines, const float *sines,
                       uint32_t head_dim) {
    uint32_t half = head_dim / 2;
    for (uint32_t i = 0; i < head_dim; i++) {
        uint32_t p = i < half ? i + half : i - half;
        float input = bf16_to_f32(head[i]);
        float paired = bf16_to_f32(head[p]);
        float signed_paired = i < half ? -paired : paired;
        out[i] = f32_to_bf16(input * cosines[i] + signed_paired * sines[i]);
    }
}

/* attention_single_pass, causal, one query row per head (decode), GQA:
 * crates/stark-engine/src/backends/cpu/kernel/attention/attention_single_pass.rs:11-133.
 * keys/values: [sequence_length, kv_heads, head_dim] bf16; queries [heads, head_dim]; out [heads, head_dim]. */
void so_attention_decode_bf16(const uint16_t *queries, const uint16_t *keys, const uint16_t *values, uint16_t *out,
                              uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t sequence_length,
                              float scale, int threads) {
    const uint32_t gqa = heads / kv_heads;
    const size_t seq_stride = (size_t)kv_heads * head_dim;
    (void)threads;
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
    for (int64_t head = 0; head < (int64_t)heads; head++) {
        uint32_t kvh = (uint32_t)head / gqa;
        float q[512], o[512];
        for (uint32_t j = 0; j < head_dim; j++) {
            q[j] = scale * bf16_to_f32(queries[(size_t)head * head_dim + j]);
            o[j] = 0.0f;
        }
        float max_score = -INFINITY, sum_exp = 0.0f;
        for (uint32_t i = 0; i < sequence_length; i++) {
            const uint16_t *kr = keys + (size_t)i * seq_stride + (size_t)kvh * head_dim;
            float score = 0.0f;
            for (uint32_t j = 0; j < head_dim; j++) score += q[j] * bf16_to_f32(kr[j]);
            float new_max = fmaxf(max_score, score);
            float factor = expf(max_score - new_max);
            float e = expf(score - new_max);
            max_score = new_max;
            sum_exp = sum_exp * factor + e;
            const uint16_t *vr = values + (size_t)i * seq_stride + (size_t)kvh * head_dim;
            for (uint32_t j = 0; j < head_dim; j++) o[j] = o[j] * factor + e * bf16_to_f32(vr[j]);
        }
        for (uint32_t j = 0; j < head_dim; j++) out[(size_t)head * head_dim + j] = f32_to_bf16(o[j] / sum_exp);
    }
}

/* gated_act_mul on a fused [up; gate] row, SiLU alpha 1, bf16:
 * crates/stark-engine/src/backends/cpu/kernel/gated_act_mul/gated_act_mul.rs:66-100,
 * crates/stark-engine/src/backends/common/gpu_types/activation_type.rs:37-49 */
void so_swiglu_bf16(const uint16_t *fused, uint16_t *out, uint32_t gated_dim) {
    for (uint32_t g = 0; g < gated_dim; g++) {
        float value = bf16_to_f32(fused[g]);
        float gate = bf16_to_f32(fused[gated_dim + g]);
        float activated = bf16_round(gate / (1.0f + expf(-1.0f * gate)));
        out[g] = f32_to_bf16(bf16_round(value * activated));
    }
}

/* input_embedding_lookup, quantized ScaleBias table, bf16 row:
 * crates/stark-engine/src/backends/cpu/kernel/embedding/input_embedding_lookup.rs:59-105 */
void so_embedding_row_bf16(const uint8_t *codes, const uint16_t *scales, const uint16_t *biases, uint32_t token,
                           uint32_t vocab, uint32_t dim, uint32_t bits, uint32_t group, uint16_t *out) {
    if (token >= vocab) {
        memset(out, 0, (size_t)dim * 2);
        return;
    }
    size_t groups = (dim + group - 1) / group;
    for (uint32_t c = 0; c < dim; c++) {
        size_t index = (size_t)token * groups + c / group;
        float scale = bf16_to_f32(scales[index]);
        float bias = bf16_to_f32(biases[index]);
        float code = (float)so_packed_code(codes, bits, (size_t)token * dim + c);
        float deq = scale * code + bias;
        out[c] = f32_to_bf16(deq * 1.0f);
    }
}

/* Greedy token: first index of the maximum; any non-finite logit => UINT32_MAX.
 * crates/stark-engine/src/backends/cpu/kernel/sampling/unified_sampling.rs:36-45,108-116 */
uint32_t so_argmax_bf16(const uint16_t *logits, uint32_t vocab) {
    uint32_t best = UINT32_MAX;
    float best_value = -INFINITY;
    for (uint32_t i = 0; i < vocab; i++) {
        float v = bf16_to_f32(logits[i]);
        if (!isfinite(v)) return UINT32_MAX;
        if (best == UINT32_MAX || v > best_value) {
            best = i;
            best_value = v;
        }
    }
    return best;
}

uint32_t so_argmax_f32(const float *logits, uint32_t vocab) {
    uint32_t best = UINT32_MAX;
    float best_value = -INFINITY;
    for (uint32_t i = 0; i < vocab; i++) {
        if (!isfinite(logits[i])) return UINT32_MAX;
        if (best == UINT32_MAX || logits[i] > best_value) {
            best = i;
            best_value = logits[i];
        }
    }
    return best;
}

/* Full-vocabulary log-probabilities in f64:
 * crates/stark-score/src/scoring.rs:299-336  log p_i = logit_i - (max + ln sum exp(logit - max)) */
void so_log_softmax_f64(const float *logits, double *out, uint32_t vocab) {
    double maximum = -INFINITY;
    for (uint32_t i = 0; i < vocab; i++)
        if ((double)logits[i] > maximum) maximum = (double)logits[i];
    double sum = 0.0;
    for (uint32_t i = 0; i < vocab; i++) sum += exp((double)logits[i] - maximum);
    double lse = maximum + log(sum);
    for (uint32_t i = 0; i < vocab; i++) out[i] = (double)logits[i] - lse;
}

/* hybrid::math::softmax: crates/stark-engine/src/engine/hybrid/math.rs:36-51 */
int so_softmax_f32(const float *x, float *out, uint32_t count) {
    if (count == 0) return SO_INVALID;
    float maximum = -INFINITY;
    for (uint32_t i = 0; i < count; i++) {
        if (isnan(x[i]) || x[i] == INFINITY) return SO_INVALID;
        maximum = fmaxf(maximum, x[i]);
    }
    if (!isfinite(maximum)) return SO_INVALID;
    float sum = 0.0f;
    for (uint32_t i = 0; i < count; i++) {
        out[i] = expf(x[i] - maximum);
        sum += out[i];
    }
    if (!isfinite(sum) || sum <= 0.0f) return SO_INVALID;
    for (uint32_t i = 0; i < count; i++) out[i] /= sum;
    return SO_OK;
}

/* hybrid::math::topk: stable by (value desc, index asc). math.rs:55-66 */
int so_topk_f32(const float *x, uint32_t count, uint32_t k, uint32_t *indices) {
    if (k == 0 || k > count) return SO_INVALID;
    for (uint32_t i = 0; i < count; i++)
        if (isnan(x[i])) return SO_INVALID;
    uint8_t *taken = (uint8_t *)calloc(count, 1);
    for (uint32_t r = 0; r < k; r++) {
        uint32_t best = UINT32_MAX;
        for (uint32_t i = 0; i < count; i++) {
            if (taken[i]) continue;
            if (best == UINT32_MAX || x[i] > x[best]) best = i;
        }
        taken[best] = 1;
        indices[r] = best;
    }
    free(taken);
    return SO_OK;
}

/* moe_route: softmax over all experts, iterative top-k (first maximum wins),
 * renormalise over the selected, optional bf16 rounding of logits / weights.
 * crates/stark-engine/src/backends/cpu/kernel/moe.rs:25-82 */
int so_moe_route(const float *logits, uint32_t *ids, float *weights, uint32_t rows, uint32_t experts,
                 uint32_t active, uint32_t round_weights, uint32_t round_logits) {
    float *x = (float *)malloc(sizeof(float) * (experts ? experts : 1));
    for (uint32_t row = 0; row < rows; row++) {
        const float *source = logits + (size_t)row * experts;
        uint32_t *rid = ids + (size_t)row * active;
        float *rw = weights + (size_t)row * active;
        int valid = experts >= 1 && experts <= 1024 && active >= 1 && active <= 32 && active <= experts;
        for (uint32_t e = 0; e < experts; e++) {
            x[e] = round_logits ? bf16_round(source[e]) : source[e];
            if (!isfinite(x[e])) valid = 0;
        }
        float maximum = -INFINITY;
        for (uint32_t e = 0; e < experts; e++) maximum = fmaxf(maximum, x[e]);
        float denominator = 0.0f;
        for (uint32_t e = 0; e < experts; e++) denominator += expf(x[e] - maximum);
        float selected_sum = 0.0f;
        for (uint32_t rank = 0; rank < active; rank++) {
            float best = -INFINITY;
            uint32_t selected = 0;
            for (uint32_t e = 0; e < experts; e++) {
                int used = 0;
                for (uint32_t r = 0; r < rank; r++)
                    if (rid[r] == e) used = 1;
                if (!used && x[e] > best) {
                    best = x[e];
                    selected = e;
                }
            }
            rid[rank] = valid ? selected : 0;
            rw[rank] = expf(best - maximum) / denominator;
            selected_sum += rw[rank];
        }
        for (uint32_t rank = 0; rank < active; rank++) {
            rw[rank] /= selected_sum;
            if (round_weights) rw[rank] = bf16_round(rw[rank]);
            if (!valid) rw[rank] = NAN;
        }
    }
    free(x);
    return SO_OK;
}

/* ------------------------------------------------ dense decoder (bf16 graph) */

typedef struct {
    const uint8_t *codes;   /* [n, k*bits/8] MLX row-major packed codes */
    const uint16_t *scales; /* [n, k/group] bf16 */
    const uint16_t *biases; /* [n, k/group] bf16 */
    uint32_t n, k, bits, group;
} so_qmat;

typedef struct {
    const float *attn_norm; /* [hidden] f32 */
    const float *mlp_norm;  /* [hidden] */
    const float *q_norm;    /* [head_dim] */
    const float *k_norm;    /* [head_dim] */
    so_qmat qkv;            /* [(q_heads + 2 kv_heads) * head_dim, hidden], rows [q; k; v] */
    so_qmat o;              /* [hidden, q_heads*head_dim] */
    so_qmat upgate;         /* [2*inter, hidden], rows [up; gate] */
    so_qmat down;           /* [hidden, inter] */
} so_dense_layer;

typedef struct {
    uint32_t layers, hidden, q_heads, kv_heads, head_dim, inter, vocab;
    float eps, rope_theta;
    so_qmat embed;   /* [vocab, hidden] */
    so_qmat lm_head; /* [vocab, hidden]; same planes as embed when tied */
    const float *final_norm;
    const so_dense_layer *layer;
} so_dense_model;

typedef struct {
    uint16_t *keys;   /* [layers, capacity, kv_heads*head_dim] bf16 */
    uint16_t *values; /* same */
    uint32_t capacity;
    uint32_t position; /* rows already in the cache */
} so_dense_state;

static void qmv(const so_qmat *w, const uint16_t *x, uint16_t *y, int threads) {
    so_affine_matvec_bf16(w->codes, w->scales, w->biases, x, y, 1, w->n, w->k, w->bits, w->group, 0, 0, 0, 0,
                          threads);
}

/* One decode row through the Qwen3 dense graph with the bf16 rounding points of
 * the converted-model path:
 *   wiring   crates/stark-engine/src/encodable_block/transformer_layer.rs:549-659
 *            crates/stark-engine/src/encodable_block/mixer/attention/mode.rs:377-461
 *            crates/stark-engine/src/encodable_block/mlp/dense.rs:99-115
 *            crates/stark-engine/src/encodable_block/decoder.rs:494-555
 * logits_out may be NULL (cache-only ingest of a prompt row); hidden_out (the
 * final normalized row, [hidden] bf16) may be NULL. */
int so_dense_step(const so_dense_model *m, so_dense_state *s, uint32_t token, uint16_t *logits_out,
                  uint16_t *hidden_out, int threads) {
    if (s->position >= s->capacity || token >= m->vocab) return SO_INVALID;
    const uint32_t D = m->hidden, hd = m->head_dim, QH = m->q_heads, KH = m->kv_heads, I = m->inter;
    const uint32_t qkv_n = (QH + 2 * KH) * hd;
    const size_t kv_row = (size_t)KH * hd;
    uint16_t *hidden = (uint16_t *)malloc(2 * (size_t)D);
    uint16_t *shortcut = (uint16_t *)malloc(2 * (size_t)D);
    uint16_t *normed = (uint16_t *)malloc(2 * (size_t)D);
    uint16_t *qkv = (uint16_t *)malloc(2 * (size_t)qkv_n);
    uint16_t *attn = (uint16_t *)malloc(2 * (size_t)QH * hd);
    uint16_t *fused = (uint16_t *)malloc(2 * (size_t)2 * I);
    uint16_t *act = (uint16_t *)malloc(2 * (size_t)I);
    uint16_t *tmp = (uint16_t *)malloc(2 * (size_t)hd);
    float *cosines = (float *)malloc(4 * (size_t)hd), *sines = (float *)malloc(4 * (size_t)hd);
    const uint32_t pos = s->position;
    so_rope_coeffs(pos, hd, m->rope_theta, cosines, sines);
    const float scale = 1.0f / sqrtf((float)hd);

    so_embedding_row_bf16(m->embed.codes, m->embed.scales, m->embed.biases, token, m->vocab, D, m->embed.bits,
                          m->embed.group, hidden);
    for (uint32_t l = 0; l < m->layers; l++) {
        const so_dense_layer *L = &m->layer[l];
        /* pre_mixer_norm: Copy on layer 0, Add afterwards (transformer_layer.rs:250-264) */
        so_rmsnorm_bf16(hidden, L->attn_norm, normed, shortcut, 1, D, m->eps, l > 0);
        qmv(&L->qkv, normed, qkv, threads);
        so_head_norm_bf16(qkv, L->q_norm, 0, QH, hd, m->eps);
        so_head_norm_bf16(qkv, L->k_norm, QH, KH, hd, m->eps);
        uint16_t *kc = s->keys + ((size_t)l * s->capacity + pos) * kv_row;
        uint16_t *vc = s->values + ((size_t)l * s->capacity + pos) * kv_row;
        for (uint32_t h = 0; h < QH; h++) {
            so_rope_head_bf16(qkv + (size_t)h * hd, tmp, cosines, sines, hd);
            memcpy(qkv + (size_t)h * hd, tmp, 2 * (size_t)hd);
        }
        for (uint32_t h = 0; h < KH; h++)
            so_rope_head_bf16(qkv + (size_t)(QH + h) * hd, kc + (size_t)h * hd, cosines, sines, hd);
        memcpy(vc, qkv + (size_t)(QH + KH) * hd, 2 * kv_row);
        so_attention_decode_bf16(qkv, s->keys + (size_t)l * s->capacity * kv_row,
                                 s->values + (size_t)l * s->capacity * kv_row, attn, QH, KH, hd, pos + 1, scale,
                                 threads);
        qmv(&L->o, attn, hidden, threads);
        so_rmsnorm_bf16(hidden, L->mlp_norm, normed, shortcut, 1, D, m->eps, 1);
        qmv(&L->upgate, normed, fused, threads);
        so_swiglu_bf16(fused, act, I);
        qmv(&L->down, act, hidden, threads);
    }
    s->position = pos + 1;
    if (logits_out || hidden_out) {
        so_rmsnorm_bf16(hidden, m->final_norm, normed, shortcut, 1, D, m->eps, 1);
        if (hidden_out) memcpy(hidden_out, normed, 2 * (size_t)D);
        if (logits_out) qmv(&m->lm_head, normed, logits_out, threads);
    }
    free(hidden);
    free(shortcut);
    free(normed);
    free(qkv);
    free(attn);
    free(fused);
    free(act);
    free(tmp);
    free(cosines);
    free(sines);
    return SO_OK;
}

/* One row through the dense multi-token-prediction head:
 *   fuse     crates/stark-engine/src/encodable_block/qwen_mtp.rs:322-352 -- joined = [embedding_norm(e) ; hidden_norm(h)]
 *            with e the embedding row of `token` and h the target's normalized hidden of the row before; fusion
 *            linear [hidden, 2 hidden]
 *   layer    the head's transformer: ONE decoder layer with its own cache, then its output norm (qwen_mtp.rs:277-300;
 *            the layer is the graph of so_dense_step)
 *   readout  the target's read-out over the normalized output; that output is also the hidden of the next
 *            draft step (crates/stark-engine/src/engine/language_model/dense_mtp.rs:291-372)
 * `m` supplies the dimensions, the embedding table and the read-out; `s` is the head's own one-layer cache.
 * logits_out and hidden_out both NULL: cache-only row (qwen_mtp.rs:302-320, keys and values only). */
int so_mtp_head_step(const so_dense_model *m, const so_dense_layer *L, const so_qmat *fusion, const float *embed_norm,
                     const float *hidden_norm, const float *out_norm, so_dense_state *s, uint32_t token,
                     const uint16_t *hidden_in, uint16_t *logits_out, uint16_t *hidden_out, int threads) {
    if (s->position >= s->capacity || token >= m->vocab) return SO_INVALID;
    const uint32_t D = m->hidden, hd = m->head_dim, QH = m->q_heads, KH = m->kv_heads, I = m->inter;
    if (fusion->n != D || fusion->k != 2 * D) return SO_INVALID;
    const uint32_t qkv_n = (QH + 2 * KH) * hd;
    const size_t kv_row = (size_t)KH * hd;
    uint16_t *joined = (uint16_t *)malloc(2 * (size_t)2 * D);
    uint16_t *hidden = (uint16_t *)malloc(2 * (size_t)D);
    uint16_t *shortcut = (uint16_t *)malloc(2 * (size_t)D);
    uint16_t *normed = (uint16_t *)malloc(2 * (size_t)D);
    uint16_t *qkv = (uint16_t *)malloc(2 * (size_t)qkv_n);
    uint16_t *attn = (uint16_t *)malloc(2 * (size_t)QH * hd);
    uint16_t *fused = (uint16_t *)malloc(2 * (size_t)2 * I);
    uint16_t *act = (uint16_t *)malloc(2 * (size_t)I);
    uint16_t *tmp = (uint16_t *)malloc(2 * (size_t)hd);
    float *cosines = (float *)malloc(4 * (size_t)hd), *sines = (float *)malloc(4 * (size_t)hd);
    const uint32_t pos = s->position;
    so_rope_coeffs(pos, hd, m->rope_theta, cosines, sines);
    const float scale = 1.0f / sqrtf((float)hd);

    so_embedding_row_bf16(m->embed.codes, m->embed.scales, m->embed.biases, token, m->vocab, D, m->embed.bits,
                          m->embed.group, hidden);
    so_rmsnorm_bf16(hidden, embed_norm, joined, shortcut, 1, D, m->eps, 0);
    so_rmsnorm_bf16(hidden_in, hidden_norm, joined + D, shortcut, 1, D, m->eps, 0);
    qmv(fusion, joined, hidden, threads);

    so_rmsnorm_bf16(hidden, L->attn_norm, normed, shortcut, 1, D, m->eps, 0);
    qmv(&L->qkv, normed, qkv, threads);
    so_head_norm_bf16(qkv, L->q_norm, 0, QH, hd, m->eps);
    so_head_norm_bf16(qkv, L->k_norm, QH, KH, hd, m->eps);
    uint16_t *kc = s->keys + (size_t)pos * kv_row, *vc = s->values + (size_t)pos * kv_row;
    for (uint32_t h = 0; h < QH; h++) {
        so_rope_head_bf16(qkv + (size_t)h * hd, tmp, cosines, sines, hd);
        memcpy(qkv + (size_t)h * hd, tmp, 2 * (size_t)hd);
    }
    for (uint32_t h = 0; h < KH; h++)
        so_rope_head_bf16(qkv + (size_t)(QH + h) * hd, kc + (size_t)h * hd, cosines, sines, hd);
    memcpy(vc, qkv + (size_t)(QH + KH) * hd, 2 * kv_row);
    s->position = pos + 1;
    if (logits_out || hidden_out) {
        so_attention_decode_bf16(qkv, s->keys, s->values, attn, QH, KH, hd, pos + 1, scale, threads);
        qmv(&L->o, attn, hidden, threads);
        so_rmsnorm_bf16(hidden, L->mlp_norm, normed, shortcut, 1, D, m->eps, 1);
        qmv(&L->upgate, normed, fused, threads);
        so_swiglu_bf16(fused, act, I);
        qmv(&L->down, act, hidden, threads);
        so_rmsnorm_bf16(hidden, out_norm, normed, shortcut, 1, D, m->eps, 1);
        if (hidden_out) memcpy(hidden_out, normed, 2 * (size_t)D);
        if (logits_out) qmv(&m->lm_head, normed, logits_out, threads);
    }
    free(joined);
    free(hidden);
    free(shortcut);
    free(normed);
    free(qkv);
    free(attn);
    free(fused);
    free(act);
    free(tmp);
    free(cosines);
    free(sines);
    return SO_OK;
}

int so_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------ routed experts (f32 host path) */

/* hybrid::math::sigmoid / silu: crates/stark-engine/src/engine/hybrid/math.rs:5-16 */
static inline float sigmoid_f32(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    float e = expf(x);
    return e / (1.0f + e);
}
float so_silu_f32(float x) { return x * sigmoid_f32(x); }

/* Routed-expert feed-forward of the hybrid host path, without the shared expert:
 * crates/stark-engine/src/engine/hybrid/qwen.rs:872-905 -- top-k of the router scores (value
 * descending, index ascending), softmax over the SELECTED scores, per expert
 * down(silu(gate x) * (up x)), mixture in selection order.  Banks are GGUF rows
 * [experts, rows, columns] as selected_matvec reads them (weights.rs:1612-1689). */
int so_moe_ffn_f32(uint32_t kind_gate_up, const uint8_t *gate_bank, const uint8_t *up_bank, uint32_t kind_down,
                   const uint8_t *down_bank, const float *scores, const float *x, float *out, uint32_t experts,
                   uint32_t active, uint32_t hidden, uint32_t inter, uint32_t *ids_out, float *probs_out,
                   int threads) {
    uint32_t be, bb, de, db;
    if (so_block_layout(kind_gate_up, &be, &bb) != SO_OK || so_block_layout(kind_down, &de, &db) != SO_OK)
        return SO_INVALID;
    if (active == 0 || active > experts || active > 64 || hidden % be || inter % de) return SO_INVALID;
    uint32_t ids[64];
    float sel[64], prob[64];
    if (so_topk_f32(scores, experts, active, ids) != SO_OK) return SO_INVALID;
    for (uint32_t r = 0; r < active; r++) sel[r] = scores[ids[r]];
    if (so_softmax_f32(sel, prob, active) != SO_OK) return SO_INVALID;
    const size_t gu_bytes = (size_t)inter * (hidden / be) * bb;  /* one expert of a gate / up bank */
    const size_t dn_bytes = (size_t)hidden * (inter / de) * db;
    float *gate = (float *)malloc(sizeof(float) * inter), *up = (float *)malloc(sizeof(float) * inter);
    float *eo = (float *)malloc(sizeof(float) * hidden);
    for (uint32_t i = 0; i < hidden; i++) out[i] = 0.0f;
    for (uint32_t r = 0; r < active; r++) {
        so_gguf_matvec_f32(kind_gate_up, gate_bank + ids[r] * gu_bytes, x, gate, inter, hidden, threads);
        so_gguf_matvec_f32(kind_gate_up, up_bank + ids[r] * gu_bytes, x, up, inter, hidden, threads);
        for (uint32_t i = 0; i < inter; i++) gate[i] = so_silu_f32(gate[i]) * up[i];
        so_gguf_matvec_f32(kind_down, down_bank + ids[r] * dn_bytes, gate, eo, hidden, inter, threads);
        for (uint32_t i = 0; i < hidden; i++) out[i] += prob[r] * eo[i];
        if (ids_out) ids_out[r] = ids[r];
        if (probs_out) probs_out[r] = prob[r];
    }
    free(gate);
    free(up);
    free(eo);
    return SO_OK;
}

/* Dense f32 matvec, sequential f32 sum (router "gate" projection on the host path). */
void so_dense_matvec_f32(const float *w, const float *x, float *y, uint32_t rows, uint32_t columns) {
    for (uint32_t r = 0; r < rows; r++) {
        float total = 0.0f;
        for (uint32_t c = 0; c < columns; c++) total += w[(size_t)r * columns + c] * x[c];
        y[r] = total;
    }
}

/* ------------------------------------------------------------ routed-expert decoder (f32 host path) */

/* `rope` of the hybrid host graphs (crates/stark-engine/src/engine/hybrid/ripple.rs:653-666, the same
 * in flint.rs:412-425): angle = position * theta^(-(2i)/d) in f32, half-split pairing (i, i + d/2). */
void so_rope_f32(float *head, uint32_t dim, uint32_t position, float theta) {
    const uint32_t half = dim / 2;
    for (uint32_t i = 0; i < half; i++) {
        const float angle = (float)position * powf(theta, -((float)(2 * i)) / (float)dim);
        const float sn = sinf(angle), cs = cosf(angle);
        const float a = head[i], b = head[i + half];
        head[i] = a * cs - b * sn;
        head[i + half] = a * sn + b * cs;
    }
}

/* One token of a routed-expert decoder on the hybrid host path's conventions (f32 activations, GGUF
 * blocks decoded as decode_block, sequential f32 sums).  The reference ships no model of exactly this
 * shape; the step is composed of its operators:
 *   rms_norm                                math.rs:18-34
 *   q/k/v projections, per-head norm, rope, causal attention over the f32 cache, o projection
 *                                           ripple.rs:668-741 (no blend, no gate, no window)
 *   router scores -> top-k -> softmax over the selected -> expert mixture
 *                                           qwen.rs:872-899 (no shared expert), math.rs:36-66
 *   x += update (pre-norm residual), final norm, output projection
 *                                           ripple.rs:474-482 (without the post norms)
 * Attention matrices, the token table and the output matrix are Q8_0, expert banks Q4_K. */
typedef struct {
    uint32_t vocab, hidden, layers, q_heads, kv_heads, head_dim, experts, active, inter, context;
    float eps, theta;
    const uint8_t *embed, *output;               /* Q8_0 [vocab, hidden] */
    const float *final_norm;                     /* [hidden] */
    const float *const *attn_norm, *const *ffn_norm, *const *q_norm, *const *k_norm;
    const uint8_t *const *wq, *const *wk, *const *wv, *const *wo; /* Q8_0 */
    const float *const *router;                  /* f32 [experts, hidden] */
    const uint8_t *const *gate, *const *up, *const *down; /* Q4_K banks [experts, rows, columns] */
} so_moe_model;

/* keys / values: [layers][context][kv_heads * head_dim] f32, filled up to `position`.  logits may be
 * NULL (a prompt token that only fills the cache).  ids_out (may be NULL): [layers][active]. */
int so_moe_step(const so_moe_model *m, float *keys, float *values, uint32_t position, uint32_t token,
                float *logits, uint32_t *ids_out, int threads) {
    const uint32_t H = m->hidden, D = m->head_dim, QH = m->q_heads, KV = m->kv_heads;
    if (token >= m->vocab || position >= m->context || H % 256u || QH % KV) return SO_INVALID;
    const uint32_t kind_q8 = 8, kind_q4k = 12; /* ggml type ids */
    const size_t kv_row = (size_t)KV * D;
    float *x = (float *)malloc(sizeof(float) * H), *n = (float *)malloc(sizeof(float) * H);
    float *q = (float *)malloc(sizeof(float) * QH * D), *att = (float *)malloc(sizeof(float) * QH * D);
    float *upd = (float *)malloc(sizeof(float) * H), *scores = (float *)malloc(sizeof(float) * m->experts);
    float *sc = (float *)malloc(sizeof(float) * (position + 1)), *pr = (float *)malloc(sizeof(float) * (position + 1));
    float *tmp = (float *)malloc(sizeof(float) * D);
    int rc = so_gguf_decode_row(kind_q8, m->embed + (size_t)token * (H / 32u) * 34u, x, H);
    for (uint32_t l = 0; l < m->layers && rc == SO_OK; l++) {
        float *kc = keys + ((size_t)l * m->context + position) * kv_row;
        float *vc = values + ((size_t)l * m->context + position) * kv_row;
        rc |= so_rmsnorm_f32(x, m->attn_norm[l], n, H, m->eps);
        rc |= so_gguf_matvec_f32(kind_q8, m->wq[l], n, q, QH * D, H, threads);
        rc |= so_gguf_matvec_f32(kind_q8, m->wk[l], n, kc, KV * D, H, threads);
        rc |= so_gguf_matvec_f32(kind_q8, m->wv[l], n, vc, KV * D, H, threads);
        if (rc != SO_OK) break;
        for (uint32_t h = 0; h < QH; h++) {
            rc |= so_rmsnorm_f32(q + h * D, m->q_norm[l], tmp, D, m->eps);
            memcpy(q + h * D, tmp, sizeof(float) * D);
            so_rope_f32(q + h * D, D, position, m->theta);
        }
        for (uint32_t h = 0; h < KV; h++) {
            rc |= so_rmsnorm_f32(kc + h * D, m->k_norm[l], tmp, D, m->eps);
            memcpy(kc + h * D, tmp, sizeof(float) * D);
            so_rope_f32(kc + h * D, D, position, m->theta);
        }
        const float scale = 1.0f / sqrtf((float)D);
        for (uint32_t h = 0; h < QH; h++) {
            const uint32_t begin = h / (QH / KV) * D;
            const float *qh = q + h * D;
            float *out = att + h * D;
            for (uint32_t t = 0; t <= position; t++) {
                const float *k = keys + ((size_t)l * m->context + t) * kv_row + begin;
                float dot = 0.0f;
                for (uint32_t i = 0; i < D; i++) dot += qh[i] * k[i];
                sc[t] = dot * scale;
            }
            rc |= so_softmax_f32(sc, pr, position + 1);
            for (uint32_t i = 0; i < D; i++) out[i] = 0.0f;
            for (uint32_t t = 0; t <= position; t++) {
                const float *v = values + ((size_t)l * m->context + t) * kv_row + begin;
                for (uint32_t i = 0; i < D; i++) out[i] += pr[t] * v[i];
            }
        }
        rc |= so_gguf_matvec_f32(kind_q8, m->wo[l], att, upd, H, QH * D, threads);
        for (uint32_t i = 0; i < H; i++) x[i] += upd[i];
        rc |= so_rmsnorm_f32(x, m->ffn_norm[l], n, H, m->eps);
        so_dense_matvec_f32(m->router[l], n, scores, m->experts, H);
        rc |= so_moe_ffn_f32(kind_q4k, m->gate[l], m->up[l], kind_q4k, m->down[l], scores, n, upd, m->experts, m->active,
                             H, m->inter, ids_out ? ids_out + (size_t)l * m->active : NULL, NULL, threads);
        for (uint32_t i = 0; i < H; i++) x[i] += upd[i];
    }
    if (rc == SO_OK && logits) {
        rc |= so_rmsnorm_f32(x, m->final_norm, n, H, m->eps);
        rc |= so_gguf_matvec_f32(kind_q8, m->output, n, logits, m->vocab, H, threads);
    }
    free(x), free(n), free(q), free(att), free(upd), free(scores), free(sc), free(pr), free(tmp);
    return rc == SO_OK ? SO_OK : SO_INVALID;
}

/* ------------------------------------------------------------------------------------------------
 * Stochastic sampling of the converted-model path.
 *   Philox4x32-10 counter-based generator, Gumbel noise, index -> (counter offset, word) mapping:
 *     crates/stark-engine/src/encodable_block/sampling/gumbel.rs:1-85
 *   per-position seed derivation (the 64-bit finalizer of MurmurHash3):
 *     crates/stark-engine/src/encodable_block/sampling/prng.rs:12-22
 *   the sampler itself (finite check, temperature with overflow centring, top-k / top-p / min-p as one
 *   prefix of the descending order, Gumbel-max, first index of the maximum):
 *     crates/stark-engine/src/backends/cpu/kernel/sampling/unified_sampling.rs:15-117
 */
static void philox_round(uint32_t c[4], const uint32_t k[2]) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k[0], n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k[1], n3 = (uint32_t)p0;
    c[0] = n0, c[1] = n1, c[2] = n2, c[3] = n3;
}

void so_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c[4] = {ctr[0], ctr[1], ctr[2], ctr[3]}, k[2] = {key[0], key[1]};
    philox_round(c, k);
    for (int i = 0; i < 9; ++i) {
        k[0] += 0x9E3779B9u;
        k[1] += 0xBB67AE85u;
        philox_round(c, k);
    }
    memcpy(out, c, sizeof c);
}

float so_unit_interval(uint32_t word) {
    uint32_t v = word >> 8;
    if (v < 1u) v = 1u;
    return (float)v * (1.0f / 16777216.0f);
}

float so_gumbel_float(uint64_t key, uint32_t offset, uint32_t word) {
    const uint32_t ctr[4] = {offset, 0u, 0u, 0u}, k[2] = {(uint32_t)key, (uint32_t)(key >> 32)};
    uint32_t out[4];
    so_philox4x32_10(ctr, k, out);
    return -logf(-logf(so_unit_interval(out[word])));
}

void so_revidx(uint32_t logit_idx, uint32_t vocab, uint32_t *offset, uint32_t *word) {
    const uint32_t thread_idx = logit_idx % 1024u;
    const uint32_t thread_offset = ((vocab + 4095u) / 4096u) * thread_idx;
    const uint32_t block_idx = logit_idx / 1024u;
    *offset = thread_offset + block_idx / 4u;
    *word = block_idx % 4u;
}

uint64_t so_prng_derive(uint64_t seed, uint64_t index) {
    uint64_t h = seed + index;
    h ^= h >> 33;
    h *= 0xff51afd7ed558ccdULL;
    h ^= h >> 33;
    h *= 0xc4ceb9fe1a85ec53ULL;
    h ^= h >> 33;
    return h;
}

typedef struct {
    float v;
    uint32_t i;
} so_ranked;
static int so_ranked_cmp(const void *pa, const void *pb) {
    const so_ranked *a = (const so_ranked *)pa, *b = (const so_ranked *)pb;
    if (a->v > b->v) return -1;
    if (a->v < b->v) return 1;
    return a->i < b->i ? -1 : (a->i > b->i ? 1 : 0);
}

/* ---- the generation worker's host sampler (crates/stark-generate/src/hybrid.rs) ---- */

/* `uniform` (hybrid.rs:1103-1111): one SplitMix64 step, the top 53 bits as a double in [0, 1). */
double so_splitmix64_uniform(uint64_t *state) {
    *state += 0x9e3779b97f4a7c15ull;
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return (double)((z ^ (z >> 31)) >> 11) * (1.0 / 9007199254740992.0);
}

/* `descending_sample_key` (hybrid.rs:1324-1328): ascending integer order of the key = descending
 * `total_cmp` order of the value (signed zeros stay distinct). */
uint32_t so_descending_sample_key(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    const uint32_t mask = ((bits & 0x80000000u) ? 0xffffffffu : 0u) | 0x80000000u;
    return ~(bits ^ mask);
}

static int so_u64_cmp(const void *pa, const void *pb) {
    const uint64_t a = *(const uint64_t *)pa, b = *(const uint64_t *)pb;
    return a < b ? -1 : (a > b ? 1 : 0);
}

/* `sample_with_mapper` over `sampling_distribution` (hybrid.rs:1122-1212) for Sampling::Stochastic:
 * all logits finite, candidates = the first k of the descending (total order, then lower id) sequence
 * (`sampling_indices`, :1265-1288, every branch of which yields that prefix), probabilities
 * exp(f64((l - max) / temperature)) with the subtraction and the division in f32 (:138-165), their
 * sequential f64 total, the min-p / top-p prefix (:1192-1204), then one SplitMix64 draw scaled by the kept
 * mass and a sequential scan (:1134-1142).  flags: 4 top_k, 8 top_p, 16 min_p.  Returns the token,
 * UINT32_MAX for an empty or non-finite row or k = 0; *rng advances by one step only when a token is drawn. */
uint32_t so_host_sampling_f64(const float *logits, uint32_t vocab, uint32_t flags, uint64_t *rng, float temperature,
                              uint32_t top_k, float top_p, float min_p) {
    if (vocab == 0) return 0xffffffffu;
    for (uint32_t i = 0; i < vocab; ++i)
        if (!isfinite(logits[i])) return 0xffffffffu;
    uint32_t k = vocab;
    if ((flags & 4u) && top_k < k) k = top_k;
    if (k == 0) return 0xffffffffu;
    uint64_t *order = (uint64_t *)malloc((size_t)vocab * sizeof(uint64_t));
    for (uint32_t i = 0; i < vocab; ++i) order[i] = ((uint64_t)so_descending_sample_key(logits[i]) << 32) | i;
    qsort(order, vocab, sizeof(uint64_t), so_u64_cmp);
    double *p = (double *)malloc((size_t)k * sizeof(double));
    const float max = logits[(uint32_t)order[0]];
    double total = 0.0;
    for (uint32_t n = 0; n < k; ++n) {
        const float arg = (logits[(uint32_t)order[n]] - max) / temperature;
        p[n] = exp((double)arg);
        total += p[n];
    }
    uint32_t kept = 0;
    double cumulative = 0.0;
    for (uint32_t n = 0; n < k; ++n) {
        if (kept > 0 && (((flags & 16u) && p[n] < (double)min_p) || ((flags & 8u) && cumulative / total >= (double)top_p)))
            break;
        cumulative += p[n];
        kept += 1;
    }
    const double target = so_splitmix64_uniform(rng) * cumulative;
    uint32_t token = (uint32_t)order[kept - 1];
    double mass = 0.0;
    for (uint32_t n = 0; n < kept; ++n) {
        mass += p[n];
        if (target < mass) {
            token = (uint32_t)order[n];
            break;
        }
    }
    free(p);
    free(order);
    return token;
}

/* flags: 1 stochastic, 2 temperature, 4 top_k, 8 top_p, 16 min_p.  Returns the token, UINT32_MAX if a
 * logit is not finite (or nothing finite is left). */
uint32_t so_unified_sampling_f32(const float *in, uint32_t vocab, uint32_t flags, uint64_t seed, float temperature,
                                 uint32_t top_k, float top_p, float min_p) {
    float *l = (float *)malloc((size_t)vocab * sizeof(float));
    uint32_t result = 0xffffffffu;
    for (uint32_t i = 0; i < vocab; ++i) {
        l[i] = in[i];
        if (!isfinite(l[i])) {
            free(l);
            return result;
        }
    }
    if (flags & 2u) {
        const float recip = 1.0f / temperature;
        int center = 0;
        for (uint32_t i = 0; i < vocab; ++i)
            if (isfinite(l[i]) && !isfinite(l[i] * recip)) center = 1;
        float shift = 0.0f;
        if (center) {
            shift = -INFINITY;
            for (uint32_t i = 0; i < vocab; ++i) shift = fmaxf(shift, l[i]);
        }
        for (uint32_t i = 0; i < vocab; ++i) {
            if (center) l[i] -= shift;
            l[i] *= recip;
        }
    }
    if (flags & (4u | 8u | 16u)) {
        so_ranked *s = (so_ranked *)malloc((size_t)vocab * sizeof(so_ranked));
        for (uint32_t i = 0; i < vocab; ++i) s[i].v = l[i], s[i].i = i;
        qsort(s, vocab, sizeof(so_ranked), so_ranked_cmp);
        const float top = s[0].v;
        float norm = 0.0f;
        for (uint32_t i = 0; i < vocab; ++i) norm += expf(s[i].v - top);
        for (uint32_t i = 0; i < vocab; ++i) l[i] = -INFINITY;
        float mass = 0.0f;
        for (uint32_t n = 0; n < vocab; ++n) {
            if (((flags & 4u) && n >= top_k) || ((flags & 8u) && mass >= top_p) ||
                ((flags & 16u) && s[n].v < top + logf(min_p)))
                break;
            l[s[n].i] = s[n].v;
            mass += expf(s[n].v - top) / norm;
        }
        free(s);
    }
    if (flags & 1u) {
        for (uint32_t i = 0; i < vocab; ++i) {
            uint32_t off, word;
            so_revidx(i, vocab, &off, &word);
            l[i] += so_gumbel_float(seed, off, word);
        }
    }
    float best = -INFINITY;
    int have = 0;
    for (uint32_t i = 0; i < vocab; ++i) {  /* max_by with ties to the lower index; NaN compares equal */
        if (!have || l[i] > best) {
            if (!have || l[i] > best) {
                best = l[i];
                result = i;
                have = 1;
            }
        }
    }
    if (!have || !isfinite(best)) result = 0xffffffffu;
    free(l);
    return result;
}
