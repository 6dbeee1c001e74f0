/*
 * stark_b200.h -- C ABI of the B200 (sm_100a) decode engine for Stark's token loop.
 *
 * The boundary follows the reference's own foreign-engine ABI
 * (vendor/glm-exl3-bridge/include/stark_glm.h:16-175, bound from Rust in
 * crates/stark-engine/src/engine/hybrid/glm_exl3_ffi.rs:1-140): opaque handles,
 * uint32_t status codes, versioned POD structs {struct_size, abi_version, ...},
 * caller-owned buffers, serial (one host thread per handle) use, explicit destroy.
 * No C++ or framework types cross it; nothing is written to stdout/stderr.
 *
 * Two groups of entry points:
 *   (1) the model surface -- the FFI image of hybrid::Model / LanguageModel
 *       (load, reset, prefill, step, full-vocabulary read-out, prefix rewind);
 *   (2) per-operator calls (quantized matvec, norms, RoPE, attention, router,
 *       log-softmax) that play the role of the reference's per-kernel
 *       `XKernel::encode` API (crates/stark-engine/build/common/traitgen.rs:56-66)
 *       for parity tests and micro-benchmarks.
 *
 * Every pointer argument carries a `location` (host or device).  Host pointers
 * are copied through the library's own staging buffers inside the call.
 */
#ifndef STARK_B200_H
#define STARK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define STARK_B200_ABI_VERSION 1u

typedef struct stark_b200_qmatrix stark_b200_qmatrix;
typedef struct stark_b200_model stark_b200_model;

/* Same numbering as stark_glm_status (stark_glm.h:18-32). */
typedef uint32_t stark_b200_status;
enum {
    STARK_B200_OK = 0,
    STARK_B200_INVALID_ARGUMENT = 1,
    STARK_B200_ABI_MISMATCH = 2,
    STARK_B200_CONTEXT_LIMIT = 3,
    STARK_B200_CANCELLED = 4,
    STARK_B200_UNSUPPORTED = 5,
    STARK_B200_OUT_OF_MEMORY = 6,
    STARK_B200_IO_FAILURE = 7,
    STARK_B200_DEVICE_FAILURE = 8,
    STARK_B200_RELOAD_REQUIRED = 9,
    STARK_B200_BUSY = 10,
    STARK_B200_INVALID_STATE = 11
};

/* Where a caller's buffer lives. */
#define STARK_B200_HOST 0u
#define STARK_B200_DEVICE 1u

/* Element types of activation vectors. */
#define STARK_B200_BF16 0u /* converted-model path: bf16 in/out, f32 accumulate */
#define STARK_B200_F32 1u  /* hybrid host path conventions: f32 in/out */

/* Plane (scale/bias) element kinds, numbered like the reference's tensor kinds
 * (crates/stark-engine/src/engine/hybrid/weights.rs:1207). */
#define STARK_B200_PLANE_F32 0u
#define STARK_B200_PLANE_F16 1u
#define STARK_B200_PLANE_BF16 30u

/* GGUF block kinds (ggml type ids; weights.rs:2565-2584). */
#define STARK_B200_GGUF_Q8_0 8u
#define STARK_B200_GGUF_Q4_K 12u

/* stark_glm_abi_version / stark_glm_status_name (stark_glm.h:82-83). */
uint32_t stark_b200_abi_version(void);
const char *stark_b200_status_name(uint32_t status);

/* Device plumbing for callers that do not bring their own allocator. */
stark_b200_status stark_b200_device_count(int32_t *out_count);
stark_b200_status stark_b200_set_device(int32_t device);
stark_b200_status stark_b200_device_malloc(void **out_ptr, size_t bytes);
stark_b200_status stark_b200_device_free(void *ptr);
stark_b200_status stark_b200_memcpy_h2d(void *dst_device, const void *src_host, size_t bytes, void *stream);
stark_b200_status stark_b200_memcpy_d2h(void *dst_host, const void *src_device, size_t bytes, void *stream);
stark_b200_status stark_b200_stream_synchronize(void *stream);
/* Reads and clears the device error word that kernels set when one of their bounded waits ran
 * out (0 = no error).  A non-zero word means the results of that launch are not valid. */
stark_b200_status stark_b200_take_device_error(uint32_t *out_word);

/* ------------------------------------------------------------------------------------------
 * Quantized matrices.
 *
 * An MLX-affine matrix W[rows, columns]: w = scale * q + bias, q unsigned `bits` wide, packed
 * LSB-first along columns (8 nibbles per uint32 for 4 bits), one (scale, bias) per `group`
 * consecutive columns.  Replaces the operands of MatmulB::Quantized
 * (crates/stark-engine/src/backends/common/kernel/matmul/arguments.rs:7-24) and of
 * Weights::affine_row (crates/stark-engine/src/engine/hybrid/weights.rs:1284-1309).
 * scale_layout 0: planes [rows, groups] (MLX native); 1: planes [groups, plane_pitch]
 * (the converted-model layout, backends/common/kernel/matmul/mod.rs:120-156).
 * The create call copies and re-tiles the data into device memory; the caller's buffers are
 * not referenced afterwards.
 */
typedef struct stark_b200_affine_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t rows;
    uint32_t columns;
    uint32_t bits;         /* 4 or 8 */
    uint32_t group;        /* 64 */
    uint32_t plane_kind;   /* STARK_B200_PLANE_* */
    uint32_t scale_layout; /* 0 or 1 */
    uint32_t plane_pitch;  /* round_up4(rows) for layout 1, ignored for layout 0 */
    uint32_t location;     /* STARK_B200_HOST / _DEVICE for codes, scales, biases */
    uint32_t pair_halves;  /* 1: rows r and r + rows/2 are a fused [up; gate] pair */
    uint32_t reserved;
} stark_b200_affine_desc;

stark_b200_status stark_b200_qmatrix_create_affine(const void *codes, const void *scales, const void *biases,
                                                   const stark_b200_affine_desc *desc,
                                                   stark_b200_qmatrix **out_matrix);
/* GGUF rows: `rows` rows of columns/block consecutive blocks, as decode_values reads them
 * (crates/stark-engine/src/engine/hybrid/weights.rs:2880-2895). */
stark_b200_status stark_b200_qmatrix_create_gguf(const void *blocks, uint32_t kind, uint32_t rows,
                                                 uint32_t columns, uint32_t location,
                                                 stark_b200_qmatrix **out_matrix);
stark_b200_status stark_b200_qmatrix_destroy(stark_b200_qmatrix **matrix);
/* Bytes the matrix occupies in device memory (codes + planes, after re-tiling). */
stark_b200_status stark_b200_qmatrix_device_bytes(const stark_b200_qmatrix *matrix, uint64_t *out_bytes);
/* Integer codes recovered from the re-tiled device copy through the same extraction the matvec
 * kernels use; dst[row * columns + column], one byte per code.  Must equal packed_code
 * (crates/stark-engine/src/backends/cpu/kernel/matmul/reference.rs:91-104) bit for bit. */
stark_b200_status stark_b200_qmatrix_unpack_codes(const stark_b200_qmatrix *matrix, uint8_t *dst_host,
                                                  size_t count);

/* y[m, rows] = x[m, columns] * W^T.  Replaces MatmulKernel::encode for a quantized B with
 * m <= 8 input rows (crates/stark-engine/src/backends/cpu/kernel/matmul/kernel.rs:168-285) and
 * Weights::matvec (weights.rs:1311-1350, 2511-2553).  io_type selects bf16 or f32 vectors. */
stark_b200_status stark_b200_op_qmv(const stark_b200_qmatrix *matrix, const void *x, void *y, uint32_t m,
                                    uint32_t io_type, uint32_t location, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* STARK_B200_H */
