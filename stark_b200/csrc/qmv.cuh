// Quantized matrix handle and the launch interface of the fused-dequant matvec kernels.
#pragma once
#include "common.cuh"

namespace sb {

// Storage formats of a re-tiled quantized matrix in device memory.
enum QFormat : uint32_t {
    kFmtAffine4 = 0,  // MLX affine, 4 bit, group 64, bf16 planes: 576-byte records
    kFmtAffine8 = 1,  // MLX affine, 8 bit, group 64, bf16 planes: 1088-byte records
    kFmtQ8_0 = 2,     // GGUF Q8_0: 16 rows x 64 columns per record, f16 block scales
    kFmtQ4_K = 3,     // GGUF Q4_K re-tiled: 16 rows x 256 columns per 2304-byte super-record (qmv_q4k.cu)
    kFmtQ4_KRaw = 4,  // GGUF Q4_K in the source byte layout (row-wise kernel; STARK_B200_Q4K_ROWS=1)
    kFmtQ8_0T = 5,    // GGUF Q8_0 re-tiled: 16 rows x 256 columns per 4352-byte super-record (qmv_b8.cu)
    kFmtAffine8T = 6, // MLX affine 8-bit re-tiled the same way
};

// One record covers 16 rows x 64 columns (one quantization group per row).
//   bytes [0, 512): lane L (0..31) owns 16 bytes = 4 words; word j, nibble p (bits 4p..4p+3) holds
//                   W[row0 + g + 8*(p&1)][64*kg + 16*t + 4*j + 2*((p>>1)&1) + (p>>2)],  g = L>>2, t = L&3.
//                   That is exactly the A-fragment order of mma.m16n8k16 after the lop3 extraction
//                   in dequant_a4_word(), so a lane needs one 128-bit load per record and no shuffles.
//   bytes [512, 544): 16 bf16 scales, index 2*g + h <-> row row0 + g + 8*h
//   bytes [544, 576): 16 bf16 biases, same order
// Records are ordered [row tile][column group], so a CTA's share of the matrix is one contiguous
// byte range that streams through bulk copies.  576 B per 1024 weights = 0.5625 B per weight, the
// same as the MLX layout.
constexpr uint32_t kA4RecordBytes = 576;
constexpr uint32_t kA8RecordBytes = 1088;
constexpr uint32_t kMaxStageRecords = 32;

struct QMatrix {
    QFormat format;
    uint32_t rows;         // logical rows N
    uint32_t columns;      // K
    uint32_t row_tiles;    // ceil(N / 16) (even when pair_halves)
    uint32_t groups;       // K / 64
    uint32_t pair_halves;  // storage tile 2j = rows 16j.., tile 2j+1 = rows N/2 + 16j..
    uint32_t record_bytes;
    uint32_t experts;  // > 1: a bank of `experts` matrices of rows x columns (row-wise formats only)
    uint8_t *data;  // device
    size_t bytes;
    int device;
};

// First logical row of storage tile `tile`.
__host__ __device__ inline uint32_t tile_row0(uint32_t tile, uint32_t pair_halves, uint32_t rows) {
    if (!pair_halves) return tile * 16u;
    return (tile >> 1) * 16u + ((tile & 1u) ? rows / 2u : 0u);
}

enum QmvPrologue : uint32_t {
    kProPlain = 0,    // x is the input vector (bf16 or f32)
    kProRmsNorm = 1,  // x = bf16(bf16(h * rms_inv) * bf16(norm_w)), h bf16
    kProStaged = 2,   // the kernel before this one left the row ready to use (QmvStagedRow): a plain copy
};
// A matvec input as the kernel keeps it in shared memory, written once by the kernel that produces the row (the
// tensor-parallel reduction, which holds the whole new residual row anyway) instead of once per consuming CTA:
//   [columns] f16      the normalized row times an exact power of two (largest element in [2^14, 2^15))
//   [columns / 64] f32 per-group sums of the normalized (unscaled) row
//   f32                the factor that undoes the scale
__host__ __device__ inline size_t qmv_staged_bytes(uint32_t columns) {
    return ((size_t)columns * 2u + (size_t)(columns / 64u) * 4u + 16u + 15u) & ~(size_t)15u;
}
enum QmvEpilogue : uint32_t {
    kEpiStore = 0,     // y[row] = value (bf16 or f32)
    kEpiResidual = 1,  // y[row] = bf16(bf16(value) + resid[row])   (resid may alias y)
    kEpiSwiGlu = 2,    // pair_halves matrix: y[r] = bf16(up[r] * bf16(silu(gate[r])))
    kEpiLogits = 3,    // y[row] = bf16(value) and a per-CTA (max, first index) partial
    kEpiPartialF32 = 4,  // y[row] = value as f32, bf16 input: this rank's share of a K-split product
    kEpiPush = 5,        // the f32 share goes to every rank's receive buffer as {value, ticket} packets
};

// Tensor-parallel exchange hooks of a matvec (see tp.cuh).  A K-split projection pushes its f32 share
// into every rank's receive buffer over peer mappings (kEpiPush) as 8-byte packets {value, ticket},
// each written with one 64-bit store: a packet is valid exactly when its ticket is the exchange's, so
// the producer needs no fence, no flag and no arrival counter, and the data is usable the moment it
// lands.  The matvec that consumes the sum (kProRmsNorm with `recv` set) polls the packets of all ranks
// while it loads its input, forms
//   h' = bf16(bf16(sum over ranks, in rank order) + h)
// in its prologue -- the rounding of the projection output and the residual add of the reference
// graph -- normalizes h' as usual, and block 0 stores h' for the next residual.  Tickets are
// tokens * ticket_mul + ticket_add with `tokens` a device word that advances once per token, so every
// exchange of a run has its own non-zero value and nothing is ever reset.
constexpr uint32_t kMaxExchangeRanks = 8;
struct QmvExchange {
    uint32_t ranks;
    unsigned long long *push[kMaxExchangeRanks];  // kEpiPush: on rank r, this rank's row of packets
    const unsigned long long *recv;               // consumer: local [kMaxExchangeRanks][columns] packets
    uint16_t *h_out;                              // consumer: [columns] bf16, written by block 0
    const uint32_t *tokens;
    uint32_t ticket_mul, ticket_add;
    unsigned long long wait_ns;  // consumer: how long to poll for a rank's packets
};

struct QmvArgs {
    const QMatrix *matrix;
    const void *x;  // [m, K]
    void *y;        // [m, N] (or [m, N/2] for kEpiSwiGlu)
    uint32_t m;     // input rows, 1..8
    uint32_t io_type;
    QmvPrologue prologue;
    QmvEpilogue epilogue;
    const float *norm_weight;  // kProRmsNorm
    const uint16_t *norm_weight_bf16;  // optional: the same weights already rounded to bf16 (copied, not converted)
    const void *staged;        // kProStaged: the row as qmv_staged_bytes describes it (device memory)
    float eps;
    const void *resid;        // kEpiResidual
    float *partial_max;       // kEpiLogits: [grid] per-CTA maxima
    uint32_t *partial_index;  // kEpiLogits: [grid] per-CTA first index of the maximum
    uint32_t *error_word;     // device word, OR-ed with kErr* bits
    TraceSlot *trace;         // optional timeline slot of this launch
    bool pdl;                 // launch with programmatic stream serialization
    uint32_t *out_grid;       // optional: number of CTAs launched
    const QmvExchange *exchange;  // optional tensor-parallel hooks
    bool roomy;                   // no small kernel needs shared memory beside this launch: take a deeper ring
};

stark_b200_status qmv_launch(const QmvArgs &args, cudaStream_t stream);
// Ring-stage geometry for a matrix with `groups` column groups: records per stage, records per
// consumer warp, and whether the stage is ragged (needs per-record predicates).
void qmv_pick_stage(uint32_t groups, uint32_t *records, uint32_t *rpw, bool *pred);

// A handful of input rows against one pass over the matrix (qmv_multi.cu): y[r] = W x[r] for r < m <= 8, bf16 in
// and out.  norm_weight != nullptr: every row goes through the RMS norm first (columns <= 4096).
constexpr uint32_t kQmvMultiMaxRows = 8;
struct QmvMultiArgs {
    const QMatrix *matrix;
    const uint16_t *x;   // [m, K] bf16
    uint32_t x_stride;   // elements between rows (0 = K)
    uint32_t m;
    uint16_t *y;         // [m, y_stride]; kEpiResidual reads and rewrites it
    uint32_t y_stride;
    const float *norm_weight;
    float eps;
    QmvEpilogue epilogue;  // kEpiStore, kEpiResidual or kEpiSwiGlu
    uint32_t *error_word;
    bool pdl;
};
bool qmv_multi_supports(const QMatrix *w, uint32_t m, bool norm);
stark_b200_status qmv_multi_launch(const QmvMultiArgs &args, cudaStream_t stream);

// Re-tiling (device kernels; inputs already in device memory).
stark_b200_status qmatrix_from_affine_device(const uint8_t *codes, const void *scales, const void *biases,
                                             const stark_b200_affine_desc &desc, cudaStream_t stream,
                                             QMatrix **out);
stark_b200_status qmatrix_unpack_codes_device(const QMatrix *m, uint8_t *dst_device, cudaStream_t stream);
void qmatrix_free(QMatrix *m);

// Tensor-core Q4_K (qmv_q4k.cu): re-tile a device copy of the source blocks into m->data, multiply, decode.
size_t q4kt_bytes(uint32_t experts, uint32_t rows, uint32_t columns);
stark_b200_status q4kt_retile(const uint8_t *blocks_device, QMatrix *m, cudaStream_t stream);
// pdl: launch with programmatic stream serialization (the kernel awaits its predecessor itself).
// x_mul (f32 input only): the input is silu(x) * x_mul, the gated activation of the expert feed-forward.
stark_b200_status q4kt_launch(const QMatrix *m, const void *x, size_t x_stride, void *y, uint32_t batch,
                              const uint32_t *expert_ids, uint32_t io_type, cudaStream_t stream, bool pdl = false,
                              const float *x_mul = nullptr);
stark_b200_status q4kt_dequantize(const QMatrix *m, uint32_t expert, uint32_t row, float *out_device,
                                  uint8_t *codes_device, cudaStream_t stream);

// Tensor-core 8-bit formats (qmv_b8.cu): Q8_0 and MLX affine 8-bit, re-tiled from device copies of the source.
size_t b8t_bytes(uint32_t experts, uint32_t rows, uint32_t columns);
stark_b200_status b8t_retile(const uint8_t *codes, const uint16_t *scales, const uint16_t *biases, QMatrix *m,
                             cudaStream_t stream);
stark_b200_status b8t_launch(const QMatrix *m, const void *x, size_t x_stride, void *y, uint32_t batch,
                             const uint32_t *expert_ids, uint32_t io_type, cudaStream_t stream, bool pdl = false);
stark_b200_status b8t_dequantize(const QMatrix *m, uint32_t expert, uint32_t row, float *out_device,
                                 uint8_t *codes_device, cudaStream_t stream);

// Row-wise kernels for the formats kept in the reference's byte layout (qmv_rows.cu).
bool qmv_rows_supports(const QMatrix *m);
// y[b, rows] = W[expert_ids[b]] x_b for b < batch (expert_ids == nullptr: the only matrix);
// x_stride = elements between consecutive inputs, 0 if all launch rows share one input.
// pdl only affects the re-tiled tensor-core formats; the streaming kernels launch fully serialized.
stark_b200_status qmv_rows_launch(const QMatrix *m, const void *x, size_t x_stride, void *y, uint32_t batch,
                                  const uint32_t *expert_ids, uint32_t io_type, cudaStream_t stream, bool pdl = false);
// One row dequantized to f32 (and / or its integer codes, one byte each), device outputs.
stark_b200_status qmv_rows_dequantize(const QMatrix *m, uint32_t expert, uint32_t row, float *out_device,
                                      uint8_t *codes_device, cudaStream_t stream);

}  // namespace sb
