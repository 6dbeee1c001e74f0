// extern "C" entry points for the formats kept in the reference's byte layout (GGUF Q8_0 / Q4_K,
// MLX affine 8-bit), for expert banks and for the routed-expert feed-forward.
#include <new>
#include <vector>

#include "context.cuh"
#include "ops.cuh"
#include "qmv.cuh"

using namespace sb;

namespace {

struct Staged {
    std::vector<void *> ptrs;
    ~Staged() {
        for (void *p : ptrs) cudaFree(p);
    }
    template <typename T>
    stark_b200_status in(const T *host, size_t count, T **dev) {
        *dev = nullptr;
        SB_CUDA(cudaMalloc(dev, count * sizeof(T) ? count * sizeof(T) : 1));
        ptrs.push_back(*dev);
        if (host) SB_CUDA(cudaMemcpy(*dev, host, count * sizeof(T), cudaMemcpyHostToDevice));
        return STARK_B200_OK;
    }
};

#define SB_TRY(expr)                        \
    do {                                    \
        stark_b200_status _s = (expr);      \
        if (_s != STARK_B200_OK) return _s; \
    } while (0)

size_t gguf_row_bytes(uint32_t kind, uint32_t columns) {
    if (kind == STARK_B200_GGUF_Q8_0) return (size_t)(columns / 32u) * 34u;
    if (kind == STARK_B200_GGUF_Q4_K) return (size_t)(columns / 256u) * 144u;
    return 0;
}

stark_b200_status make_gguf(const void *blocks, uint32_t kind, uint32_t experts, uint32_t rows, uint32_t columns,
                            uint32_t location, stark_b200_qmatrix **out) {
    if (!blocks || !out) return STARK_B200_INVALID_ARGUMENT;
    *out = nullptr;
    if (kind != STARK_B200_GGUF_Q8_0 && kind != STARK_B200_GGUF_Q4_K) return STARK_B200_UNSUPPORTED;
    const uint32_t block = kind == STARK_B200_GGUF_Q8_0 ? 32u : 256u;
    if (rows == 0 || columns == 0 || experts == 0 || columns % block != 0) return STARK_B200_INVALID_ARGUMENT;
    QMatrix *m = new (std::nothrow) QMatrix();
    if (!m) return STARK_B200_OUT_OF_MEMORY;
    static const bool q4k_rows = [] {
        const char *e = getenv("STARK_B200_Q4K_ROWS");
        return e && e[0] == '1';
    }();
    static const bool b8_rows = [] {  // STARK_B200_B8_ROWS=1 keeps the source layout and the row-wise kernel
        const char *e = getenv("STARK_B200_B8_ROWS");
        return e && e[0] == '1';
    }();
    // the tensor-core layouts cut rows into 256-column super-records; other widths keep the source layout
    const bool tiled = kind == STARK_B200_GGUF_Q4_K ? !q4k_rows : (!b8_rows && columns % 256u == 0);
    m->format = kind == STARK_B200_GGUF_Q8_0 ? (tiled ? kFmtQ8_0T : kFmtQ8_0) : (tiled ? kFmtQ4_K : kFmtQ4_KRaw);
    m->rows = rows;
    m->columns = columns;
    m->row_tiles = tiled ? (rows + 15u) / 16u : 0;
    m->groups = columns / 64u;
    m->pair_halves = 0;
    m->record_bytes = 0;
    m->experts = experts;
    const size_t source_bytes = gguf_row_bytes(kind, columns) * rows * experts;
    m->bytes = !tiled ? source_bytes
                      : (kind == STARK_B200_GGUF_Q4_K ? q4kt_bytes(experts, rows, columns) : b8t_bytes(experts, rows, columns));
    cudaGetDevice(&m->device);
    const cudaMemcpyKind dir = location == STARK_B200_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    cudaError_t e = cudaMalloc(&m->data, m->bytes);
    if (e == cudaSuccess && !tiled) e = cudaMemcpy(m->data, blocks, m->bytes, dir);
    if (e == cudaSuccess && tiled) {
        // re-tiled into tensor-core fragment order: stage the source bytes, re-tile, drop the copy
        uint8_t *staging = nullptr;
        e = cudaMalloc(&staging, source_bytes);
        if (e == cudaSuccess) e = cudaMemcpy(staging, blocks, source_bytes, dir);
        if (e == cudaSuccess) {
            const stark_b200_status rs = kind == STARK_B200_GGUF_Q4_K ? q4kt_retile(staging, m, nullptr)
                                                                      : b8t_retile(staging, nullptr, nullptr, m, nullptr);
            if (rs != STARK_B200_OK) e = cudaErrorUnknown;
        }
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        cudaFree(staging);
    }
    if (e != cudaSuccess) {
        qmatrix_free(m);
        return cuda_status(e);
    }
    *out = reinterpret_cast<stark_b200_qmatrix *>(m);
    return STARK_B200_OK;
}

}  // namespace

extern "C" {

stark_b200_status stark_b200_qmatrix_create_gguf(const void *blocks, uint32_t kind, uint32_t rows, uint32_t columns,
                                                 uint32_t location, stark_b200_qmatrix **out_matrix) {
    return make_gguf(blocks, kind, 1, rows, columns, location, out_matrix);
}

stark_b200_status stark_b200_qmatrix_create_gguf_bank(const void *blocks, uint32_t kind, uint32_t experts,
                                                      uint32_t rows, uint32_t columns, uint32_t location,
                                                      stark_b200_qmatrix **out_matrix) {
    return make_gguf(blocks, kind, experts, rows, columns, location, out_matrix);
}

stark_b200_status stark_b200_qmatrix_dequantize_row(const stark_b200_qmatrix *matrix, uint32_t expert, uint32_t row,
                                                    float *dst_host) {
    const QMatrix *m = reinterpret_cast<const QMatrix *>(matrix);
    if (!m || !dst_host) return STARK_B200_INVALID_ARGUMENT;
    if (!qmv_rows_supports(m)) return STARK_B200_UNSUPPORTED;
    Staged st;
    float *d;
    SB_TRY(st.in((const float *)nullptr, m->columns, &d));
    SB_TRY(qmv_rows_dequantize(m, expert, row, d, nullptr, 0));
    SB_CUDA(cudaMemcpy(dst_host, d, (size_t)m->columns * 4u, cudaMemcpyDeviceToHost));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_qmv_experts(const stark_b200_qmatrix *bank, const uint32_t *expert_ids,
                                            uint32_t count, const void *x, uint32_t shared_input, void *y,
                                            uint32_t io_type, uint32_t location, void *stream) {
    const QMatrix *m = reinterpret_cast<const QMatrix *>(bank);
    if (!m || !expert_ids || !x || !y || count == 0 || count > 64 || io_type > STARK_B200_F32)
        return STARK_B200_INVALID_ARGUMENT;
    if (!qmv_rows_supports(m)) return STARK_B200_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t esz = io_type == STARK_B200_F32 ? 4u : 2u;
    const size_t x_rows = shared_input ? 1u : count;
    if (location == STARK_B200_DEVICE)
        return qmv_rows_launch(m, x, shared_input ? 0 : m->columns, y, count, expert_ids, io_type, s);
    for (uint32_t i = 0; i < count; ++i)
        if (expert_ids[i] >= m->experts) return STARK_B200_INVALID_ARGUMENT;  // selected_matvec (weights.rs:1623)
    Staged st;
    uint8_t *dx, *dy;
    uint32_t *di;
    SB_TRY(st.in((const uint8_t *)x, x_rows * m->columns * esz, &dx));
    SB_TRY(st.in((const uint8_t *)nullptr, (size_t)count * m->rows * esz, &dy));
    SB_TRY(st.in(expert_ids, count, &di));
    SB_TRY(qmv_rows_launch(m, dx, shared_input ? 0 : m->columns, dy, count, di, io_type, s));
    SB_CUDA(cudaMemcpyAsync(y, dy, (size_t)count * m->rows * esz, cudaMemcpyDeviceToHost, s));
    SB_CUDA(cudaStreamSynchronize(s));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_dense_matvec_f32(const float *w, const float *x, float *y, uint32_t rows,
                                                 uint32_t columns, uint32_t location, void *stream) {
    if (!w || !x || !y || rows == 0 || columns == 0) return STARK_B200_INVALID_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (location == STARK_B200_DEVICE) return dense_matvec_f32_launch(w, x, y, rows, columns, s);
    Staged st;
    float *dw, *dx, *dy;
    SB_TRY(st.in(w, (size_t)rows * columns, &dw));
    SB_TRY(st.in(x, columns, &dx));
    SB_TRY(st.in((const float *)nullptr, rows, &dy));
    SB_TRY(dense_matvec_f32_launch(dw, dx, dy, rows, columns, s));
    SB_CUDA(cudaMemcpyAsync(y, dy, (size_t)rows * 4u, cudaMemcpyDeviceToHost, s));
    SB_CUDA(cudaStreamSynchronize(s));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_moe_ffn(const stark_b200_qmatrix *gate_bank, const stark_b200_qmatrix *up_bank,
                                        const stark_b200_qmatrix *down_bank, const float *scores, const float *x,
                                        float *out, uint32_t active, uint32_t *ids_out, float *probs_out,
                                        uint32_t location, void *stream) {
    const QMatrix *g = reinterpret_cast<const QMatrix *>(gate_bank);
    const QMatrix *u = reinterpret_cast<const QMatrix *>(up_bank);
    const QMatrix *d = reinterpret_cast<const QMatrix *>(down_bank);
    if (!g || !u || !d || !scores || !x || !out) return STARK_B200_INVALID_ARGUMENT;
    if (!qmv_rows_supports(g) || !qmv_rows_supports(u) || !qmv_rows_supports(d)) return STARK_B200_UNSUPPORTED;
    const uint32_t experts = g->experts, inter = g->rows, hidden = g->columns;
    if (u->experts != experts || d->experts != experts || u->rows != inter || u->columns != hidden ||
        d->rows != hidden || d->columns != inter || active == 0 || active > experts || active > 32)
        return STARK_B200_INVALID_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    Staged st;
    const float *ds = scores, *dx = x;
    float *dout = out;
    if (location == STARK_B200_HOST) {
        float *a, *b, *c;
        SB_TRY(st.in(scores, experts, &a));
        SB_TRY(st.in(x, hidden, &b));
        SB_TRY(st.in((const float *)nullptr, hidden, &c));
        ds = a;
        dx = b;
        dout = c;
    }
    uint32_t *ids;
    float *probs, *gate, *up, *eo;
    SB_TRY(st.in((const uint32_t *)nullptr, active, &ids));
    SB_TRY(st.in((const float *)nullptr, active, &probs));
    SB_TRY(st.in((const float *)nullptr, (size_t)active * inter, &gate));
    SB_TRY(st.in((const float *)nullptr, (size_t)active * inter, &up));
    SB_TRY(st.in((const float *)nullptr, (size_t)active * hidden, &eo));
    SB_TRY(moe_select_launch(ds, experts, active, ids, probs, s));
    SB_TRY(qmv_rows_launch(g, dx, 0, gate, active, ids, STARK_B200_F32, s));
    SB_TRY(qmv_rows_launch(u, dx, 0, up, active, ids, STARK_B200_F32, s));
    SB_TRY(silu_mul_f32_launch(gate, up, active * inter, s));
    SB_TRY(qmv_rows_launch(d, gate, inter, eo, active, ids, STARK_B200_F32, s));
    SB_TRY(weighted_sum_launch(eo, probs, dout, active, hidden, s));
    if (location == STARK_B200_HOST) SB_CUDA(cudaMemcpyAsync(out, dout, (size_t)hidden * 4u, cudaMemcpyDeviceToHost, s));
    if (ids_out) SB_CUDA(cudaMemcpyAsync(ids_out, ids, active * 4u, cudaMemcpyDeviceToHost, s));
    if (probs_out) SB_CUDA(cudaMemcpyAsync(probs_out, probs, active * 4u, cudaMemcpyDeviceToHost, s));
    SB_CUDA(cudaStreamSynchronize(s));
    return STARK_B200_OK;
}

}  // extern "C"
