// extern "C" surface of libstark_b200.so (declared in include/stark_b200.h).
// No exception crosses the boundary and nothing is printed.
#include <cmath>
#include <cstdlib>
#include <mutex>
#include <new>

#include "context.cuh"
#include "qmv.cuh"
#include "prefill.cuh"

namespace sb {

static std::mutex g_ctx_mutex;
static DeviceContext g_ctx[64];

DeviceContext *device_context() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    DeviceContext &c = g_ctx[dev];
    if (c.device != dev) {
        uint32_t *word = nullptr;
        if (cudaMalloc(&word, 256) != cudaSuccess) return nullptr;
        if (cudaMemset(word, 0, 256) != cudaSuccess) {
            cudaFree(word);
            return nullptr;
        }
        c.error_word = word;
        c.device = dev;
    }
    return &c;
}

stark_b200_status ensure_buffer(void **buf, size_t *have, size_t want) {
    if (*have >= want && *buf) return STARK_B200_OK;
    if (*buf) cudaFree(*buf);
    *buf = nullptr;
    *have = 0;
    size_t cap = want < 4096 ? 4096 : want;
    SB_CUDA(cudaMalloc(buf, cap));
    *have = cap;
    return STARK_B200_OK;
}

}  // namespace sb

using namespace sb;

// Programmatic dependent launch between consecutive kernels of a stream (on unless STARK_B200_PDL=0).
static bool pdl_enabled() {
    static const bool on = [] {
        const char *e = getenv("STARK_B200_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

extern "C" {

uint32_t stark_b200_abi_version(void) { return STARK_B200_ABI_VERSION; }

const char *stark_b200_status_name(uint32_t status) {
    switch (status) {
        case STARK_B200_OK: return "ok";
        case STARK_B200_INVALID_ARGUMENT: return "invalid_argument";
        case STARK_B200_ABI_MISMATCH: return "abi_mismatch";
        case STARK_B200_CONTEXT_LIMIT: return "context_limit";
        case STARK_B200_CANCELLED: return "cancelled";
        case STARK_B200_UNSUPPORTED: return "unsupported";
        case STARK_B200_OUT_OF_MEMORY: return "out_of_memory";
        case STARK_B200_IO_FAILURE: return "io_failure";
        case STARK_B200_DEVICE_FAILURE: return "device_failure";
        case STARK_B200_RELOAD_REQUIRED: return "reload_required";
        case STARK_B200_BUSY: return "busy";
        case STARK_B200_INVALID_STATE: return "invalid_state";
        default: return "unknown";
    }
}

const char *stark_b200_last_cuda_error(void) { return cudaGetErrorName(last_cuda_error()); }

stark_b200_status stark_b200_device_count(int32_t *out_count) {
    if (!out_count) return STARK_B200_INVALID_ARGUMENT;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        *out_count = 0;
        return STARK_B200_DEVICE_FAILURE;
    }
    *out_count = n;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_device_memory(uint64_t *out_free_bytes, uint64_t *out_total_bytes) {
    if (!out_free_bytes || !out_total_bytes) return STARK_B200_INVALID_ARGUMENT;
    size_t free_bytes = 0, total_bytes = 0;
    SB_CUDA(cudaMemGetInfo(&free_bytes, &total_bytes));
    *out_free_bytes = free_bytes;
    *out_total_bytes = total_bytes;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_set_device(int32_t device) {
    SB_CUDA(cudaSetDevice(device));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_device_malloc(void **out_ptr, size_t bytes) {
    if (!out_ptr) return STARK_B200_INVALID_ARGUMENT;
    *out_ptr = nullptr;
    SB_CUDA(cudaMalloc(out_ptr, bytes ? bytes : 1));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_device_free(void *ptr) {
    SB_CUDA(cudaFree(ptr));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream) {
    SB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream) {
    SB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_stream_synchronize(void *stream) {
    SB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_take_device_error(uint32_t *out_word) {
    if (!out_word) return STARK_B200_INVALID_ARGUMENT;
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    SB_CUDA(cudaMemcpy(out_word, ctx->error_word, 4, cudaMemcpyDeviceToHost));
    if (*out_word) SB_CUDA(cudaMemset(ctx->error_word, 0, 4));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_qmatrix_create_affine(const void *codes, const void *scales, const void *biases,
                                                   const stark_b200_affine_desc *desc,
                                                   stark_b200_qmatrix **out_matrix) {
    if (!codes || !scales || !biases || !desc || !out_matrix) return STARK_B200_INVALID_ARGUMENT;
    *out_matrix = nullptr;
    if (desc->struct_size != sizeof(stark_b200_affine_desc) || desc->abi_version != STARK_B200_ABI_VERSION)
        return STARK_B200_ABI_MISMATCH;
    if (desc->rows == 0 || desc->columns == 0 || desc->group == 0 || desc->columns % desc->group != 0)
        return STARK_B200_INVALID_ARGUMENT;
    const size_t code_bytes = (size_t)desc->rows * desc->columns * desc->bits / 8u;
    const size_t groups = desc->columns / desc->group;
    const size_t plane_elems = desc->scale_layout == 0 ? (size_t)desc->rows * groups : groups * desc->plane_pitch;
    const size_t plane_bytes = plane_elems * (desc->plane_kind == STARK_B200_PLANE_F32 ? 4u : 2u);
    QMatrix *m = nullptr;
    stark_b200_status st;
    if (desc->bits == 8) {
        // 8-bit affine keeps the reference's byte layout: codes, then the scale plane, then the bias plane
        if (desc->group != 64 || desc->plane_kind != STARK_B200_PLANE_BF16 || desc->scale_layout != 0 || desc->pair_halves)
            return STARK_B200_UNSUPPORTED;
        m = new (std::nothrow) QMatrix();
        if (!m) return STARK_B200_OUT_OF_MEMORY;
        static const bool b8_rows = [] {  // STARK_B200_B8_ROWS=1 keeps the source layout and the row-wise kernel
            const char *e = getenv("STARK_B200_B8_ROWS");
            return e && e[0] == '1';
        }();
        const bool tiled = !b8_rows && desc->columns % 256u == 0;  // tensor-core layout (qmv_b8.cu)
        m->format = tiled ? kFmtAffine8T : kFmtAffine8;
        m->rows = desc->rows;
        m->columns = desc->columns;
        m->row_tiles = tiled ? (desc->rows + 15u) / 16u : 0;
        m->groups = desc->columns / 64u;
        m->experts = 1;
        m->bytes = tiled ? b8t_bytes(1, desc->rows, desc->columns) : code_bytes + 2u * plane_bytes;
        cudaGetDevice(&m->device);
        const cudaMemcpyKind kind = desc->location == STARK_B200_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
        cudaError_t e = cudaMalloc(&m->data, m->bytes);
        uint8_t *staging = nullptr;
        uint8_t *dst = m->data;
        if (e == cudaSuccess && tiled) {
            e = cudaMalloc(&staging, code_bytes + 2u * plane_bytes);
            dst = staging;
        }
        if (e == cudaSuccess) e = cudaMemcpy(dst, codes, code_bytes, kind);
        if (e == cudaSuccess) e = cudaMemcpy(dst + code_bytes, scales, plane_bytes, kind);
        if (e == cudaSuccess) e = cudaMemcpy(dst + code_bytes + plane_bytes, biases, plane_bytes, kind);
        if (e == cudaSuccess && tiled) {
            if (b8t_retile(staging, reinterpret_cast<const uint16_t *>(staging + code_bytes),
                           reinterpret_cast<const uint16_t *>(staging + code_bytes + plane_bytes), m, nullptr) != STARK_B200_OK)
                e = cudaErrorUnknown;
            if (e == cudaSuccess) e = cudaDeviceSynchronize();
        }
        cudaFree(staging);
        if (e != cudaSuccess) {
            qmatrix_free(m);
            return cuda_status(e);
        }
        *out_matrix = reinterpret_cast<stark_b200_qmatrix *>(m);
        return STARK_B200_OK;
    }
    if (desc->location == STARK_B200_DEVICE) {
        st = qmatrix_from_affine_device((const uint8_t *)codes, scales, biases, *desc, 0, &m);
        if (st == STARK_B200_OK) st = cuda_status(cudaStreamSynchronize(0));
    } else {
        uint8_t *dc = nullptr, *ds = nullptr, *db = nullptr;
        cudaError_t e = cudaMalloc(&dc, code_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&ds, plane_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&db, plane_bytes);
        if (e == cudaSuccess) e = cudaMemcpy(dc, codes, code_bytes, cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMemcpy(ds, scales, plane_bytes, cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMemcpy(db, biases, plane_bytes, cudaMemcpyHostToDevice);
        st = cuda_status(e);
        if (st == STARK_B200_OK) st = qmatrix_from_affine_device(dc, ds, db, *desc, 0, &m);
        if (st == STARK_B200_OK) st = cuda_status(cudaStreamSynchronize(0));
        cudaFree(dc);
        cudaFree(ds);
        cudaFree(db);
    }
    if (st != STARK_B200_OK) {
        qmatrix_free(m);
        return st;
    }
    *out_matrix = reinterpret_cast<stark_b200_qmatrix *>(m);
    return STARK_B200_OK;
}

stark_b200_status stark_b200_qmatrix_destroy(stark_b200_qmatrix **matrix) {
    if (!matrix) return STARK_B200_INVALID_ARGUMENT;
    qmatrix_free(reinterpret_cast<QMatrix *>(*matrix));
    *matrix = nullptr;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_qmatrix_device_bytes(const stark_b200_qmatrix *matrix, uint64_t *out_bytes) {
    if (!matrix || !out_bytes) return STARK_B200_INVALID_ARGUMENT;
    *out_bytes = reinterpret_cast<const QMatrix *>(matrix)->bytes;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_qmatrix_unpack_codes(const stark_b200_qmatrix *matrix, uint8_t *dst_host,
                                                  size_t count) {
    const QMatrix *m = reinterpret_cast<const QMatrix *>(matrix);
    if (!m || !dst_host || count != (size_t)m->rows * m->columns) return STARK_B200_INVALID_ARGUMENT;
    uint8_t *d = nullptr;
    SB_CUDA(cudaMalloc(&d, count));
    stark_b200_status st = STARK_B200_OK;
    if (qmv_rows_supports(m)) {
        if (m->experts > 1) st = STARK_B200_UNSUPPORTED;
        for (uint32_t row = 0; row < m->rows && st == STARK_B200_OK; ++row)
            st = qmv_rows_dequantize(m, 0, row, nullptr, d + (size_t)row * m->columns, 0);
    } else {
        st = qmatrix_unpack_codes_device(m, d, 0);
    }
    if (st == STARK_B200_OK) st = cuda_status(cudaMemcpy(dst_host, d, count, cudaMemcpyDeviceToHost));
    cudaFree(d);
    return st;
}

stark_b200_status stark_b200_op_qmv(const stark_b200_qmatrix *matrix, const void *x, void *y, uint32_t m,
                                    uint32_t io_type, uint32_t location, void *stream) {
    const QMatrix *w = reinterpret_cast<const QMatrix *>(matrix);
    if (!w || !x || !y || m == 0 || m > 8 || io_type > STARK_B200_F32) return STARK_B200_INVALID_ARGUMENT;
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t esz = io_type == STARK_B200_F32 ? 4u : 2u;
    const size_t xin = (size_t)w->columns * esz, yout = (size_t)w->rows * esz;
    const uint8_t *dx = (const uint8_t *)x;
    uint8_t *dy = (uint8_t *)y;
    if (location == STARK_B200_HOST) {
        stark_b200_status st = ensure_buffer(&ctx->stage_in, &ctx->stage_in_bytes, xin * m);
        if (st != STARK_B200_OK) return st;
        st = ensure_buffer(&ctx->stage_out, &ctx->stage_out_bytes, yout * m);
        if (st != STARK_B200_OK) return st;
        SB_CUDA(cudaMemcpyAsync(ctx->stage_in, x, xin * m, cudaMemcpyHostToDevice, s));
        dx = (const uint8_t *)ctx->stage_in;
        dy = (uint8_t *)ctx->stage_out;
    }
    if (qmv_rows_supports(w)) {
        stark_b200_status st = qmv_rows_launch(w, dx, w->columns, dy, m, nullptr, io_type, s);
        if (st != STARK_B200_OK) return st;
    }
    for (uint32_t row = 0; row < m && !qmv_rows_supports(w); ++row) {
        QmvArgs a{};
        a.matrix = w;
        a.x = dx + row * xin;
        a.y = dy + row * yout;
        a.m = 1;
        a.io_type = io_type;
        a.prologue = kProPlain;
        a.epilogue = kEpiStore;
        a.error_word = ctx->error_word;
        a.pdl = location == STARK_B200_DEVICE && pdl_enabled();
        stark_b200_status st = qmv_launch(a, s);
        if (st != STARK_B200_OK) return st;
    }
    if (location == STARK_B200_HOST) {
        SB_CUDA(cudaMemcpyAsync(y, ctx->stage_out, yout * m, cudaMemcpyDeviceToHost, s));
        SB_CUDA(cudaStreamSynchronize(s));
    }
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_qgemm(const stark_b200_qmatrix *matrix, const void *x, void *y, uint32_t m,
                                      uint32_t epilogue, uint32_t location, void *stream) {
    QMatrix *w = const_cast<QMatrix *>(reinterpret_cast<const QMatrix *>(matrix));
    if (!w || !x || !y || m == 0 || epilogue > 2u) return STARK_B200_INVALID_ARGUMENT;
    if (w->format != kFmtAffine4) return STARK_B200_UNSUPPORTED;
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    cudaStream_t s = (cudaStream_t)stream;
    stark_b200_status st;
    const uint32_t out_cols = epilogue == 2u ? w->rows / 2u : w->rows;
    const size_t xin = (size_t)m * w->columns * 2u, yout = (size_t)m * out_cols * 2u;
    const uint16_t *dx = (const uint16_t *)x;
    uint16_t *dy = (uint16_t *)y;
    if (location == STARK_B200_HOST) {
        if ((st = ensure_buffer(&ctx->stage_in, &ctx->stage_in_bytes, xin)) != STARK_B200_OK) return st;
        if ((st = ensure_buffer(&ctx->stage_out, &ctx->stage_out_bytes, yout)) != STARK_B200_OK) return st;
        SB_CUDA(cudaMemcpyAsync(ctx->stage_in, x, xin, cudaMemcpyHostToDevice, s));
        if (epilogue == 1u) SB_CUDA(cudaMemcpyAsync(ctx->stage_out, y, yout, cudaMemcpyHostToDevice, s));
        dx = (const uint16_t *)ctx->stage_in;
        dy = (uint16_t *)ctx->stage_out;
    }
    GemmArgs a{};
    a.w = w;
    a.x = dx;
    a.x_rows = m;
    a.m = m;
    a.out = dy;
    a.ld_out = out_cols;
    a.epilogue = epilogue == 0u ? kEpiStore : (epilogue == 1u ? kEpiResidual : kEpiSwiGlu);
    a.error_word = ctx->error_word;
    if ((st = prefill_gemm_launch(a, s)) != STARK_B200_OK) return st;
    if (location == STARK_B200_HOST) {
        SB_CUDA(cudaMemcpyAsync(y, ctx->stage_out, yout, cudaMemcpyDeviceToHost, s));
        SB_CUDA(cudaStreamSynchronize(s));
    }
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_qmv_rows(const stark_b200_qmatrix *matrix, const void *x, void *y, uint32_t m,
                                         uint32_t epilogue, const float *norm_weight_host, float eps, uint32_t location,
                                         void *stream) {
    QMatrix *w = const_cast<QMatrix *>(reinterpret_cast<const QMatrix *>(matrix));
    if (!w || !x || !y || m == 0 || m > kQmvMultiMaxRows || epilogue > 2u) return STARK_B200_INVALID_ARGUMENT;
    if (!qmv_multi_supports(w, m, norm_weight_host != nullptr)) return STARK_B200_UNSUPPORTED;
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    cudaStream_t s = (cudaStream_t)stream;
    stark_b200_status st;
    const uint32_t out_cols = epilogue == 2u ? w->rows / 2u : w->rows;
    const size_t xin = (size_t)m * w->columns * 2u, yout = (size_t)m * out_cols * 2u;
    const size_t norm_bytes = norm_weight_host ? (size_t)w->columns * 4u : 0u;
    const uint16_t *dx = (const uint16_t *)x;
    uint16_t *dy = (uint16_t *)y;
    const float *dnorm = nullptr;
    if (location == STARK_B200_HOST) {
        // input rows, then the norm weights, in the one staging buffer (16-byte aligned parts)
        const size_t xin_padded = (xin + 15u) & ~(size_t)15u;
        if ((st = ensure_buffer(&ctx->stage_in, &ctx->stage_in_bytes, xin_padded + norm_bytes)) != STARK_B200_OK) return st;
        if ((st = ensure_buffer(&ctx->stage_out, &ctx->stage_out_bytes, yout)) != STARK_B200_OK) return st;
        SB_CUDA(cudaMemcpyAsync(ctx->stage_in, x, xin, cudaMemcpyHostToDevice, s));
        if (norm_bytes) {
            SB_CUDA(cudaMemcpyAsync((uint8_t *)ctx->stage_in + xin_padded, norm_weight_host, norm_bytes, cudaMemcpyHostToDevice, s));
            dnorm = (const float *)((uint8_t *)ctx->stage_in + xin_padded);
        }
        if (epilogue == 1u) SB_CUDA(cudaMemcpyAsync(ctx->stage_out, y, yout, cudaMemcpyHostToDevice, s));
        dx = (const uint16_t *)ctx->stage_in;
        dy = (uint16_t *)ctx->stage_out;
    } else {
        dnorm = norm_weight_host;  // with device buffers the weights are a device pointer too
    }
    QmvMultiArgs a{};
    a.matrix = w;
    a.x = dx;
    a.x_stride = w->columns;
    a.m = m;
    a.y = dy;
    a.y_stride = out_cols;
    a.norm_weight = dnorm;
    a.eps = eps;
    a.epilogue = epilogue == 0u ? kEpiStore : (epilogue == 1u ? kEpiResidual : kEpiSwiGlu);
    a.error_word = ctx->error_word;
    if ((st = qmv_multi_launch(a, s)) != STARK_B200_OK) return st;
    if (location == STARK_B200_HOST) {
        SB_CUDA(cudaMemcpyAsync(y, ctx->stage_out, yout, cudaMemcpyDeviceToHost, s));
        SB_CUDA(cudaStreamSynchronize(s));
    }
    return STARK_B200_OK;
}

struct stark_b200_graph {
    cudaGraph_t graph;
    cudaGraphExec_t exec;
};

stark_b200_status stark_b200_graph_begin(void *stream) {
    if (!device_context()) return STARK_B200_DEVICE_FAILURE;
    SB_CUDA(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_graph_end(void *stream, stark_b200_graph **out_graph) {
    if (!out_graph) return STARK_B200_INVALID_ARGUMENT;
    *out_graph = nullptr;
    cudaGraph_t g = nullptr;
    SB_CUDA(cudaStreamEndCapture((cudaStream_t)stream, &g));
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        return cuda_status(e);
    }
    stark_b200_graph *out = new (std::nothrow) stark_b200_graph{g, exec};
    if (!out) {
        cudaGraphExecDestroy(exec);
        cudaGraphDestroy(g);
        return STARK_B200_OUT_OF_MEMORY;
    }
    *out_graph = out;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_graph_launch(stark_b200_graph *graph, void *stream) {
    if (!graph) return STARK_B200_INVALID_ARGUMENT;
    SB_CUDA(cudaGraphLaunch(graph->exec, (cudaStream_t)stream));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_graph_destroy(stark_b200_graph **graph) {
    if (!graph) return STARK_B200_INVALID_ARGUMENT;
    if (*graph) {
        cudaGraphExecDestroy((*graph)->exec);
        cudaGraphDestroy((*graph)->graph);
        delete *graph;
        *graph = nullptr;
    }
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_prefill_attention(const void *qkv, const void *keys, const void *values,
                                                  const int32_t *block_table, uint32_t num_blocks, void *out, uint32_t m,
                                                  uint32_t first_pos, uint32_t q_heads, uint32_t kv_heads,
                                                  uint32_t variant) {
    if (!qkv || !keys || !values || !block_table || !out || m == 0 || num_blocks == 0 || kv_heads == 0 || q_heads == 0 ||
        q_heads % kv_heads != 0 || variant > 1u)
        return STARK_B200_INVALID_ARGUMENT;
    if ((uint64_t)first_pos + m > (uint64_t)num_blocks * kPageTokens) return STARK_B200_CONTEXT_LIMIT;
    for (uint32_t i = 0; i < num_blocks; ++i)
        if (block_table[i] < 0 || (uint32_t)block_table[i] >= num_blocks) return STARK_B200_INVALID_ARGUMENT;
    if (!device_context()) return STARK_B200_DEVICE_FAILURE;
    const size_t heads = q_heads + 2u * (size_t)kv_heads;
    const size_t qkv_bytes = (size_t)m * heads * kHeadDim * 2u, out_bytes = (size_t)m * q_heads * kHeadDim * 2u;
    const size_t cache_bytes = (size_t)num_blocks * kv_heads * kPageTokens * kHeadDim * 2u;
    uint16_t *dq = nullptr, *dk = nullptr, *dv = nullptr, *dout = nullptr;
    int32_t *dtable = nullptr;
    stark_b200_status st = STARK_B200_OK;
    auto ok = [&](cudaError_t e) {
        if (e != cudaSuccess && st == STARK_B200_OK) st = cuda_status(e);
        return e == cudaSuccess;
    };
    if (ok(cudaMalloc(&dq, qkv_bytes)) && ok(cudaMalloc(&dk, cache_bytes)) && ok(cudaMalloc(&dv, cache_bytes)) &&
        ok(cudaMalloc(&dout, out_bytes)) && ok(cudaMalloc(&dtable, (size_t)num_blocks * 4u)) &&
        ok(cudaMemcpy(dq, qkv, qkv_bytes, cudaMemcpyHostToDevice)) && ok(cudaMemcpy(dk, keys, cache_bytes, cudaMemcpyHostToDevice)) &&
        ok(cudaMemcpy(dv, values, cache_bytes, cudaMemcpyHostToDevice)) && ok(cudaMemset(dout, 0, out_bytes)) &&
        ok(cudaMemcpy(dtable, block_table, (size_t)num_blocks * 4u, cudaMemcpyHostToDevice))) {
        PrefillAttnArgs a{dq, KvLayer{dk, dv}, dtable, dout, m, first_pos, q_heads, kv_heads, 1.0f / sqrtf((float)kHeadDim)};
        a.num_blocks = variant == 1u ? num_blocks : 0u;  // without the cache's extent: the mma.sync kernel
        st = variant == 1u ? prefill_attention_tc_launch(a, nullptr) : prefill_attention_launch(a, nullptr);
        if (st == STARK_B200_OK && ok(cudaDeviceSynchronize())) ok(cudaMemcpy(out, dout, out_bytes, cudaMemcpyDeviceToHost));
    }
    cudaFree(dq);
    cudaFree(dk);
    cudaFree(dv);
    cudaFree(dout);
    cudaFree(dtable);
    return st;
}

}  // extern "C"
