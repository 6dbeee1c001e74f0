// extern "C" entry points of the model surface and of the small operators.
#include <cmath>
#include <cstring>
#include <new>
#include <vector>

#include "model.cuh"
#include "tunables.cuh"

using namespace sb;

namespace {

inline Model *M(stark_b200_model *m) { return reinterpret_cast<Model *>(m); }

__global__ void bf16_to_f32_kernel(const uint16_t *in, float *out, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        out[i] = bf16_bits_to_f32(in[i]);
}

// Temporary device mirrors of host buffers for the per-operator calls.
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

#define SB_TRY(expr)                                \
    do {                                            \
        stark_b200_status _s = (expr);              \
        if (_s != STARK_B200_OK) return _s;         \
    } while (0)

}  // namespace

extern "C" {

stark_b200_status stark_b200_op_rmsnorm(const void *input, const float *scales, void *output, void *shortcut,
                                        uint32_t count, float epsilon, uint32_t residual_add, uint32_t location,
                                        void *stream) {
    if (!input || !scales || !output || count == 0 || (residual_add && !shortcut)) return STARK_B200_INVALID_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (location == STARK_B200_DEVICE)
        return rmsnorm_launch((const uint16_t *)input, scales, (uint16_t *)output, (uint16_t *)shortcut, count,
                              epsilon, residual_add != 0, s);
    Staged st;
    uint16_t *din, *dout, *dsc = nullptr;
    float *dw;
    SB_TRY(st.in((const uint16_t *)input, count, &din));
    SB_TRY(st.in(scales, count, &dw));
    SB_TRY(st.in((const uint16_t *)nullptr, count, &dout));
    if (shortcut) SB_TRY(st.in((const uint16_t *)shortcut, count, &dsc));
    SB_TRY(rmsnorm_launch(din, dw, dout, dsc, count, epsilon, residual_add != 0, s));
    SB_CUDA(cudaMemcpyAsync(output, dout, count * 2, cudaMemcpyDeviceToHost, s));
    if (shortcut) SB_CUDA(cudaMemcpyAsync(shortcut, dsc, count * 2, cudaMemcpyDeviceToHost, s));
    SB_CUDA(cudaStreamSynchronize(s));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_swiglu(const void *fused, void *out, uint32_t gated_dim, uint32_t location,
                                       void *stream) {
    if (!fused || !out || gated_dim == 0) return STARK_B200_INVALID_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (location == STARK_B200_DEVICE) return swiglu_launch((const uint16_t *)fused, (uint16_t *)out, gated_dim, s);
    Staged st;
    uint16_t *din, *dout;
    SB_TRY(st.in((const uint16_t *)fused, (size_t)2 * gated_dim, &din));
    SB_TRY(st.in((const uint16_t *)nullptr, gated_dim, &dout));
    SB_TRY(swiglu_launch(din, dout, gated_dim, s));
    SB_CUDA(cudaMemcpyAsync(out, dout, (size_t)gated_dim * 2, cudaMemcpyDeviceToHost, s));
    SB_CUDA(cudaStreamSynchronize(s));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_qmv_swiglu(const stark_b200_qmatrix *matrix, const void *x, void *out,
                                           uint32_t location, void *stream) {
    const QMatrix *w = reinterpret_cast<const QMatrix *>(matrix);
    if (!w || !x || !out || !w->pair_halves) return STARK_B200_INVALID_ARGUMENT;
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    cudaStream_t s = (cudaStream_t)stream;
    Staged st;
    const uint16_t *dx = (const uint16_t *)x;
    uint16_t *dy = (uint16_t *)out;
    if (location == STARK_B200_HOST) {
        uint16_t *a, *b;
        SB_TRY(st.in((const uint16_t *)x, w->columns, &a));
        SB_TRY(st.in((const uint16_t *)nullptr, w->rows / 2u, &b));
        dx = a;
        dy = b;
    }
    QmvArgs a{};
    a.matrix = w;
    a.x = dx;
    a.y = dy;
    a.m = 1;
    a.io_type = STARK_B200_BF16;
    a.prologue = kProPlain;
    a.epilogue = kEpiSwiGlu;
    a.error_word = ctx->error_word;
    a.pdl = location == STARK_B200_DEVICE;
    SB_TRY(qmv_launch(a, s));
    if (location == STARK_B200_HOST) {
        SB_CUDA(cudaMemcpyAsync(out, dy, (size_t)(w->rows / 2u) * 2, cudaMemcpyDeviceToHost, s));
        SB_CUDA(cudaStreamSynchronize(s));
    }
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_argmax(const void *logits_bf16, uint32_t vocab, uint32_t *out_index,
                                       uint32_t location, void *stream) {
    if (!logits_bf16 || !out_index || vocab == 0) return STARK_B200_INVALID_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (location == STARK_B200_DEVICE) return argmax_bf16_launch((const uint16_t *)logits_bf16, vocab, out_index, s);
    Staged st;
    uint16_t *din;
    uint32_t *dout;
    SB_TRY(st.in((const uint16_t *)logits_bf16, vocab, &din));
    SB_TRY(st.in((const uint32_t *)nullptr, 1, &dout));
    SB_TRY(argmax_bf16_launch(din, vocab, dout, s));
    SB_CUDA(cudaMemcpyAsync(out_index, dout, 4, cudaMemcpyDeviceToHost, s));
    SB_CUDA(cudaStreamSynchronize(s));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_log_softmax(const float *logits, double *out, uint32_t vocab, uint32_t location,
                                            void *stream) {
    if (!logits || !out || vocab == 0) return STARK_B200_INVALID_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (location == STARK_B200_DEVICE) return log_softmax_launch(logits, out, vocab, nullptr, s);
    Staged st;
    float *din;
    double *dout;
    SB_TRY(st.in(logits, vocab, &din));
    SB_TRY(st.in((const double *)nullptr, vocab, &dout));
    SB_TRY(log_softmax_launch(din, dout, vocab, nullptr, s));
    SB_CUDA(cudaMemcpyAsync(out, dout, (size_t)vocab * 8, cudaMemcpyDeviceToHost, s));
    SB_CUDA(cudaStreamSynchronize(s));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_moe_route(const float *logits, uint32_t *ids, float *weights, uint32_t rows,
                                          uint32_t experts, uint32_t active, uint32_t round_weights,
                                          uint32_t round_logits, uint32_t location, void *stream) {
    if (!logits || !ids || !weights || rows == 0 || experts == 0 || active == 0) return STARK_B200_INVALID_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (location == STARK_B200_DEVICE)
        return moe_route_launch(logits, ids, weights, rows, experts, active, round_weights != 0, round_logits != 0, s);
    Staged st;
    float *dl, *dw;
    uint32_t *di;
    SB_TRY(st.in(logits, (size_t)rows * experts, &dl));
    SB_TRY(st.in((const uint32_t *)nullptr, (size_t)rows * active, &di));
    SB_TRY(st.in((const float *)nullptr, (size_t)rows * active, &dw));
    SB_CUDA(cudaMemsetAsync(di, 0, (size_t)rows * active * 4, s));
    SB_TRY(moe_route_launch(dl, di, dw, rows, experts, active, round_weights != 0, round_logits != 0, s));
    SB_CUDA(cudaMemcpyAsync(ids, di, (size_t)rows * active * 4, cudaMemcpyDeviceToHost, s));
    SB_CUDA(cudaMemcpyAsync(weights, dw, (size_t)rows * active * 4, cudaMemcpyDeviceToHost, s));
    SB_CUDA(cudaStreamSynchronize(s));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_attention_decode(const void *qkv, void *keys, void *values, void *out,
                                                 const float *q_norm, const float *k_norm,
                                                 const stark_b200_attention_desc *d) {
    if (!qkv || !keys || !values || !out || !d) return STARK_B200_INVALID_ARGUMENT;
    if (d->struct_size != sizeof(stark_b200_attention_desc) || d->abi_version != STARK_B200_ABI_VERSION)
        return STARK_B200_ABI_MISMATCH;
    if (d->head_dim != kHeadDim || d->kv_heads == 0 || d->q_heads % d->kv_heads != 0) return STARK_B200_UNSUPPORTED;
    if (d->position >= d->capacity) return STARK_B200_CONTEXT_LIMIT;
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    const uint32_t H = d->q_heads, KH = d->kv_heads, pos = d->position;
    const uint32_t blocks = pos / kPageTokens + 1u;
    const size_t page_elems = (size_t)KH * kPageTokens * kHeadDim;
    // host [row, kv_head, 128] -> paged [block, kv_head, row_in_block, 128]
    std::vector<uint16_t> pk(blocks * page_elems, 0), pv(blocks * page_elems, 0);
    const uint16_t *hk = (const uint16_t *)keys, *hv = (const uint16_t *)values;
    for (uint32_t r = 0; r < pos; ++r)
        for (uint32_t h = 0; h < KH; ++h) {
            const size_t dst = (((size_t)(r / kPageTokens) * KH + h) * kPageTokens + r % kPageTokens) * kHeadDim;
            const size_t src = ((size_t)r * KH + h) * kHeadDim;
            memcpy(&pk[dst], &hk[src], kHeadDim * 2);
            memcpy(&pv[dst], &hv[src], kHeadDim * 2);
        }
    std::vector<int32_t> table(blocks);
    for (uint32_t b = 0; b < blocks; ++b) table[b] = (int32_t)b;
    // RoPE coefficients of this position (rope.rs:346-440)
    std::vector<float> cs(kHeadDim * (size_t)(pos + 1u), 0.0f), sn(kHeadDim * (size_t)(pos + 1u), 0.0f);
    if (d->rope_theta > 0.0f)
        for (uint32_t pair = 0; pair < kHeadDim / 2u; ++pair) {
            const float inv = 1.0f / powf(d->rope_theta, (float)(pair * 2u) / (float)kHeadDim);
            const float e = (float)pos * inv;
            const float s = sinf(e) * 1.0f, c = cosf(e) * 1.0f;
            sn[(size_t)pos * kHeadDim + pair] = sn[(size_t)pos * kHeadDim + pair + 64u] = s;
            cs[(size_t)pos * kHeadDim + pair] = cs[(size_t)pos * kHeadDim + pair + 64u] = c;
        }
    const uint32_t splits = d->splits ? std::min(d->splits, kMaxAttnSplits) : std::min<uint32_t>(kMaxAttnSplits, 8u);
    Staged st;
    uint16_t *dq, *dk, *dv, *dout;
    int32_t *dt;
    float *dqn = nullptr, *dkn = nullptr, *dcs = nullptr, *dsn = nullptr, *dscr;
    uint32_t *dcnt;
    StepState hs{pos, 0, 0, 0}, *dstate;
    SB_TRY(st.in((const uint16_t *)qkv, (size_t)(H + 2u * KH) * kHeadDim, &dq));
    SB_TRY(st.in(pk.data(), pk.size(), &dk));
    SB_TRY(st.in(pv.data(), pv.size(), &dv));
    SB_TRY(st.in((const uint16_t *)nullptr, (size_t)H * kHeadDim, &dout));
    SB_TRY(st.in(table.data(), table.size(), &dt));
    if (q_norm) SB_TRY(st.in(q_norm, kHeadDim, &dqn));
    if (k_norm) SB_TRY(st.in(k_norm, kHeadDim, &dkn));
    if (d->rope_theta > 0.0f) {
        SB_TRY(st.in(cs.data(), cs.size(), &dcs));
        SB_TRY(st.in(sn.data(), sn.size(), &dsn));
    }
    SB_TRY(st.in((const float *)nullptr, attention_scratch_floats(H, KH, splits), &dscr));
    SB_TRY(st.in((const uint32_t *)nullptr, KH, &dcnt));
    SB_CUDA(cudaMemset(dcnt, 0, KH * 4));
    SB_TRY(st.in(&hs, 1, &dstate));
    AttnArgs a{};
    a.qkv = dq;
    a.out = dout;
    a.kv = KvLayer{dk, dv};
    a.block_table = dt;
    a.q_norm = dqn;
    a.k_norm = dkn;
    a.rope_cos = dcs;
    a.rope_sin = dsn;
    a.state = dstate;
    a.eps = d->epsilon;
    a.scale = 1.0f / sqrtf((float)kHeadDim);
    a.q_heads = H;
    a.kv_heads = KH;
    a.splits = splits;
    a.scratch = dscr;
    a.counters = dcnt;
    a.error_word = ctx->error_word;
    a.pdl = false;
    SB_TRY(attention_decode_launch(a, 0));
    SB_CUDA(cudaMemcpy(out, dout, (size_t)H * kHeadDim * 2, cudaMemcpyDeviceToHost));
    // the appended row back into the caller's row-major cache
    std::vector<uint16_t> bk(page_elems), bv(page_elems);
    const uint32_t nb = pos / kPageTokens;
    SB_CUDA(cudaMemcpy(bk.data(), dk + (size_t)nb * page_elems, page_elems * 2, cudaMemcpyDeviceToHost));
    SB_CUDA(cudaMemcpy(bv.data(), dv + (size_t)nb * page_elems, page_elems * 2, cudaMemcpyDeviceToHost));
    uint16_t *ok = (uint16_t *)keys, *ov = (uint16_t *)values;
    for (uint32_t h = 0; h < KH; ++h) {
        const size_t src = ((size_t)h * kPageTokens + pos % kPageTokens) * kHeadDim;
        memcpy(&ok[((size_t)pos * KH + h) * kHeadDim], &bk[src], kHeadDim * 2);
        memcpy(&ov[((size_t)pos * KH + h) * kHeadDim], &bv[src], kHeadDim * 2);
    }
    return STARK_B200_OK;
}

// ------------------------------------------------------------------------------------------ model

stark_b200_status stark_b200_model_create(const stark_b200_dense_config *config, stark_b200_model **out_model) {
    if (!config || !out_model) return STARK_B200_INVALID_ARGUMENT;
    *out_model = nullptr;
    if (config->struct_size != sizeof(stark_b200_dense_config) || config->abi_version != STARK_B200_ABI_VERSION)
        return STARK_B200_ABI_MISMATCH;
    if (!device_context()) return STARK_B200_DEVICE_FAILURE;
    Model *m = nullptr;
    stark_b200_status st = model_create(*config, &m);
    if (st != STARK_B200_OK) return st;
    *out_model = reinterpret_cast<stark_b200_model *>(m);
    return STARK_B200_OK;
}

stark_b200_status stark_b200_model_set_affine(stark_b200_model *model, uint32_t layer, uint32_t which,
                                              const void *codes, const void *scales, const void *biases,
                                              const stark_b200_affine_desc *desc) {
    if (!model || !desc) return STARK_B200_INVALID_ARGUMENT;
    stark_b200_affine_desc d = *desc;
    d.pair_halves = which == STARK_B200_MAT_UPGATE ? 1u : 0u;
    stark_b200_qmatrix *q = nullptr;
    stark_b200_status st = stark_b200_qmatrix_create_affine(codes, scales, biases, &d, &q);
    if (st != STARK_B200_OK) return st;
    st = model_set_matrix(M(model), layer, which, reinterpret_cast<QMatrix *>(q));
    if (st != STARK_B200_OK) stark_b200_qmatrix_destroy(&q);
    return st;
}

stark_b200_status stark_b200_model_set_vector(stark_b200_model *model, uint32_t layer, uint32_t which,
                                              const float *data, uint32_t count) {
    if (!model || !data) return STARK_B200_INVALID_ARGUMENT;
    return model_set_vector(M(model), layer, which, data, count);
}

stark_b200_status stark_b200_model_tp_init(stark_b200_model *model, uint32_t rank, uint32_t ranks,
                                           uint32_t vocab_offset, uint32_t vocab_total, uint8_t handle_out[64]) {
    if (!model || !handle_out) return STARK_B200_INVALID_ARGUMENT;
    return model_tp_init(M(model), rank, ranks, vocab_offset, vocab_total, handle_out);
}

stark_b200_status stark_b200_model_tp_connect(stark_b200_model *model, const uint8_t *handles, size_t handle_bytes) {
    if (!model || !handles) return STARK_B200_INVALID_ARGUMENT;
    if (handle_bytes != (size_t)M(model)->tp.size * 64u) return STARK_B200_INVALID_ARGUMENT;
    return model_tp_connect(M(model), handles);
}

stark_b200_status stark_b200_model_tp_set_wait(stark_b200_model *model, uint64_t nanoseconds) {
    if (!model) return STARK_B200_INVALID_ARGUMENT;
    return model_tp_set_wait(M(model), nanoseconds);
}

stark_b200_status stark_b200_model_tp_connect_unanswered(stark_b200_model *model) {
    if (!model) return STARK_B200_INVALID_ARGUMENT;
    return model_tp_connect_unanswered(M(model));
}

stark_b200_status stark_b200_model_tp_rows_init(stark_b200_model *model, uint8_t handle_out[64]) {
    if (!model || !handle_out) return STARK_B200_INVALID_ARGUMENT;
    return model_tp_rows_init(M(model), handle_out);
}

stark_b200_status stark_b200_model_tp_rows_connect(stark_b200_model *model, const uint8_t *handles, size_t handle_bytes) {
    if (!model || !handles) return STARK_B200_INVALID_ARGUMENT;
    if (handle_bytes != (size_t)M(model)->tp.size * 64u) return STARK_B200_INVALID_ARGUMENT;
    return model_tp_rows_connect(M(model), handles);
}

stark_b200_status stark_b200_model_finalize(stark_b200_model *model) {
    if (!model) return STARK_B200_INVALID_ARGUMENT;
    return model_finalize(M(model));
}

stark_b200_status stark_b200_destroy(stark_b200_model **model) {
    if (!model) return STARK_B200_INVALID_ARGUMENT;
    if (*model) {
        cudaStreamSynchronize(M(*model)->stream);
        delete M(*model);
        *model = nullptr;
    }
    return STARK_B200_OK;
}

stark_b200_status stark_b200_reset(stark_b200_model *model) {
    if (!model) return STARK_B200_INVALID_ARGUMENT;
    if (M(model)->fenced) return STARK_B200_RELOAD_REQUIRED;
    return model_reset(M(model));
}

stark_b200_status stark_b200_drain(stark_b200_model *model) {
    if (!model) return STARK_B200_INVALID_ARGUMENT;
    return model_drain(M(model));
}

stark_b200_status stark_b200_cancel(stark_b200_model *model) {
    if (!model) return STARK_B200_INVALID_ARGUMENT;
    M(model)->cancel_requested = true;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_prefill(stark_b200_model *model, const uint32_t *token_ids, size_t count) {
    if (!model || !token_ids) return STARK_B200_INVALID_ARGUMENT;
    return model_prefill(M(model), token_ids, count);
}

stark_b200_status stark_b200_step(stark_b200_model *model, uint32_t token_id) {
    if (!model) return STARK_B200_INVALID_ARGUMENT;
    return model_step(M(model), token_id, false);
}

stark_b200_status stark_b200_readout_f32(stark_b200_model *model, float *dst, size_t count) {
    if (!model || !dst) return STARK_B200_INVALID_ARGUMENT;
    return model_readout_f32(M(model), dst, count);
}

stark_b200_status stark_b200_readout_bf16(stark_b200_model *model, uint16_t *dst, size_t count) {
    if (!model || !dst) return STARK_B200_INVALID_ARGUMENT;
    return model_readout_bf16(M(model), dst, count);
}

stark_b200_status stark_b200_readout_logprobs_f32(stark_b200_model *model, float *dst, size_t count) {
    if (!model || !dst) return STARK_B200_INVALID_ARGUMENT;
    Model *m = M(model);
    if (!m->has_logits) return STARK_B200_INVALID_STATE;
    if (m->tp.size > 1u) return STARK_B200_UNSUPPORTED;  // a shard's logits do not normalise alone
    if (count != m->cfg.vocab) return STARK_B200_INVALID_ARGUMENT;
    Staged st;
    float *df;
    double *dd;
    SB_TRY(st.in((const float *)nullptr, count, &df));
    SB_TRY(st.in((const double *)nullptr, count, &dd));
    bf16_to_f32_kernel<<<148, 256, 0, m->stream>>>(m->logits, df, (uint32_t)count);
    SB_TRY(log_softmax_launch(df, dd, (uint32_t)count, nullptr, m->stream));
    std::vector<double> host(count);
    SB_CUDA(cudaMemcpyAsync(host.data(), dd, count * 8, cudaMemcpyDeviceToHost, m->stream));
    SB_CUDA(cudaStreamSynchronize(m->stream));
    for (size_t i = 0; i < count; ++i) dst[i] = (float)host[i];
    return STARK_B200_OK;
}

stark_b200_status stark_b200_sample(stark_b200_model *model, const stark_b200_sampling *params, uint32_t *out_token) {
    if (!model || !params || !out_token) return STARK_B200_INVALID_ARGUMENT;
    if (params->struct_size != sizeof(stark_b200_sampling)) return STARK_B200_ABI_MISMATCH;
    Model *m = M(model);
    if (!m->has_logits) return STARK_B200_INVALID_STATE;
    if (m->tp.size > 1u) return STARK_B200_UNSUPPORTED;
    SB_TRY(sampling_validate(*params, m->cfg.vocab));
    if (!m->sample_scratch) SB_CUDA(cudaMalloc(&m->sample_scratch, sampling_scratch_bytes(m->cfg.vocab) + 16u));
    // the token lands behind the working arrays
    uint32_t *out = reinterpret_cast<uint32_t *>(static_cast<uint8_t *>(m->sample_scratch) +
                                                 sampling_scratch_bytes(m->cfg.vocab));
    SB_TRY(sampling_launch(m->logits, STARK_B200_BF16, m->cfg.vocab, *params, m->sample_scratch, out, m->stream));
    SB_CUDA(cudaMemcpyAsync(out_token, out, 4, cudaMemcpyDeviceToHost, m->stream));
    SB_CUDA(cudaStreamSynchronize(m->stream));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_op_sample(const void *logits, uint32_t vocab, uint32_t io_type,
                                       const stark_b200_sampling *params, uint32_t *out_token, uint32_t location,
                                       void *stream) {
    if (!logits || !params || !out_token || io_type > STARK_B200_F32) return STARK_B200_INVALID_ARGUMENT;
    if (params->struct_size != sizeof(stark_b200_sampling)) return STARK_B200_ABI_MISMATCH;
    SB_TRY(sampling_validate(*params, vocab));
    cudaStream_t s = (cudaStream_t)stream;
    Staged st;
    const uint8_t *din = static_cast<const uint8_t *>(logits);
    if (location == STARK_B200_HOST) {
        uint8_t *copy;
        SB_TRY(st.in(static_cast<const uint8_t *>(logits), (size_t)vocab * (io_type == STARK_B200_F32 ? 4u : 2u), &copy));
        din = copy;
    }
    uint8_t *scratch;
    SB_TRY(st.in((const uint8_t *)nullptr, sampling_scratch_bytes(vocab) + 16u, &scratch));
    uint32_t *out = reinterpret_cast<uint32_t *>(scratch + sampling_scratch_bytes(vocab));
    SB_TRY(sampling_launch(din, io_type, vocab, *params, scratch, out, s));
    SB_CUDA(cudaMemcpyAsync(out_token, out, 4, cudaMemcpyDeviceToHost, s));
    SB_CUDA(cudaStreamSynchronize(s));
    return STARK_B200_OK;
}

stark_b200_status stark_b200_argmax(stark_b200_model *model, uint32_t *out_token) {
    if (!model || !out_token) return STARK_B200_INVALID_ARGUMENT;
    return model_next_token(M(model), out_token);
}

stark_b200_status stark_b200_generate_greedy(stark_b200_model *model, uint32_t steps, uint32_t *out_tokens) {
    if (!model || !out_tokens) return STARK_B200_INVALID_ARGUMENT;
    return model_generate_greedy(M(model), steps, out_tokens);
}

stark_b200_status stark_b200_rewind(stark_b200_model *model, uint64_t position) {
    if (!model) return STARK_B200_INVALID_ARGUMENT;
    return model_rewind(M(model), position);
}

stark_b200_status stark_b200_set_tunable(const char *name, uint32_t value) {
    return set_tunable(name, value) ? STARK_B200_OK : STARK_B200_INVALID_ARGUMENT;
}

stark_b200_status stark_b200_model_recapture(stark_b200_model *model) {
    if (!model) return STARK_B200_INVALID_ARGUMENT;
    if (M(model)->tp.size > 1u) return STARK_B200_UNSUPPORTED;
    return model_recapture(M(model));
}

stark_b200_status stark_b200_mtp_initial(stark_b200_model *model, uint32_t *out_pending) {
    if (!model || !out_pending) return STARK_B200_INVALID_ARGUMENT;
    Model *m = M(model);
    if (!m->mtp.enabled) return STARK_B200_UNSUPPORTED;
    if (!m->mtp.has_pending || !m->has_logits) return STARK_B200_INVALID_STATE;
    return model_next_token(m, out_pending);
}

stark_b200_status stark_b200_mtp_round(stark_b200_model *model, uint32_t pending, uint32_t drafts, uint32_t policy,
                                       uint32_t accept_mask, stark_b200_mtp_round_result *out) {
    if (!model || !out) return STARK_B200_INVALID_ARGUMENT;
    if (out->struct_size != sizeof(stark_b200_mtp_round_result) || out->abi_version != STARK_B200_ABI_VERSION)
        return STARK_B200_ABI_MISMATCH;
    return mtp_round(M(model), pending, drafts, policy, accept_mask, out);
}

stark_b200_status stark_b200_mtp_round_lookup(stark_b200_model *model, uint32_t pending, const uint32_t *proposals,
                                              uint32_t count, uint32_t policy, uint32_t accept_mask,
                                              stark_b200_mtp_round_result *out) {
    if (!model || !out || (count && !proposals)) return STARK_B200_INVALID_ARGUMENT;
    if (out->struct_size != sizeof(stark_b200_mtp_round_result) || out->abi_version != STARK_B200_ABI_VERSION)
        return STARK_B200_ABI_MISMATCH;
    static const uint32_t none = 0;
    return mtp_round(M(model), pending, count, policy, accept_mask, out, count ? proposals : &none);
}

stark_b200_status stark_b200_mtp_commit(stark_b200_model *model, uint32_t accepted, uint32_t next_pending,
                                        stark_b200_mtp_round_result *out) {
    if (!model || !out) return STARK_B200_INVALID_ARGUMENT;
    if (out->struct_size != sizeof(stark_b200_mtp_round_result) || out->abi_version != STARK_B200_ABI_VERSION)
        return STARK_B200_ABI_MISMATCH;
    return mtp_commit(M(model), accepted, next_pending, out);
}

stark_b200_status stark_b200_mtp_readout_row_f32(stark_b200_model *model, uint32_t row, float *dst, size_t count) {
    if (!model || !dst) return STARK_B200_INVALID_ARGUMENT;
    return mtp_readout_row_f32(M(model), row, dst, count);
}

stark_b200_status stark_b200_model_stream(stark_b200_model *model, void **out_stream) {
    if (!model || !out_stream) return STARK_B200_INVALID_ARGUMENT;
    *out_stream = (void *)M(model)->stream;
    return STARK_B200_OK;
}

stark_b200_status stark_b200_read_trace(stark_b200_model *model, uint64_t *dst, size_t count) {
    if (!model || !dst) return STARK_B200_INVALID_ARGUMENT;
    return model_read_trace(M(model), reinterpret_cast<unsigned long long *>(dst), count);
}

stark_b200_status stark_b200_get_info(stark_b200_model *model, stark_b200_info *info) {
    if (!model || !info) return STARK_B200_INVALID_ARGUMENT;
    if (info->struct_size != sizeof(stark_b200_info) || info->abi_version != STARK_B200_ABI_VERSION)
        return STARK_B200_ABI_MISMATCH;
    Model *m = M(model);
    info->vocab_size = m->cfg.vocab;
    info->prefill_chunk_tokens = 1024;
    info->context_tokens = m->cfg.context_tokens;
    info->position = m->position;
    info->capabilities = STARK_B200_CAP_FULL_F32_READOUT | STARK_B200_CAP_SERIAL_DECODE |
                         STARK_B200_CAP_PREFIX_REWIND | STARK_B200_CAP_DEVICE_GREEDY;
    info->fenced = m->fenced ? 1u : 0u;
    info->launches_per_step = m->step_launches;
    uint64_t wb = 0;
    for (auto &L : m->layers)
        for (QMatrix *q : {L.qkv, L.o, L.upgate, L.down})
            if (q) wb += q->bytes;
    if (m->embed) wb += m->embed->bytes;
    if (m->lm_head && m->lm_head != m->embed) wb += m->lm_head->bytes;
    info->weight_bytes = wb;
    info->kv_bytes_per_token = (uint64_t)m->cfg.layers * 2u * m->cfg.kv_heads * kHeadDim * 2u;
    info->launches_issued = m->launches_issued;
    info->trace_slots = m->trace ? m->trace_slots : 0u;
    info->persistent = m->use_mega ? 1u : 0u;
    return STARK_B200_OK;
}

}  // extern "C"
