// Dense Qwen3-shaped decode engine: one recorded launch sequence (CUDA graph with programmatic
// dependent launch between its kernels) per token, replayed with the position and token read from
// device memory.  Mirrors the reference's decode pass
//   crates/stark-engine/src/engine/language_model/stream/stream.rs:787-1217 (one submission per token,
//   on-device token chaining) and its layer wiring
//   crates/stark-engine/src/encodable_block/transformer_layer.rs:549-659.
//
// Per layer the sequence is five kernels:
//   qkv    = W_qkv  rmsnorm(h)                      matvec, norm fused in the prologue
//   attn   = attention(rope(norm(q)), cache + k, v)  one kernel: QK-norm, RoPE, KV append, split-KV, merge
//   h      = bf16(bf16(W_o attn) + h)                matvec, residual fused in the epilogue
//   act    = silu(gate) * up,  [up; gate] = W rmsnorm(h)
//   h      = bf16(bf16(W_down act) + h)
// then logits = W_head rmsnorm(h) with the greedy read-out fused into the matvec epilogue.
#include "model.cuh"
#include "mega.cuh"
#include "prefill.cuh"
#include "tunables.cuh"

#include <cmath>
#include <cstring>
#include <new>
#include <vector>

namespace sb {

namespace {

template <typename T>
stark_b200_status dmalloc(T **p, size_t count) {
    *p = nullptr;
    SB_CUDA(cudaMalloc(p, count * sizeof(T) ? count * sizeof(T) : 1));
    return STARK_B200_OK;
}

// Size of the token id space: the embedding table's rows (under tensor parallelism cfg.vocab is the
// read-out shard of this rank).
uint32_t input_vocab(const Model *m) { return m->tp.size > 1u ? m->tp_vocab_total : m->cfg.vocab; }

bool pdl_on() { return tunables().pdl != 0u; }

// CTAs per KV head of the decode attention: about one CTA per SM in total, so that every CTA can be resident
// beside the matvec before it and fetch its cache tiles while that matvec runs (measured on the 8-KV-head
// shape: 18 per head beats 16, 20, 24 and 32).
uint32_t default_attn_splits(uint32_t kv_heads) {
    return std::min<uint32_t>(kMaxAttnSplits, std::max<uint32_t>(1u, 148u / kv_heads));
}

}  // namespace

Model::~Model() {
    if (step_graph) cudaGraphExecDestroy(step_graph);
    if (ingest_graph) cudaGraphExecDestroy(ingest_graph);
    for (auto &L : layers) {
        qmatrix_free(L.qkv);
        qmatrix_free(L.o);
        qmatrix_free(L.upgate);
        qmatrix_free(L.down);
        qmatrix_free(L.o_rows);
        qmatrix_free(L.down_rows);
        cudaFree(L.attn_norm);
        cudaFree(L.mlp_norm);
        cudaFree(L.attn_norm_b16);
        cudaFree(L.mlp_norm_b16);
        cudaFree(L.q_norm);
        cudaFree(L.k_norm);
        cudaFree(L.kv.keys);
        cudaFree(L.kv.values);
    }
    mtp_destroy(this);
    if (lm_head != embed) qmatrix_free(lm_head);
    qmatrix_free(embed);
    cudaFree(final_norm);
    cudaFree(final_norm_b16);
    cudaFree(block_table);
    cudaFree(rope_cos);
    cudaFree(rope_sin);
    cudaFree(state);
    cudaFree(pending);
    cudaFree(generated);
    cudaFree(trace);
    cudaFree(tp_staged);
    cudaFree(mega_ops);
    cudaFree(mega_ingest_ops);
    cudaFree(mega_done);
    cudaFree(mega_scratch);
    cudaFree(h);
    cudaFree(h_alt);
    cudaFree(qkv);
    cudaFree(attn);
    cudaFree(act);
    cudaFree(logits);
    cudaFree(attn_scratch);
    cudaFree(attn_counters);
    cudaFree(partial_max);
    cudaFree(partial_index);
    if (tp_connected)
        for (uint32_t r = 0; r < tp.size; ++r)
            if (r != tp.rank && tp.base[r]) {
                if (tp_stand_ins) cudaFree(tp.base[r]);
                else cudaIpcCloseMemHandle(tp.base[r]);
            }
    if (tp_rows_connected)
        for (uint32_t r = 0; r < tp_rows.size; ++r)
            if (r != tp_rows.rank && tp_rows.base[r]) cudaIpcCloseMemHandle(tp_rows.base[r]);
    cudaFree(chunk_tokens);
    if (!tp_rows_local) {  // under tensor parallelism these two live inside the rows region
        cudaFree(chunk_h);
        cudaFree(chunk_act);
    }
    cudaFree(chunk_x);
    cudaFree(chunk_qkv);
    cudaFree(chunk_attn);
    cudaFree(tp_rows_local);
    cudaFree(tp_rows_arrive);
    cudaFree(rows_attn_partials);
    cudaFree(tp_local);
    cudaFree(sample_scratch);
    cudaFree(tp_seq);
    if (host_state) cudaFreeHost(host_state);
    if (host_logits) cudaFreeHost(host_logits);
    if (stream) cudaStreamDestroy(stream);
}

stark_b200_status model_create(const stark_b200_dense_config &c, Model **out) {
    *out = nullptr;
    if (c.layers == 0 || c.hidden == 0 || c.hidden % 64u != 0 || c.head_dim != kHeadDim || c.kv_heads == 0 ||
        c.q_heads % c.kv_heads != 0 || c.q_heads / c.kv_heads > 8u || c.inter == 0 || c.inter % 64u != 0 ||
        c.vocab == 0 || c.context_tokens == 0 || !(c.eps > 0.0f) || !(c.rope_theta > 0.0f))
        return STARK_B200_INVALID_ARGUMENT;
    Model *m = new (std::nothrow) Model();
    if (!m) return STARK_B200_OUT_OF_MEMORY;
    m->cfg = c;
    if (c.reserved > 1u) {  // the field counts draft-head layers: 0 or 1
        delete m;
        return STARK_B200_INVALID_ARGUMENT;
    }
    cudaGetDevice(&m->device);
    m->layers.resize(c.layers + c.reserved);  // the draft head's layer (with its own cache) comes last
    stark_b200_status st = STARK_B200_OK;
    auto fail = [&](stark_b200_status s) {
        delete m;
        return s;
    };
    if (cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) != cudaSuccess) return fail(STARK_B200_DEVICE_FAILURE);

    // KV pages: identity block table sized for the context (rounded up to whole pages).
    m->num_blocks = (c.context_tokens + kPageTokens - 1u) / kPageTokens;
    const size_t page_elems = (size_t)c.kv_heads * kPageTokens * kHeadDim;
    for (auto &L : m->layers) {
        if ((st = dmalloc(&L.kv.keys, m->num_blocks * page_elems)) != STARK_B200_OK) return fail(st);
        if ((st = dmalloc(&L.kv.values, m->num_blocks * page_elems)) != STARK_B200_OK) return fail(st);
        if (cudaMemset(L.kv.keys, 0, m->num_blocks * page_elems * 2) != cudaSuccess ||
            cudaMemset(L.kv.values, 0, m->num_blocks * page_elems * 2) != cudaSuccess)
            return fail(STARK_B200_DEVICE_FAILURE);
    }
    std::vector<int32_t> table(m->num_blocks);
    for (uint32_t i = 0; i < m->num_blocks; ++i) table[i] = (int32_t)i;
    if ((st = dmalloc(&m->block_table, m->num_blocks)) != STARK_B200_OK) return fail(st);
    if (cudaMemcpy(m->block_table, table.data(), table.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess)
        return fail(STARK_B200_DEVICE_FAILURE);

    // RoPE tables on the host with the reference's formulas and operation order
    // (crates/stark-engine/src/encodable_block/mixer/attention/rope.rs:346-440, UnscaledRoPEConfig).
    {
        const uint32_t positions = m->num_blocks * kPageTokens;
        std::vector<float> cs((size_t)positions * kHeadDim), sn((size_t)positions * kHeadDim);
        const uint32_t half = kHeadDim / 2u;
        for (uint32_t pair = 0; pair < half; ++pair) {
            const float inv = 1.0f / powf(c.rope_theta, (float)(pair * 2u) / (float)kHeadDim);
            for (uint32_t pos = 0; pos < positions; ++pos) {
                const float e = (float)pos * inv;
                const float s = sinf(e) * 1.0f, co = cosf(e) * 1.0f;
                sn[(size_t)pos * kHeadDim + pair] = s;
                sn[(size_t)pos * kHeadDim + pair + half] = s;
                cs[(size_t)pos * kHeadDim + pair] = co;
                cs[(size_t)pos * kHeadDim + pair + half] = co;
            }
        }
        if ((st = dmalloc(&m->rope_cos, cs.size())) != STARK_B200_OK) return fail(st);
        if ((st = dmalloc(&m->rope_sin, sn.size())) != STARK_B200_OK) return fail(st);
        if (cudaMemcpy(m->rope_cos, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMemcpy(m->rope_sin, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess)
            return fail(STARK_B200_DEVICE_FAILURE);
    }

    const uint32_t qkv_n = (c.q_heads + 2u * c.kv_heads) * kHeadDim;
    // CTAs per KV head: at most ~1.3 attention CTAs per SM in total.  One of them fits beside the two
    // resident CTAs of the matvec before it and fetches its cache tiles while that matvec runs; more
    // splits than that start cold.
    m->attn_splits = default_attn_splits(c.kv_heads);
    if (tunables().attn_splits) m->attn_splits = tunables().attn_splits;  // tuning: CTAs per KV head
    if ((st = dmalloc(&m->state, 1)) != STARK_B200_OK) return fail(st);
    if ((st = dmalloc(&m->pending, (size_t)c.context_tokens + 1u)) != STARK_B200_OK) return fail(st);
    if ((st = dmalloc(&m->generated, (size_t)c.context_tokens + 1u)) != STARK_B200_OK) return fail(st);
    if ((st = dmalloc(&m->h, c.hidden)) != STARK_B200_OK) return fail(st);
    if ((st = dmalloc(&m->h_alt, c.hidden)) != STARK_B200_OK) return fail(st);
    if ((st = dmalloc(&m->qkv, qkv_n)) != STARK_B200_OK) return fail(st);
    if ((st = dmalloc(&m->attn, c.q_heads * kHeadDim)) != STARK_B200_OK) return fail(st);
    if ((st = dmalloc(&m->act, c.inter)) != STARK_B200_OK) return fail(st);
    if ((st = dmalloc(&m->logits, c.vocab)) != STARK_B200_OK) return fail(st);
    if ((st = dmalloc(&m->attn_scratch, attention_scratch_floats(c.q_heads, c.kv_heads, kMaxAttnSplits))) !=
        STARK_B200_OK)
        return fail(st);
    if ((st = dmalloc(&m->attn_counters, c.kv_heads)) != STARK_B200_OK) return fail(st);
    if ((st = dmalloc(&m->partial_max, 1024)) != STARK_B200_OK) return fail(st);
    if ((st = dmalloc(&m->partial_index, 1024)) != STARK_B200_OK) return fail(st);
    if (const char *e = getenv("STARK_B200_TRACE")) {
        if (e[0] == '1') {  // one slot per launch
            m->trace_slots = 1u + 7u * c.layers + 3u;  // up to 7 launches per layer with tensor-parallel reductions
            if ((st = dmalloc(&m->trace, m->trace_slots)) != STARK_B200_OK) return fail(st);
        }
    }
    if (cudaMemset(m->attn_counters, 0, c.kv_heads * 4) != cudaSuccess ||
        cudaMemset(m->state, 0, sizeof(StepState)) != cudaSuccess)
        return fail(STARK_B200_DEVICE_FAILURE);
    if (cudaMallocHost(&m->host_state, sizeof(StepState)) != cudaSuccess ||
        cudaMallocHost(&m->host_logits, (size_t)c.vocab * 2u) != cudaSuccess)
        return fail(STARK_B200_OUT_OF_MEMORY);
    if (c.reserved == 1u && (st = mtp_create(m)) != STARK_B200_OK) return fail(st);
    *out = m;
    return STARK_B200_OK;
}

static stark_b200_status upload_f32(float **dst, const float *src, size_t n) {
    if (*dst) cudaFree(*dst);
    stark_b200_status st = dmalloc(dst, n);
    if (st != STARK_B200_OK) return st;
    SB_CUDA(cudaMemcpy(*dst, src, n * 4, cudaMemcpyHostToDevice));
    return STARK_B200_OK;
}

// The row norms multiply by bf16(weight) (normalization.rs:157-161): the rounded copy is made once, here.
static stark_b200_status upload_norm(float **dst, uint16_t **dst_b16, const float *src, size_t n) {
    stark_b200_status st = upload_f32(dst, src, n);
    if (st != STARK_B200_OK) return st;
    std::vector<uint16_t> rounded(n);
    for (size_t i = 0; i < n; ++i) rounded[i] = f32_to_bf16_bits(src[i]);
    if (*dst_b16) cudaFree(*dst_b16);
    if ((st = dmalloc(dst_b16, n)) != STARK_B200_OK) return st;
    SB_CUDA(cudaMemcpy(*dst_b16, rounded.data(), n * 2, cudaMemcpyHostToDevice));
    return STARK_B200_OK;
}

stark_b200_status model_set_vector(Model *m, uint32_t layer, uint32_t which, const float *data, uint32_t count) {
    if (m->finalized) return STARK_B200_INVALID_STATE;
    const auto &c = m->cfg;
    if (count != (which == STARK_B200_VEC_Q_NORM || which == STARK_B200_VEC_K_NORM ? kHeadDim : c.hidden) || count % 8u != 0)
        return STARK_B200_INVALID_ARGUMENT;
    if (which == STARK_B200_VEC_FINAL_NORM) return upload_norm(&m->final_norm, &m->final_norm_b16, data, count);
    if (which >= STARK_B200_VEC_MTP_EMBED_NORM && which <= STARK_B200_VEC_MTP_OUT_NORM) {
        if (!m->mtp.enabled) return STARK_B200_INVALID_STATE;
        float **slot = which == STARK_B200_VEC_MTP_EMBED_NORM ? &m->mtp.embed_norm
                       : (which == STARK_B200_VEC_MTP_HIDDEN_NORM ? &m->mtp.hidden_norm : &m->mtp.out_norm);
        return upload_f32(slot, data, count);
    }
    if (layer >= m->layers.size()) return STARK_B200_INVALID_ARGUMENT;  // layers, then the draft head's layer
    auto &L = m->layers[layer];
    switch (which) {
        case STARK_B200_VEC_ATTN_NORM: return upload_norm(&L.attn_norm, &L.attn_norm_b16, data, count);
        case STARK_B200_VEC_MLP_NORM: return upload_norm(&L.mlp_norm, &L.mlp_norm_b16, data, count);
        case STARK_B200_VEC_Q_NORM: return count == kHeadDim ? upload_f32(&L.q_norm, data, count) : STARK_B200_INVALID_ARGUMENT;
        case STARK_B200_VEC_K_NORM: return count == kHeadDim ? upload_f32(&L.k_norm, data, count) : STARK_B200_INVALID_ARGUMENT;
        default: return STARK_B200_INVALID_ARGUMENT;
    }
}

stark_b200_status model_set_matrix(Model *m, uint32_t layer, uint32_t which, QMatrix *q) {
    if (m->finalized) return STARK_B200_INVALID_STATE;
    const auto &c = m->cfg;
    const uint32_t qkv_n = (c.q_heads + 2u * c.kv_heads) * kHeadDim;
    auto put = [&](QMatrix **slot, uint32_t rows, uint32_t cols, bool pair) -> stark_b200_status {
        if (q->rows != rows || q->columns != cols || (q->pair_halves != 0) != pair) return STARK_B200_INVALID_ARGUMENT;
        if (*slot && *slot != q) qmatrix_free(*slot);
        *slot = q;
        return STARK_B200_OK;
    };
    if (which == STARK_B200_MAT_EMBED) {
        stark_b200_status st = put(&m->embed, input_vocab(m), c.hidden, false);
        if (st == STARK_B200_OK && c.tied) m->lm_head = m->embed;
        return st;
    }
    if (which == STARK_B200_MAT_LM_HEAD) {
        if (c.tied) return STARK_B200_INVALID_ARGUMENT;
        return put(&m->lm_head, c.vocab, c.hidden, false);
    }
    if (which == STARK_B200_MAT_MTP_FUSION) {
        if (!m->mtp.enabled) return STARK_B200_INVALID_STATE;
        return put(&m->mtp.fusion, c.hidden, 2u * c.hidden, false);
    }
    if (layer >= m->layers.size()) return STARK_B200_INVALID_ARGUMENT;  // layers, then the draft head's layer
    auto &L = m->layers[layer];
    switch (which) {
        case STARK_B200_MAT_QKV: return put(&L.qkv, qkv_n, c.hidden, false);
        case STARK_B200_MAT_O: return put(&L.o, c.hidden, c.q_heads * kHeadDim, false);
        case STARK_B200_MAT_UPGATE: return put(&L.upgate, 2u * c.inter, c.hidden, true);
        case STARK_B200_MAT_DOWN: return put(&L.down, c.hidden, c.inter, false);
        case STARK_B200_MAT_O_ROWS:
            if (m->tp.size < 2u || c.hidden % m->tp.size) return STARK_B200_INVALID_STATE;
            return put(&L.o_rows, c.hidden / m->tp.size, c.q_heads * m->tp.size * kHeadDim, false);
        case STARK_B200_MAT_DOWN_ROWS:
            if (m->tp.size < 2u || c.hidden % m->tp.size) return STARK_B200_INVALID_STATE;
            return put(&L.down_rows, c.hidden / m->tp.size, c.inter * m->tp.size, false);
        default: return STARK_B200_INVALID_ARGUMENT;
    }
}

// Issues the kernels of one token on m->stream.  full == false stops after the last layer
// (cache-only ingest of a prompt row) and takes the next token from the pending list.
static stark_b200_status issue_token(Model *m, bool full, uint32_t *launches) {
    const auto &c = m->cfg;
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    const bool pdl = pdl_on();
    cudaStream_t s = m->stream;
    stark_b200_status st;
    uint32_t n = 0;
    if ((st = embedding_row_launch(m->embed, m->state, m->h, pdl, s)) != STARK_B200_OK) return st;
    ++n;
    auto slot = [&](uint32_t index) -> TraceSlot * { return m->trace ? m->trace + index : nullptr; };
    const bool tp = m->tp.size > 1u;
    // Tensor parallel: a K-split projection pushes its share to every rank and the next matvec sums
    // the shares, adds the residual and stores the new residual stream into the other of two buffers
    // (its own blocks still read the old one).  2 exchanges per layer; exchange 2l+1 (after `down`) is
    // consumed by the next layer's qkv, the last one by the read-out matvec or the ingest close.
    const uint32_t per_token = 2u * c.layers;
    uint32_t *tokens = m->tp_seq;
    uint16_t *hcur = m->h, *hnext = m->h_alt;
    QmvExchange hooks{};
    // Two ways to close an exchange.  Default: a small kernel sums the packets once, in place, between the
    // producing and the consuming matvec (2 extra launches per layer).  STARK_B200_TP_FUSED=1: the consuming
    // matvec sums them in its prologue -- no extra launch, but every one of its CTAs reads every packet,
    // which costs more than the launch (8B on 2 GPUs: 535 tok/s fused, 612 with the kernel).
    static const bool fused = [] {
        const char *e = getenv("STARK_B200_TP_FUSED");
        return e && e[0] == '1';
    }();
    stark_b200_status consume_status = STARK_B200_OK;
    auto consume = [&](QmvArgs &a, uint32_t index) {
        if (fused) {
            hooks = tp_consumer_hooks(m->tp, index, per_token, tokens, hnext);
            a.exchange = &hooks;
            std::swap(hcur, hnext);  // after this matvec the residual stream lives in the other buffer
        } else {
            TraceSlot *own = a.trace;  // the reduction takes the slot, the matvec the next one
            if (tunables().tp_stage && m->tp_staged && a.prologue == kProRmsNorm) {
                // the reduction holds the whole new row: it also normalizes and scales it for this matvec
                consume_status = tp_reduce_stage_launch(m->tp, index, per_token, tokens, hcur, a.norm_weight, c.eps,
                                                        m->tp_staged, ctx->error_word, own, pdl, s);
                a.prologue = kProStaged;
                a.staged = m->tp_staged;
            } else {
                consume_status = tp_reduce_residual_launch(m->tp, index, per_token, tokens, hcur, ctx->error_word, own, pdl, s);
            }
            a.trace = slot(n++);
        }
    };
    auto produce = [&](QmvArgs &a, uint32_t index) {
        hooks = tp_producer_hooks(m->tp, index, per_token, tokens);
        a.exchange = &hooks;
        a.epilogue = kEpiPush;
        a.resid = nullptr;
    };
    for (uint32_t l = 0; l < c.layers; ++l) {
        auto &L = m->layers[l];
        QmvArgs a{};
        a.m = 1;
        a.io_type = STARK_B200_BF16;
        a.error_word = ctx->error_word;
        a.pdl = pdl;
        a.eps = c.eps;
        // qkv = W_qkv rmsnorm(h)
        a.matrix = L.qkv;
        a.x = hcur;
        a.y = m->qkv;
        a.prologue = kProRmsNorm;
        a.norm_weight = L.attn_norm;
        a.norm_weight_bf16 = L.attn_norm_b16;
        a.epilogue = kEpiStore;
        a.trace = slot(n++);
        if (tp && l > 0) consume(a, 2u * l - 1u);
        if (consume_status != STARK_B200_OK) return consume_status;
        if ((st = qmv_launch(a, s)) != STARK_B200_OK) return st;
        a.exchange = nullptr;
        // attention with fused QK-norm, RoPE and KV append
        AttnArgs at{};
        at.qkv = m->qkv;
        at.out = m->attn;
        at.kv = L.kv;
        at.block_table = m->block_table;
        at.q_norm = L.q_norm;
        at.k_norm = L.k_norm;
        at.rope_cos = m->rope_cos;
        at.rope_sin = m->rope_sin;
        at.state = m->state;
        at.eps = c.eps;
        at.scale = 1.0f / sqrtf((float)kHeadDim);
        at.q_heads = c.q_heads;
        at.kv_heads = c.kv_heads;
        at.splits = m->attn_splits;
        at.scratch = m->attn_scratch;
        at.counters = m->attn_counters;
        at.error_word = ctx->error_word;
        at.pdl = pdl;
        at.trace = slot(n++);
        if ((st = attention_decode_launch(at, s)) != STARK_B200_OK) return st;
        // h = bf16(bf16(W_o attn) + h)
        a.matrix = L.o;
        a.x = m->attn;
        a.y = hcur;
        a.resid = hcur;
        a.prologue = kProPlain;
        a.epilogue = kEpiResidual;
        a.trace = slot(n++);
        if (tp) produce(a, 2u * l);
        if ((st = qmv_launch(a, s)) != STARK_B200_OK) return st;
        a.exchange = nullptr;
        // act = silu(gate) * up
        a.matrix = L.upgate;
        a.x = hcur;
        a.y = m->act;
        a.prologue = kProRmsNorm;
        a.norm_weight = L.mlp_norm;
        a.norm_weight_bf16 = L.mlp_norm_b16;
        a.epilogue = kEpiSwiGlu;
        a.roomy = true;  // followed by the down projection, then the next layer's qkv: no attention CTA to host
        a.trace = slot(n++);
        if (tp) consume(a, 2u * l);
        if (consume_status != STARK_B200_OK) return consume_status;
        if ((st = qmv_launch(a, s)) != STARK_B200_OK) return st;
        a.exchange = nullptr;
        // h = bf16(bf16(W_down act) + h)
        a.matrix = L.down;
        a.x = m->act;
        a.y = hcur;
        a.resid = hcur;
        a.prologue = kProPlain;
        a.epilogue = kEpiResidual;
        a.trace = slot(n++);
        if (tp) produce(a, 2u * l + 1u);
        if ((st = qmv_launch(a, s)) != STARK_B200_OK) return st;
    }
    if (full) {
        QmvArgs a{};
        a.m = 1;
        a.io_type = STARK_B200_BF16;
        a.error_word = ctx->error_word;
        a.pdl = pdl;
        a.eps = c.eps;
        a.matrix = m->lm_head;
        a.x = hcur;
        a.y = m->logits;
        a.prologue = kProRmsNorm;
        a.norm_weight = m->final_norm;
        a.norm_weight_bf16 = m->final_norm_b16;
        a.epilogue = kEpiLogits;
        a.roomy = true;
        a.partial_max = m->partial_max;
        a.partial_index = m->partial_index;
        uint32_t grid = 0;
        a.out_grid = &grid;
        a.trace = slot(n++);
        if (tp) consume(a, per_token - 1u);
        if (consume_status != STARK_B200_OK) return consume_status;
        if ((st = qmv_launch(a, s)) != STARK_B200_OK) return st;
        st = tp ? tp_argmax_finalize_launch(m->tp, tokens, m->partial_max, m->partial_index, grid,
                                            m->tp_vocab_offset, m->state, m->generated, ctx->error_word, pdl, s)
                : argmax_finalize_launch(m->partial_max, m->partial_index, grid, m->state, m->generated, true, pdl, s);
        if (st != STARK_B200_OK) return st;
        n += 1;
    } else {
        st = tp ? tp_ingest_advance_launch(m->tp, per_token - 1u, per_token, tokens, m->state, m->pending,
                                           ctx->error_word, pdl, s)
                : ingest_advance_launch(m->state, m->pending, pdl, s);
        if (st != STARK_B200_OK) return st;
        n += 1;
    }
    if (launches) *launches = n;
    return STARK_B200_OK;
}

// Persistent-kernel path: builds the operator lists (full token / cache-only prompt row).
static stark_b200_status build_mega(Model *m) {
    const auto &c = m->cfg;
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    int sms = 0;
    SB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, m->device));
    m->mega_grid = (uint32_t)sms;
    m->mega_splits = std::max(1u, std::min<uint32_t>(kMaxAttnSplits, m->mega_grid / c.kv_heads));
    std::vector<MegaOp> ops;
    uint32_t max_columns = 0, stage_capacity = 0;
    auto gemv = [&](const QMatrix *w, const uint16_t *x, uint16_t *y, uint32_t pro, const float *nw, uint32_t epi,
                    const uint16_t *resid, uint32_t dep) {
        MegaOp o{};
        o.type = kOpGemv;
        o.dep = dep;
        o.participants = m->mega_grid;
        o.w = w->data;
        o.x = x;
        o.y = y;
        o.norm_weight = nw;
        o.resid = resid;
        o.rows = w->rows;
        o.row_tiles = w->row_tiles;
        o.groups = w->groups;
        bool pred = false;
        qmv_pick_stage(w->groups, &o.stage_records, &o.rpw, &pred);
        // the persistent kernel has 16 consumer warps: records per warp and raggedness follow from that
        o.rpw = (o.stage_records + 15u) / 16u;
        o.pred = (o.stage_records % 16u != 0u) ? 1u : 0u;
        o.stages_per_tile = w->groups / o.stage_records;
        o.pair_halves = w->pair_halves;
        o.unit_tiles = epi == kEpiSwiGlu ? 2u : 1u;
        o.prologue = pro;
        o.epilogue = epi;
        max_columns = std::max(max_columns, w->columns);
        stage_capacity = std::max(stage_capacity, (o.stage_records * kA4RecordBytes + 127u) & ~127u);
        ops.push_back(o);
        return (uint32_t)ops.size() - 1u;
    };
    MegaOp e{};
    e.type = kOpEmbed;
    e.dep = 0xffffffffu;
    e.participants = 1;
    ops.push_back(e);
    uint32_t last = 0;
    for (uint32_t l = 0; l < c.layers; ++l) {
        auto &L = m->layers[l];
        const uint32_t q = gemv(L.qkv, m->h, m->qkv, kProRmsNorm, L.attn_norm, kEpiStore, nullptr, last);
        MegaOp ap{};
        ap.type = kOpAttnPartial;
        ap.dep = q;
        ap.participants = c.kv_heads * m->mega_splits;
        ap.keys = L.kv.keys;
        ap.values = L.kv.values;
        ap.q_norm = L.q_norm;
        ap.k_norm = L.k_norm;
        ops.push_back(ap);
        MegaOp am{};
        am.type = kOpAttnMerge;
        am.dep = (uint32_t)ops.size() - 1u;
        am.participants = c.kv_heads;
        ops.push_back(am);
        const uint32_t o = gemv(L.o, m->attn, m->h, kProPlain, nullptr, kEpiResidual, m->h, (uint32_t)ops.size() - 1u);
        const uint32_t u = gemv(L.upgate, m->h, m->act, kProRmsNorm, L.mlp_norm, kEpiSwiGlu, nullptr, o);
        last = gemv(L.down, m->act, m->h, kProPlain, nullptr, kEpiResidual, m->h, u);
    }
    std::vector<MegaOp> ingest = ops;
    const uint32_t head = gemv(m->lm_head, m->h, m->logits, kProRmsNorm, m->final_norm, kEpiLogits, nullptr, last);
    MegaOp fin{};
    fin.type = kOpFinalize;
    fin.dep = head;
    fin.participants = 1;
    ops.push_back(fin);
    MegaOp adv{};
    adv.type = kOpIngestAdvance;
    adv.dep = last;
    adv.participants = 1;
    ingest.push_back(adv);
    if (c.kv_heads * m->mega_splits > m->mega_grid || c.kv_heads > m->mega_grid) return STARK_B200_UNSUPPORTED;

    stark_b200_status st;
    if ((st = dmalloc(&m->mega_ops, ops.size())) != STARK_B200_OK) return st;
    if ((st = dmalloc(&m->mega_ingest_ops, ingest.size())) != STARK_B200_OK) return st;
    if ((st = dmalloc(&m->mega_done, ops.size() + 1)) != STARK_B200_OK) return st;
    if ((st = dmalloc(&m->mega_scratch, attention_scratch_floats(c.q_heads, c.kv_heads, m->mega_splits))) != STARK_B200_OK)
        return st;
    SB_CUDA(cudaMemcpy(m->mega_ops, ops.data(), ops.size() * sizeof(MegaOp), cudaMemcpyHostToDevice));
    SB_CUDA(cudaMemcpy(m->mega_ingest_ops, ingest.data(), ingest.size() * sizeof(MegaOp), cudaMemcpyHostToDevice));
    SB_CUDA(cudaMemset(m->mega_done, 0, (ops.size() + 1) * sizeof(unsigned long long)));
    m->mega_num_ops = (uint32_t)ops.size();
    m->mega_num_ingest_ops = (uint32_t)ingest.size();

    MegaParams p{};
    p.stage_capacity = stage_capacity;
    p.max_columns = max_columns;
    uint32_t stages = 8;
    while (stages > 2 && mega_smem_bytes(stages, stage_capacity, max_columns) > 225u * 1024u) --stages;
    p.num_stages = stages;
    m->mega_smem = mega_smem_bytes(stages, stage_capacity, max_columns);
    if (m->mega_smem > 227u * 1024u) return STARK_B200_UNSUPPORTED;
    p.state = m->state;
    p.done = m->mega_done;
    p.embed = m->embed->data;
    p.embed_rows = m->embed->rows;
    p.embed_columns = m->embed->columns;
    p.h = m->h;
    p.qkv = m->qkv;
    p.attn = m->attn;
    p.block_table = m->block_table;
    p.rope_cos = m->rope_cos;
    p.rope_sin = m->rope_sin;
    p.attn_scratch = m->mega_scratch;
    p.eps = c.eps;
    p.attn_scale = 1.0f / sqrtf((float)kHeadDim);
    p.q_heads = c.q_heads;
    p.kv_heads = c.kv_heads;
    p.attn_splits = m->mega_splits;
    p.partial_max = m->partial_max;
    p.partial_index = m->partial_index;
    p.generated = m->generated;
    p.pending = m->pending;
    p.error_word = ctx->error_word;
    p.trace = m->trace;
    m->mega_full = p;
    m->mega_full.ops = m->mega_ops;
    m->mega_full.num_ops = m->mega_num_ops;
    m->mega_ingest = p;
    m->mega_ingest.ops = m->mega_ingest_ops;
    m->mega_ingest.num_ops = m->mega_num_ingest_ops;
    return STARK_B200_OK;
}

// One token on the model's stream: the recorded launch sequence, or the persistent kernel.
static stark_b200_status launch_token(Model *m, bool full) {
    if (m->use_mega) {
        SB_CUDA(cudaMemsetAsync(m->mega_done, 0, (m->mega_num_ops + 1u) * sizeof(unsigned long long), m->stream));
        return mega_launch(full ? m->mega_full : m->mega_ingest, m->mega_grid, m->mega_smem, m->stream);
    }
    SB_CUDA(cudaGraphLaunch(full ? m->step_graph : m->ingest_graph, m->stream));
    return STARK_B200_OK;
}

static stark_b200_status capture(Model *m, bool full, cudaGraphExec_t *exec, uint32_t *launches) {
    SB_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
    stark_b200_status st = issue_token(m, full, launches);
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(m->stream, &g);
    if (st != STARK_B200_OK) {
        if (g) cudaGraphDestroy(g);
        return st;
    }
    if (e != cudaSuccess) return cuda_status(e);
    e = cudaGraphInstantiate(exec, g, 0);
    cudaGraphDestroy(g);
    return cuda_status(e);
}

stark_b200_status model_tp_init(Model *m, uint32_t rank, uint32_t size, uint32_t vocab_offset, uint32_t vocab_total,
                                uint8_t *handle_out) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the interface");
    if (m->finalized || m->tp_local) return STARK_B200_INVALID_STATE;
    if (size < 2u || size > kMaxTpRanks || rank >= size || m->cfg.tied || m->cfg.hidden % 4u != 0 ||
        (uint64_t)vocab_offset + m->cfg.vocab > vocab_total)
        return STARK_B200_INVALID_ARGUMENT;
    const size_t bytes = tp_region_bytes(m->cfg.hidden);
    SB_CUDA(cudaMalloc(&m->tp_local, bytes));
    SB_CUDA(cudaMemset(m->tp_local, 0, bytes));
    stark_b200_status st = dmalloc(&m->tp_seq, 4);
    if (st != STARK_B200_OK) return st;
    SB_CUDA(cudaMalloc(&m->tp_staged, qmv_staged_bytes(m->cfg.hidden)));
    SB_CUDA(cudaMemset(m->tp_staged, 0, qmv_staged_bytes(m->cfg.hidden)));
    SB_CUDA(cudaMemset(m->tp_seq, 0, 16u));
    SB_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t handle;
    SB_CUDA(cudaIpcGetMemHandle(&handle, m->tp_local));
    memcpy(handle_out, &handle, 64);
    m->tp.rank = rank;
    m->tp.size = size;
    m->tp.hidden = m->cfg.hidden;
    m->tp.wait_ns = kDefaultPeerWaitNs;
    m->tp.base[rank] = m->tp_local;
    m->tp_vocab_offset = vocab_offset;
    m->tp_vocab_total = vocab_total;
    return STARK_B200_OK;
}

stark_b200_status model_tp_connect(Model *m, const uint8_t *handles) {
    if (m->finalized || !m->tp_local || m->tp_connected) return STARK_B200_INVALID_STATE;
    for (uint32_t r = 0; r < m->tp.size; ++r) {
        if (r == m->tp.rank) continue;
        cudaIpcMemHandle_t handle;
        memcpy(&handle, handles + (size_t)r * 64u, 64);
        void *p = nullptr;
        SB_CUDA(cudaIpcOpenMemHandle(&p, handle, cudaIpcMemLazyEnablePeerAccess));
        m->tp.base[r] = static_cast<uint8_t *>(p);
    }
    m->tp_connected = true;
    return STARK_B200_OK;
}

stark_b200_status model_tp_rows_init(Model *m, uint8_t *handle_out) {
    if (m->finalized || !m->tp_local || m->tp_rows_local || m->tp_stand_ins || m->chunk_h) return STARK_B200_INVALID_STATE;
    const auto &c = m->cfg;
    const size_t bytes = tp_rows_region_bytes(kPrefillBatchRows, c.hidden, (size_t)c.q_heads * m->tp.size * kHeadDim,
                                              (size_t)c.inter * m->tp.size);
    SB_CUDA(cudaMalloc(&m->tp_rows_local, bytes));
    SB_CUDA(cudaMemset(m->tp_rows_local, 0, kTpRowsHeaderBytes));
    stark_b200_status st = dmalloc(&m->tp_rows_arrive, 1);
    if (st != STARK_B200_OK) return st;
    SB_CUDA(cudaMemset(m->tp_rows_arrive, 0, 4u));
    SB_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t handle;
    SB_CUDA(cudaIpcGetMemHandle(&handle, m->tp_rows_local));
    memcpy(handle_out, &handle, 64);
    m->tp_rows.rank = m->tp.rank;
    m->tp_rows.size = m->tp.size;
    m->tp_rows.base[m->tp.rank] = m->tp_rows_local;
    return STARK_B200_OK;
}

stark_b200_status model_tp_rows_connect(Model *m, const uint8_t *handles) {
    if (m->finalized || !m->tp_rows_local || m->tp_rows_connected) return STARK_B200_INVALID_STATE;
    for (uint32_t r = 0; r < m->tp_rows.size; ++r) {
        if (r == m->tp_rows.rank) continue;
        cudaIpcMemHandle_t handle;
        memcpy(&handle, handles + (size_t)r * 64u, 64);
        void *p = nullptr;
        SB_CUDA(cudaIpcOpenMemHandle(&p, handle, cudaIpcMemLazyEnablePeerAccess));
        m->tp_rows.base[r] = static_cast<uint8_t *>(p);
    }
    m->tp_rows_connected = true;
    return STARK_B200_OK;
}

// Between init and finalize: how long this rank's kernels wait for a peer (the value is part of the recorded
// launch sequences).
stark_b200_status model_tp_set_wait(Model *m, uint64_t nanoseconds) {
    if (m->finalized || !m->tp_local) return STARK_B200_INVALID_STATE;
    if (nanoseconds < 1000ull || nanoseconds > 600000000000ull) return STARK_B200_INVALID_ARGUMENT;
    m->tp.wait_ns = nanoseconds;
    return STARK_B200_OK;
}

// Connects the rank to peers that never answer: every other rank's region is a zeroed local allocation that
// nobody writes.  The rank's own pushes land there harmlessly; its waits for the peers' packets run out after
// the wait limit and surface as a device failure.  This is how the bounded wait is exercised on one GPU without
// hanging or faulting anything.
stark_b200_status model_tp_connect_unanswered(Model *m) {
    if (m->finalized || !m->tp_local || m->tp_connected) return STARK_B200_INVALID_STATE;
    const size_t bytes = tp_region_bytes(m->cfg.hidden);
    for (uint32_t r = 0; r < m->tp.size; ++r) {
        if (r == m->tp.rank) continue;
        uint8_t *p = nullptr;
        SB_CUDA(cudaMalloc(&p, bytes));
        SB_CUDA(cudaMemset(p, 0, bytes));
        m->tp.base[r] = p;
    }
    m->tp_connected = true;
    m->tp_stand_ins = true;
    return STARK_B200_OK;
}

stark_b200_status model_finalize(Model *m) {
    if (m->finalized) return STARK_B200_INVALID_STATE;
    if (!m->embed || !m->lm_head || !m->final_norm) return STARK_B200_INVALID_STATE;
    if (m->tp.size > 1u && !m->tp_connected) return STARK_B200_INVALID_STATE;
    for (auto &L : m->layers)
        if (!L.qkv || !L.o || !L.upgate || !L.down || !L.attn_norm || !L.mlp_norm || !L.q_norm || !L.k_norm)
            return STARK_B200_INVALID_STATE;
    // One eager pass first (function attributes and lazily created library state must exist before
    // a recording), on a scratch position; then record both sequences.
    stark_b200_status st = model_reset(m);
    if (st != STARK_B200_OK) return st;
    // Tensor parallel: this first pass is where every rank's kernels are loaded, and on a machine that has not run
    // the library yet one rank can take seconds longer over that than another.  That is start-up skew, not a peer
    // that left: the first pass waits a minute for its peers; the recorded sequences keep the configured limit.
    const unsigned long long configured_wait = m->tp.wait_ns;
    if (m->tp.size > 1u && !m->tp_stand_ins) m->tp.wait_ns = std::max<unsigned long long>(configured_wait, 60000000000ull);
    st = issue_token(m, true, nullptr);
    if (st == STARK_B200_OK) st = issue_token(m, false, nullptr);
    m->tp.wait_ns = configured_wait;
    if (st != STARK_B200_OK) return st;
    SB_CUDA(cudaStreamSynchronize(m->stream));
    if ((st = capture(m, true, &m->step_graph, &m->step_launches)) != STARK_B200_OK) return st;
    if ((st = capture(m, false, &m->ingest_graph, &m->ingest_launches)) != STARK_B200_OK) return st;
    if (const char *e = getenv("STARK_B200_MEGA")) m->use_mega = e[0] == '1' && m->tp.size <= 1u;
    if (m->use_mega) {
        if (m->trace) {  // one slot per operator instead of one per launch
            cudaFree(m->trace);
            m->trace = nullptr;
            m->trace_slots = 4u + 6u * m->cfg.layers;
            if ((st = dmalloc(&m->trace, m->trace_slots)) != STARK_B200_OK) return st;
        }
        if ((st = build_mega(m)) != STARK_B200_OK) return st;
        m->step_launches = 1;
        m->ingest_launches = 1;
    }
    if ((st = mtp_finalize(m)) != STARK_B200_OK) return st;
    m->finalized = true;
    return model_reset(m);
}

// Records both launch sequences again with the current launch-shape settings.  Cache and position are kept.
stark_b200_status model_recapture(Model *m) {
    if (!m->finalized || m->fenced) return STARK_B200_INVALID_STATE;
    if (m->use_mega) return STARK_B200_UNSUPPORTED;
    SB_CUDA(cudaStreamSynchronize(m->stream));
    m->attn_splits = tunables().attn_splits ? tunables().attn_splits : default_attn_splits(m->cfg.kv_heads);
    // one eager pass on a scratch copy of the step state (first use of a kernel instance sets its attributes)
    StepState saved;
    SB_CUDA(cudaMemcpy(&saved, m->state, sizeof(StepState), cudaMemcpyDeviceToHost));
    stark_b200_status st;
    if ((st = issue_token(m, true, nullptr)) != STARK_B200_OK) return st;
    if ((st = issue_token(m, false, nullptr)) != STARK_B200_OK) return st;
    SB_CUDA(cudaStreamSynchronize(m->stream));
    SB_CUDA(cudaMemcpy(m->state, &saved, sizeof(StepState), cudaMemcpyHostToDevice));
    cudaGraphExec_t step = nullptr, ingest = nullptr;
    uint32_t step_n = 0, ingest_n = 0;
    if ((st = capture(m, true, &step, &step_n)) != STARK_B200_OK) return st;
    if ((st = capture(m, false, &ingest, &ingest_n)) != STARK_B200_OK) {
        cudaGraphExecDestroy(step);
        return st;
    }
    cudaGraphExecDestroy(m->step_graph);
    cudaGraphExecDestroy(m->ingest_graph);
    m->step_graph = step;
    m->ingest_graph = ingest;
    m->step_launches = step_n;
    m->ingest_launches = ingest_n;
    m->has_logits = false;
    return STARK_B200_OK;
}

stark_b200_status model_reset(Model *m) {
    SB_CUDA(cudaMemsetAsync(m->state, 0, sizeof(StepState), m->stream));
    SB_CUDA(cudaMemsetAsync(m->attn_counters, 0, m->cfg.kv_heads * 4, m->stream));
    if (m->mega_done)
        SB_CUDA(cudaMemsetAsync(m->mega_done, 0, (m->mega_num_ops + 1u) * sizeof(unsigned long long), m->stream));
    SB_CUDA(cudaStreamSynchronize(m->stream));
    m->position = 0;
    m->has_logits = false;
    return mtp_reset(m);
}

stark_b200_status model_rewind(Model *m, uint64_t position) {
    if (position > m->position) return STARK_B200_INVALID_ARGUMENT;
    // the draft head's cache would need the hidden row before the cut, which is not kept
    if (m->mtp.enabled && position != 0) return STARK_B200_UNSUPPORTED;
    if (m->mtp.enabled) mtp_reset(m);
    const uint32_t pos = (uint32_t)position;
    SB_CUDA(cudaMemcpyAsync(&m->state->position, &pos, 4, cudaMemcpyHostToDevice, m->stream));
    SB_CUDA(cudaStreamSynchronize(m->stream));
    m->position = position;
    m->has_logits = false;
    return STARK_B200_OK;
}

// Feeds `count` tokens; the last one runs the full sequence so that logits and the greedy token
// are available afterwards (hybrid::Model: ingest all but the last, then step the last;
// crates/stark-score/src/scoring.rs:453-489).
stark_b200_status model_prefill(Model *m, const uint32_t *ids, size_t count) {
    if (!m->finalized || m->fenced || m->mtp.open_rows) return STARK_B200_INVALID_STATE;
    if (count == 0) return STARK_B200_INVALID_ARGUMENT;
    if (m->position + count > m->cfg.context_tokens) return STARK_B200_CONTEXT_LIMIT;
    for (size_t i = 0; i < count; ++i)
        if (ids[i] >= input_vocab(m)) return STARK_B200_INVALID_ARGUMENT;
    // All rows but the last only fill the cache: enough of them go through the batched path (tensor-core
    // contraction over whole chunks), after which the last row is an ordinary token at its position.
    const bool batched = tunables().prefill_batch && model_batched_prefill_ready(m);
    if (m->mtp.enabled && (!batched || (m->position > 0 && !m->mtp.has_pending))) return STARK_B200_UNSUPPORTED;
    if (batched && (m->mtp.enabled || count - 1 >= tunables().prefill_min_rows)) {
        if (m->mtp.enabled && m->position > 0) {
            // a continued prompt: the pair (first new token, hidden of the last row so far) enters the head's cache
            SB_CUDA(cudaMemcpyAsync(m->chunk_tokens, ids, 4, cudaMemcpyHostToDevice, m->stream));
            stark_b200_status ps = mtp_prime_continue(m);
            if (ps != STARK_B200_OK) return ps;
        }
        stark_b200_status bs = model_prefill_batched(m, ids, count - 1, count);
        if (bs == STARK_B200_CANCELLED) {
            m->cancel_requested = false;
            cudaStreamSynchronize(m->stream);
            model_reset(m);
            return bs;
        }
        if (bs != STARK_B200_OK) return bs;
        StepState last{};
        last.position = (uint32_t)(m->position + count - 1);
        last.token = ids[count - 1];
        SB_CUDA(cudaMemcpyAsync(m->state, &last, sizeof(last), cudaMemcpyHostToDevice, m->stream));
        stark_b200_status ls = launch_token(m, true);
        if (ls != STARK_B200_OK) return ls;
        m->position += count;
        m->has_logits = true;
        m->launches_issued += m->step_launches;
        return mtp_after_prompt(m);
    }
    // pending[0 .. count-2] = ids[1 ..]; the ingest-advance kernel pops one per row
    if (count > 1) SB_CUDA(cudaMemcpyAsync(m->pending, ids + 1, (count - 1) * 4, cudaMemcpyHostToDevice, m->stream));
    StepState hs{};
    hs.position = (uint32_t)m->position;
    hs.token = ids[0];
    hs.next_token = 0;
    hs.cursor = 0;
    SB_CUDA(cudaMemcpyAsync(m->state, &hs, sizeof(hs), cudaMemcpyHostToDevice, m->stream));
    for (size_t i = 0; i + 1 < count; ++i) {
        if (m->cancel_requested) {
            m->cancel_requested = false;
            cudaStreamSynchronize(m->stream);
            m->fenced = false;
            model_reset(m);
            return STARK_B200_CANCELLED;
        }
        stark_b200_status ls = launch_token(m, false);
        if (ls != STARK_B200_OK) return ls;
    }
    {
        stark_b200_status ls = launch_token(m, true);
        if (ls != STARK_B200_OK) return ls;
    }
    m->position += count;
    m->has_logits = true;
    m->launches_issued += (count - 1) * m->ingest_launches + m->step_launches;
    return STARK_B200_OK;
}

stark_b200_status model_step(Model *m, uint32_t token, bool chained) {
    if (!m->finalized || m->fenced || m->mtp.open_rows) return STARK_B200_INVALID_STATE;
    if (m->position + 1 > m->cfg.context_tokens) return STARK_B200_CONTEXT_LIMIT;
    if (!chained) {
        if (token >= input_vocab(m)) return STARK_B200_INVALID_ARGUMENT;
        SB_CUDA(cudaMemcpyAsync(&m->state->token, &token, 4, cudaMemcpyHostToDevice, m->stream));
    }
    {
        stark_b200_status ls = launch_token(m, true);
        if (ls != STARK_B200_OK) return ls;
    }
    m->position += 1;
    m->has_logits = true;
    m->launches_issued += m->step_launches;
    return STARK_B200_OK;
}

static stark_b200_status check_device_error(Model *m) {
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    uint32_t word = 0;
    SB_CUDA(cudaMemcpyAsync(&word, ctx->error_word, 4, cudaMemcpyDeviceToHost, m->stream));
    SB_CUDA(cudaStreamSynchronize(m->stream));
    if (word) {
        m->fenced = true;
        return STARK_B200_DEVICE_FAILURE;
    }
    return STARK_B200_OK;
}

stark_b200_status model_drain(Model *m) {
    cudaError_t e = cudaStreamSynchronize(m->stream);
    if (e != cudaSuccess) {
        m->fenced = true;
        return cuda_status(e);
    }
    return check_device_error(m);
}

stark_b200_status model_next_token(Model *m, uint32_t *out) {
    if (!m->has_logits) return STARK_B200_INVALID_STATE;
    SB_CUDA(cudaMemcpyAsync(m->host_state, m->state, sizeof(StepState), cudaMemcpyDeviceToHost, m->stream));
    SB_CUDA(cudaStreamSynchronize(m->stream));
    *out = m->host_state->next_token;
    return STARK_B200_OK;
}

stark_b200_status model_readout_bf16(Model *m, uint16_t *dst, size_t count) {
    if (!m->has_logits) return STARK_B200_INVALID_STATE;
    if (count != m->cfg.vocab) return STARK_B200_INVALID_ARGUMENT;
    SB_CUDA(cudaMemcpyAsync(m->host_logits, m->logits, count * 2, cudaMemcpyDeviceToHost, m->stream));
    SB_CUDA(cudaStreamSynchronize(m->stream));
    memcpy(dst, m->host_logits, count * 2);
    return STARK_B200_OK;
}

stark_b200_status model_readout_f32(Model *m, float *dst, size_t count) {
    if (!m->has_logits) return STARK_B200_INVALID_STATE;
    if (count != m->cfg.vocab) return STARK_B200_INVALID_ARGUMENT;
    SB_CUDA(cudaMemcpyAsync(m->host_logits, m->logits, count * 2, cudaMemcpyDeviceToHost, m->stream));
    SB_CUDA(cudaStreamSynchronize(m->stream));
    for (size_t i = 0; i < count; ++i) dst[i] = bf16_bits_to_f32(m->host_logits[i]);
    return STARK_B200_OK;
}

// Greedy decode of `steps` tokens chained on the device: the step sequence writes its own next
// input.  Token ids come back through one small device-to-host copy per step, all asynchronous;
// the host synchronises once at the end.
stark_b200_status model_generate_greedy(Model *m, uint32_t steps, uint32_t *out_tokens) {
    if (!m->finalized || m->fenced || !m->has_logits) return STARK_B200_INVALID_STATE;
    if (m->position + steps > m->cfg.context_tokens) return STARK_B200_CONTEXT_LIMIT;
    uint32_t *pinned = nullptr;
    SB_CUDA(cudaMallocHost(&pinned, (size_t)(steps + 1u) * 4u));
    // out[0] is the token sampled from the logits already present (the prompt's last row); the
    // rest are appended to the device-side list by each step and fetched in one copy at the end.
    const uint32_t window[2] = {0u, steps};
    cudaError_t e = cudaMemcpyAsync(&pinned[0], &m->state->next_token, 4, cudaMemcpyDeviceToHost, m->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&m->state->gen_cursor, window, 8, cudaMemcpyHostToDevice, m->stream);
    for (uint32_t i = 0; i < steps && e == cudaSuccess; ++i) {
        if (launch_token(m, true) != STARK_B200_OK) e = last_cuda_error() != cudaSuccess ? last_cuda_error() : cudaErrorUnknown;
    }
    if (e == cudaSuccess && steps)
        e = cudaMemcpyAsync(&pinned[1], m->generated, (size_t)steps * 4u, cudaMemcpyDeviceToHost, m->stream);
    const uint32_t closed[2] = {0u, 0u};
    if (e == cudaSuccess) e = cudaMemcpyAsync(&m->state->gen_cursor, closed, 8, cudaMemcpyHostToDevice, m->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    if (e == cudaSuccess) memcpy(out_tokens, pinned, (size_t)(steps + 1u) * 4u);
    cudaFreeHost(pinned);
    if (e != cudaSuccess) {
        m->fenced = true;
        return cuda_status(e);
    }
    m->position += steps;
    m->launches_issued += (uint64_t)steps * m->step_launches;
    return check_device_error(m);
}

// Copies out the timeline slots of the launches issued since the last call and re-arms them.
stark_b200_status model_read_trace(Model *m, unsigned long long *dst, size_t count) {
    if (!m->trace) return STARK_B200_UNSUPPORTED;
    if (count != (size_t)m->trace_slots * kTraceFields) return STARK_B200_INVALID_ARGUMENT;
    SB_CUDA(cudaStreamSynchronize(m->stream));
    SB_CUDA(cudaMemcpy(dst, m->trace, count * 8u, cudaMemcpyDeviceToHost));
    std::vector<TraceSlot> init(m->trace_slots, TraceSlot{~0ull, ~0ull, 0ull, 0ull, 0ull, 0ull});
    SB_CUDA(cudaMemcpy(m->trace, init.data(), count * 8u, cudaMemcpyHostToDevice));
    return STARK_B200_OK;
}

}  // namespace sb
