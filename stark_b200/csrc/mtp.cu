// Dense multi-token prediction: a one-layer draft head proposes tokens, the target verifies all of them in one
// (k + 1)-row pass on the tensor cores, the accepted rows stay in the caches and the rest is rewound.
// Follows the reference's round (crates/stark-engine/src/engine/language_model/dense_mtp.rs:786-886):
//   drafts  k x  head([token], hidden)  -> proposal; the head's normalized output is the next step's hidden
//   verify       target([pending, d1 .. dk]) -> k + 1 rows of logits and of normalized hidden
//   accept       row i confirms proposal i + 1 while the sampler's pick equals it; the first other pick ends the
//                round and becomes the next pending token
//   commit       target keeps 1 + accepted rows; the head keeps its first draft row and replays the accepted
//                proposals with the TARGET's hidden rows (cache only)
// Sampling here is greedy (draft = arg-max of the head, target = arg-max of the row), which reproduces plain
// greedy decoding token for token, or -- for timing with a fixed work mix -- an acceptance pattern given by the
// caller.  The verify rows' logits stay readable until the next round for a host-side sampler.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "model.cuh"
#include "prefill.cuh"
#include "tunables.cuh"

namespace sb {

namespace {

template <typename T>
stark_b200_status dalloc(T **p, size_t count) {
    *p = nullptr;
    SB_CUDA(cudaMalloc(p, count * sizeof(T)));
    return STARK_B200_OK;
}

ModelLayer &head_layer(Model *m) { return m->layers[m->cfg.layers]; }

// One draft step on m->stream: reads state->token / state->position of the head, appends to its cache, leaves
// the logits in m->logits, the greedy pick in the head's state (token := pick, position += 1) and in the
// generated list, and its normalized output in draft_in.
stark_b200_status issue_draft_step(Model *m) {
    const auto &c = m->cfg;
    MtpHead &h = m->mtp;
    ModelLayer &L = head_layer(m);
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    cudaStream_t s = m->stream;
    const bool pdl = false;
    stark_b200_status st;
    // [norm_e(embedding) ; norm_h(hidden)]
    if ((st = embedding_row_launch(m->embed, h.state, h.embedded, pdl, s)) != STARK_B200_OK) return st;
    if ((st = rmsnorm_rows_launch(h.embedded, h.embed_norm, h.joined, 1, c.hidden, c.eps, s)) != STARK_B200_OK) return st;
    if ((st = rmsnorm_rows_launch(h.draft_in, h.hidden_norm, h.joined + c.hidden, 1, c.hidden, c.eps, s)) != STARK_B200_OK) return st;
    QmvArgs a{};
    a.m = 1;
    a.io_type = STARK_B200_BF16;
    a.error_word = ctx->error_word;
    a.pdl = pdl;
    a.eps = c.eps;
    // fusion: [D, 2D] over the joined row
    a.matrix = h.fusion;
    a.x = h.joined;
    a.y = h.stream_h;
    a.prologue = kProPlain;
    a.epilogue = kEpiStore;
    if ((st = qmv_launch(a, s)) != STARK_B200_OK) return st;
    // the head's decoder layer, same operators as a target layer
    a.matrix = L.qkv;
    a.x = h.stream_h;
    a.y = m->qkv;
    a.prologue = kProRmsNorm;
    a.norm_weight = L.attn_norm;
    a.norm_weight_bf16 = L.attn_norm_b16;
    if ((st = qmv_launch(a, s)) != STARK_B200_OK) return st;
    AttnArgs at{};
    at.qkv = m->qkv;
    at.out = m->attn;
    at.kv = L.kv;
    at.block_table = m->block_table;
    at.q_norm = L.q_norm;
    at.k_norm = L.k_norm;
    at.rope_cos = m->rope_cos;
    at.rope_sin = m->rope_sin;
    at.state = h.state;
    at.eps = c.eps;
    at.scale = 1.0f / sqrtf((float)kHeadDim);
    at.q_heads = c.q_heads;
    at.kv_heads = c.kv_heads;
    at.splits = m->attn_splits;
    at.scratch = m->attn_scratch;
    at.counters = m->attn_counters;
    at.error_word = ctx->error_word;
    at.pdl = pdl;
    if ((st = attention_decode_launch(at, s)) != STARK_B200_OK) return st;
    a.matrix = L.o;
    a.x = m->attn;
    a.y = h.stream_h;
    a.resid = h.stream_h;
    a.prologue = kProPlain;
    a.norm_weight = nullptr;
    a.norm_weight_bf16 = nullptr;
    a.epilogue = kEpiResidual;
    if ((st = qmv_launch(a, s)) != STARK_B200_OK) return st;
    a.matrix = L.upgate;
    a.x = h.stream_h;
    a.y = m->act;
    a.resid = nullptr;
    a.prologue = kProRmsNorm;
    a.norm_weight = L.mlp_norm;
    a.norm_weight_bf16 = L.mlp_norm_b16;
    a.epilogue = kEpiSwiGlu;
    if ((st = qmv_launch(a, s)) != STARK_B200_OK) return st;
    a.matrix = L.down;
    a.x = m->act;
    a.y = h.stream_h;
    a.resid = h.stream_h;
    a.prologue = kProPlain;
    a.norm_weight = nullptr;
    a.norm_weight_bf16 = nullptr;
    a.epilogue = kEpiResidual;
    if ((st = qmv_launch(a, s)) != STARK_B200_OK) return st;
    // output norm: the next step's hidden input, and the row the shared read-out multiplies
    if ((st = rmsnorm_rows_launch(h.stream_h, h.out_norm, h.draft_in, 1, c.hidden, c.eps, s)) != STARK_B200_OK) return st;
    a.matrix = m->lm_head;
    a.x = h.draft_in;
    a.y = m->logits;
    a.resid = nullptr;
    a.epilogue = kEpiLogits;
    a.partial_max = m->partial_max;
    a.partial_index = m->partial_index;
    uint32_t grid = 0;
    a.out_grid = &grid;
    if ((st = qmv_launch(a, s)) != STARK_B200_OK) return st;
    // proposals are appended at chunk_tokens[1 ..]: chunk_tokens[0] is the round's pending token
    return argmax_finalize_launch(m->partial_max, m->partial_index, grid, h.state, m->chunk_tokens + 1, true, pdl, s);
}

// Cache-only rows of the head for `rows` pairs (tokens on the device, hidden rows [rows, D] normalized by the
// target's final norm) at the head's positions first_pos ..: fuse, layer norm, qkv, per-head norm + RoPE + append.
stark_b200_status head_cache_rows(Model *m, const uint32_t *tokens_device, const uint16_t *hidden_rows, uint32_t rows,
                                  uint32_t first_pos) {
    const auto &c = m->cfg;
    MtpHead &h = m->mtp;
    ModelLayer &L = head_layer(m);
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    cudaStream_t s = m->stream;
    stark_b200_status st;
    if ((st = embed_rows_launch(m->embed, tokens_device, rows, h.rows_e, s)) != STARK_B200_OK) return st;
    if ((st = rmsnorm_rows_launch(h.rows_e, h.embed_norm, h.rows_j, rows, c.hidden, c.eps, s, 0, 2u * c.hidden)) != STARK_B200_OK) return st;
    if ((st = rmsnorm_rows_launch(hidden_rows, h.hidden_norm, h.rows_j + c.hidden, rows, c.hidden, c.eps, s, 0, 2u * c.hidden)) != STARK_B200_OK) return st;
    GemmArgs g{};
    g.x_rows = kPrefillBatchRows;
    g.m = rows;
    g.error_word = ctx->error_word;
    g.w = h.fusion;
    g.x = h.rows_j;
    g.out = h.rows_e;  // the embedding rows are consumed: the fused rows take their place
    g.ld_out = c.hidden;
    g.epilogue = kEpiStore;
    if ((st = prefill_gemm_launch(g, s)) != STARK_B200_OK) return st;
    if ((st = rmsnorm_rows_launch(h.rows_e, L.attn_norm, h.rows_j, rows, c.hidden, c.eps, s)) != STARK_B200_OK) return st;
    g.w = L.qkv;
    g.x = h.rows_j;
    g.out = m->chunk_qkv;
    g.ld_out = (c.q_heads + 2u * c.kv_heads) * kHeadDim;
    if ((st = prefill_gemm_launch(g, s)) != STARK_B200_OK) return st;
    RopeAppendArgs ra{m->chunk_qkv, L.kv, m->block_table, L.q_norm, L.k_norm, m->rope_cos, m->rope_sin,
                      rows, first_pos, c.q_heads, c.kv_heads, c.eps};
    if ((st = rope_append_rows_launch(ra, s)) != STARK_B200_OK) return st;
    m->launches_issued += 7;
    return STARK_B200_OK;
}

}  // namespace

stark_b200_status mtp_create(Model *m) {
    const auto &c = m->cfg;
    MtpHead &h = m->mtp;
    h.enabled = true;
    stark_b200_status st;
    if ((st = dalloc(&h.state, 1)) != STARK_B200_OK) return st;
    SB_CUDA(cudaMemset(h.state, 0, sizeof(StepState)));
    if ((st = dalloc(&h.last_hidden, c.hidden)) != STARK_B200_OK) return st;
    if ((st = dalloc(&h.draft_in, c.hidden)) != STARK_B200_OK) return st;
    if ((st = dalloc(&h.joined, 2u * (size_t)c.hidden)) != STARK_B200_OK) return st;
    if ((st = dalloc(&h.embedded, c.hidden)) != STARK_B200_OK) return st;
    if ((st = dalloc(&h.stream_h, c.hidden)) != STARK_B200_OK) return st;
    if ((st = dalloc(&h.rows_e, (size_t)kPrefillBatchRows * c.hidden)) != STARK_B200_OK) return st;
    if ((st = dalloc(&h.rows_j, (size_t)kPrefillBatchRows * 2u * c.hidden)) != STARK_B200_OK) return st;
    if ((st = dalloc(&h.rows_hidden, (size_t)16u * c.hidden)) != STARK_B200_OK) return st;
    if ((st = dalloc(&h.rows_logits, (size_t)16u * c.vocab)) != STARK_B200_OK) return st;
    if ((st = dalloc(&h.rows_pick, 16)) != STARK_B200_OK) return st;
    SB_CUDA(cudaMallocHost(&h.host_words, 64 * sizeof(uint32_t)));
    return STARK_B200_OK;
}

void mtp_destroy(Model *m) {
    MtpHead &h = m->mtp;
    if (h.draft_graph) cudaGraphExecDestroy(h.draft_graph);
    qmatrix_free(h.fusion);
    cudaFree(h.embed_norm);
    cudaFree(h.hidden_norm);
    cudaFree(h.out_norm);
    cudaFree(h.state);
    cudaFree(h.last_hidden);
    cudaFree(h.draft_in);
    cudaFree(h.joined);
    cudaFree(h.embedded);
    cudaFree(h.stream_h);
    cudaFree(h.rows_e);
    cudaFree(h.rows_j);
    cudaFree(h.rows_hidden);
    cudaFree(h.rows_logits);
    cudaFree(h.rows_pick);
    if (h.host_words) cudaFreeHost(h.host_words);
}

// Called at the end of model_finalize: one eager draft step (kernel attributes), then the step is recorded.
stark_b200_status mtp_finalize(Model *m) {
    MtpHead &h = m->mtp;
    if (!h.enabled) return STARK_B200_OK;
    if (!h.fusion || !h.embed_norm || !h.hidden_norm || !h.out_norm) return STARK_B200_INVALID_STATE;
    if (h.fusion->rows != m->cfg.hidden || h.fusion->columns != 2u * m->cfg.hidden || m->tp.size > 1u || m->cfg.vocab % 128u != 0)
        return STARK_B200_UNSUPPORTED;
    stark_b200_status st = ensure_chunk_buffers(m);
    if (st != STARK_B200_OK) return st;
    SB_CUDA(cudaMemsetAsync(h.state, 0, sizeof(StepState), m->stream));
    SB_CUDA(cudaMemsetAsync(h.draft_in, 0, (size_t)m->cfg.hidden * 2u, m->stream));
    if ((st = issue_draft_step(m)) != STARK_B200_OK) return st;
    SB_CUDA(cudaStreamSynchronize(m->stream));
    SB_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
    st = issue_draft_step(m);
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(m->stream, &g);
    if (st != STARK_B200_OK) {
        if (g) cudaGraphDestroy(g);
        return st;
    }
    if (e != cudaSuccess) return cuda_status(e);
    e = cudaGraphInstantiate(&h.draft_graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return cuda_status(e);
    return mtp_reset(m);
}

stark_b200_status mtp_reset(Model *m) {
    MtpHead &h = m->mtp;
    if (!h.enabled) return STARK_B200_OK;
    SB_CUDA(cudaMemsetAsync(h.state, 0, sizeof(StepState), m->stream));
    h.position = 0;
    h.has_pending = false;
    h.verified_rows = 0;
    h.open_rows = 0;
    h.open_serial = false;
    return STARK_B200_OK;
}

stark_b200_status mtp_prime_rows(Model *m, uint32_t mrows, uint32_t pairs, uint32_t first_pos) {
    const auto &c = m->cfg;
    MtpHead &h = m->mtp;
    if (pairs == 0) return STARK_B200_OK;
    if (pairs > mrows || h.position != first_pos) return STARK_B200_INVALID_STATE;
    // normalized hidden of every row of the chunk (the target's final norm: dense_mtp.rs:262-266); chunk_x is
    // free once the layers are done
    stark_b200_status st = rmsnorm_rows_launch(m->chunk_h, m->final_norm, m->chunk_x, pairs, c.hidden, c.eps, m->stream);
    if (st != STARK_B200_OK) return st;
    // pair i = (token of row i + 1, hidden of row i): the tokens start one entry into the chunk's id list
    if ((st = head_cache_rows(m, m->chunk_tokens + 1, m->chunk_x, pairs, first_pos)) != STARK_B200_OK) return st;
    h.position += pairs;
    return STARK_B200_OK;
}

stark_b200_status mtp_prime_continue(Model *m) {
    MtpHead &h = m->mtp;
    if (h.position + 1 != m->position) return STARK_B200_INVALID_STATE;
    stark_b200_status st = head_cache_rows(m, m->chunk_tokens, h.last_hidden, 1, (uint32_t)h.position);
    if (st != STARK_B200_OK) return st;
    h.position += 1;
    h.has_pending = false;
    return STARK_B200_OK;
}

stark_b200_status mtp_after_prompt(Model *m) {
    MtpHead &h = m->mtp;
    if (!h.enabled) return STARK_B200_OK;
    // m->h holds the last row's final residual stream; the head's cache holds one row less than the target's
    if (h.position + 1 != m->position) return STARK_B200_INVALID_STATE;
    stark_b200_status st = rmsnorm_rows_launch(m->h, m->final_norm, h.last_hidden, 1, m->cfg.hidden, m->cfg.eps, m->stream);
    if (st != STARK_B200_OK) return st;
    h.has_pending = true;
    h.verified_rows = 0;
    return STARK_B200_OK;
}

// proposals == nullptr: the head drafts `drafts` tokens.  Otherwise the caller proposes them (tokens it copied from
// the request's own context: a prompt-lookup round, engine/hybrid/mtp_policy.rs `RoundPlan::Lookup`), no head
// step runs, and the head's cache gets the pending row written instead ("head advance").
stark_b200_status mtp_round(Model *m, uint32_t pending, uint32_t drafts, uint32_t policy, uint32_t accept_mask,
                            stark_b200_mtp_round_result *out, const uint32_t *proposals) {
    const auto &c = m->cfg;
    MtpHead &h = m->mtp;
    if (!h.enabled) return STARK_B200_UNSUPPORTED;
    if (!m->finalized || m->fenced || !h.has_pending) return STARK_B200_INVALID_STATE;
    if (drafts > kMaxMtpDrafts || pending >= c.vocab || policy > STARK_B200_MTP_HELD) return STARK_B200_INVALID_ARGUMENT;
    if (h.open_rows) return STARK_B200_INVALID_STATE;  // a held round has to be committed first
    if (m->position + drafts + 1u > c.context_tokens) return STARK_B200_CONTEXT_LIMIT;
    if (h.position + 1 != m->position) return STARK_B200_INVALID_STATE;
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    cudaStream_t s = m->stream;
    const uint32_t rows = drafts + 1u;
    const uint32_t prefix = (uint32_t)h.position;
    stark_b200_status st;

    if (drafts == 0) {
        // A round without proposals is one ordinary token: the recorded one-token sequence (every launch a
        // programmatic dependent of the one before) instead of a one-row pass of the several-rows kernels.  The
        // head's cache gets the pair (pending, previous hidden) first, while that hidden row is still there.
        SB_CUDA(cudaMemcpyAsync(m->chunk_tokens, &pending, 4, cudaMemcpyHostToDevice, s));
        if ((st = head_cache_rows(m, m->chunk_tokens, h.last_hidden, 1, prefix)) != STARK_B200_OK) return st;
        if ((st = model_step(m, pending, false)) != STARK_B200_OK) return st;
        if ((st = rmsnorm_rows_launch(m->h, m->final_norm, h.last_hidden, 1, c.hidden, c.eps, s)) != STARK_B200_OK) return st;
        SB_CUDA(cudaMemcpyAsync(h.rows_logits, m->logits, (size_t)c.vocab * 2u, cudaMemcpyDeviceToDevice, s));
        SB_CUDA(cudaMemcpyAsync(h.host_words, &m->state->next_token, 4, cudaMemcpyDeviceToHost, s));
        SB_CUDA(cudaMemcpyAsync(h.host_words + 32, ctx->error_word, 4, cudaMemcpyDeviceToHost, s));
        const cudaError_t se = cudaStreamSynchronize(s);
        if (se != cudaSuccess || h.host_words[32]) {
            m->fenced = true;
            return se != cudaSuccess ? cuda_status(se) : STARK_B200_DEVICE_FAILURE;
        }
        if (h.host_words[0] >= c.vocab) return STARK_B200_DEVICE_FAILURE;  // a non-finite row
        const uint32_t picked = h.host_words[0];
        h.host_words[0] = pending;  // the committed input, where a held round's commit looks for it
        h.position = prefix + 1u;
        h.verified_rows = 1;
        if (policy == STARK_B200_MTP_HELD) {  // the caller samples from row 0 and closes the round with mtp_commit(0, token)
            h.open_rows = 1;
            h.open_serial = true;
            h.open_prefix = prefix;
        }
        memset(out->tokens, 0, sizeof(out->tokens));
        out->count = 1;
        out->accepted = 0;
        out->proposed = 0;
        out->next_pending = picked;
        out->tokens[0] = pending;
        out->position = m->position;
        return STARK_B200_OK;
    }

    // ---- drafts, chained on the device: state.token = pending, proposals appended at chunk_tokens[1 ..]
    StepState hs{};
    hs.position = prefix;
    hs.token = pending;
    hs.gen_cursor = 0;
    hs.gen_capacity = drafts;
    SB_CUDA(cudaMemcpyAsync(h.state, &hs, sizeof(hs), cudaMemcpyHostToDevice, s));
    SB_CUDA(cudaMemcpyAsync(m->chunk_tokens, &pending, 4, cudaMemcpyHostToDevice, s));
    if (proposals) {
        for (uint32_t d = 0; d < drafts; ++d)
            if (proposals[d] >= c.vocab) return STARK_B200_INVALID_ARGUMENT;
        // pageable host memory: the copy is staged before the call returns, the caller's array may go away
        if (drafts) SB_CUDA(cudaMemcpyAsync(m->chunk_tokens + 1, proposals, (size_t)drafts * 4u, cudaMemcpyHostToDevice, s));
    } else {
        SB_CUDA(cudaMemcpyAsync(h.draft_in, h.last_hidden, (size_t)c.hidden * 2u, cudaMemcpyDeviceToDevice, s));
        for (uint32_t d = 0; d < drafts; ++d) SB_CUDA(cudaGraphLaunch(h.draft_graph, s));
        m->launches_issued += 12ull * drafts;
    }

    // ---- verify: the target over [pending, d1 .. dk] at its own positions; logits and hidden of every row
    if ((st = model_rows_pass(m, m->chunk_tokens, rows, (uint32_t)m->position)) != STARK_B200_OK) return st;
    if ((st = rmsnorm_rows_launch(m->chunk_h, m->final_norm, h.rows_hidden, rows, c.hidden, c.eps, s)) != STARK_B200_OK) return st;
    GemmArgs g{};
    g.w = m->lm_head;
    g.x = h.rows_hidden;
    g.x_rows = 16;
    g.m = rows;
    g.out = h.rows_logits;
    g.ld_out = c.vocab;
    g.epilogue = kEpiStore;
    g.error_word = ctx->error_word;
    if ((st = prefill_gemm_launch(g, s)) != STARK_B200_OK) return st;
    if ((st = argmax_rows_launch(h.rows_logits, rows, c.vocab, h.rows_pick, s)) != STARK_B200_OK) return st;
    m->launches_issued += 3;

    // ---- accept on the host: the proposals and the target's pick of every row in one small read-back
    SB_CUDA(cudaMemcpyAsync(h.host_words, m->chunk_tokens, (size_t)rows * 4u, cudaMemcpyDeviceToHost, s));
    SB_CUDA(cudaMemcpyAsync(h.host_words + 16, h.rows_pick, (size_t)rows * 4u, cudaMemcpyDeviceToHost, s));
    SB_CUDA(cudaMemcpyAsync(h.host_words + 32, ctx->error_word, 4, cudaMemcpyDeviceToHost, s));
    cudaError_t e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        m->fenced = true;
        return cuda_status(e);
    }
    if (h.host_words[32]) {  // a bounded wait ran out in one of the round's kernels
        m->fenced = true;
        return STARK_B200_DEVICE_FAILURE;
    }
    const uint32_t *inputs = h.host_words, *picks = h.host_words + 16;
    for (uint32_t i = 0; i < rows; ++i)
        if (picks[i] >= c.vocab) return STARK_B200_DEVICE_FAILURE;  // a non-finite row
    h.verified_rows = rows;
    h.open_rows = rows;
    h.open_prefix = prefix;
    h.open_head_advance = drafts == 0 || proposals != nullptr;
    if (policy == STARK_B200_MTP_HELD) {
        // the caller decides: every row's logits can be read now, mtp_commit closes the round
        memset(out->tokens, 0, sizeof(out->tokens));
        out->count = rows;
        out->accepted = 0;
        out->proposed = drafts;
        out->next_pending = picks[0];
        for (uint32_t i = 0; i < rows; ++i) out->tokens[i] = inputs[i];
        out->position = m->position;
        return STARK_B200_OK;
    }
    uint32_t accepted = 0;
    for (;;) {
        const bool has_proposal = accepted + 1u < rows;
        bool take = has_proposal && inputs[accepted + 1u] == picks[accepted];
        if (policy == STARK_B200_MTP_FORCED && has_proposal) take = ((accept_mask >> accepted) & 1u) != 0u;
        if (!take) break;
        ++accepted;
    }
    return mtp_commit(m, accepted, picks[accepted], out);
}

// Closes the round mtp_round left open (or finishes one it decided itself): the target keeps 1 + accepted rows, the
// head keeps its first draft row and replays the accepted proposals against the target's hidden rows.
stark_b200_status mtp_commit(Model *m, uint32_t accepted, uint32_t next_pending, stark_b200_mtp_round_result *out) {
    const auto &c = m->cfg;
    MtpHead &h = m->mtp;
    if (!h.enabled) return STARK_B200_UNSUPPORTED;
    if (!m->finalized || m->fenced || h.open_rows == 0) return STARK_B200_INVALID_STATE;
    if (accepted + 1u > h.open_rows || next_pending >= c.vocab) return STARK_B200_INVALID_ARGUMENT;
    cudaStream_t s = m->stream;
    stark_b200_status st;
    const uint32_t rows = h.open_rows, prefix = h.open_prefix;
    const uint32_t *inputs = h.host_words;
    h.open_rows = 0;
    if (h.open_serial) {  // a round without proposals already is one committed token
        h.open_serial = false;
        if (accepted != 0) return STARK_B200_INVALID_ARGUMENT;
        memset(out->tokens, 0, sizeof(out->tokens));
        out->count = 1;
        out->accepted = 0;
        out->proposed = 0;
        out->next_pending = next_pending;
        out->tokens[0] = inputs[0];
        out->position = m->position;
        return STARK_B200_OK;
    }
    const uint32_t count = accepted + 1u;
    m->position += count;
    const uint32_t pos32 = (uint32_t)m->position;
    SB_CUDA(cudaMemcpyAsync(&m->state->position, &pos32, 4, cudaMemcpyHostToDevice, s));
    h.position = prefix;
    if (h.open_head_advance) {
        // no draft step ran: the pair (pending, previous hidden) still has to enter the head's cache
        if ((st = head_cache_rows(m, m->chunk_tokens, h.last_hidden, 1, prefix)) != STARK_B200_OK) return st;
    }
    h.position = prefix + 1u;
    if (accepted) {
        if ((st = head_cache_rows(m, m->chunk_tokens + 1, h.rows_hidden, accepted, prefix + 1u)) != STARK_B200_OK) return st;
        h.position += accepted;
    }
    SB_CUDA(cudaMemcpyAsync(h.last_hidden, h.rows_hidden + (size_t)(count - 1u) * c.hidden, (size_t)c.hidden * 2u,
                            cudaMemcpyDeviceToDevice, s));
    m->has_logits = false;

    memset(out->tokens, 0, sizeof(out->tokens));
    out->count = count;
    out->accepted = accepted;
    out->proposed = rows - 1u;
    out->next_pending = next_pending;
    for (uint32_t i = 0; i < count; ++i) out->tokens[i] = inputs[i];
    out->position = m->position;
    return STARK_B200_OK;  // the commit's launches run on; the next round (or a drain) observes them
}

stark_b200_status mtp_readout_row_f32(Model *m, uint32_t row, float *dst, size_t count) {
    MtpHead &h = m->mtp;
    if (!h.enabled) return STARK_B200_UNSUPPORTED;
    if (row >= h.verified_rows) return STARK_B200_INVALID_STATE;
    if (count != m->cfg.vocab) return STARK_B200_INVALID_ARGUMENT;
    SB_CUDA(cudaMemcpyAsync(m->host_logits, h.rows_logits + (size_t)row * m->cfg.vocab, count * 2u, cudaMemcpyDeviceToHost,
                            m->stream));
    SB_CUDA(cudaStreamSynchronize(m->stream));
    for (size_t i = 0; i < count; ++i) dst[i] = bf16_bits_to_f32(m->host_logits[i]);
    return STARK_B200_OK;
}

}  // namespace sb
