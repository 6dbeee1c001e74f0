// Batched prompt ingest of the dense decoder: up to 4096 rows at a time through the tensor-core contraction and
// the row-wise operators, layer by layer, leaving the rows' keys and values in the paged cache exactly where the
// one-token path would have put them.  Mirrors the reference's prefill loop
// (crates/stark-engine/src/engine/language_model/stream/stream.rs:441-686: chunks of 1024 rows, each a batched
// pass over the layers; the prompt's last row then goes through the sampling pass).  The rows of a pass are
// independent, so the larger pass here changes no value.
#include <algorithm>
#include <cmath>

#include "model.cuh"
#include "prefill.cuh"
#include "tunables.cuh"

namespace sb {

namespace {

template <typename T>
stark_b200_status dmalloc_rows(T **p, size_t count) {
    *p = nullptr;
    SB_CUDA(cudaMalloc(p, count * sizeof(T)));
    return STARK_B200_OK;
}

// byte offsets of the three row buffers inside the rows region (tp.cuh)
size_t rows_region_h(const Model *) { return kTpRowsHeaderBytes; }
size_t rows_region_attn(const Model *m) { return rows_region_h(m) + (size_t)kPrefillBatchRows * m->cfg.hidden * 2u; }
size_t rows_region_act(const Model *m) {
    return rows_region_attn(m) + (size_t)kPrefillBatchRows * m->cfg.q_heads * m->tp.size * kHeadDim * 2u;
}

}  // namespace

stark_b200_status ensure_chunk_buffers(Model *m) {
    if (m->chunk_h) return STARK_B200_OK;
    const auto &c = m->cfg;
    const size_t rows = kPrefillBatchRows;
    const uint32_t qkv_n = (c.q_heads + 2u * c.kv_heads) * kHeadDim;
    stark_b200_status st;
    if ((st = dmalloc_rows(&m->chunk_tokens, rows + 8u)) != STARK_B200_OK) return st;
    if (m->tp_rows_local) {
        // whole rows of all ranks, inside the exported region: the peers store their column slices there
        m->chunk_h = reinterpret_cast<uint16_t *>(m->tp_rows_local + rows_region_h(m));
        m->chunk_act = reinterpret_cast<uint16_t *>(m->tp_rows_local + rows_region_act(m));
    } else {
        if ((st = dmalloc_rows(&m->chunk_h, rows * c.hidden)) != STARK_B200_OK) return st;
        if ((st = dmalloc_rows(&m->chunk_act, rows * c.inter)) != STARK_B200_OK) return st;
    }
    if ((st = dmalloc_rows(&m->chunk_x, rows * c.hidden)) != STARK_B200_OK) return st;
    if ((st = dmalloc_rows(&m->chunk_qkv, rows * qkv_n)) != STARK_B200_OK) return st;
    if ((st = dmalloc_rows(&m->chunk_attn, rows * c.q_heads * kHeadDim)) != STARK_B200_OK) return st;
    if ((st = dmalloc_rows(&m->rows_attn_partials, prefill_attention_partial_floats(c.q_heads, kPrefillAttnMaxSplits))) != STARK_B200_OK)
        return st;
    return STARK_B200_OK;
}

// Whether the batched path can take this model's prompt rows: one GPU, the recorded-launch token path, layer
// matrices whose rows fill whole 128-feature tiles (examined once, at first use).
bool model_batched_prefill_ready(Model *m) {
    if (m->prefill_state == 2u) return false;
    if (m->prefill_state == 1u) return true;
    m->prefill_state = 2u;
    if (m->use_mega) return false;
    const bool tp = m->tp.size > 1u;
    // tensor parallel: needs the rows region and the row cuts of o and down; otherwise rows take the token path
    if (tp && !m->tp_rows_connected) return false;
    for (auto &L : m->layers)  // the draft head's layer, if any, included
        for (QMatrix *q : {L.qkv, tp ? L.o_rows : L.o, L.upgate, tp ? L.down_rows : L.down}) {
            if (!q || q->rows % 128u != 0 || q->columns % 64u != 0) return false;
        }
    if (m->cfg.hidden > 12288u || ensure_chunk_buffers(m) != STARK_B200_OK) return false;
    m->prefill_state = 1u;
    return true;
}

// One chunk of rows whose token ids are already on the device, at cache positions first_pos .. first_pos + mrows:
// embedding, then every layer of the target.  Leaves the rows' final residual stream in m->chunk_h.
stark_b200_status model_rows_pass(Model *m, const uint32_t *tokens_device, uint32_t mrows, uint32_t first_pos) {
    const auto &c = m->cfg;
    DeviceContext *ctx = device_context();
    if (!ctx) return STARK_B200_DEVICE_FAILURE;
    if (mrows == 0 || mrows > kPrefillBatchRows) return STARK_B200_INVALID_ARGUMENT;
    cudaStream_t s = m->stream;
    const uint32_t qkv_n = (c.q_heads + 2u * c.kv_heads) * kHeadDim;
    const float scale = 1.0f / sqrtf((float)kHeadDim);
    stark_b200_status st;
    // the few-rows form of the attention adds a merge launch per layer (same rule as prefill_attention_launch)
    const bool split_rows = mrows <= 16u && std::min((first_pos + mrows - 1u) / kPageTokens + 1u,
                                                      std::min(kPrefillAttnMaxSplits, std::max(1u, 296u / c.kv_heads))) >= 2u;
    // a handful of rows: the several-rows matvec normalizes the rows in its own prologue
    const bool fused_norm = tunables().rows_matvec && qmv_multi_supports(m->layers[0].qkv, mrows, true) &&
                            qmv_multi_supports(m->layers[0].upgate, mrows, true);
    // Tensor parallel (tp.cuh): every rank holds whole rows of h; its contractions produce column slices -- of the
    // attention output, of the new h (o and down cut by output rows), of the gated activation -- which the ranks
    // then copy into one another's buffers.  Four gathers per layer.
    const bool tp = m->tp.size > 1u;
    const uint32_t ranks = tp ? m->tp.size : 1u, rank = tp ? m->tp.rank : 0u;
    const uint32_t attn_local = c.q_heads * kHeadDim, attn_width = attn_local * ranks, inter_total = c.inter * ranks;
    const uint32_t h_slice = c.hidden / ranks;
    uint16_t *attn_rows = tp ? reinterpret_cast<uint16_t *>(m->tp_rows_local + rows_region_attn(m)) : m->chunk_attn;
    // More than a handful of rows: the contraction's epilogue can store its tiles to the peers itself
    // (tp_rows_push 1: always, 0: never, 2: between two ranks only).  Measured on the 8B shape, 4 096 rows: with one
    // peer the stores ride under the contraction (55.8 ms a pass against 57.1 with the copy kernel); with three
    // peers they hold the CTA, and with it the SM, three times as long, and the copy kernel -- 592 CTAs that do
    // nothing else -- wins (41.2 ms against 43.7; pushing only from the one contraction of several waves: 43.1).
    const uint32_t push_mode = tp && mrows > kPrefillSmallRows ? tunables().tp_rows_push : 0u;
    const bool push = push_mode == 1u || (push_mode == 2u && ranks == 2u);
    auto peers_of = [&](GemmArgs &g, size_t region_offset) {  // the place of g.out in the other ranks' buffers
        g.peers = 0;
        if (!push) return;
        for (uint32_t r = 0; r < ranks; ++r)
            if (r != rank) g.peer_out[g.peers++] = reinterpret_cast<uint16_t *>(m->tp_rows.base[r] + region_offset);
    };
    uint32_t gathers = 0;
    // a rank group's first pass loads these kernels and allocates the row buffers: start-up skew between ranks is
    // given a minute, later passes the configured limit
    const unsigned long long rows_wait =
        m->tp_rows_ticket == 0 ? std::max<unsigned long long>(m->tp.wait_ns, 60000000000ull) : m->tp.wait_ns;
    auto gather = [&](const uint16_t *src, uint32_t src_ld, size_t dst_offset, uint32_t dst_ld, uint32_t column,
                      uint32_t width, bool own) -> stark_b200_status {
        m->tp_rows.wait_ns = rows_wait;
        TpGatherArgs ga{src, src_ld, dst_offset, dst_ld, column, width, mrows, own, ++m->tp_rows_ticket};
        ++gathers;
        return tp_rows_gather_launch(m->tp_rows, ga, m->tp_rows_arrive, ctx->error_word, s);
    };
    if ((st = embed_rows_launch(m->embed, tokens_device, mrows, m->chunk_h, s)) != STARK_B200_OK) return st;
    for (uint32_t l = 0; l < c.layers; ++l) {
        auto &L = m->layers[l];
        GemmArgs g{};
        g.x_rows = kPrefillBatchRows;
        g.m = mrows;
        g.error_word = ctx->error_word;
        // qkv = W_qkv rmsnorm(h)
        if (fused_norm) {
            QmvMultiArgs q{L.qkv, m->chunk_h, c.hidden, mrows, m->chunk_qkv, qkv_n, L.attn_norm, c.eps, kEpiStore,
                           ctx->error_word, true};
            if ((st = qmv_multi_launch(q, s)) != STARK_B200_OK) return st;
        } else {
            if ((st = rmsnorm_rows_launch(m->chunk_h, L.attn_norm, m->chunk_x, mrows, c.hidden, c.eps, s)) != STARK_B200_OK) return st;
            g.w = L.qkv;
            g.x = m->chunk_x;
            g.out = m->chunk_qkv;
            g.ld_out = qkv_n;
            g.epilogue = kEpiStore;
            if ((st = prefill_gemm_launch(g, s)) != STARK_B200_OK) return st;
        }
        // per-head norm, RoPE, cache append; causal attention over the cache
        RopeAppendArgs ra{m->chunk_qkv, L.kv, m->block_table, L.q_norm, L.k_norm, m->rope_cos, m->rope_sin,
                          mrows, first_pos, c.q_heads, c.kv_heads, c.eps};
        if ((st = rope_append_rows_launch(ra, s)) != STARK_B200_OK) return st;
        PrefillAttnArgs pa{m->chunk_qkv, L.kv, m->block_table, m->chunk_attn, mrows, first_pos, c.q_heads, c.kv_heads, scale};
        pa.partials = m->rows_attn_partials;
        pa.max_splits = kPrefillAttnMaxSplits;
        pa.num_blocks = m->num_blocks;
        if ((st = prefill_attention_launch(pa, s)) != STARK_B200_OK) return st;
        if (tp && (st = gather(m->chunk_attn, attn_local, rows_region_attn(m), attn_width, rank * attn_local, attn_local,
                               true)) != STARK_B200_OK)
            return st;
        // h = bf16(bf16(W_o attn) + h); tensor parallel: this rank's columns of h, in place, then gathered
        g.w = tp ? L.o_rows : L.o;
        g.x = attn_rows;
        g.out = m->chunk_h + (size_t)rank * h_slice;
        g.ld_out = c.hidden;
        g.epilogue = kEpiResidual;
        peers_of(g, rows_region_h(m) + (size_t)rank * h_slice * 2u);
        if ((st = prefill_gemm_launch(g, s)) != STARK_B200_OK) return st;
        g.peers = 0;
        if (tp && (st = gather(m->chunk_h + (size_t)rank * h_slice, c.hidden, rows_region_h(m), c.hidden, rank * h_slice,
                               push ? 0u : h_slice, false)) != STARK_B200_OK)
            return st;
        // act = silu(gate) * up
        uint16_t *act_slice = m->chunk_act + (size_t)rank * c.inter;  // this rank's columns of the whole rows
        if (fused_norm) {
            QmvMultiArgs q{L.upgate, m->chunk_h, c.hidden, mrows, act_slice, inter_total, L.mlp_norm, c.eps, kEpiSwiGlu,
                           ctx->error_word, true};
            if ((st = qmv_multi_launch(q, s)) != STARK_B200_OK) return st;
        } else {
            if ((st = rmsnorm_rows_launch(m->chunk_h, L.mlp_norm, m->chunk_x, mrows, c.hidden, c.eps, s)) != STARK_B200_OK) return st;
            g.w = L.upgate;
            g.x = m->chunk_x;
            g.out = act_slice;
            g.ld_out = inter_total;
            g.epilogue = kEpiSwiGlu;
            peers_of(g, rows_region_act(m) + (size_t)rank * c.inter * 2u);
            if ((st = prefill_gemm_launch(g, s)) != STARK_B200_OK) return st;
            g.peers = 0;
        }
        if (tp && (st = gather(act_slice, inter_total, rows_region_act(m), inter_total, rank * c.inter,
                               push ? 0u : c.inter, false)) != STARK_B200_OK)
            return st;
        // h = bf16(bf16(W_down act) + h)
        g.w = tp ? L.down_rows : L.down;
        g.x = m->chunk_act;
        g.out = m->chunk_h + (size_t)rank * h_slice;
        g.ld_out = c.hidden;
        g.epilogue = kEpiResidual;
        peers_of(g, rows_region_h(m) + (size_t)rank * h_slice * 2u);
        if ((st = prefill_gemm_launch(g, s)) != STARK_B200_OK) return st;
        g.peers = 0;
        if (tp && (st = gather(m->chunk_h + (size_t)rank * h_slice, c.hidden, rows_region_h(m), c.hidden, rank * h_slice,
                               push ? 0u : h_slice, false)) != STARK_B200_OK)
            return st;
    }
    m->launches_issued += 1u + (fused_norm ? 6u : 8u) * c.layers + (split_rows ? c.layers : 0u) + gathers;
    return STARK_B200_OK;
}

// Ingests `rows` prompt rows starting at position m->position (cache only: no logits).  The caller has checked
// ids and the context limit.  With a draft head loaded, every chunk also primes the head's cache with the pairs
// (next prompt token, this row's normalized hidden): dense_mtp.rs:462-584.
stark_b200_status model_prefill_batched(Model *m, const uint32_t *ids, size_t rows, size_t ids_total) {
    stark_b200_status st;
    for (size_t done = 0; done < rows; done += kPrefillBatchRows) {
        if (m->cancel_requested) return STARK_B200_CANCELLED;
        const uint32_t mrows = (uint32_t)std::min<size_t>(kPrefillBatchRows, rows - done);
        const uint32_t first_pos = (uint32_t)(m->position + done);
        // one extra id when there is one: the head's pairs need the token after each row
        const size_t upload = std::min<size_t>((size_t)mrows + 1u, ids_total - done);
        SB_CUDA(cudaMemcpyAsync(m->chunk_tokens, ids + done, upload * 4u, cudaMemcpyHostToDevice, m->stream));
        if ((st = model_rows_pass(m, m->chunk_tokens, mrows, first_pos)) != STARK_B200_OK) return st;
        if (m->mtp.enabled && (st = mtp_prime_rows(m, mrows, (uint32_t)(upload - 1u), first_pos)) != STARK_B200_OK) return st;
    }
    return STARK_B200_OK;
}

}  // namespace sb
