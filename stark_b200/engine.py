"""Host-side mirror of the reference's engine-level operator surface for the token loop.

``DenseModel`` follows ``hybrid::Model`` (crates/stark-engine/src/engine/hybrid/mod.rs:347-1428):
``load`` -> ``reset`` -> ``ingest_prefix`` / ``prefill`` -> ``step(token) -> logits`` with the same
argument meaning and error behaviour (invalid token or context overflow raise and leave the model
reset).  All arithmetic happens in ``libstark_b200.so``; this class only marshals.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import StarkB200Error, check


def _rows(t: dict, lo: int, hi: int) -> dict:
    """Rows [lo, hi) of a quantized matrix in the MLX layout (codes and planes are row-major)."""
    return dict(t, codes=t["codes"][lo:hi], scales=t["scales"][lo:hi], biases=t["biases"][lo:hi], n=hi - lo)


def _columns(t: dict, lo: int, hi: int) -> dict:
    """Columns [lo, hi) of a quantized matrix; the cut must fall on quantization-group boundaries."""
    g, per_word = t["group"], 32 // t["bits"]
    if lo % g or hi % g:
        raise ValueError("a column shard must consist of whole quantization groups")
    return dict(t, codes=t["codes"][:, lo // per_word:hi // per_word], scales=t["scales"][:, lo // g:hi // g],
                biases=t["biases"][:, lo // g:hi // g], k=hi - lo)


def _stack(parts: list) -> dict:
    return dict(parts[0], codes=np.concatenate([p["codes"] for p in parts]),
                scales=np.concatenate([p["scales"] for p in parts]),
                biases=np.concatenate([p["biases"] for p in parts]), n=sum(p["n"] for p in parts))


def vocab_shard(vocab: int, rank: int, ranks: int) -> tuple[int, int]:
    """Rows [lo, hi) of the read-out matrix owned by `rank`: equal runs of whole 16-row tiles, the
    last rank taking what is left."""
    per = -(-vocab // (16 * ranks)) * 16
    lo = min(vocab, rank * per)
    return lo, min(vocab, lo + per)


def shard_dense(cfg: dict, weights: dict, rank: int, ranks: int) -> tuple[dict, dict, int]:
    """This rank's share of a dense decoder under tensor parallelism.

    qkv and up||gate are cut by output rows (whole heads, the KV cache follows the KV heads), the o- and
    down-projections by input columns (whole quantization groups), the read-out by vocabulary rows; the
    embedding table and all norm vectors stay whole.  For batched prompt passes a rank also gets its output rows
    of the whole o- and down-projection (`o_rows`, `down_rows`: 1/ranks of each again).  Returns (local config, local weights, first
    vocabulary row of the read-out shard).  The reference runs on one device; this is how the same
    graph (crates/stark-engine/src/encodable_block/transformer_layer.rs:549-659) is spread over several.
    """
    from .artifact import row_major_planes
    weights = dict(weights, embed=row_major_planes(weights["embed"]), lm_head=row_major_planes(weights["lm_head"]),
                   layers=[dict(lw, **{k: row_major_planes(lw[k]) for k in ("qkv", "o", "upgate", "down")})
                           for lw in weights["layers"]])
    hq, hkv, hd, inter, hidden = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], cfg["inter"], cfg["hidden"]
    if hq % ranks or hkv % ranks or inter % (16 * ranks) or (inter // ranks) % 64:
        raise ValueError(f"{ranks} ranks do not divide heads {hq}/{hkv} or width {inter} into whole shards")
    ql, kl, il = hq // ranks, hkv // ranks, inter // ranks
    lo, hi = vocab_shard(cfg["vocab"], rank, ranks)
    if hi <= lo:
        raise ValueError("empty read-out shard")
    local = dict(cfg, q_heads=ql, kv_heads=kl, inter=il, vocab=hi - lo, tied=False, vocab_total=cfg["vocab"])
    k0, v0 = hq * hd, (hq + hkv) * hd
    layers = []
    for lw in weights["layers"]:
        qkv = _stack([_rows(lw["qkv"], rank * ql * hd, (rank + 1) * ql * hd),
                      _rows(lw["qkv"], k0 + rank * kl * hd, k0 + (rank + 1) * kl * hd),
                      _rows(lw["qkv"], v0 + rank * kl * hd, v0 + (rank + 1) * kl * hd)])
        upgate = _stack([_rows(lw["upgate"], rank * il, (rank + 1) * il),
                         _rows(lw["upgate"], inter + rank * il, inter + (rank + 1) * il)])
        layer = dict(lw, qkv=qkv, upgate=upgate, o=_columns(lw["o"], rank * ql * hd, (rank + 1) * ql * hd),
                     down=_columns(lw["down"], rank * il, (rank + 1) * il))
        if hidden % (128 * ranks) == 0:
            # prompt passes: the same two projections cut by output rows over all columns (whole output elements,
            # gathered between ranks instead of reduced)
            hs = hidden // ranks
            layer.update(o_rows=_rows(lw["o"], rank * hs, (rank + 1) * hs),
                         down_rows=_rows(lw["down"], rank * hs, (rank + 1) * hs))
        layers.append(layer)
    out = dict(weights, layers=layers, lm_head=_rows(weights["lm_head"], lo, hi))
    return local, out, lo


class TensorParallel:
    """Rank layout of a tensor-parallel group plus the one host-side collective the engine needs:
    ``all_gather(bytes) -> [bytes per rank]`` (for example ``torch.distributed.all_gather_object``)."""

    def __init__(self, rank: int, ranks: int, all_gather, wait_ns: int | None = None, unanswered: bool = False,
                 rows: bool = True):
        self.rank, self.ranks, self.all_gather = int(rank), int(ranks), all_gather
        # rows: batched prompt passes across the ranks (False: prompt rows take the token path)
        self.rows = bool(rows) and not unanswered
        # wait_ns: how long a kernel of this rank waits for a peer's data before it reports a device failure
        # (library default 4 s).  unanswered: connect to stand-in peers nobody writes (exercises that limit).
        self.wait_ns, self.unanswered = wait_ns, bool(unanswered)


class DenseModel:
    PREFIX_CHUNK_TOKENS = 1024  # crates/stark-generate/src/prefix_cache.rs:14

    def __init__(self, cfg: dict, context_tokens: int):
        self.cfg = dict(cfg)
        self.context_tokens = int(context_tokens)
        self.tp = None
        self._h = C.c_void_p()
        c = _lib.DenseConfig(C.sizeof(_lib.DenseConfig), _lib.ABI_VERSION, cfg["layers"], cfg["hidden"],
                             cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], cfg["inter"], cfg["vocab"],
                             int(cfg["tied"]), self.context_tokens, cfg["eps"], cfg["rope_theta"],
                             1 if cfg.get("mtp") else 0)
        check(_lib.load().stark_b200_model_create(C.byref(c), C.byref(self._h)), "model_create")

    # ------------------------------------------------------------------ loading
    def _set_matrix(self, layer: int, which: int, t: dict):
        lib = _lib.load()
        d = _lib.AffineDesc(C.sizeof(_lib.AffineDesc), _lib.ABI_VERSION, t["n"], t["k"], t["bits"], t["group"],
                            _lib.PLANE_BF16, int(t.get("scale_layout", 0)), int(t.get("plane_pitch", 0)), _lib.HOST,
                            0, 0)
        codes = np.ascontiguousarray(t["codes"])
        scales = np.ascontiguousarray(t["scales"], np.uint16)
        biases = np.ascontiguousarray(t["biases"], np.uint16)
        check(lib.stark_b200_model_set_affine(self._h, layer, which, codes.ctypes.data, scales.ctypes.data,
                                              biases.ctypes.data, C.byref(d)), "model_set_affine")

    def _set_vector(self, layer: int, which: int, v: np.ndarray):
        v = np.ascontiguousarray(v, np.float32)
        check(_lib.load().stark_b200_model_set_vector(self._h, layer, which, v.ctypes.data, v.size),
              "model_set_vector")

    @classmethod
    def load(cls, cfg: dict, weights: dict, context_tokens: int, tp: "TensorParallel | None" = None) -> "DenseModel":
        """Build from in-memory tensors in the reference's MLX layout (see ``stark_b200.synthetic``).

        With ``tp`` the call is collective: every rank passes the WHOLE model's config and weights and
        keeps its own shard (``shard_dense``); the ranks' exchange buffers are connected before the
        launch sequences are recorded.
        """
        if tp is not None and tp.ranks > 1:
            cfg, weights, vocab_offset = shard_dense(cfg, weights, tp.rank, tp.ranks)
        else:
            tp = None
        m = cls(cfg, context_tokens)
        if tp is not None:
            m.tp, m.vocab_offset, m.vocab_total = tp, vocab_offset, cfg["vocab_total"]
            handle = (C.c_uint8 * 64)()
            check(_lib.load().stark_b200_model_tp_init(m._h, tp.rank, tp.ranks, vocab_offset, cfg["vocab_total"],
                                                       handle), "model_tp_init")
            if tp.wait_ns is not None:
                check(_lib.load().stark_b200_model_tp_set_wait(m._h, int(tp.wait_ns)), "model_tp_set_wait")
            if tp.unanswered:
                check(_lib.load().stark_b200_model_tp_connect_unanswered(m._h), "model_tp_connect_unanswered")
            else:
                handles = b"".join(tp.all_gather(bytes(handle)))
                check(_lib.load().stark_b200_model_tp_connect(m._h, handles, len(handles)), "model_tp_connect")
                if tp.rows and all("o_rows" in lw for lw in weights["layers"]):
                    # batched prompt passes: a second exported region holds whole rows gathered from the ranks
                    check(_lib.load().stark_b200_model_tp_rows_init(m._h, handle), "model_tp_rows_init")
                    handles = b"".join(tp.all_gather(bytes(handle)))
                    check(_lib.load().stark_b200_model_tp_rows_connect(m._h, handles, len(handles)),
                          "model_tp_rows_connect")
        m._set_matrix(0, _lib.MAT_EMBED, weights["embed"])
        if not cfg["tied"]:
            m._set_matrix(0, _lib.MAT_LM_HEAD, weights["lm_head"])
        m._set_vector(0, _lib.VEC_FINAL_NORM, weights["final_norm"])
        for i, lw in enumerate(weights["layers"]):
            m._set_matrix(i, _lib.MAT_QKV, lw["qkv"])
            m._set_matrix(i, _lib.MAT_O, lw["o"])
            m._set_matrix(i, _lib.MAT_UPGATE, lw["upgate"])
            m._set_matrix(i, _lib.MAT_DOWN, lw["down"])
            if tp is not None and tp.rows and "o_rows" in lw:
                m._set_matrix(i, _lib.MAT_O_ROWS, lw["o_rows"])
                m._set_matrix(i, _lib.MAT_DOWN_ROWS, lw["down_rows"])
            m._set_vector(i, _lib.VEC_ATTN_NORM, lw["attn_norm"])
            m._set_vector(i, _lib.VEC_MLP_NORM, lw["mlp_norm"])
            m._set_vector(i, _lib.VEC_Q_NORM, lw["q_norm"])
            m._set_vector(i, _lib.VEC_K_NORM, lw["k_norm"])
        if cfg.get("mtp"):
            # the draft head (qwen_mtp.rs:36-330): its decoder layer is stored after the target's layers
            head, at = weights["mtp"], cfg["layers"]
            m._set_matrix(at, _lib.MAT_MTP_FUSION, head["fusion"])
            for which, key in ((_lib.MAT_QKV, "qkv"), (_lib.MAT_O, "o"), (_lib.MAT_UPGATE, "upgate"), (_lib.MAT_DOWN, "down")):
                m._set_matrix(at, which, head["layer"][key])
            for which, key in ((_lib.VEC_ATTN_NORM, "attn_norm"), (_lib.VEC_MLP_NORM, "mlp_norm"),
                               (_lib.VEC_Q_NORM, "q_norm"), (_lib.VEC_K_NORM, "k_norm")):
                m._set_vector(at, which, head["layer"][key])
            m._set_vector(at, _lib.VEC_MTP_EMBED_NORM, head["embed_norm"])
            m._set_vector(at, _lib.VEC_MTP_HIDDEN_NORM, head["hidden_norm"])
            m._set_vector(at, _lib.VEC_MTP_OUT_NORM, head["out_norm"])
        if tp is not None:
            tp.all_gather(b"")  # every rank has uploaded its shard: the recording pass below is collective
        check(_lib.load().stark_b200_model_finalize(m._h), "model_finalize")
        return m

    @classmethod
    def from_artifact(cls, directory, context_tokens: int, tp: "TensorParallel | None" = None) -> "DenseModel":
        """Load a converted-model directory (``config.json`` + ``model.safetensors`` in the reference's
        layout, see ``stark_b200.artifact``); the analogue of ``Engine::new`` -> ``load_language_model``
        (crates/stark-engine/src/engine/language_model/mod.rs:72-127)."""
        from .artifact import read_artifact
        cfg, weights = read_artifact(directory)
        return cls.load(cfg, weights, context_tokens, tp=tp)

    @classmethod
    def load_path(cls, directory, context_tokens: int = 0) -> "DenseModel":
        """The same artifact through the library's own loader (``stark_b200_load``): what a host that is not
        Python calls.  The Python object only wraps the handle it gets back."""
        from .artifact import read_artifact
        path = str(directory).encode("utf-8")
        opts = _lib.LoadOptions(C.sizeof(_lib.LoadOptions), _lib.ABI_VERSION, int(context_tokens), 0)
        handle = C.c_void_p()
        check(_lib.load().stark_b200_load(path, len(path), C.byref(opts), C.byref(handle)), "load")
        m = cls.__new__(cls)
        m._h, m.tp = handle, None
        info = m.info()
        m.context_tokens = int(info.context_tokens)
        m.cfg = dict(vocab=int(info.vocab_size))
        return m

    def _gather_vocab(self, local: np.ndarray) -> np.ndarray:
        """Whole-vocabulary vector from the ranks' read-out shards (identity on one GPU)."""
        if self.tp is None:
            return local
        parts = self.tp.all_gather(local.tobytes())
        return np.concatenate([np.frombuffer(p, local.dtype) for p in parts])

    # ------------------------------------------------------------------ token loop
    def reset(self):
        check(_lib.load().stark_b200_reset(self._h), "reset")

    def _guard(self, status: int, where: str):
        if status != 0:
            # hybrid::Model resets itself after any error (mod.rs:876-885)
            if status not in (_lib.STATUS_NAMES.index("reload_required"),):
                _lib.load().stark_b200_reset(self._h)
            raise StarkB200Error(status, where)

    def prefill(self, token_ids) -> None:
        ids = np.ascontiguousarray(token_ids, np.uint32)
        if self.tp is not None:
            # Ranks wait for one another on the device with a time limit: line the hosts up where a
            # request starts, so that host-side skew (tokenising, scoring) is not charged to that limit.
            self.tp.all_gather(b"")
        self._guard(_lib.load().stark_b200_prefill(self._h, ids.ctypes.data, ids.size), "prefill")

    def ingest_prefix(self, token_ids) -> None:
        self.prefill(token_ids)

    def step(self, token: int) -> np.ndarray:
        """Feed one token, return the full-vocabulary logits (f32) of its row."""
        self._guard(_lib.load().stark_b200_step(self._h, int(token)), "step")
        return self.logits()

    def step_async(self, token: int) -> None:
        self._guard(_lib.load().stark_b200_step(self._h, int(token)), "step")

    def logits(self) -> np.ndarray:
        out = np.empty(self.cfg["vocab"], np.float32)
        self._guard(_lib.load().stark_b200_readout_f32(self._h, out.ctypes.data, out.size), "readout_f32")
        return self._gather_vocab(out)

    def logits_bf16(self) -> np.ndarray:
        out = np.empty(self.cfg["vocab"], np.uint16)
        self._guard(_lib.load().stark_b200_readout_bf16(self._h, out.ctypes.data, out.size), "readout_bf16")
        return self._gather_vocab(out)

    def log_probabilities(self) -> np.ndarray:
        if self.tp is not None:  # normalise over the gathered vocabulary with the same f64 kernel
            from . import ops
            return ops.log_softmax(self.logits()).astype(np.float32)
        out = np.empty(self.cfg["vocab"], np.float32)
        self._guard(_lib.load().stark_b200_readout_logprobs_f32(self._h, out.ctypes.data, out.size),
                    "readout_logprobs_f32")
        return out

    def argmax(self) -> int:
        t = C.c_uint32(0)
        self._guard(_lib.load().stark_b200_argmax(self._h, C.byref(t)), "argmax")
        return t.value

    def sample(self, seed=None, temperature=None, top_k=None, top_p=None, min_p=None, ordered: bool = False) -> int:
        """One token from the last row's logits through the device sampler (the reference's unified
        sampler; ``seed`` is the per-position seed, see ``position_seed``).  ``ordered`` selects the
        generation worker's host-sampler semantics instead (crates/stark-generate/src/hybrid.rs:1122-1212);
        ``seed`` is then the SplitMix64 state before the draw."""
        params = _lib.sampling(seed, temperature, top_k, top_p, min_p, ordered)
        t = C.c_uint32(0)
        self._guard(_lib.load().stark_b200_sample(self._h, C.byref(params), C.byref(t)), "sample")
        return t.value

    def generate_greedy(self, steps: int) -> np.ndarray:
        out = np.empty(steps + 1, np.uint32)
        self._guard(_lib.load().stark_b200_generate_greedy(self._h, steps, out.ctypes.data), "generate_greedy")
        return out

    def rewind(self, position: int) -> None:
        check(_lib.load().stark_b200_rewind(self._h, position), "rewind")

    def drain(self) -> None:
        check(_lib.load().stark_b200_drain(self._h), "drain")

    def cancel(self) -> None:
        check(_lib.load().stark_b200_cancel(self._h), "cancel")

    def info(self) -> _lib.Info:
        i = _lib.Info()
        i.struct_size = C.sizeof(_lib.Info)
        i.abi_version = _lib.ABI_VERSION
        check(_lib.load().stark_b200_get_info(self._h, C.byref(i)), "get_info")
        return i

    def read_trace(self) -> np.ndarray:
        """Timeline of the launches since the last call, ``uint64[launches_per_step, 6]`` (ns): first CTA
        entered, first wait returned, last prologue done, last CTA left, last CTA entered, last wait returned."""
        n = self.info().trace_slots
        out = np.empty((n, 6), np.uint64)
        check(_lib.load().stark_b200_read_trace(self._h, out.ctypes.data, out.size), "read_trace")
        return out

    # ------------------------------------------------------------------ multi-token prediction
    def mtp_initial(self) -> int:
        """After ``prefill``: the pending token (greedy pick of the prompt's last row), not yet committed."""
        t = C.c_uint32(0)
        self._guard(_lib.load().stark_b200_mtp_initial(self._h, C.byref(t)), "mtp_initial")
        return t.value

    def mtp_round(self, pending: int, drafts: int, accept_mask: int | None = None, held: bool = False) -> dict:
        """One speculative round (``LanguageModel::dense_mtp_round``, dense_mtp.rs:661-886): ``drafts`` proposals of
        the head, one target pass over ``drafts + 1`` rows, acceptance, commit.  Greedy acceptance unless
        ``accept_mask`` gives the pattern (bit i accepts proposal i).  Returns the committed tokens (the first is
        ``pending``), the accepted count and the next pending token.  ``held``: stop after the target pass --
        ``tokens`` are the pending token and all proposals, the caller reads rows with ``mtp_row_logits``, decides,
        and closes the round with ``mtp_commit``."""
        r = _lib.MtpRoundResult()
        r.struct_size, r.abi_version = C.sizeof(_lib.MtpRoundResult), _lib.ABI_VERSION
        policy = _lib.MTP_HELD if held else (_lib.MTP_GREEDY if accept_mask is None else _lib.MTP_FORCED)
        self._guard(_lib.load().stark_b200_mtp_round(self._h, int(pending), int(drafts), policy, int(accept_mask or 0),
                                                     C.byref(r)), "mtp_round")
        return dict(tokens=[int(t) for t in r.tokens[:r.count]], accepted=int(r.accepted), proposed=int(r.proposed),
                    next_pending=int(r.next_pending), position=int(r.position))

    def mtp_commit(self, accepted: int, next_pending: int) -> dict:
        """Closes a held round: ``accepted`` proposals are kept, ``next_pending`` is what the caller's sampler drew
        after the last kept row (``stark_b200_mtp_commit``)."""
        r = _lib.MtpRoundResult()
        r.struct_size, r.abi_version = C.sizeof(_lib.MtpRoundResult), _lib.ABI_VERSION
        self._guard(_lib.load().stark_b200_mtp_commit(self._h, int(accepted), int(next_pending), C.byref(r)), "mtp_commit")
        return dict(tokens=[int(t) for t in r.tokens[:r.count]], accepted=int(r.accepted), proposed=int(r.proposed),
                    next_pending=int(r.next_pending), position=int(r.position))

    def mtp_round_lookup(self, pending: int, proposals, accept_mask: int | None = None, held: bool = False) -> dict:
        """A round whose proposals the caller supplies (prompt lookup: tokens copied from the request's own
        context, engine/hybrid/mtp_lookup.rs) instead of the head; otherwise as ``mtp_round``."""
        r = _lib.MtpRoundResult()
        r.struct_size, r.abi_version = C.sizeof(_lib.MtpRoundResult), _lib.ABI_VERSION
        p = np.ascontiguousarray(proposals, np.uint32).reshape(-1)
        policy = _lib.MTP_HELD if held else (_lib.MTP_GREEDY if accept_mask is None else _lib.MTP_FORCED)
        self._guard(_lib.load().stark_b200_mtp_round_lookup(self._h, int(pending), p.ctypes.data if p.size else None,
                                                            p.size, policy, int(accept_mask or 0), C.byref(r)),
                    "mtp_round_lookup")
        return dict(tokens=[int(t) for t in r.tokens[:r.count]], accepted=int(r.accepted), proposed=int(r.proposed),
                    next_pending=int(r.next_pending), position=int(r.position))

    def mtp_row_logits(self, row: int) -> np.ndarray:
        """Full-vocabulary logits (f32) of one row of the last round's target pass."""
        out = np.empty(self.cfg["vocab"], np.float32)
        self._guard(_lib.load().stark_b200_mtp_readout_row_f32(self._h, int(row), out.ctypes.data, out.size),
                    "mtp_readout_row_f32")
        return out

    def recapture(self, **tunables: int) -> None:
        """Sets launch-shape settings (``stark_b200_set_tunable`` names) and records the token sequences again."""
        for name, value in tunables.items():
            check(_lib.load().stark_b200_set_tunable(name.encode(), int(value)), f"set_tunable {name}")
        check(_lib.load().stark_b200_model_recapture(self._h), "model_recapture")

    def stream(self) -> int:
        """The cudaStream_t the model issues its work on (an integer handle)."""
        p = C.c_void_p()
        check(_lib.load().stark_b200_model_stream(self._h, C.byref(p)), "model_stream")
        return p.value or 0

    @property
    def position(self) -> int:
        return int(self.info().position)

    def close(self, collective: bool = True):
        if self._h and self._h.value and self.tp is not None and collective:
            # peers read this rank's exchange buffers: nobody unmaps before everybody is idle
            try:
                _lib.load().stark_b200_drain(self._h)
                self.tp.all_gather(b"")
            except Exception:
                pass
        if self._h and self._h.value:
            _lib.load().stark_b200_destroy(C.byref(self._h))

    def __del__(self):
        try:
            self.close(collective=False)
        except Exception:
            pass


def position_seed(seed: int, position: int) -> int:
    """Per-position sampling seed, ``PRng::derive`` (crates/stark-engine/src/encodable_block/sampling/prng.rs:12-22):
    the 64-bit MurmurHash3 finalizer of ``seed + position``."""
    mask = (1 << 64) - 1
    h = (seed + position) & mask
    h ^= h >> 33
    h = (h * 0xFF51AFD7ED558CCD) & mask
    h ^= h >> 33
    h = (h * 0xC4CEB9FE1A85EC53) & mask
    h ^= h >> 33
    return h


def reusable_prefix_rows(previous_prompt_len: int, common_prefix: int, new_prompt_len: int,
                         chunk: int = DenseModel.PREFIX_CHUNK_TOKENS) -> int:
    """Rows of the previous request that the next one may reuse.

    crates/stark-generate/src/prefix_cache.rs:44-99: the retained prefix is the previous prompt cut
    to whole chunks strictly below its final chunk; reuse is the common prefix with it, cut to whole
    chunks strictly below the new prompt's final chunk.
    """
    if previous_prompt_len <= 0 or new_prompt_len <= 0:
        return 0
    retained = ((previous_prompt_len - 1) // chunk) * chunk
    limit = ((new_prompt_len - 1) // chunk) * chunk
    return (min(common_prefix, retained, limit) // chunk) * chunk


class ExpertParallel:
    """Rank layout of an expert-parallel group plus the one host-side collective the engine needs:
    ``all_gather(bytes) -> [bytes per rank]`` (for example ``torch.distributed.all_gather_object``)."""

    def __init__(self, rank: int, ranks: int, all_gather, wait_ns: int | None = None):
        self.rank, self.ranks, self.all_gather, self.wait_ns = int(rank), int(ranks), all_gather, wait_ns


def expert_shard(bank: np.ndarray, rank: int, ranks: int) -> np.ndarray:
    """Rank ``rank``'s experts of a bank whose first axis counts experts: the contiguous block
    ``[rank * E / ranks, (rank + 1) * E / ranks)``."""
    experts = bank.shape[0]
    if experts % ranks:
        raise ValueError("the expert count must be a multiple of the rank count")
    per = experts // ranks
    return bank[rank * per:(rank + 1) * per]


def expert_owner(expert: int, experts: int, ranks: int) -> int:
    return int(expert) // (experts // ranks)


class MoEModel:
    """A routed-expert decoder on the conventions of the reference's hybrid host path (f32 activations and
    logits, GGUF Q8_0 attention / token table / output, Q4_K expert banks), with the surface of
    ``hybrid::Model`` (crates/stark-engine/src/engine/hybrid/mod.rs:347,863,897,990): ``load``, ``reset``,
    ``ingest``, ``step -> logits``.  Any failing call leaves the model reset, as the reference does."""

    def __init__(self, cfg: dict, context_tokens: int, ep: "ExpertParallel | None" = None):
        self.cfg = dict(cfg)
        self.context_tokens = int(context_tokens)
        self.ep = ep if ep is not None and ep.ranks > 1 else None
        self._h = C.c_void_p()
        self._matrices = []  # the handle borrows them
        c = _lib.MoeConfig(C.sizeof(_lib.MoeConfig), cfg["vocab"], cfg["hidden"], cfg["layers"], cfg["q_heads"],
                           cfg["kv_heads"], cfg["head_dim"], cfg["experts"], cfg["active"], cfg["inter"],
                           self.context_tokens, cfg["eps"], cfg["rope_theta"])
        check(_lib.load().stark_b200_moe_model_create(C.byref(c), C.byref(self._h)), "moe_model_create")
        if self.ep is not None:
            # collective: every rank allocates its exchange region, the 64-byte handles travel over the host-side
            # collective, every rank maps every other rank's region
            if cfg["experts"] % self.ep.ranks:
                raise ValueError("the expert count must be a multiple of the rank count")
            handle = (C.c_uint8 * 64)()
            check(_lib.load().stark_b200_moe_model_ep_init(self._h, self.ep.rank, self.ep.ranks, handle), "moe_model_ep_init")
            if self.ep.wait_ns is not None:
                check(_lib.load().stark_b200_moe_model_ep_set_wait(self._h, int(self.ep.wait_ns)), "moe_model_ep_set_wait")
            handles = b"".join(self.ep.all_gather(bytes(handle)))
            buf = (C.c_uint8 * len(handles)).from_buffer_copy(handles)
            check(_lib.load().stark_b200_moe_model_ep_connect(self._h, buf, len(handles)), "moe_model_ep_connect")

    def _matrix(self, kind: int, layer: int, blocks: np.ndarray, ggml_kind: int, rows: int, columns: int,
                experts: int = 0):
        from .ops import QMatrix
        q = QMatrix.from_gguf(blocks, ggml_kind, rows, columns, experts)
        self._matrices.append(q)
        check(_lib.load().stark_b200_moe_model_set_matrix(self._h, kind, layer, q._h), "moe_model_set_matrix")

    def _tensor(self, kind: int, layer: int, a: np.ndarray):
        a = np.ascontiguousarray(a)
        check(_lib.load().stark_b200_moe_model_set_tensor(self._h, kind, layer, a.ctypes.data, a.nbytes),
              "moe_model_set_tensor")

    def set_layer(self, layer: int, w: dict) -> None:
        """One layer's tensors (``stark_b200.synthetic.moe_layer_weights`` layout); uploads as it goes, so a
        large model can be streamed layer by layer."""
        c, L = self.cfg, _lib
        qd, kd = c["q_heads"] * c["head_dim"], c["kv_heads"] * c["head_dim"]
        Q8_0, Q4_K = 8, 12
        self._matrix(L.MOE_MAT_QKV, layer, w["qkv"], Q8_0, qd + 2 * kd, c["hidden"])
        self._matrix(L.MOE_MAT_O, layer, w["o"], Q8_0, c["hidden"], qd)
        gate, up, down = (np.asarray(w[k], np.uint8).reshape(c["experts"], -1) for k in ("gate", "up", "down"))
        local = c["experts"]
        if self.ep is not None:  # this rank's contiguous share of the expert banks
            gate, up, down = (expert_shard(a, self.ep.rank, self.ep.ranks) for a in (gate, up, down))
            local = c["experts"] // self.ep.ranks
        gate_up = np.concatenate([gate.reshape(-1), up.reshape(-1)])
        self._matrix(L.MOE_MAT_GATE_UP, layer, gate_up, Q4_K, c["inter"], c["hidden"], 2 * local)
        self._matrix(L.MOE_MAT_DOWN, layer, down.reshape(-1), Q4_K, c["hidden"], c["inter"], local)
        self._tensor(L.MOE_ROUTER, layer, np.asarray(w["router"], np.float32))
        for kind, name in ((L.MOE_ATTN_NORM, "attn_norm"), (L.MOE_FFN_NORM, "ffn_norm"), (L.MOE_Q_NORM, "q_norm"),
                           (L.MOE_K_NORM, "k_norm")):
            self._tensor(kind, layer, np.asarray(w[name], np.float32))

    def set_globals(self, token_table: np.ndarray, output: np.ndarray, final_norm: np.ndarray) -> None:
        c, L = self.cfg, _lib
        self._tensor(L.MOE_TOKEN_TABLE, 0, np.asarray(token_table, np.uint8))
        self._matrix(L.MOE_MAT_OUTPUT, 0, output, 8, c["vocab"], c["hidden"])
        self._tensor(L.MOE_FINAL_NORM, 0, np.asarray(final_norm, np.float32))

    @classmethod
    def load(cls, cfg: dict, weights: dict, context_tokens: int, ep: "ExpertParallel | None" = None) -> "MoEModel":
        """With ``ep`` the call is collective: every rank passes the whole model's weights and keeps the experts
        it owns (``expert_shard``); attention, router, token table and read-out are replicated."""
        m = cls(cfg, context_tokens, ep)
        m.set_globals(weights["token_table"], weights["output"], weights["final_norm"])
        for layer, w in enumerate(weights["layers"]):
            m.set_layer(layer, w)
        return m

    def _line_up(self) -> None:
        """Expert parallel: the calls that start a request are collective.  Ranks meet on the host first, so that
        no rank's kernels sit waiting for a peer that is still busy with something else (the device-side wait is
        bounded and would report a failure).  Single steps do not meet: ranks that step together drift by host
        jitter only."""
        if self.ep is not None:
            self.ep.all_gather(b"")

    def reset(self) -> None:
        self._line_up()
        check(_lib.load().stark_b200_moe_model_reset(self._h), "moe_model_reset")

    def ingest(self, tokens) -> None:
        self._line_up()
        t = np.ascontiguousarray(tokens, np.uint32).reshape(-1)
        check(_lib.load().stark_b200_moe_model_ingest(self._h, t.ctypes.data, t.size), "moe_model_ingest")

    def step(self, token: int, want_logits: bool = True):
        out = np.empty(self.cfg["vocab"], np.float32) if want_logits else None
        check(_lib.load().stark_b200_moe_model_step(self._h, int(token), out.ctypes.data if want_logits else None,
                                                    self.cfg["vocab"] if want_logits else 0), "moe_model_step")
        return out

    def generate_greedy(self, first: int, steps: int) -> np.ndarray:
        self._line_up()
        out = np.empty(steps, np.uint32)
        check(_lib.load().stark_b200_moe_model_generate_greedy(self._h, int(first), steps, out.ctypes.data),
              "moe_model_generate_greedy")
        return out

    def last_experts(self) -> np.ndarray:
        out = np.empty((self.cfg["layers"], self.cfg["active"]), np.uint32)
        check(_lib.load().stark_b200_moe_model_last_experts(self._h, out.ctypes.data, out.size), "moe_model_last_experts")
        return out

    @property
    def position(self) -> int:
        p = C.c_uint32(0)
        check(_lib.load().stark_b200_moe_model_position(self._h, C.byref(p)), "moe_model_position")
        return p.value

    @property
    def launches_per_token(self) -> int:
        p = C.c_uint32(0)
        check(_lib.load().stark_b200_moe_model_launches_per_token(self._h, C.byref(p)), "moe_model_launches_per_token")
        return p.value

    @property
    def stream(self) -> int:
        p = C.c_void_p()
        check(_lib.load().stark_b200_moe_model_stream(self._h, C.byref(p)), "moe_model_stream")
        return p.value or 0

    def weight_bytes_per_token(self) -> int:
        """Bytes of weights one decode token reads: attention and output matrices whole, the active experts
        of each bank, the router, one row of the token table."""
        c = self.cfg
        qd, kd = c["q_heads"] * c["head_dim"], c["kv_heads"] * c["head_dim"]
        q8 = lambda n: n // 32 * 34
        q4 = lambda n: n // 256 * 144
        ranks = self.ep.ranks if self.ep is not None else 1   # a rank reads the selected experts it owns: active / ranks on average
        per_layer = q8((qd + 2 * kd) * c["hidden"]) + q8(c["hidden"] * qd) + 4 * c["experts"] * c["hidden"] \
            + 3 * c["active"] * q4(c["inter"] * c["hidden"]) // ranks
        return c["layers"] * per_layer + q8(c["vocab"] * c["hidden"]) + q8(c["hidden"])

    def close(self) -> None:
        if self._h:
            _lib.load().stark_b200_moe_model_destroy(C.byref(self._h))
            self._h = C.c_void_p()
        for q in self._matrices:
            q.destroy()
        self._matrices = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
