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


class DenseModel:
    PREFIX_CHUNK_TOKENS = 1024  # crates/stark-generate/src/prefix_cache.rs:14

    def __init__(self, cfg: dict, context_tokens: int):
        self.cfg = dict(cfg)
        self.context_tokens = int(context_tokens)
        self._h = C.c_void_p()
        c = _lib.DenseConfig(C.sizeof(_lib.DenseConfig), _lib.ABI_VERSION, cfg["layers"], cfg["hidden"],
                             cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], cfg["inter"], cfg["vocab"],
                             int(cfg["tied"]), self.context_tokens, cfg["eps"], cfg["rope_theta"], 0)
        check(_lib.load().stark_b200_model_create(C.byref(c), C.byref(self._h)), "model_create")

    # ------------------------------------------------------------------ loading
    def _set_matrix(self, layer: int, which: int, t: dict):
        lib = _lib.load()
        d = _lib.AffineDesc(C.sizeof(_lib.AffineDesc), _lib.ABI_VERSION, t["n"], t["k"], t["bits"], t["group"],
                            _lib.PLANE_BF16, 0, 0, _lib.HOST, 0, 0)
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
    def load(cls, cfg: dict, weights: dict, context_tokens: int) -> "DenseModel":
        """Build from in-memory tensors in the reference's MLX layout (see ``stark_b200.synthetic``)."""
        m = cls(cfg, context_tokens)
        m._set_matrix(0, _lib.MAT_EMBED, weights["embed"])
        if not cfg["tied"]:
            m._set_matrix(0, _lib.MAT_LM_HEAD, weights["lm_head"])
        m._set_vector(0, _lib.VEC_FINAL_NORM, weights["final_norm"])
        for i, lw in enumerate(weights["layers"]):
            m._set_matrix(i, _lib.MAT_QKV, lw["qkv"])
            m._set_matrix(i, _lib.MAT_O, lw["o"])
            m._set_matrix(i, _lib.MAT_UPGATE, lw["upgate"])
            m._set_matrix(i, _lib.MAT_DOWN, lw["down"])
            m._set_vector(i, _lib.VEC_ATTN_NORM, lw["attn_norm"])
            m._set_vector(i, _lib.VEC_MLP_NORM, lw["mlp_norm"])
            m._set_vector(i, _lib.VEC_Q_NORM, lw["q_norm"])
            m._set_vector(i, _lib.VEC_K_NORM, lw["k_norm"])
        check(_lib.load().stark_b200_model_finalize(m._h), "model_finalize")
        return m

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
        return out

    def logits_bf16(self) -> np.ndarray:
        out = np.empty(self.cfg["vocab"], np.uint16)
        self._guard(_lib.load().stark_b200_readout_bf16(self._h, out.ctypes.data, out.size), "readout_bf16")
        return out

    def log_probabilities(self) -> np.ndarray:
        out = np.empty(self.cfg["vocab"], np.float32)
        self._guard(_lib.load().stark_b200_readout_logprobs_f32(self._h, out.ctypes.data, out.size),
                    "readout_logprobs_f32")
        return out

    def argmax(self) -> int:
        t = C.c_uint32(0)
        self._guard(_lib.load().stark_b200_argmax(self._h, C.byref(t)), "argmax")
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
        """Timeline of the launches since the last call, ``uint64[launches_per_step, 4]`` (ns)."""
        n = self.info().trace_slots
        out = np.empty((n, 4), np.uint64)
        check(_lib.load().stark_b200_read_trace(self._h, out.ctypes.data, out.size), "read_trace")
        return out

    def stream(self) -> int:
        """The cudaStream_t the model issues its work on (an integer handle)."""
        p = C.c_void_p()
        check(_lib.load().stark_b200_model_stream(self._h, C.byref(p)), "model_stream")
        return p.value or 0

    @property
    def position(self) -> int:
        return int(self.info().position)

    def close(self):
        if self._h and self._h.value:
            _lib.load().stark_b200_destroy(C.byref(self._h))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


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
