"""ctypes front-end of the CPU oracle (``stark_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke`` and by the
CPU-baseline / reference legs of ``bench.py``.  The product package never imports this module.

The C file restates the reference's Rust CPU kernels (each function cites the file and lines it
follows); this module only marshals numpy arrays into it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "libstark_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compile ``stark_oracle.c`` with the recipe in ``oracle/Makefile``."""
    src = _HERE / "stark_oracle.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.run(["make", "-C", str(_HERE), "-B", "libstark_oracle.so"], check=True, env=env,
                       stdout=subprocess.DEVNULL)
    return _SO


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(_SO))
        _lib.so_packed_code.restype = C.c_uint8
        _lib.so_packed_code.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t]
        _lib.so_f32_to_bf16.restype = C.c_uint16
        _lib.so_f32_to_bf16.argtypes = [C.c_float]
        _lib.so_bf16_to_f32.restype = C.c_float
        _lib.so_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.so_f16_to_f32.restype = C.c_float
        _lib.so_f16_to_f32.argtypes = [C.c_uint16]
        _lib.so_argmax_bf16.restype = C.c_uint32
        _lib.so_argmax_f32.restype = C.c_uint32
        _lib.so_rope_coeffs.argtypes = [C.c_uint32, C.c_uint32, C.c_float, C.c_void_p, C.c_void_p]
        _lib.so_dense_step.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_int]
    return _lib


def max_threads() -> int:
    return int(lib().so_max_threads())


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


# ----------------------------------------------------------------------------- bf16 helpers

def f32_to_bf16(x) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16), NaN kept quiet (half::bf16::from_f32)."""
    u = _c(x, np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), rounded)


def bf16_to_f32(h) -> np.ndarray:
    return (_c(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


# ----------------------------------------------------------------------------- integer unpack

def packed_code(codes: np.ndarray, bits: int, index: int) -> int:
    codes = _c(codes, np.uint8)
    return int(lib().so_packed_code(_p(codes), bits, index))


def unpack_codes(codes: np.ndarray, bits: int, count: int) -> np.ndarray:
    codes = _c(codes.view(np.uint8).reshape(-1), np.uint8)
    out = np.empty(count, np.uint8)
    lib().so_unpack_codes(_p(codes), C.c_size_t(bits), C.c_size_t(count), _p(out))
    return out


# ----------------------------------------------------------------------------- affine matvec

def affine_matvec_bf16(codes, scales, biases, a, n, k, bits=4, group=64, m=1, scale_layout=0, npad=0,
                       correction=0, signed_codes=0, threads=1) -> np.ndarray:
    """Path-A quantized matmul: bf16 in, f32 accumulate, bf16 out (bit patterns, uint16)."""
    codes = _c(codes.view(np.uint8).reshape(-1), np.uint8)
    scales = _c(scales, np.uint16)
    biases = None if biases is None else _c(biases, np.uint16)
    a = _c(a, np.uint16)
    d = np.empty((m, n), np.uint16)
    rc = lib().so_affine_matvec_bf16(_p(codes), _p(scales), _p(biases), _p(a), _p(d), m, n, k, bits, group,
                                     scale_layout, npad, correction, signed_codes, threads)
    if rc:
        raise ValueError("invalid affine matvec arguments")
    return d


def affine_matvec_f32(codes, scales, biases, plane_kind, x, rows, columns, bits=4, group=64, threads=1):
    """Path-B host matvec: f32 in/out, planes f32 (0) / f16 (1) / bf16 (30)."""
    codes = _c(np.ascontiguousarray(codes).view(np.uint8).reshape(-1), np.uint8)
    scales, biases = np.ascontiguousarray(scales), np.ascontiguousarray(biases)
    x = _c(x, np.float32)
    y = np.empty(rows, np.float32)
    rc = lib().so_affine_matvec_f32(_p(codes), _p(scales), _p(biases), plane_kind, _p(x), _p(y), rows, columns,
                                    bits, group, threads)
    if rc:
        raise ValueError("invalid matvec input shape or values")
    return y


def affine_row_f32(codes, scales, biases, plane_kind, row, columns, bits=4, group=64):
    codes = _c(codes.view(np.uint8).reshape(-1), np.uint8)
    out = np.empty(columns, np.float32)
    rc = lib().so_affine_row_f32(_p(codes), _p(scales), _p(biases), plane_kind, _p(out), row, columns, bits, group)
    if rc:
        raise ValueError("invalid affine row arguments")
    return out


# ----------------------------------------------------------------------------- GGUF blocks

Q8_0, Q4_K = 8, 12
BLOCK = {Q8_0: (32, 34), Q4_K: (256, 144)}


def decode_block(kind: int, block: np.ndarray) -> np.ndarray:
    elements, size = BLOCK[kind]
    block = _c(block, np.uint8)
    if block.size != size:
        raise ValueError("invalid quantization block size")
    out = np.empty(elements, np.float32)
    if lib().so_decode_block(kind, _p(block), _p(out)):
        raise ValueError("unsupported weight block format")
    return out


def q4k_unpack(block: np.ndarray):
    block = _c(block, np.uint8)
    codes = np.empty(256, np.uint8)
    sc = np.empty(8, np.uint8)
    mn = np.empty(8, np.uint8)
    lib().so_q4k_unpack(_p(block), _p(codes), _p(sc), _p(mn))
    return codes, sc, mn


def gguf_matvec_f32(kind, data, x, rows, columns, threads=1):
    data = _c(data, np.uint8)
    x = _c(x, np.float32)
    y = np.empty(rows, np.float32)
    if lib().so_gguf_matvec_f32(kind, _p(data), _p(x), _p(y), rows, columns, threads):
        raise ValueError("invalid matvec input shape or values")
    return y


def gguf_decode_row(kind, data, columns):
    data = _c(data, np.uint8)
    out = np.empty(columns, np.float32)
    if lib().so_gguf_decode_row(kind, _p(data), _p(out), columns):
        raise ValueError("invalid encoded row size")
    return out


# ----------------------------------------------------------------------------- small ops

def rmsnorm_bf16(x, scales, eps, shortcut=None, residual_add=False):
    """Returns (normed, new_shortcut_or_None); bf16 bit patterns."""
    x = _c(x, np.uint16)
    batch, count = (1, x.size) if x.ndim == 1 else x.shape
    scales = _c(scales, np.float32)
    out = np.empty_like(x)
    sc = None if shortcut is None else _c(shortcut, np.uint16).copy()
    lib().so_rmsnorm_bf16(_p(x), _p(scales), _p(out), _p(sc), batch, count, C.c_float(eps), int(residual_add))
    return out, sc


def rmsnorm_f32(x, weight, eps):
    x = _c(x, np.float32)
    weight = _c(weight, np.float32)
    if x.size != weight.size:
        raise ValueError("RMS normalization dimensions or values")
    out = np.empty_like(x)
    if lib().so_rmsnorm_f32(_p(x), _p(weight), _p(out), x.size, C.c_float(eps)):
        raise ValueError("RMS normalization dimensions or values")
    return out


def head_norm_bf16(row, scales, head_offset, head_count, head_dim, eps):
    row = _c(row, np.uint16).copy()
    scales = _c(scales, np.float32)
    lib().so_head_norm_bf16(_p(row), _p(scales), head_offset, head_count, head_dim, C.c_float(eps))
    return row


def rope_coeffs(position, head_dim, base):
    cos = np.empty(head_dim, np.float32)
    sin = np.empty(head_dim, np.float32)
    lib().so_rope_coeffs(position, head_dim, C.c_float(base), _p(cos), _p(sin))
    return cos, sin


def rope_head_bf16(head, cos, sin):
    head = _c(head, np.uint16)
    out = np.empty_like(head)
    lib().so_rope_head_bf16(_p(head), _p(out), _p(_c(cos, np.float32)), _p(_c(sin, np.float32)), head.size)
    return out


def attention_decode_bf16(q, keys, values, heads, kv_heads, head_dim, seq_len, scale, threads=1):
    q = _c(q, np.uint16)
    keys = _c(keys, np.uint16)
    values = _c(values, np.uint16)
    out = np.empty(heads * head_dim, np.uint16)
    lib().so_attention_decode_bf16(_p(q), _p(keys), _p(values), _p(out), heads, kv_heads, head_dim, seq_len,
                                   C.c_float(scale), threads)
    return out


def swiglu_bf16(fused, gated_dim):
    fused = _c(fused, np.uint16)
    out = np.empty(gated_dim, np.uint16)
    lib().so_swiglu_bf16(_p(fused), _p(out), gated_dim)
    return out


def embedding_row_bf16(codes, scales, biases, token, vocab, dim, bits=4, group=64):
    codes = _c(codes.view(np.uint8).reshape(-1), np.uint8)
    out = np.empty(dim, np.uint16)
    lib().so_embedding_row_bf16(_p(codes), _p(_c(scales, np.uint16)), _p(_c(biases, np.uint16)), token, vocab, dim,
                                bits, group, _p(out))
    return out


def argmax_bf16(logits) -> int:
    logits = _c(logits, np.uint16)
    return int(lib().so_argmax_bf16(_p(logits), logits.size))


def argmax_f32(logits) -> int:
    logits = _c(logits, np.float32)
    return int(lib().so_argmax_f32(_p(logits), logits.size))


def philox4x32_10(ctr, key) -> np.ndarray:
    """gumbel.rs:16-46: ten rounds, key bumped by the Weyl constants between rounds."""
    ctr, key, out = _c(ctr, np.uint32), _c(key, np.uint32), np.zeros(4, np.uint32)
    lib().so_philox4x32_10(_p(ctr), _p(key), _p(out))
    return out


def unit_interval(word: int) -> float:
    f = lib().so_unit_interval
    f.restype, f.argtypes = C.c_float, [C.c_uint32]
    return float(f(word))


def gumbel_float(key: int, offset: int, word: int) -> float:
    f = lib().so_gumbel_float
    f.restype, f.argtypes = C.c_float, [C.c_uint64, C.c_uint32, C.c_uint32]
    return float(f(key, offset, word))


def revidx(index: int, vocab: int) -> tuple[int, int]:
    off, word = C.c_uint32(0), C.c_uint32(0)
    lib().so_revidx(C.c_uint32(index), C.c_uint32(vocab), C.byref(off), C.byref(word))
    return off.value, word.value


def prng_derive(seed: int, index: int) -> int:
    f = lib().so_prng_derive
    f.restype, f.argtypes = C.c_uint64, [C.c_uint64, C.c_uint64]
    return int(f(seed, index))


def unified_sampling(logits, seed=None, temperature=None, top_k=None, top_p=None, min_p=None) -> int:
    """unified_sampling.rs:15-117 on one row of f32 logits; ``seed`` None = greedy."""
    logits = _c(logits, np.float32)
    flags = (1 if seed is not None else 0) | (2 if temperature is not None else 0) | (4 if top_k is not None else 0) \
        | (8 if top_p is not None else 0) | (16 if min_p is not None else 0)
    f = lib().so_unified_sampling_f32
    f.restype = C.c_uint32
    f.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64, C.c_float, C.c_uint32, C.c_float, C.c_float]
    return int(f(_p(logits), logits.size, flags, seed or 0, temperature or 1.0, top_k or 0, top_p or 1.0, min_p or 0.0))


SPLITMIX64_STEP = 0x9E3779B97F4A7C15


def splitmix64_uniform(state: int) -> tuple[float, int]:
    """`uniform` (crates/stark-generate/src/hybrid.rs:1103-1111): (value in [0, 1), advanced state)."""
    st = C.c_uint64(state & (2**64 - 1))
    f = lib().so_splitmix64_uniform
    f.restype, f.argtypes = C.c_double, [C.POINTER(C.c_uint64)]
    return float(f(C.byref(st))), int(st.value)


def descending_sample_key(value: float) -> int:
    f = lib().so_descending_sample_key
    f.restype, f.argtypes = C.c_uint32, [C.c_float]
    return int(f(value))


def host_sampling(logits, rng: int, temperature: float = 1.0, top_k=None, top_p=None, min_p=None) -> tuple[int, int]:
    """The generation worker's stochastic host sampler (hybrid.rs:1122-1212): (token, advanced rng state);
    token 0xffffffff for an empty or non-finite row."""
    logits = _c(logits, np.float32)
    flags = (4 if top_k is not None else 0) | (8 if top_p is not None else 0) | (16 if min_p is not None else 0)
    st = C.c_uint64(rng & (2**64 - 1))
    f = lib().so_host_sampling_f64
    f.restype = C.c_uint32
    f.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint64), C.c_float, C.c_uint32, C.c_float, C.c_float]
    tok = int(f(_p(logits), logits.size, flags, C.byref(st), temperature, top_k or 0, top_p or 1.0, min_p or 0.0))
    return tok, int(st.value)


def log_softmax_f64(logits) -> np.ndarray:
    logits = _c(logits, np.float32)
    out = np.empty(logits.size, np.float64)
    lib().so_log_softmax_f64(_p(logits), _p(out), logits.size)
    return out


def softmax_f32(x):
    x = _c(x, np.float32)
    out = np.empty_like(x)
    if lib().so_softmax_f32(_p(x), _p(out), x.size):
        raise ValueError("softmax input")
    return out


def topk_f32(x, k):
    x = _c(x, np.float32)
    out = np.empty(k, np.uint32)
    if lib().so_topk_f32(_p(x), x.size, k, _p(out)):
        raise ValueError("top-k input")
    return out


def moe_route(logits, experts, active, round_weights=False, round_logits=False):
    logits = _c(logits, np.float32).reshape(-1, experts)
    rows = logits.shape[0]
    ids = np.zeros((rows, active), np.uint32)
    weights = np.zeros((rows, active), np.float32)
    lib().so_moe_route(_p(logits), _p(ids), _p(weights), rows, experts, active, int(round_weights),
                       int(round_logits))
    return ids, weights


# ----------------------------------------------------------------------------- dense decoder

class _QMat(C.Structure):
    _fields_ = [("codes", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p),
                ("n", C.c_uint32), ("k", C.c_uint32), ("bits", C.c_uint32), ("group", C.c_uint32)]


class _Layer(C.Structure):
    _fields_ = [("attn_norm", C.c_void_p), ("mlp_norm", C.c_void_p), ("q_norm", C.c_void_p),
                ("k_norm", C.c_void_p), ("qkv", _QMat), ("o", _QMat), ("upgate", _QMat), ("down", _QMat)]


class _Model(C.Structure):
    _fields_ = [("layers", C.c_uint32), ("hidden", C.c_uint32), ("q_heads", C.c_uint32),
                ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("inter", C.c_uint32), ("vocab", C.c_uint32),
                ("eps", C.c_float), ("rope_theta", C.c_float), ("embed", _QMat), ("lm_head", _QMat),
                ("final_norm", C.c_void_p), ("layer", C.POINTER(_Layer))]


class _State(C.Structure):
    _fields_ = [("keys", C.c_void_p), ("values", C.c_void_p), ("capacity", C.c_uint32), ("position", C.c_uint32)]


def _qmat(t: dict) -> _QMat:
    return _QMat(t["codes"].ctypes.data, t["scales"].ctypes.data, t["biases"].ctypes.data,
                 t["n"], t["k"], t["bits"], t["group"])


class DenseOracle:
    """Qwen3-shaped dense decoder on the CPU with the converted-model bf16 rounding points.

    ``weights`` is the dict produced by ``stark_b200.synthetic.dense_weights`` (numpy arrays in the
    MLX layout); the arrays are referenced, not copied, and must outlive this object.
    """

    def __init__(self, cfg: dict, weights: dict, capacity: int, threads: int | None = None):
        self.cfg = cfg
        self.w = weights
        self.threads = threads or max_threads()
        L = cfg["layers"]
        self._layers = (_Layer * L)()
        for i in range(L):
            lw = weights["layers"][i]
            self._layers[i] = _Layer(lw["attn_norm"].ctypes.data, lw["mlp_norm"].ctypes.data,
                                     lw["q_norm"].ctypes.data, lw["k_norm"].ctypes.data,
                                     _qmat(lw["qkv"]), _qmat(lw["o"]), _qmat(lw["upgate"]), _qmat(lw["down"]))
        self._model = _Model(L, cfg["hidden"], cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], cfg["inter"],
                             cfg["vocab"], cfg["eps"], cfg["rope_theta"], _qmat(weights["embed"]),
                             _qmat(weights["lm_head"]), weights["final_norm"].ctypes.data, self._layers)
        kv_row = cfg["kv_heads"] * cfg["head_dim"]
        self.keys = np.zeros((L, capacity, kv_row), np.uint16)
        self.values = np.zeros((L, capacity, kv_row), np.uint16)
        self._state = _State(self.keys.ctypes.data, self.values.ctypes.data, capacity, 0)

    @property
    def position(self) -> int:
        return int(self._state.position)

    def reset(self, position: int = 0):
        self._state.position = position

    def ingest(self, token: int):
        if lib().so_dense_step(C.byref(self._model), C.byref(self._state), token, None, None, self.threads):
            raise ValueError("invalid token or context overflow")

    def step(self, token: int, want_hidden: bool = False):
        """Returns bf16 logits (uint16 bit patterns) [vocab] (and the final normed row)."""
        logits = np.empty(self.cfg["vocab"], np.uint16)
        hidden = np.empty(self.cfg["hidden"], np.uint16) if want_hidden else None
        if lib().so_dense_step(C.byref(self._model), C.byref(self._state), token, _p(logits), _p(hidden),
                               self.threads):
            raise ValueError("invalid token or context overflow")
        return (logits, hidden) if want_hidden else logits


class MtpHeadOracle:
    """The dense multi-token-prediction head on the CPU (``so_mtp_head_step``): fusion of the token's embedding
    with the target's normalized hidden row, one decoder layer with its own cache, output norm, the target's
    read-out.  ``target`` is the ``DenseOracle`` whose tables and dimensions it shares; ``head`` is the dict of
    ``stark_b200.synthetic.mtp_weights``."""

    def __init__(self, target: "DenseOracle", head: dict, capacity: int):
        self.target, self.head, cfg = target, head, target.cfg
        lw = head["layer"]
        self._layer = _Layer(lw["attn_norm"].ctypes.data, lw["mlp_norm"].ctypes.data, lw["q_norm"].ctypes.data,
                             lw["k_norm"].ctypes.data, _qmat(lw["qkv"]), _qmat(lw["o"]), _qmat(lw["upgate"]),
                             _qmat(lw["down"]))
        self._fusion = _qmat(head["fusion"])
        kv_row = cfg["kv_heads"] * cfg["head_dim"]
        self.keys = np.zeros((capacity, kv_row), np.uint16)
        self.values = np.zeros((capacity, kv_row), np.uint16)
        self._state = _State(self.keys.ctypes.data, self.values.ctypes.data, capacity, 0)

    @property
    def position(self) -> int:
        return int(self._state.position)

    def rewind(self, position: int) -> None:
        self._state.position = position

    def _run(self, token: int, hidden, logits, out_hidden):
        hidden = _c(hidden, np.uint16)
        h = self.head
        if lib().so_mtp_head_step(C.byref(self.target._model), C.byref(self._layer), C.byref(self._fusion),
                                  _p(_c(h["embed_norm"], np.float32)), _p(_c(h["hidden_norm"], np.float32)),
                                  _p(_c(h["out_norm"], np.float32)), C.byref(self._state), int(token), _p(hidden),
                                  _p(logits), _p(out_hidden), self.target.threads):
            raise ValueError("invalid token, geometry or context overflow")

    def cache_row(self, token: int, hidden) -> None:
        """A cache-only row: the pair (token, normalized hidden of the row before it)."""
        self._run(token, hidden, None, None)

    def step(self, token: int, hidden):
        """(logits, normalized output): bf16 bit patterns; the output is the hidden of the next draft step."""
        logits = np.empty(self.target.cfg["vocab"], np.uint16)
        out = np.empty(self.target.cfg["hidden"], np.uint16)
        self._run(token, hidden, logits, out)
        return logits, out


# ----------------------------------------------------------------------------- routed experts (f32 host path)

def silu_f32(x: float) -> float:
    lib().so_silu_f32.restype = C.c_float
    return float(lib().so_silu_f32(C.c_float(x)))


def dense_matvec_f32(w, x):
    w = _c(w, np.float32)
    x = _c(x, np.float32)
    y = np.empty(w.shape[0], np.float32)
    lib().so_dense_matvec_f32(_p(w), _p(x), _p(y), w.shape[0], w.shape[1])
    return y


def moe_ffn_f32(kind_gate_up, gate_bank, up_bank, kind_down, down_bank, scores, x, experts, active, hidden, inter,
                threads=1):
    """Returns (out, ids, probabilities) of the routed-expert feed-forward."""
    gate_bank, up_bank, down_bank = _c(gate_bank, np.uint8), _c(up_bank, np.uint8), _c(down_bank, np.uint8)
    scores, x = _c(scores, np.float32), _c(x, np.float32)
    out = np.empty(hidden, np.float32)
    ids = np.empty(active, np.uint32)
    probs = np.empty(active, np.float32)
    rc = lib().so_moe_ffn_f32(kind_gate_up, _p(gate_bank), _p(up_bank), kind_down, _p(down_bank), _p(scores), _p(x),
                              _p(out), experts, active, hidden, inter, _p(ids), _p(probs), threads)
    if rc:
        raise ValueError("invalid expert geometry or inputs")
    return out, ids, probs


class _SoMoeModel(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("vocab", "hidden", "layers", "q_heads", "kv_heads", "head_dim", "experts",
                                          "active", "inter", "context")] + [
        ("eps", C.c_float), ("theta", C.c_float), ("embed", C.c_void_p), ("output", C.c_void_p),
        ("final_norm", C.c_void_p)] + [(n, C.POINTER(C.c_void_p)) for n in (
            "attn_norm", "ffn_norm", "q_norm", "k_norm", "wq", "wk", "wv", "wo", "router", "gate", "up", "down")]


class MoEDecoder:
    """The routed-expert decoder step of the hybrid host path (`so_moe_step`), over weights in the layout
    of ``stark_b200.synthetic.moe_weights`` ([q; k; v] rows fused in one Q8_0 array)."""

    def __init__(self, cfg: dict, weights: dict, context_tokens: int, threads: int = 0):
        self.cfg, self.context, self.threads = dict(cfg), int(context_tokens), threads or max_threads()
        self._keep = []
        L = cfg["layers"]
        qd, kd = cfg["q_heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"]

        def hold(a, dtype):
            a = np.ascontiguousarray(a, dtype)
            self._keep.append(a)
            return a.ctypes.data

        def per_layer(fn):
            arr = (C.c_void_p * L)(*[fn(w) for w in weights["layers"]])
            self._keep.append(arr)
            return C.cast(arr, C.POINTER(C.c_void_p))

        m = _SoMoeModel(cfg["vocab"], cfg["hidden"], L, cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"],
                        cfg["experts"], cfg["active"], cfg["inter"], self.context, cfg["eps"], cfg["rope_theta"])
        m.embed, m.output = hold(weights["token_table"], np.uint8), hold(weights["output"], np.uint8)
        m.final_norm = hold(weights["final_norm"], np.float32)
        rows = lambda w, lo, hi: np.asarray(w["qkv"], np.uint8).reshape(qd + 2 * kd, -1)[lo:hi]
        m.wq = per_layer(lambda w: hold(rows(w, 0, qd), np.uint8))
        m.wk = per_layer(lambda w: hold(rows(w, qd, qd + kd), np.uint8))
        m.wv = per_layer(lambda w: hold(rows(w, qd + kd, qd + 2 * kd), np.uint8))
        m.wo = per_layer(lambda w: hold(w["o"], np.uint8))
        for name in ("attn_norm", "ffn_norm", "q_norm", "k_norm", "router"):
            setattr(m, name, per_layer(lambda w, n=name: hold(w[n], np.float32)))
        for name in ("gate", "up", "down"):
            setattr(m, name, per_layer(lambda w, n=name: hold(w[n], np.uint8)))
        self._m = m
        kv = L * self.context * kd
        self.keys, self.values = np.zeros(kv, np.float32), np.zeros(kv, np.float32)
        self.position = 0
        self.last_experts = np.zeros((L, cfg["active"]), np.uint32)

    def reset(self):
        self.position = 0

    def step(self, token: int, want_logits: bool = True):
        logits = np.empty(self.cfg["vocab"], np.float32) if want_logits else None
        f = lib().so_moe_step
        f.restype = C.c_int
        f.argtypes = [C.POINTER(_SoMoeModel), C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p,
                      C.c_int]
        rc = f(C.byref(self._m), _p(self.keys), _p(self.values), self.position, int(token),
               _p(logits) if want_logits else None, _p(self.last_experts), self.threads)
        if rc != 0:
            raise ValueError("moe step")
        self.position += 1
        return logits

    def ingest(self, tokens):
        for t in tokens:
            self.step(int(t), want_logits=False)
