"""Host-side mirror of the reference's per-operator interface, over the C ABI.

Names follow the reference: a quantized ``B`` operand with MLX-affine planes
(``MatmulB::Quantized``, crates/stark-engine/src/backends/common/kernel/matmul/arguments.rs:7-24)
becomes :class:`QMatrix`; ``MatmulKernel::encode`` / ``Weights::matvec`` become :meth:`QMatrix.matvec`.
Arrays crossing this layer are numpy arrays of bit patterns (``uint16`` for bf16) or f32; device
pointers are plain integers.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import BF16, DEVICE, F32, HOST, check


def _ptr(a: np.ndarray) -> C.c_void_p:
    return a.ctypes.data_as(C.c_void_p)


def device_count() -> int:
    n = C.c_int32(0)
    _lib.load().stark_b200_device_count(C.byref(n))
    return n.value


def take_device_error() -> int:
    w = C.c_uint32(0)
    check(_lib.load().stark_b200_take_device_error(C.byref(w)), "take_device_error")
    return w.value


class DeviceBuffer:
    """A raw device allocation owned by the library's allocator."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        check(_lib.load().stark_b200_device_malloc(C.byref(p), self.nbytes), "device_malloc")
        self.ptr = p.value

    def upload(self, a: np.ndarray, stream: int = 0) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        lib = _lib.load()
        check(lib.stark_b200_memcpy_h2d(self.ptr, _ptr(a), a.nbytes, stream), "memcpy_h2d")
        check(lib.stark_b200_stream_synchronize(stream), "stream_synchronize")
        return self

    def download(self, dtype, count: int, stream: int = 0) -> np.ndarray:
        out = np.empty(count, dtype)
        lib = _lib.load()
        check(lib.stark_b200_memcpy_d2h(_ptr(out), self.ptr, out.nbytes, stream), "memcpy_d2h")
        check(lib.stark_b200_stream_synchronize(stream), "stream_synchronize")
        return out

    def free(self):
        if self.ptr:
            _lib.load().stark_b200_device_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class QMatrix:
    """A quantized weight matrix resident (re-tiled) in device memory."""

    def __init__(self, handle: int, rows: int, columns: int, pair_halves: bool = False):
        self._h = C.c_void_p(handle)
        self.rows, self.columns, self.pair_halves = rows, columns, pair_halves

    @classmethod
    def from_affine(cls, codes: np.ndarray, scales: np.ndarray, biases: np.ndarray, rows: int, columns: int,
                    bits: int = 4, group: int = 64, plane_kind: int = _lib.PLANE_BF16, scale_layout: int = 0,
                    plane_pitch: int = 0, pair_halves: bool = False) -> "QMatrix":
        """codes: MLX ``uint32[rows, columns*bits/32]`` (or the same bytes as uint8); planes: bit patterns."""
        codes = np.ascontiguousarray(codes)
        scales = np.ascontiguousarray(scales)
        biases = np.ascontiguousarray(biases)
        if codes.nbytes != rows * columns * bits // 8:
            raise ValueError("inconsistent affine planes")
        d = _lib.AffineDesc(C.sizeof(_lib.AffineDesc), _lib.ABI_VERSION, rows, columns, bits, group, plane_kind,
                            scale_layout, plane_pitch, HOST, int(pair_halves), 0)
        h = C.c_void_p()
        check(_lib.load().stark_b200_qmatrix_create_affine(_ptr(codes), _ptr(scales), _ptr(biases), C.byref(d),
                                                           C.byref(h)), "qmatrix_create_affine")
        return cls(h.value, rows, columns, pair_halves)

    @property
    def handle(self) -> int:
        return self._h.value

    def device_bytes(self) -> int:
        n = C.c_uint64(0)
        check(_lib.load().stark_b200_qmatrix_device_bytes(self._h, C.byref(n)), "qmatrix_device_bytes")
        return n.value

    def unpack_codes(self) -> np.ndarray:
        out = np.empty(self.rows * self.columns, np.uint8)
        check(_lib.load().stark_b200_qmatrix_unpack_codes(self._h, _ptr(out), out.size), "qmatrix_unpack_codes")
        return out.reshape(self.rows, self.columns)

    def matvec(self, x: np.ndarray, io_type: int = BF16) -> np.ndarray:
        """y = W x through host buffers (copies in and out inside the call)."""
        dt = np.float32 if io_type == F32 else np.uint16
        x = np.ascontiguousarray(x, dtype=dt)
        m = 1 if x.ndim == 1 else x.shape[0]
        if x.size != m * self.columns:
            raise ValueError("invalid matvec input shape or values")
        y = np.empty((m, self.rows), dt)
        check(_lib.load().stark_b200_op_qmv(self._h, _ptr(x), _ptr(y), m, io_type, HOST, None), "op_qmv")
        return y[0] if x.ndim == 1 else y

    def gemm(self, x: np.ndarray, epilogue: int = 0, residual: np.ndarray | None = None) -> np.ndarray:
        """Y = X W^T for many bf16 rows at once on the tensor cores (``stark_b200_op_qgemm``).
        epilogue 0: store; 1: ``bf16(bf16(product) + residual)``; 2: SwiGLU over a pair-ordered matrix."""
        x = np.ascontiguousarray(x, np.uint16)
        m = x.shape[0]
        if x.ndim != 2 or x.shape[1] != self.columns:
            raise ValueError("invalid gemm input shape")
        cols = self.rows // 2 if epilogue == 2 else self.rows
        y = np.ascontiguousarray(residual, np.uint16).copy() if epilogue == 1 else np.empty((m, cols), np.uint16)
        if y.shape != (m, cols):
            raise ValueError("invalid residual shape")
        check(_lib.load().stark_b200_op_qgemm(self._h, _ptr(x), _ptr(y), m, epilogue, HOST, None), "op_qgemm")
        return y

    def matvec_rows(self, x: np.ndarray, epilogue: int = 0, residual: np.ndarray | None = None,
                    norm_weight: np.ndarray | None = None, eps: float = 1e-6) -> np.ndarray:
        """Up to 8 bf16 rows against one pass over the matrix (``stark_b200_op_qmv_rows``): the verify pass of a
        speculative round.  ``norm_weight``: RMS norm of every row in the kernel's prologue.  Epilogues as ``gemm``."""
        x = np.ascontiguousarray(x, np.uint16)
        m = x.shape[0]
        if x.ndim != 2 or x.shape[1] != self.columns:
            raise ValueError("invalid input shape")
        cols = self.rows // 2 if epilogue == 2 else self.rows
        y = np.ascontiguousarray(residual, np.uint16).copy() if epilogue == 1 else np.empty((m, cols), np.uint16)
        if y.shape != (m, cols):
            raise ValueError("invalid residual shape")
        nw = None if norm_weight is None else np.ascontiguousarray(norm_weight, np.float32)
        if nw is not None and nw.shape != (self.columns,):
            raise ValueError("invalid norm weight shape")
        check(_lib.load().stark_b200_op_qmv_rows(self._h, _ptr(x), _ptr(y), m, epilogue, None if nw is None else _ptr(nw),
                                                 float(eps), HOST, None), "op_qmv_rows")
        return y

    def matvec_device(self, x_ptr: int, y_ptr: int, m: int = 1, io_type: int = BF16, stream: int = 0) -> None:
        check(_lib.load().stark_b200_op_qmv(self._h, x_ptr, y_ptr, m, io_type, DEVICE, stream), "op_qmv")

    def destroy(self):
        if self._h and self._h.value:
            _lib.load().stark_b200_qmatrix_destroy(C.byref(self._h))

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class Graph:
    """A recorded sequence of per-operator launches (device pointers only), replayed as one CUDA graph."""

    def __init__(self, stream: int):
        self.stream = stream
        self._h = C.c_void_p()

    def __enter__(self):
        check(_lib.load().stark_b200_graph_begin(self.stream), "graph_begin")
        return self

    def __exit__(self, exc_type, exc, tb):
        st = _lib.load().stark_b200_graph_end(self.stream, C.byref(self._h))
        if exc_type is None:
            check(st, "graph_end")
        return False

    def launch(self, stream: int | None = None):
        check(_lib.load().stark_b200_graph_launch(self._h, self.stream if stream is None else stream),
              "graph_launch")

    def destroy(self):
        if self._h and self._h.value:
            _lib.load().stark_b200_graph_destroy(C.byref(self._h))

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


# ----------------------------------------------------------------------------- small operators (host buffers)

def rmsnorm(x: np.ndarray, scales: np.ndarray, eps: float, shortcut: np.ndarray | None = None,
            residual_add: bool = False):
    """Returns (normed, shortcut_after) as bf16 bit patterns; mirrors Normalization::encode."""
    x = np.ascontiguousarray(x, np.uint16)
    scales = np.ascontiguousarray(scales, np.float32)
    out = np.empty_like(x)
    sc = None if shortcut is None else np.ascontiguousarray(shortcut, np.uint16).copy()
    check(_lib.load().stark_b200_op_rmsnorm(_ptr(x), _ptr(scales), _ptr(out), None if sc is None else _ptr(sc),
                                            x.size, eps, int(residual_add), HOST, None), "op_rmsnorm")
    return out, sc


def swiglu(fused: np.ndarray, gated_dim: int) -> np.ndarray:
    fused = np.ascontiguousarray(fused, np.uint16)
    out = np.empty(gated_dim, np.uint16)
    check(_lib.load().stark_b200_op_swiglu(_ptr(fused), _ptr(out), gated_dim, HOST, None), "op_swiglu")
    return out


def qmv_swiglu(q: QMatrix, x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.uint16)
    out = np.empty(q.rows // 2, np.uint16)
    check(_lib.load().stark_b200_op_qmv_swiglu(q._h, _ptr(x), _ptr(out), HOST, None), "op_qmv_swiglu")
    return out


def argmax(logits_bf16: np.ndarray) -> int:
    logits = np.ascontiguousarray(logits_bf16, np.uint16)
    out = C.c_uint32(0)
    check(_lib.load().stark_b200_op_argmax(_ptr(logits), logits.size, C.byref(out), HOST, None), "op_argmax")
    return out.value


def log_softmax(logits: np.ndarray) -> np.ndarray:
    logits = np.ascontiguousarray(logits, np.float32)
    out = np.empty(logits.size, np.float64)
    check(_lib.load().stark_b200_op_log_softmax(_ptr(logits), _ptr(out), logits.size, HOST, None),
          "op_log_softmax")
    return out


def sample(logits: np.ndarray, seed=None, temperature=None, top_k=None, top_p=None, min_p=None,
           ordered: bool = False) -> int:
    """One token from one row of logits (f32, or bf16 bit patterns as uint16) through the device sampler.
    ``ordered``: the generation worker's host-sampler semantics; ``seed`` is then the SplitMix64 state
    before the draw (advance it by ``_lib.SPLITMIX64_STEP`` per sampled token)."""
    logits = np.ascontiguousarray(logits)
    io = _lib.F32 if logits.dtype == np.float32 else _lib.BF16
    params = _lib.sampling(seed, temperature, top_k, top_p, min_p, ordered)
    tok = C.c_uint32(0)
    check(_lib.load().stark_b200_op_sample(_ptr(logits), logits.size, io, C.byref(params), C.byref(tok), HOST, None),
          "op_sample")
    return tok.value


def moe_route(logits: np.ndarray, experts: int, active: int, round_weights=False, round_logits=False):
    logits = np.ascontiguousarray(logits, np.float32).reshape(-1, experts)
    rows = logits.shape[0]
    ids = np.zeros((rows, active), np.uint32)
    weights = np.zeros((rows, active), np.float32)
    check(_lib.load().stark_b200_op_moe_route(_ptr(logits), _ptr(ids), _ptr(weights), rows, experts, active,
                                              int(round_weights), int(round_logits), HOST, None), "op_moe_route")
    return ids, weights


def attention_decode(qkv: np.ndarray, keys: np.ndarray, values: np.ndarray, q_heads: int, kv_heads: int,
                     position: int, eps: float = 1e-6, rope_theta: float = 1e6, q_norm=None, k_norm=None,
                     splits: int = 0) -> np.ndarray:
    """One decode row of attention with fused QK-norm, RoPE and cache append.

    keys/values: ``uint16[capacity, kv_heads, 128]`` with ``position`` valid rows; row ``position`` is
    written in place.  Returns ``uint16[q_heads * 128]``.
    """
    qkv = np.ascontiguousarray(qkv, np.uint16)
    assert keys.flags.c_contiguous and values.flags.c_contiguous and keys.dtype == np.uint16
    capacity = keys.shape[0]
    out = np.empty(q_heads * 128, np.uint16)
    d = _lib.AttentionDesc(C.sizeof(_lib.AttentionDesc), _lib.ABI_VERSION, q_heads, kv_heads, 128, position,
                           capacity, splits, eps, rope_theta)
    qn = None if q_norm is None else _ptr(np.ascontiguousarray(q_norm, np.float32))
    kn = None if k_norm is None else _ptr(np.ascontiguousarray(k_norm, np.float32))
    check(_lib.load().stark_b200_op_attention_decode(_ptr(qkv), _ptr(keys), _ptr(values), _ptr(out), qn, kn,
                                                     C.byref(d)), "op_attention_decode")
    return out


def prompt_attention(qkv: np.ndarray, keys: np.ndarray, values: np.ndarray, block_table: np.ndarray, first_pos: int,
                     q_heads: int, kv_heads: int, tensor_memory: bool = True) -> np.ndarray:
    """Causal attention of the rows of one prompt pass over a paged cache (attention_single_pass.rs:11-133, many rows).

    qkv: ``uint16[m, q_heads + 2 kv_heads, 128]`` with the query heads already normalized and rotated; keys / values:
    ``uint16[pages, kv_heads, 64, 128]`` holding positions ``0 .. first_pos + m - 1`` (the pass's own rows included)
    through ``block_table`` (``int32[pages]``: logical page -> physical page).  ``tensor_memory`` selects the tcgen05
    kernel (more than 16 rows) over the mma.sync one.  Returns ``uint16[m, q_heads, 128]``.
    """
    qkv = np.ascontiguousarray(qkv, np.uint16)
    keys, values = np.ascontiguousarray(keys, np.uint16), np.ascontiguousarray(values, np.uint16)
    table = np.ascontiguousarray(block_table, np.int32)
    m = qkv.shape[0]
    assert qkv.shape[1:] == (q_heads + 2 * kv_heads, 128) and keys.shape == values.shape == (len(table), kv_heads, 64, 128)
    out = np.zeros((m, q_heads, 128), np.uint16)
    check(_lib.load().stark_b200_op_prefill_attention(_ptr(qkv), _ptr(keys), _ptr(values), _ptr(table), len(table),
                                                      _ptr(out), m, int(first_pos), q_heads, kv_heads,
                                                      1 if tensor_memory else 0), "op_prefill_attention")
    return out


# ----------------------------------------------------------------------------- GGUF / 8-bit matrices, expert banks

def _qmatrix_from_gguf(blocks: np.ndarray, kind: int, rows: int, columns: int, experts: int = 0) -> QMatrix:
    blocks = np.ascontiguousarray(blocks, np.uint8)
    h = C.c_void_p()
    lib = _lib.load()
    if experts:
        check(lib.stark_b200_qmatrix_create_gguf_bank(_ptr(blocks), kind, experts, rows, columns, HOST, C.byref(h)),
              "qmatrix_create_gguf_bank")
    else:
        check(lib.stark_b200_qmatrix_create_gguf(_ptr(blocks), kind, rows, columns, HOST, C.byref(h)),
              "qmatrix_create_gguf")
    q = QMatrix(h.value, rows, columns)
    q.experts = experts or 1
    return q


QMatrix.from_gguf = staticmethod(_qmatrix_from_gguf)


def dequantize_row(q: QMatrix, row: int, expert: int = 0) -> np.ndarray:
    out = np.empty(q.columns, np.float32)
    check(_lib.load().stark_b200_qmatrix_dequantize_row(q._h, expert, row, _ptr(out)), "qmatrix_dequantize_row")
    return out


def matvec_experts(bank: QMatrix, expert_ids, x: np.ndarray, shared_input: bool, io_type: int = F32) -> np.ndarray:
    """``Weights::selected_matvec``: y[i] = W[expert_ids[i]] x_i (or x if shared)."""
    ids = np.ascontiguousarray(expert_ids, np.uint32)
    dt = np.float32 if io_type == F32 else np.uint16
    x = np.ascontiguousarray(x, dt)
    y = np.empty((ids.size, bank.rows), dt)
    check(_lib.load().stark_b200_op_qmv_experts(bank._h, _ptr(ids), ids.size, _ptr(x), int(shared_input), _ptr(y),
                                                io_type, HOST, None), "op_qmv_experts")
    return y


def dense_matvec_f32(w: np.ndarray, x: np.ndarray) -> np.ndarray:
    w = np.ascontiguousarray(w, np.float32)
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(w.shape[0], np.float32)
    check(_lib.load().stark_b200_op_dense_matvec_f32(_ptr(w), _ptr(x), _ptr(y), w.shape[0], w.shape[1], HOST, None),
          "op_dense_matvec_f32")
    return y


def moe_ffn(gate: QMatrix, up: QMatrix, down: QMatrix, scores: np.ndarray, x: np.ndarray, active: int):
    """Routed-expert feed-forward (hybrid host path).  Returns (out, ids, probabilities)."""
    scores = np.ascontiguousarray(scores, np.float32)
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(down.rows, np.float32)
    ids = np.empty(active, np.uint32)
    probs = np.empty(active, np.float32)
    check(_lib.load().stark_b200_op_moe_ffn(gate._h, up._h, down._h, _ptr(scores), _ptr(x), _ptr(out), active,
                                            _ptr(ids), _ptr(probs), HOST, None), "op_moe_ffn")
    return out, ids, probs
