"""ctypes binding of ``libstark_b200.so`` (the C ABI in ``include/stark_b200.h``).

The library is the product: there is no Python or CPU fallback.  If it has not been built, or a
call returns a non-zero status, this module raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libstark_b200.so"

ABI_VERSION = 1
HOST, DEVICE = 0, 1
BF16, F32 = 0, 1
PLANE_F32, PLANE_F16, PLANE_BF16 = 0, 1, 30
GGUF_Q8_0, GGUF_Q4_K = 8, 12

STATUS_NAMES = ["ok", "invalid_argument", "abi_mismatch", "context_limit", "cancelled", "unsupported",
                "out_of_memory", "io_failure", "device_failure", "reload_required", "busy", "invalid_state"]


class StarkB200Error(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else "unknown"
        super().__init__(f"{where}: {name} ({status})")


class AffineDesc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "struct_size", "abi_version", "rows", "columns", "bits", "group", "plane_kind", "scale_layout",
        "plane_pitch", "location", "pair_halves", "reserved")]


class AttentionDesc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("struct_size", "abi_version", "q_heads", "kv_heads", "head_dim",
                                          "position", "capacity", "splits")] + [("epsilon", C.c_float),
                                                                                 ("rope_theta", C.c_float)]


class DenseConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("struct_size", "abi_version", "layers", "hidden", "q_heads", "kv_heads",
                                          "head_dim", "inter", "vocab", "tied", "context_tokens")] + [
        ("eps", C.c_float), ("rope_theta", C.c_float), ("reserved", C.c_uint32)]


class MoeConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("struct_size", "vocab", "hidden", "layers", "q_heads", "kv_heads", "head_dim",
                                          "experts", "active_experts", "expert_intermediate", "context_tokens")] + [
        ("rms_eps", C.c_float), ("rope_theta", C.c_float)]


MOE_MAT_QKV, MOE_MAT_O, MOE_MAT_GATE_UP, MOE_MAT_DOWN, MOE_MAT_OUTPUT = range(5)
(MOE_ATTN_NORM, MOE_FFN_NORM, MOE_Q_NORM, MOE_K_NORM, MOE_FINAL_NORM, MOE_ROUTER, MOE_TOKEN_TABLE) = range(7)


class Info(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("abi_version", C.c_uint32), ("vocab_size", C.c_uint32),
                ("prefill_chunk_tokens", C.c_uint32), ("context_tokens", C.c_uint64), ("position", C.c_uint64),
                ("capabilities", C.c_uint64), ("fenced", C.c_uint32), ("launches_per_step", C.c_uint32),
                ("weight_bytes", C.c_uint64), ("kv_bytes_per_token", C.c_uint64), ("launches_issued", C.c_uint64),
                ("trace_slots", C.c_uint32), ("persistent", C.c_uint32)]


(MAT_EMBED, MAT_LM_HEAD, MAT_QKV, MAT_O, MAT_UPGATE, MAT_DOWN, MAT_MTP_FUSION, MAT_O_ROWS,
 MAT_DOWN_ROWS) = range(9)
(VEC_FINAL_NORM, VEC_ATTN_NORM, VEC_MLP_NORM, VEC_Q_NORM, VEC_K_NORM, VEC_MTP_EMBED_NORM, VEC_MTP_HIDDEN_NORM,
 VEC_MTP_OUT_NORM) = range(8)
MTP_GREEDY, MTP_FORCED, MTP_HELD = 0, 1, 2


class LoadOptions(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("abi_version", C.c_uint32), ("context_tokens", C.c_uint64),
                ("flags", C.c_uint64)]


class MtpRoundResult(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("abi_version", C.c_uint32), ("count", C.c_uint32),
                ("accepted", C.c_uint32), ("proposed", C.c_uint32), ("next_pending", C.c_uint32),
                ("tokens", C.c_uint32 * 8), ("position", C.c_uint64)]


class Sampling(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("flags", C.c_uint32), ("seed", C.c_uint64),
                ("temperature", C.c_float), ("top_k", C.c_uint32), ("top_p", C.c_float), ("min_p", C.c_float)]


SPLITMIX64_STEP = 0x9E3779B97F4A7C15


def sampling(seed=None, temperature=None, top_k=None, top_p=None, min_p=None, ordered=False) -> Sampling:
    """``seed`` None = no noise (greedy over whatever the filters keep).  ``ordered`` selects the generation
    worker's host-sampler semantics (sorted f64 probabilities, one SplitMix64 draw; ``seed`` is the
    generator state before the draw)."""
    flags = (1 if seed is not None else 0) | (2 if temperature is not None else 0) | (4 if top_k is not None else 0) \
        | (8 if top_p is not None else 0) | (16 if min_p is not None else 0) | (32 if ordered else 0)
    return Sampling(C.sizeof(Sampling), flags, seed or 0, temperature if temperature is not None else 1.0,
                    top_k or 0, top_p if top_p is not None else 1.0, min_p if min_p is not None else 0.0)


_lib = None


def load() -> C.CDLL:
    """Load the shared library; raises if it is missing (build it with ``python -m stark_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA library has not been built "
            "(run `python -m stark_b200.build`); there is no fallback path")
    lib = C.CDLL(str(LIB_PATH))
    vp, u32, u64, sz = C.c_void_p, C.c_uint32, C.c_uint64, C.c_size_t
    sig = {
        "stark_b200_abi_version": (u32, []),
        "stark_b200_status_name": (C.c_char_p, [u32]),
        "stark_b200_last_cuda_error": (C.c_char_p, []),
        "stark_b200_device_count": (u32, [C.POINTER(C.c_int32)]),
        "stark_b200_device_memory": (u32, [C.POINTER(u64), C.POINTER(u64)]),
        "stark_b200_set_device": (u32, [C.c_int32]),
        "stark_b200_device_malloc": (u32, [C.POINTER(vp), sz]),
        "stark_b200_device_free": (u32, [vp]),
        "stark_b200_memcpy_h2d": (u32, [vp, vp, sz, vp]),
        "stark_b200_memcpy_d2h": (u32, [vp, vp, sz, vp]),
        "stark_b200_stream_synchronize": (u32, [vp]),
        "stark_b200_take_device_error": (u32, [C.POINTER(u32)]),
        "stark_b200_qmatrix_create_affine": (u32, [vp, vp, vp, C.POINTER(AffineDesc), C.POINTER(vp)]),
        "stark_b200_qmatrix_create_gguf": (u32, [vp, u32, u32, u32, u32, C.POINTER(vp)]),
        "stark_b200_qmatrix_create_gguf_bank": (u32, [vp, u32, u32, u32, u32, u32, C.POINTER(vp)]),
        "stark_b200_qmatrix_dequantize_row": (u32, [vp, u32, u32, vp]),
        "stark_b200_op_qmv_experts": (u32, [vp, vp, u32, vp, u32, vp, u32, u32, vp]),
        "stark_b200_op_dense_matvec_f32": (u32, [vp, vp, vp, u32, u32, u32, vp]),
        "stark_b200_op_moe_ffn": (u32, [vp, vp, vp, vp, vp, vp, u32, vp, vp, u32, vp]),
        "stark_b200_qmatrix_destroy": (u32, [C.POINTER(vp)]),
        "stark_b200_qmatrix_device_bytes": (u32, [vp, C.POINTER(u64)]),
        "stark_b200_qmatrix_unpack_codes": (u32, [vp, vp, sz]),
        "stark_b200_op_qmv": (u32, [vp, vp, vp, u32, u32, u32, vp]),
        "stark_b200_op_qgemm": (u32, [vp, vp, vp, u32, u32, u32, vp]),
        "stark_b200_op_qmv_rows": (u32, [vp, vp, vp, u32, u32, vp, C.c_float, u32, vp]),
        "stark_b200_op_rmsnorm": (u32, [vp, vp, vp, vp, u32, C.c_float, u32, u32, vp]),
        "stark_b200_op_swiglu": (u32, [vp, vp, u32, u32, vp]),
        "stark_b200_op_qmv_swiglu": (u32, [vp, vp, vp, u32, vp]),
        "stark_b200_op_argmax": (u32, [vp, u32, C.POINTER(u32), u32, vp]),
        "stark_b200_op_log_softmax": (u32, [vp, vp, u32, u32, vp]),
        "stark_b200_op_moe_route": (u32, [vp, vp, vp, u32, u32, u32, u32, u32, u32, vp]),
        "stark_b200_op_attention_decode": (u32, [vp, vp, vp, vp, vp, vp, C.POINTER(AttentionDesc)]),
        "stark_b200_op_attention_decode_static": (u32, [vp, vp, vp, vp, vp, vp, vp, vp, vp,
                                                        C.POINTER(AttentionDesc), vp]),
        "stark_b200_model_create": (u32, [C.POINTER(DenseConfig), C.POINTER(vp)]),
        "stark_b200_load": (u32, [C.c_char_p, sz, C.POINTER(LoadOptions), C.POINTER(vp)]),
        "stark_b200_model_set_affine": (u32, [vp, u32, u32, vp, vp, vp, C.POINTER(AffineDesc)]),
        "stark_b200_model_set_vector": (u32, [vp, u32, u32, vp, u32]),
        "stark_b200_model_tp_init": (u32, [vp, u32, u32, u32, u32, vp]),
        "stark_b200_model_tp_connect": (u32, [vp, vp, sz]),
        "stark_b200_model_tp_set_wait": (u32, [vp, u64]),
        "stark_b200_model_tp_connect_unanswered": (u32, [vp]),
        "stark_b200_op_prefill_attention": (u32, [vp, vp, vp, vp, u32, vp, u32, u32, u32, u32, u32]),
        "stark_b200_model_tp_rows_init": (u32, [vp, vp]),
        "stark_b200_model_tp_rows_connect": (u32, [vp, vp, sz]),
        "stark_b200_model_finalize": (u32, [vp]),
        "stark_b200_destroy": (u32, [C.POINTER(vp)]),
        "stark_b200_reset": (u32, [vp]),
        "stark_b200_drain": (u32, [vp]),
        "stark_b200_cancel": (u32, [vp]),
        "stark_b200_prefill": (u32, [vp, vp, sz]),
        "stark_b200_step": (u32, [vp, u32]),
        "stark_b200_readout_f32": (u32, [vp, vp, sz]),
        "stark_b200_readout_bf16": (u32, [vp, vp, sz]),
        "stark_b200_readout_logprobs_f32": (u32, [vp, vp, sz]),
        "stark_b200_argmax": (u32, [vp, C.POINTER(u32)]),
        "stark_b200_sample": (u32, [vp, C.POINTER(Sampling), C.POINTER(u32)]),
        "stark_b200_op_sample": (u32, [vp, u32, u32, C.POINTER(Sampling), C.POINTER(u32), u32, vp]),
        "stark_b200_generate_greedy": (u32, [vp, u32, vp]),
        "stark_b200_rewind": (u32, [vp, u64]),
        "stark_b200_get_info": (u32, [vp, C.POINTER(Info)]),
        "stark_b200_model_stream": (u32, [vp, C.POINTER(vp)]),
        "stark_b200_mtp_initial": (u32, [vp, C.POINTER(u32)]),
        "stark_b200_mtp_round": (u32, [vp, u32, u32, u32, u32, C.POINTER(MtpRoundResult)]),
        "stark_b200_mtp_round_lookup": (u32, [vp, u32, vp, u32, u32, u32, C.POINTER(MtpRoundResult)]),
        "stark_b200_mtp_commit": (u32, [vp, u32, u32, C.POINTER(MtpRoundResult)]),
        "stark_b200_mtp_readout_row_f32": (u32, [vp, u32, vp, sz]),
        "stark_b200_set_tunable": (u32, [C.c_char_p, u32]),
        "stark_b200_model_recapture": (u32, [vp]),
        "stark_b200_read_trace": (u32, [vp, vp, sz]),
        "stark_b200_moe_model_create": (u32, [C.POINTER(MoeConfig), C.POINTER(vp)]),
        "stark_b200_moe_model_set_matrix": (u32, [vp, u32, u32, vp]),
        "stark_b200_moe_model_set_tensor": (u32, [vp, u32, u32, vp, sz]),
        "stark_b200_moe_model_ep_init": (u32, [vp, u32, u32, vp]),
        "stark_b200_moe_model_ep_connect": (u32, [vp, vp, sz]),
        "stark_b200_moe_model_ep_set_wait": (u32, [vp, u64]),
        "stark_b200_moe_model_reset": (u32, [vp]),
        "stark_b200_moe_model_ingest": (u32, [vp, vp, u32]),
        "stark_b200_moe_model_step": (u32, [vp, u32, vp, sz]),
        "stark_b200_moe_model_generate_greedy": (u32, [vp, u32, u32, vp]),
        "stark_b200_moe_model_last_experts": (u32, [vp, vp, sz]),
        "stark_b200_moe_model_position": (u32, [vp, C.POINTER(u32)]),
        "stark_b200_moe_model_launches_per_token": (u32, [vp, C.POINTER(u32)]),
        "stark_b200_moe_model_stream": (u32, [vp, C.POINTER(vp)]),
        "stark_b200_moe_model_destroy": (u32, [C.POINTER(vp)]),
        "stark_b200_graph_begin": (u32, [vp]),
        "stark_b200_graph_end": (u32, [vp, C.POINTER(vp)]),
        "stark_b200_graph_launch": (u32, [vp, vp]),
        "stark_b200_graph_destroy": (u32, [C.POINTER(vp)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.stark_b200_abi_version() != ABI_VERSION:
        raise RuntimeError("libstark_b200.so ABI version mismatch")
    _lib = lib
    return lib


def check(status: int, where: str) -> None:
    if status != 0:
        detail = ""
        if status in (6, 8) and _lib is not None:
            detail = " [" + _lib.stark_b200_last_cuda_error().decode() + "]"
        raise StarkB200Error(status, where + detail)
