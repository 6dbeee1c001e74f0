"""Reader (and, for tests and synthetic models, writer) of the reference's converted-model artifact.

An artifact is a directory with ``config.json`` and ``model.safetensors`` in the layout the reference's
converter emits for dense Qwen3-style decoders
(tools/converter/stark_convert/qwen3.py:137-430, compressed.py:143-200, streaming.py:742-795) and its
engine loads (crates/stark-engine/src/parameters/loader.rs:80-128, 373-408;
encodable_block/weight_matrix.rs:113-216):

* ``config.json``: ``{"type": "LanguageModelConfig", "decoder_config": {...}}`` with per-layer
  ``mixer_config`` (``num_heads``, ``num_groups``, ``head_dim``), norm ``epsilon``, ``rope_config.base``,
  ``transformer_config.model_dim`` / ``hidden_dim``, ``vocab_size`` and a tied or untied embedding.
* ``model.safetensors``: 8-byte little-endian header length, JSON header, raw tensors.  A quantized
  matrix ``<m>`` is three tensors: ``<m>.weights`` (U8 ``[rows, columns*bits/8]``, the MLX packing
  byte for byte), ``<m>.scales`` and ``<m>.biases`` (BF16), whose layout the header's ``__metadata__``
  entry ``<m>.spec`` names: ``input_output`` = ``[rows, groups]``, ``output_input`` =
  ``[groups, round_up4(rows)]``.  Norm weights are ``<n>.scales`` (F32).  Matrix names: the fused
  ``[q; k; v]`` and ``[up; gate]`` projections, ``out_projection``, ``down_projection``, and the
  embedding (``decoder.embedding.embedding`` when tied, else ``input_embedding`` / ``output_embedding``).

Like the reference's loader this one refuses an artifact it does not fully understand: every tensor
must be consumed, and configuration features outside the dense path (sliding windows, biases, soft
caps, gates, other spec types or bit widths) raise ``ArtifactError``.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


class ArtifactError(ValueError):
    pass


_DTYPES = {"U8": np.uint8, "BF16": np.uint16, "F32": np.float32}
MAX_HEADER_BYTES = 100 * 1024 * 1024  # parameters/safetensors_metadata.rs:117-132


def _read_safetensors(path: Path) -> tuple[dict, dict, np.memmap]:
    size = path.stat().st_size
    with path.open("rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise ArtifactError("safetensors file is shorter than its header length field")
        (n,) = struct.unpack("<Q", raw)
        if n > MAX_HEADER_BYTES or 8 + n > size:
            raise ArtifactError("safetensors header length is out of bounds")
        header = json.loads(f.read(n).decode("utf-8"))
    metadata = header.pop("__metadata__", {}) or {}
    data = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + n)
    return header, metadata, data


def _tensor(header: dict, data: np.ndarray, name: str, dtype: str, shape: tuple, used: set) -> np.ndarray:
    if name not in header:
        raise ArtifactError(f"missing tensor {name}")
    info = header[name]
    if info["dtype"] != dtype or tuple(info["shape"]) != tuple(shape):
        raise ArtifactError(f"tensor {name} is {info['dtype']}{info['shape']}, expected {dtype}{list(shape)}")
    lo, hi = info["data_offsets"]
    nbytes = int(np.prod(shape)) * np.dtype(_DTYPES[dtype]).itemsize
    if hi - lo != nbytes or lo < 0 or hi > data.size:
        raise ArtifactError(f"tensor {name} has inconsistent data offsets")
    used.add(name)
    return np.frombuffer(data[lo:hi], dtype=_DTYPES[dtype]).reshape(shape)


def _matrix(header, metadata, data, name: str, rows: int, columns: int, used: set) -> dict:
    spec = json.loads(metadata.get(name + ".spec", "{}"))
    if spec.get("type") != "MLXSpec" or spec.get("group_size") != 64 or spec.get("bits") not in (4, 8):
        raise ArtifactError(f"{name}: only MLX affine 4/8-bit group-64 matrices are supported, got {spec}")
    bits, groups = spec["bits"], columns // 64
    codes = _tensor(header, data, name + ".weights", "U8", (rows, columns * bits // 8), used)
    if spec["layout"] == "input_output":
        shape, layout, pitch = (rows, groups), 0, 0
    elif spec["layout"] == "output_input":
        pitch = rows + (-rows % 4)
        shape, layout = (groups, pitch), 1
    else:
        raise ArtifactError(f"{name}: unknown plane layout {spec['layout']}")
    scales = _tensor(header, data, name + ".scales", "BF16", shape, used)
    biases = _tensor(header, data, name + ".biases", "BF16", shape, used)
    codes = codes.view(np.uint32).reshape(rows, columns // 8) if bits == 4 else codes
    return dict(codes=codes, scales=scales, biases=biases, n=rows, k=columns, bits=bits, group=64,
                scale_layout=layout, plane_pitch=pitch)


def row_major_planes(t: dict) -> dict:
    """The same matrix with ``[rows, groups]`` planes (what row / column sharding slices)."""
    if not t.get("scale_layout"):
        return t
    rows = t["n"]
    return dict(t, scales=np.ascontiguousarray(t["scales"][:, :rows].T),
                biases=np.ascontiguousarray(t["biases"][:, :rows].T), scale_layout=0, plane_pitch=0)


def _require(cond: bool, what: str):
    if not cond:
        raise ArtifactError(what + " is outside the dense decode path this engine implements")


def read_artifact(directory) -> tuple[dict, dict]:
    """Returns ``(cfg, weights)`` in the form ``DenseModel.load`` takes (``stark_b200.synthetic`` keys)."""
    directory = Path(directory)
    root = json.loads((directory / "config.json").read_text())
    _require(root.get("type") == "LanguageModelConfig", f"config type {root.get('type')}")
    dec = root["decoder_config"]
    tr = dec["transformer_config"]
    layers = tr["layer_configs"]
    _require(len(layers) > 0, "an empty decoder")
    first = layers[0]
    mixer, rope, norm = first["mixer_config"], first["rope_config"], first["pre_mixer_norm_config"]
    tied = {"TiedEmbeddingConfig": True, "UntiedEmbeddingConfig": False}.get(dec["embedding_config"]["type"])
    _require(tied is not None, "embedding type " + str(dec["embedding_config"]["type"]))
    for key in ("input_scale", "logit_soft_cap", "logit_scale"):
        _require(dec["embedding_config"].get(key) is None, "embedding " + key)
    _require(dec.get("ple_model_config") is None and dec.get("embedding_norm_config") is None, "embedding extras")
    for lc in layers:
        m = lc["mixer_config"]
        _require(lc == first, "layers that differ from one another")
        _require(m["type"] == "AttentionConfig" and m["is_causal"] and m["scale"] is None, "this attention form")
        _require(m["sliding_window_size"] is None and m["logit_soft_cap"] is None and not m["has_sinks"],
                 "windowed / capped / sink attention")
        _require(not (m["has_qkvg_biases"] or m["has_out_biases"] or m["has_gate"] or m["normalize_values"]
                      or m["is_kv_sharing"]), "attention biases, gates or KV sharing")
        _require(lc["mlp_config"]["type"] == "DenseMLPConfig" and lc["mlp_config"]["activation"]["type"] == "SiLU",
                 "this feed-forward form")
        _require(lc["rope_config"]["type"] == "UnscaledRoPEConfig", "scaled RoPE")
        for key in ("mixer_conv_config", "post_mixer_norm_config", "mlp_conv_config", "post_mlp_norm_config",
                    "ple_config", "kv_source_layer_index"):
            _require(lc.get(key) is None, key)
        for n in (lc["pre_mixer_norm_config"], lc["pre_mlp_norm_config"], m["query_norm_config"], m["key_norm_config"]):
            _require(n == norm and n["scale_offset"] is None and not n["subtract_mean"] and n["has_scale"]
                     and not n["has_biases"], "this norm form")
    _require(tr["output_norm_config"] == norm, "a different output norm")
    cfg = dict(layers=len(layers), hidden=tr["model_dim"], q_heads=mixer["num_heads"], kv_heads=mixer["num_groups"],
               head_dim=mixer["head_dim"], inter=tr["hidden_dim"], vocab=dec["vocab_size"], tied=tied,
               eps=float(norm["epsilon"]), rope_theta=float(rope["base"]))
    _require(cfg["head_dim"] == 128, f"head_dim {cfg['head_dim']}")

    header, metadata, data = _read_safetensors(directory / "model.safetensors")
    used: set = set()
    D, hd, inter, V = cfg["hidden"], cfg["head_dim"], cfg["inter"], cfg["vocab"]
    qw, kw = cfg["q_heads"] * hd, cfg["kv_heads"] * hd

    def mat(name, rows, columns):
        return _matrix(header, metadata, data, name, rows, columns, used)

    def vec(name, width):
        return _tensor(header, data, name + ".scales", "F32", (width,), used)

    out = {"layers": []}
    if tied:
        out["embed"] = out["lm_head"] = mat("decoder.embedding.embedding", V, D)
    else:
        out["embed"] = mat("decoder.embedding.input_embedding", V, D)
        out["lm_head"] = mat("decoder.embedding.output_embedding", V, D)
    for i in range(cfg["layers"]):
        p = f"decoder.transformer.layers.{i}"
        out["layers"].append(dict(
            attn_norm=vec(p + ".pre_mixer_norm", D), mlp_norm=vec(p + ".pre_mlp_norm", D),
            q_norm=vec(p + ".mixer.query_norm", hd), k_norm=vec(p + ".mixer.key_norm", hd),
            qkv=mat(p + ".mixer.qkvg_projection.weights", qw + 2 * kw, D),
            o=mat(p + ".mixer.out_projection.weights", D, qw),
            upgate=mat(p + ".mlp.up_projection.weights", 2 * inter, D),
            down=mat(p + ".mlp.down_projection.weights", D, inter)))
    out["final_norm"] = vec("decoder.transformer.output_norm", D)
    extra = set(header) - used
    if extra:  # language_model/mod.rs:125: every tensor must be consumed
        raise ArtifactError(f"artifact has {len(extra)} tensors the decoder does not use, e.g. {sorted(extra)[0]}")
    return cfg, out


# ----------------------------------------------------------------------------- writer (tests, synthetic models)

def write_artifact(directory, cfg: dict, weights: dict) -> None:
    """Writes ``cfg`` / ``weights`` (row-major planes) as an artifact in the converter's layout."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    norm = {"epsilon": cfg["eps"], "scale_offset": None, "upcast_mode": "only_normalization", "subtract_mean": False,
            "has_scale": True, "has_biases": False}
    rope = {"type": "UnscaledRoPEConfig", "base": cfg["rope_theta"], "max_sequence_length": 32768,
            "head_dim": cfg["head_dim"]}
    mlp = {"type": "DenseMLPConfig", "linear_config": {}, "activation": {"type": "SiLU", "alpha": 1.0},
           "has_up_biases": False, "has_down_biases": False, "gate_clipping": None, "up_clipping": None}
    mixer = {"type": "AttentionConfig", "qkvg_projection_config": {}, "out_projection_config": {},
             "query_norm_config": norm, "key_norm_config": norm, "num_heads": cfg["q_heads"],
             "num_groups": cfg["kv_heads"], "head_dim": cfg["head_dim"], "is_causal": True, "scale": None,
             "sliding_window_size": None, "logit_soft_cap": None, "has_sinks": False, "has_qkvg_biases": False,
             "has_out_biases": False, "has_gate": False, "normalize_values": False, "is_kv_sharing": False}
    layer = {"pre_mixer_norm_config": norm, "mixer_conv_config": None, "mixer_config": mixer,
             "post_mixer_norm_config": None, "pre_mlp_norm_config": norm, "mlp_conv_config": None, "mlp_config": mlp,
             "post_mlp_norm_config": None, "hidden_dim": None, "ple_config": None, "has_post_layer_scalar": False,
             "kv_source_layer_index": None, "rope_config": rope}
    root = {"type": "LanguageModelConfig", "decoder_config": {
        "embedding_config": {"type": "TiedEmbeddingConfig" if cfg["tied"] else "UntiedEmbeddingConfig",
                             "input_scale": None, "logit_soft_cap": None, "logit_scale": None},
        "transformer_config": {"layer_configs": [layer] * cfg["layers"], "output_norm_config": norm,
                               "model_dim": cfg["hidden"], "hidden_dim": cfg["inter"]},
        "vocab_size": cfg["vocab"], "ple_model_config": None, "embedding_norm_config": None}}
    (directory / "config.json").write_text(json.dumps(root, indent=4))

    tensors, metadata = [], {}

    def put(name, dtype, array):
        tensors.append((name, dtype, np.ascontiguousarray(array)))

    def mat(name, t, layout):
        t = row_major_planes(t)
        rows, groups = t["n"], t["k"] // t["group"]
        put(name + ".weights", "U8", np.ascontiguousarray(t["codes"]).view(np.uint8).reshape(rows, -1))
        for plane in ("scales", "biases"):
            src = np.asarray(t[plane], np.uint16).reshape(rows, groups)
            if layout == "output_input":
                padded = np.zeros((groups, rows + (-rows % 4)), np.uint16)
                padded[:, :rows] = src.T
                src = padded
            put(name + "." + plane, "BF16", src)
        metadata[name + ".spec"] = json.dumps({"type": "MLXSpec", "bits": t["bits"], "group_size": t["group"],
                                               "layout": layout})

    def vec(name, v):
        put(name + ".scales", "F32", np.asarray(v, np.float32))

    if cfg["tied"]:
        mat("decoder.embedding.embedding", weights["embed"], "input_output")
    else:
        mat("decoder.embedding.input_embedding", weights["embed"], "input_output")
        mat("decoder.embedding.output_embedding", weights["lm_head"], "output_input")
    for i, lw in enumerate(weights["layers"]):
        p = f"decoder.transformer.layers.{i}"
        vec(p + ".pre_mixer_norm", lw["attn_norm"])
        vec(p + ".pre_mlp_norm", lw["mlp_norm"])
        vec(p + ".mixer.query_norm", lw["q_norm"])
        vec(p + ".mixer.key_norm", lw["k_norm"])
        mat(p + ".mixer.qkvg_projection.weights", lw["qkv"], "output_input")
        mat(p + ".mixer.out_projection.weights", lw["o"], "output_input")
        mat(p + ".mlp.up_projection.weights", lw["upgate"], "output_input")
        mat(p + ".mlp.down_projection.weights", lw["down"], "output_input")
    vec("decoder.transformer.output_norm", weights["final_norm"])

    header, offset = {"__metadata__": metadata}, 0
    for name, dtype, array in tensors:
        header[name] = {"dtype": dtype, "shape": list(array.shape), "data_offsets": [offset, offset + array.nbytes]}
        offset += array.nbytes
    encoded = json.dumps(header).encode("utf-8")
    encoded += b" " * (-len(encoded) % 8)
    with (directory / "model.safetensors").open("wb") as f:
        f.write(struct.pack("<Q", len(encoded)))
        f.write(encoded)
        for _, _, array in tensors:
            f.write(array.tobytes())
