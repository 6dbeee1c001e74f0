"""The converted-model artifact (config.json + model.safetensors in the reference's layout): a
synthetic model written in that layout reads back tensor for tensor, malformed or out-of-scope
artifacts are refused, and (GPU) the engine loaded from the artifact equals the engine loaded from the
in-memory tensors bit for bit."""
import json
import struct

import numpy as np
import pytest

from stark_b200 import synthetic as S
from stark_b200.artifact import ArtifactError, read_artifact, row_major_planes, write_artifact


@pytest.fixture(scope="module")
def tiny_artifact(tmp_path_factory):
    cfg = S.CONFIGS["tiny"]
    w = S.dense_weights(cfg, seed=0)
    path = tmp_path_factory.mktemp("artifact")
    write_artifact(path, cfg, w)
    return cfg, w, path


def test_artifact_round_trips_config_and_tensors(tiny_artifact):
    cfg, w, path = tiny_artifact
    got_cfg, got = read_artifact(path)
    assert got_cfg == {k: cfg[k] for k in got_cfg}
    assert got["embed"] is got["lm_head"]  # tied
    assert np.array_equal(got["final_norm"], w["final_norm"])
    for a, b in zip(got["layers"], w["layers"]):
        for name in ("attn_norm", "mlp_norm", "q_norm", "k_norm"):
            assert np.array_equal(a[name], b[name])
        for name in ("qkv", "o", "upgate", "down"):
            t = a[name]
            assert t["scale_layout"] == 1 and t["plane_pitch"] == t["n"] + (-t["n"] % 4)  # [groups, round_up4(rows)]
            r = row_major_planes(t)
            assert np.array_equal(r["codes"], b[name]["codes"])
            assert np.array_equal(r["scales"], b[name]["scales"]) and np.array_equal(r["biases"], b[name]["biases"])
    # the header names what the reference's loader looks up
    with (path / "model.safetensors").open("rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    assert "decoder.transformer.layers.0.mixer.qkvg_projection.weights.weights" in header
    assert json.loads(header["__metadata__"]["decoder.transformer.layers.1.mlp.up_projection.weights.spec"]) == {
        "type": "MLXSpec", "bits": 4, "group_size": 64, "layout": "output_input"}
    assert header["decoder.transformer.output_norm.scales"]["dtype"] == "F32"


def test_untied_artifact_has_separate_read_out(tmp_path):
    cfg = dict(S.CONFIGS["tiny"], tied=False)
    w = S.dense_weights(cfg, seed=2)
    write_artifact(tmp_path, cfg, w)
    got_cfg, got = read_artifact(tmp_path)
    assert got_cfg["tied"] is False and got["embed"] is not got["lm_head"]
    assert got["embed"]["scale_layout"] == 0 and got["lm_head"]["scale_layout"] == 1
    assert np.array_equal(row_major_planes(got["lm_head"])["scales"], w["lm_head"]["scales"])


def test_out_of_scope_and_malformed_artifacts_are_refused(tiny_artifact, tmp_path):
    cfg, w, path = tiny_artifact
    root = json.loads((path / "config.json").read_text())
    blob = (path / "model.safetensors").read_bytes()

    def variant(mutate_config=None, mutate_header=None):
        d = tmp_path / f"v{len(list(tmp_path.iterdir()))}"
        d.mkdir()
        r = json.loads(json.dumps(root))
        if mutate_config:
            mutate_config(r)
        (d / "config.json").write_text(json.dumps(r))
        (n,) = struct.unpack("<Q", blob[:8])
        header = json.loads(blob[8:8 + n])
        if mutate_header:
            mutate_header(header)
        enc = json.dumps(header).encode()
        enc += b" " * (-len(enc) % 8)
        (d / "model.safetensors").write_bytes(struct.pack("<Q", len(enc)) + enc + blob[8 + n:])
        return d

    def window(r):
        for lc in r["decoder_config"]["transformer_config"]["layer_configs"]:
            lc["mixer_config"]["sliding_window_size"] = 4096
    with pytest.raises(ArtifactError):
        read_artifact(variant(mutate_config=window))
    with pytest.raises(ArtifactError):
        read_artifact(variant(mutate_config=lambda r: r.update(type="Qwen38LanguageModelConfig")))
    with pytest.raises(ArtifactError):  # a tensor nobody consumes
        read_artifact(variant(mutate_header=lambda h: h.update(
            {"decoder.extra.scales": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}})))
    with pytest.raises(ArtifactError):  # a missing tensor
        read_artifact(variant(mutate_header=lambda h: h.pop("decoder.transformer.output_norm.scales")))

    def five_bit(h):
        h["__metadata__"]["decoder.embedding.embedding.spec"] = json.dumps(
            {"type": "MLXSpec", "bits": 5, "group_size": 64, "layout": "input_output"})
    with pytest.raises(ArtifactError):
        read_artifact(variant(mutate_header=five_bit))
    d = tmp_path / "short"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(root))
    (d / "model.safetensors").write_bytes(struct.pack("<Q", 1 << 40))
    with pytest.raises(ArtifactError):
        read_artifact(d)


@pytest.mark.gpu
def test_engine_loaded_from_artifact_equals_engine_loaded_from_tensors(tiny_artifact):
    from stark_b200.engine import DenseModel
    cfg, w, path = tiny_artifact
    prompt = S.prompt(cfg, 40, seed=4)
    direct = DenseModel.load(cfg, w, context_tokens=128)
    direct.prefill(prompt)
    want_logits, want_tokens = direct.logits_bf16().copy(), direct.generate_greedy(6)
    direct.close()
    loaded = DenseModel.from_artifact(path, context_tokens=128)  # planes arrive as [groups, round_up4(rows)]
    loaded.prefill(prompt)
    assert np.array_equal(loaded.logits_bf16(), want_logits)
    assert np.array_equal(loaded.generate_greedy(6), want_tokens)


def _load_status(directory, context_tokens=0):
    """Status of the library's own loader (`stark_b200_load`) on a directory; a model that loads is destroyed."""
    import ctypes as C
    from stark_b200 import _lib
    lib = _lib.load()
    path = str(directory).encode()
    opts = _lib.LoadOptions(C.sizeof(_lib.LoadOptions), _lib.ABI_VERSION, context_tokens, 0)
    handle = C.c_void_p()
    status = lib.stark_b200_load(path, len(path), C.byref(opts), C.byref(handle))
    if status == 0:
        lib.stark_b200_destroy(C.byref(handle))
    return _lib.STATUS_NAMES[status]


def test_library_loader_refuses_what_the_python_reader_refuses(tiny_artifact, tmp_path):
    """The C loader walks the whole artifact (config, header, every tensor it will read, the all-consumed rule)
    before it touches the device, so its refusals can be checked without a GPU."""
    cfg, w, path = tiny_artifact
    root = json.loads((path / "config.json").read_text())
    blob = (path / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", blob[:8])

    def variant(name, mutate_config=None, mutate_header=None):
        d = tmp_path / name
        d.mkdir()
        r = json.loads(json.dumps(root))
        if mutate_config:
            mutate_config(r)
        (d / "config.json").write_text(json.dumps(r))
        header = json.loads(blob[8:8 + n])
        if mutate_header:
            mutate_header(header)
        enc = json.dumps(header).encode()
        enc += b" " * (-len(enc) % 8)
        (d / "model.safetensors").write_bytes(struct.pack("<Q", len(enc)) + enc + blob[8 + n:])
        return d

    def window(r):
        for lc in r["decoder_config"]["transformer_config"]["layer_configs"]:
            lc["mixer_config"]["sliding_window_size"] = 4096

    def five_bit(h):
        h["__metadata__"]["decoder.embedding.embedding.spec"] = json.dumps(
            {"type": "MLXSpec", "bits": 5, "group_size": 64, "layout": "input_output"})

    def wrong_shape(h):
        h["decoder.transformer.output_norm.scales"]["shape"] = [cfg["hidden"] // 2, 2]

    assert _load_status(tmp_path / "nowhere") == "io_failure"
    assert _load_status(variant("window", mutate_config=window)) == "unsupported"
    assert _load_status(variant("type", mutate_config=lambda r: r.update(type="Qwen38LanguageModelConfig"))) == "unsupported"
    assert _load_status(variant("bits", mutate_header=five_bit)) == "unsupported"
    assert _load_status(variant("extra", mutate_header=lambda h: h.update(
        {"decoder.extra.scales": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}))) == "invalid_argument"
    assert _load_status(variant("missing", mutate_header=lambda h: h.pop("decoder.transformer.output_norm.scales"))) == "invalid_argument"
    assert _load_status(variant("shape", mutate_header=wrong_shape)) == "invalid_argument"
    assert _load_status(variant("good"), context_tokens=1 << 20) == "context_limit"
    d = tmp_path / "short"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(root))
    (d / "model.safetensors").write_bytes(struct.pack("<Q", 1 << 40))
    assert _load_status(d) == "invalid_argument"
    (d / "config.json").write_text("{not json")
    assert _load_status(d) == "invalid_argument"
    # a well-formed artifact gets as far as the device: without one here, that is where it stops
    import torch
    if not torch.cuda.is_available():
        assert _load_status(variant("good2"), context_tokens=128) in ("device_failure", "out_of_memory")


@pytest.mark.gpu
def test_library_loader_equals_the_python_loader(tiny_artifact):
    from stark_b200.engine import DenseModel
    cfg, w, path = tiny_artifact
    prompt = S.prompt(cfg, 40, seed=4)
    a = DenseModel.from_artifact(path, context_tokens=128)
    a.prefill(prompt)
    want_logits, want_tokens = a.logits_bf16().copy(), a.generate_greedy(6)
    a.close()
    b = DenseModel.load_path(path, context_tokens=128)
    assert b.info().context_tokens == 128 and b.info().vocab_size == cfg["vocab"]
    b.prefill(prompt)
    assert np.array_equal(b.logits_bf16(), want_logits)
    assert np.array_equal(b.generate_greedy(6), want_tokens)
    b.close()
