"""The GGUF v3 reader against files written by the independent `gguf` package, plus the refusals the
reference's reader makes (weights.rs:2770-2866); on the GPU, a tensor read from a file multiplies like
the same bytes passed directly."""
import struct

import numpy as np
import pytest

gguf = pytest.importorskip("gguf")

from oracle import oracle as O
from stark_b200 import synthetic as S
from stark_b200.gguf_file import GGUFError, Q4_K, Q8_0, read_gguf


def _write(path, tensors, alignment=None):
    w = gguf.GGUFWriter(str(path), "llama")
    w.add_uint32("test.answer", 42)
    w.add_string("general.name", "tiny")
    w.add_array("test.list", [1, 2, 3])
    if alignment:
        w.add_custom_alignment(alignment)
    for name, arr, qt in tensors:
        if qt is None:
            w.add_tensor(name, arr)
        else:
            w.add_tensor(name, arr, raw_shape=arr.shape, raw_dtype=qt)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


@pytest.fixture(scope="module")
def sample(tmp_path_factory):
    rng = np.random.default_rng(3)
    q4 = S.q4_k_rows(rng, 48, 512)                                  # [48, 288] bytes
    q8 = S.q8_0_rows(rng, 32, 256)                                  # [32, 272] bytes
    bank = np.stack([S.q4_k_rows(rng, 16, 256) for _ in range(3)])  # [3, 16, 144]
    norm = rng.standard_normal(64).astype(np.float32)
    path = tmp_path_factory.mktemp("gguf") / "tiny.gguf"
    _write(path, [("blk.0.ffn_down.weight", q4, gguf.GGMLQuantizationType.Q4_K),
                  ("blk.0.attn_q.weight", q8, gguf.GGMLQuantizationType.Q8_0),
                  ("blk.0.ffn_gate_exps.weight", bank, gguf.GGMLQuantizationType.Q4_K),
                  ("output_norm.weight", norm, None)])
    return path, dict(q4=q4, q8=q8, bank=bank, norm=norm)


def test_reader_agrees_with_the_gguf_package(sample):
    path, src = sample
    tensors, meta = read_gguf(path)
    assert meta["test.answer"] == 42 and meta["general.name"] == "tiny" and meta["test.list"] == [1, 2, 3]
    theirs = {t.name: t for t in gguf.GGUFReader(str(path)).tensors}
    assert sorted(tensors) == sorted(theirs)
    for name, t in tensors.items():
        assert t.kind == int(theirs[name].tensor_type)
        assert list(reversed(t.shape)) == [int(d) for d in theirs[name].shape]   # slowest first here
        assert np.array_equal(t.data, np.asarray(theirs[name].data).view(np.uint8).reshape(-1))
    assert tensors["blk.0.ffn_down.weight"].shape == (48, 512) and tensors["blk.0.ffn_down.weight"].kind == Q4_K
    assert tensors["blk.0.attn_q.weight"].shape == (32, 256) and tensors["blk.0.attn_q.weight"].kind == Q8_0
    assert tensors["blk.0.ffn_gate_exps.weight"].shape == (3, 16, 256)
    assert np.array_equal(tensors["output_norm.weight"].array(), src["norm"])
    assert np.array_equal(tensors["blk.0.ffn_down.weight"].data.reshape(48, -1), src["q4"])
    # decoded through the oracle, the file's bytes are the source's values
    row = O.gguf_decode_row(O.Q4_K, tensors["blk.0.ffn_down.weight"].data.reshape(48, -1)[5], 512)
    assert np.array_equal(row, O.gguf_decode_row(O.Q4_K, src["q4"][5], 512))


def test_custom_alignment_is_honoured(tmp_path):
    x = np.arange(8, dtype=np.float32)
    _write(tmp_path / "a.gguf", [("a", x, None), ("b", x + 1, None)], alignment=256)
    tensors, meta = read_gguf(tmp_path / "a.gguf")
    assert meta["general.alignment"] == 256
    assert np.array_equal(tensors["a"].array(), x) and np.array_equal(tensors["b"].array(), x + 1)


def test_malformed_files_are_refused(sample, tmp_path):
    path, _ = sample
    blob = bytearray(path.read_bytes())

    def variant(name, mutate):
        b = bytearray(blob)
        mutate(b)
        p = tmp_path / name
        p.write_bytes(bytes(b))
        return p

    with pytest.raises(GGUFError):  # version 2
        read_gguf(variant("v2", lambda b: b.__setitem__(slice(4, 8), struct.pack("<I", 2))))
    with pytest.raises(GGUFError):  # wrong magic
        read_gguf(variant("magic", lambda b: b.__setitem__(slice(0, 4), b"GGML")))
    with pytest.raises(GGUFError):  # tensor data cut short
        read_gguf(variant("short", lambda b: b.__delitem__(slice(len(b) - 64, len(b)))))
    with pytest.raises(GGUFError):  # header cut short
        read_gguf(variant("header", lambda b: b.__delitem__(slice(40, len(b)))))
    # a type outside the reference's admitted list: patch the Q8_0 tensor's type field (value 8) to 2 (Q4_0)
    tag = b"blk.0.attn_q.weight"
    at = bytes(blob).index(tag) + len(tag) + 4 + 2 * 8   # name, rank, two dims
    assert struct.unpack("<I", blob[at:at + 4])[0] == 8
    with pytest.raises(GGUFError):
        read_gguf(variant("type", lambda b: b.__setitem__(slice(at, at + 4), struct.pack("<I", 2))))
    with pytest.raises(GGUFError):  # an offset that is not a multiple of the alignment
        read_gguf(variant("align", lambda b: b.__setitem__(slice(at + 4, at + 12), struct.pack(
            "<Q", struct.unpack("<Q", blob[at + 4:at + 12])[0] + 2))))


def test_a_file_with_types_the_engine_cannot_multiply_still_opens(tmp_path):
    """Q4_K checkpoints usually carry Q6_K tensors (output.weight, some ffn_down): the reference sizes
    every admitted type (block_layout, weights.rs:2565-2584), so such a file opens and its Q4_K / Q8_0
    tensors are usable; only the Q6_K tensor itself is refused, when asked for."""
    rng = np.random.default_rng(5)
    q4 = S.q4_k_rows(rng, 16, 256)
    q6 = rng.integers(0, 256, size=(32, 210), dtype=np.uint8)       # 32 rows x 256 columns of Q6_K blocks
    q5 = rng.integers(0, 256, size=(4, 2 * 176), dtype=np.uint8)    # Q5_K, 4 rows x 512 columns
    path = tmp_path / "mixed.gguf"
    _write(path, [("blk.0.ffn_up.weight", q4, gguf.GGMLQuantizationType.Q4_K),
                  ("output.weight", q6, gguf.GGMLQuantizationType.Q6_K),
                  ("blk.0.ffn_down.weight", q5, gguf.GGMLQuantizationType.Q5_K)])
    tensors, _ = read_gguf(path)
    assert tensors["output.weight"].kind == 14 and tensors["output.weight"].shape == (32, 256)
    assert tensors["output.weight"].data.size == 32 * 210
    assert tensors["blk.0.ffn_down.weight"].kind == 13 and tensors["blk.0.ffn_down.weight"].shape == (4, 512)
    assert np.array_equal(tensors["blk.0.ffn_up.weight"].data.reshape(16, -1), q4)
    with pytest.raises(GGUFError):
        tensors["output.weight"].qmatrix()
    with pytest.raises(GGUFError):
        tensors["output.weight"].array()


def _header(dims, kind=0, offset=0, payload=b""):
    """A minimal GGUF v3 file with one tensor whose header fields are given."""
    name = b"t"
    out = b"GGUF" + struct.pack("<IQQ", 3, 1, 0)
    out += struct.pack("<Q", len(name)) + name + struct.pack("<I", len(dims))
    out += b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", kind, offset)
    out += b"\0" * (-len(out) % 32)
    return out + payload


def test_crafted_headers_are_refused(tmp_path):
    """`product` refuses an empty dimension and a size that overflows (weights.rs:2556-2563); a wrapped
    64-bit product must not slip through the truncation check as a small tensor."""
    def read(blob, name):
        p = tmp_path / name
        p.write_bytes(blob)
        return read_gguf(p)

    tensors, _ = read(_header([4], payload=struct.pack("<4f", 1, 2, 3, 4)), "ok")
    assert tensors["t"].array().tolist() == [1.0, 2.0, 3.0, 4.0]
    with pytest.raises(GGUFError, match="empty tensor dimension"):
        read(_header([4, 0]), "zero")
    with pytest.raises(GGUFError, match="tensor size overflow"):
        read(_header([1 << 33, 1 << 33], payload=b"\0" * 64), "wrap")   # 2^66 elements, 0 modulo 2^64
    with pytest.raises(GGUFError, match="overflow"):
        read(_header([1 << 62, 2], payload=b"\0" * 64), "bytes")       # 2^63 f32 values: 2^65 bytes
    with pytest.raises(GGUFError, match="block aligned"):
        read(_header([48], kind=8, payload=b"\0" * 64), "blocks")      # Q8_0 row that is not whole blocks
    with pytest.raises(GGUFError):
        read(_header([4], offset=(1 << 64) - 32, payload=b"\0" * 64), "offset")


@pytest.mark.gpu
def test_tensors_from_a_file_multiply_like_the_source_bytes(sample):
    from stark_b200 import ops
    from stark_b200._lib import F32
    path, src = sample
    tensors, _ = read_gguf(path)
    rng = np.random.default_rng(9)
    x = rng.standard_normal(512).astype(np.float32)
    got = tensors["blk.0.ffn_down.weight"].qmatrix().matvec(x, io_type=F32)
    want = ops.QMatrix.from_gguf(src["q4"], O.Q4_K, 48, 512).matvec(x, io_type=F32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    ref = O.gguf_matvec_f32(O.Q4_K, src["q4"], x, 48, 512)
    w = np.stack([O.gguf_decode_row(O.Q4_K, src["q4"][r], 512) for r in range(48)])
    assert np.all(np.abs(got - ref) <= 2e-5 * (np.abs(w) * np.abs(x)).sum(axis=1) + 1e-12)
    x8 = rng.standard_normal(256).astype(np.float32)
    got8 = tensors["blk.0.attn_q.weight"].qmatrix().matvec(x8, io_type=F32)
    ref8 = O.gguf_matvec_f32(O.Q8_0, src["q8"], x8, 32, 256)
    w8 = np.stack([O.gguf_decode_row(O.Q8_0, src["q8"][r], 256) for r in range(32)])
    assert np.all(np.abs(got8 - ref8) <= 2e-5 * (np.abs(w8) * np.abs(x8)).sum(axis=1) + 1e-12)
    bank = tensors["blk.0.ffn_gate_exps.weight"].qmatrix()
    xe = rng.standard_normal(256).astype(np.float32)
    out = ops.matvec_experts(bank, [2, 0], xe, shared_input=True)
    for i, e in enumerate([2, 0]):
        refe = O.gguf_matvec_f32(O.Q4_K, src["bank"][e], xe, 16, 256)
        we = np.stack([O.gguf_decode_row(O.Q4_K, src["bank"][e][r], 256) for r in range(16)])
        assert np.all(np.abs(out[i] - refe) <= 2e-5 * (np.abs(we) * np.abs(xe)).sum(axis=1) + 1e-12)
