"""Pins the CPU oracle against the reference's own known answers (no GPU needed)."""
import hashlib

import numpy as np
import pytest

from oracle import oracle as O


def test_packed_code_vectors(kats):
    k = kats["packed_code_nibbles"]
    b = np.array([k["single_byte"]["byte"]], np.uint8)
    assert O.packed_code(b, 8, 0) == k["single_byte"]["bits8"]
    assert O.packed_code(b, 4, 0) == k["single_byte"]["bits4_index0"]
    assert O.packed_code(b, 4, 1) == k["single_byte"]["bits4_index1"]
    codes = np.array(k["codes"], np.uint8)
    assert [O.packed_code(codes, 4, i) for i in range(12)] == k["expected_4bit"]
    aligned = np.array(k["aligned_8bit"], np.uint8)
    assert [O.packed_code(aligned, 8, i) for i in range(4)] == k["aligned_8bit"]


@pytest.mark.parametrize("bits", [3, 5, 6])
def test_packed_code_odd_widths_round_trip(bits):
    # same construction as the reference test: code_i = (17 i + 3) mod 2^bits, packed LSB first
    expected = [(i * 17 + 3) & ((1 << bits) - 1) for i in range(64)]
    packed = np.zeros(64 * bits // 8, np.uint8)
    for i, code in enumerate(expected):
        for bit in range(bits):
            pos = i * bits + bit
            packed[pos // 8] |= ((code >> bit) & 1) << (pos % 8)
    assert [O.packed_code(packed, bits, i) for i in range(64)] == expected


def test_exact_packed_tails(kats):
    one = O.f32_to_bf16(np.ones(1, np.float32))[0]
    for case in kats["exact_packed_tails"]["cases"]:
        k, n, bits = case["k"], case["n"], case["bits"]
        codes = np.array(case["codes"], np.uint8)
        scales = np.full((n, 1), one, np.uint16)
        a = np.full(k, one, np.uint16)
        d = O.affine_matvec_bf16(codes, scales, None, a, n, k, bits=bits, group=k, correction=1)
        assert O.bf16_to_f32(d[0]).tolist() == case["expected"]


def test_gguf_block_hashes(kats):
    for case in kats["gguf_block_sha256"]["cases"]:
        elements, size = O.BLOCK[case["kind"]]
        block = np.array([(i * 73 + 41) % 256 for i in range(size)], np.uint8)
        for i, at in enumerate(case["scale_offsets"]):
            block[at:at + 2] = np.frombuffer((0x3400 if i == 0 else 0x3000).to_bytes(2, "little"), np.uint8)
        out = O.decode_block(case["kind"], block)
        assert out.size == elements
        assert hashlib.sha256(out.astype("<f4").tobytes()).hexdigest() == case["sha256"]
        with pytest.raises(ValueError):
            O.decode_block(case["kind"], block[:-1])


def test_ggml_block_sizes(kats):
    for f in kats["ggml_formats"]["formats"]:
        assert O.BLOCK[f["kind"]] == (f["block_elements"], f["block_bytes"])


def test_gguf_independent_dequantizer_agrees():
    gguf = pytest.importorskip("gguf")
    rng = np.random.default_rng(5)
    for kind, qt in ((O.Q8_0, gguf.GGMLQuantizationType.Q8_0), (O.Q4_K, gguf.GGMLQuantizationType.Q4_K)):
        elements, size = O.BLOCK[kind]
        blocks = rng.integers(0, 256, size=(64, size), dtype=np.uint8)
        # keep the f16 scale fields finite and moderate
        blocks[:, 0:2] = np.frombuffer(np.float16(0.0123).tobytes(), np.uint8)
        if kind == O.Q4_K:
            blocks[:, 2:4] = np.frombuffer(np.float16(0.0071).tobytes(), np.uint8)
        ours = np.stack([O.decode_block(kind, b) for b in blocks])
        theirs = gguf.quants.dequantize(blocks, qt).reshape(64, elements)
        # the reference evaluates d*sc*q - min*m left to right in f32; the numpy dequantizer groups the
        # products differently, so agreement is to f32 rounding, and exact on the integer fields
        np.testing.assert_allclose(ours, theirs, rtol=2e-6, atol=1e-7)


def test_mlx_plane_layout(kats):
    c = kats["mlx_plane_layout"]["case_4bit_group32"]
    codes = np.full(c["rows"] * c["columns"] // 2, c["code_byte"], np.uint8)
    scales = np.array(c["scales"], np.float32)
    biases = np.array(c["biases"], np.float32)
    r0 = O.affine_row_f32(codes, scales, biases, 0, 0, c["columns"], bits=4, group=32)
    r1 = O.affine_row_f32(codes, scales, biases, 0, 1, c["columns"], bits=4, group=32)
    assert all(r0[0::2] == c["row0_even"]) and all(r0[1::2] == c["row0_odd"])
    assert all(r1[0::2] == c["row1_even"]) and all(r1[1::2] == c["row1_odd"])
    c8 = kats["mlx_plane_layout"]["case_8bit_group32"]
    codes8 = np.full(c8["columns"], c8["code_byte"], np.uint8)
    r = O.affine_row_f32(codes8, np.array([c8["scale"]], np.float32), np.array([c8["bias"]], np.float32), 0, 0,
                         c8["columns"], bits=8, group=32)
    assert all(r == c8["value"])


def test_gguf_q8_0_rows(kats):
    c = kats["gguf_q8_0_rows"]
    data = bytearray()
    for s in c["scales_f16"]:
        data += s.to_bytes(2, "little") + bytes(range(32))
    data = np.frombuffer(bytes(data), np.uint8)
    assert O.gguf_decode_row(O.Q8_0, data[:34], 32).tolist() == [float(x) for x in range(32)]
    assert O.gguf_decode_row(O.Q8_0, data[34:], 32).tolist() == [0.5 * x for x in range(32)]
    y = O.gguf_matvec_f32(O.Q8_0, data, np.ones(32, np.float32), 2, 32)
    assert y.tolist() == [496.0, 248.0]


def test_math_kats(kats):
    m = kats["math"]
    x = np.array([float(v) for v in m["softmax_input"]], np.float32)
    assert O.softmax_f32(x).tolist() == m["softmax_expected"]
    with pytest.raises(ValueError):
        O.softmax_f32(np.array([-np.inf], np.float32))
    with pytest.raises(ValueError):
        O.softmax_f32(np.array([np.nan], np.float32))
    assert O.topk_f32(np.array(m["topk_input"], np.float32), m["topk_k"]).tolist() == m["topk_expected"]
    assert O.topk_f32(np.array(m["topk_ties_input"], np.float32), 2).tolist() == m["topk_ties_expected"]
    n = O.rmsnorm_f32(np.array(m["rms_input"]), np.array(m["rms_weight"]), m["rms_eps"])
    assert abs(n[0] - 3.0 / np.sqrt(12.5)) < 1e-6 and abs(n[1] - 8.0 / np.sqrt(12.5)) < 1e-6
    with pytest.raises(ValueError):
        O.rmsnorm_f32(np.array([1.0]), np.array([]), 1e-6)


def test_bf16_rounding_matches_numpy_mirror():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 1e3,
                        np.array([0.0, -0.0, np.inf, -np.inf, 1.00390625, 1.01171875, 3.3895314e38], np.float32)])
    ours = O.f32_to_bf16(x)
    ref = np.array([O.lib().so_f32_to_bf16(float(v)) for v in x], np.uint16)
    assert np.array_equal(ours, ref)
    # ties round to even
    assert O.lib().so_f32_to_bf16(1.00390625) == 0x3F80  # 1 + 2^-8 -> 1.0
    assert O.lib().so_f32_to_bf16(1.01171875) == 0x3F82  # 1 + 3*2^-8 -> 1 + 2^-6


def test_affine_matvec_paths_agree_on_dequantized_values():
    # bf16-in/bf16-out (converted path) vs f32 (hybrid host path): same unpack and scale*q+bias
    from stark_b200 import synthetic as S
    w = S.matvec_case(seed=3, rows=64, columns=256)
    xa = O.bf16_to_f32(w["x"])
    ya = O.bf16_to_f32(O.affine_matvec_bf16(w["codes"], w["scales"], w["biases"], w["x"], 64, 256)[0])
    yb = O.affine_matvec_f32(w["codes"], w["scales"], w["biases"], 30, xa, 64, 256)
    # same arithmetic, path A only adds the final bf16 rounding
    assert np.array_equal(O.f32_to_bf16(yb), O.f32_to_bf16(ya))
    # GroupOutput plane layout [G, round_up4(N)] gives the same result
    npad = 64
    st = np.ascontiguousarray(w["scales"].T)
    bt = np.ascontiguousarray(w["biases"].T)
    yc = O.affine_matvec_bf16(w["codes"], st, bt, w["x"], 64, 256, scale_layout=1, npad=npad)
    assert np.array_equal(yc[0], O.f32_to_bf16(ya))


def test_moe_route_first_max_and_renormalise():
    logits = np.array([[0.0, 2.0, 2.0, -1.0]], np.float32)
    ids, weights = O.moe_route(logits, 4, 2)
    assert ids.tolist() == [[1, 2]]
    np.testing.assert_allclose(weights.sum(), 1.0, rtol=1e-6)
    np.testing.assert_allclose(weights[0], [0.5, 0.5], rtol=1e-6)


def test_greedy_lowest_index_and_non_finite():
    v = O.f32_to_bf16(np.array([1.0, 3.0, 3.0, 2.0], np.float32))
    assert O.argmax_bf16(v) == 1
    v[2] = 0x7FC0
    assert O.argmax_bf16(v) == 0xFFFFFFFF
    lp = O.log_softmax_f64(np.array([0.0, 0.0], np.float32))
    np.testing.assert_allclose(lp, [-np.log(2.0)] * 2, rtol=1e-15)


def rms_boundary_input(k):
    """The input row of the reference's RMS boundary case as bf16 bits."""
    x = np.ones(k["count"], np.float32)
    for i in range(64):
        x[(i * 37 + 102) % k["count"]] = 0.0
    for i, power in enumerate(k["powers"]):
        x[(i * 37 + 102) % k["count"]] = 2.0 ** power
    x[k["probe_index"]] = k["probe_value"]
    return O.f32_to_bf16(x)


def test_rms_boundary_vector_pins_the_bf16_norm(kats):
    """The probe sits on a bf16 rounding midpoint of the normalized value, so the output bit pattern tells
    the order of the f32 sum of squares apart: the oracle must give the default policy's bits."""
    k = kats["rms_boundary"]
    x = rms_boundary_input(k)
    out, _ = O.rmsnorm_bf16(x, np.ones(k["count"], np.float32), k["epsilon"])   # scale 1.0 = no scales
    assert int(out[k["probe_index"]]) == k["expected_default_bits"]
    # the two policies really differ on this input: a float64 sum lands on the other side
    v = O.bf16_to_f32(x).astype(np.float64)
    alt = np.float32(np.float32(k["probe_value"]) * np.float32(1.0 / np.sqrt(np.float32((v * v).sum() / k["count"] + 1e-6))))
    assert int(O.f32_to_bf16(np.array([alt], np.float32))[0]) in (k["expected_default_bits"], k["expected_alternative_bits"])


def test_prefix_reuse_arithmetic(kats):
    """`reusable_prefill_rows` and `PrefixEntry::reusable` on the cases the reference's own tests hold."""
    from stark_b200.engine import reusable_prefix_rows
    k = kats["prefix_reuse"]
    for prompt, rows in k["reusable_prefill_rows"]:
        # the retained prefix of a prompt is what a longer prompt sharing all of it may reuse
        assert reusable_prefix_rows(prompt, prompt, 10 ** 9, k["chunk"]) == rows, prompt
    for case in k["reuse"]:
        got = reusable_prefix_rows(k["previous_prompt"], case["common"], case["new_prompt"], k["chunk"])
        assert got == case["expected"], case
