"""GPU parity of the GGUF (Q8_0, Q4_K) and 8-bit affine matvecs, expert banks and the routed-expert
feed-forward against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from oracle import oracle as O
from stark_b200 import synthetic as S

pytestmark = pytest.mark.gpu


def _bound(kind, data, x, rows, columns):
    """The reference's own tolerance for these comparisons: 2e-5 * sum |w x| (weights.rs:4218-4297)."""
    row_bytes = data.size // rows
    w = np.stack([O.gguf_decode_row(kind, data.reshape(rows, row_bytes)[r], columns) for r in range(rows)])
    return 2e-5 * (np.abs(w) * np.abs(x)).sum(axis=1) + 1e-12


@pytest.mark.parametrize("kind,gen", [(O.Q8_0, S.q8_0_rows), (O.Q4_K, S.q4_k_rows)])
@pytest.mark.parametrize("rows,columns", [(3, 256), (128, 2048), (2048, 1024), (768, 2048)])
def test_gguf_rows_decode_bit_exactly_and_multiply(kind, gen, rows, columns):
    from stark_b200 import ops
    from stark_b200._lib import F32
    rng = np.random.default_rng(rows + columns + kind)
    data = gen(rng, rows, columns)
    q = ops.QMatrix.from_gguf(data, kind, rows, columns)
    # bit-exact decode through the kernel's own extraction, including the 6-bit scale / min unpack
    for r in {0, rows // 2, rows - 1}:
        want = O.gguf_decode_row(kind, data[r], columns)
        got = ops.dequantize_row(q, r)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    if kind == O.Q4_K:
        codes = q.unpack_codes()
        blocks = data.reshape(-1, 144)
        want_codes = np.stack([O.q4k_unpack(b)[0] for b in blocks[: (columns // 256) * min(rows, 4)]])
        assert np.array_equal(codes[: min(rows, 4)].reshape(-1, 256), want_codes)
    x = rng.standard_normal(columns).astype(np.float32)
    got = q.matvec(x, io_type=F32)
    want = O.gguf_matvec_f32(kind, data, x, rows, columns, threads=O.max_threads())
    assert np.all(np.abs(got - want) <= _bound(kind, data, x, rows, columns))


def test_q8_0_reference_rows():
    """The reference's own row vector: d = 1.0 / 0.5, codes 0..31 (weights.rs:4299-4354)."""
    from stark_b200 import ops
    from stark_b200._lib import F32
    data = bytearray()
    for s in (0x3C00, 0x3800):
        data += s.to_bytes(2, "little") + bytes(range(32))
    data = np.frombuffer(bytes(data), np.uint8).reshape(2, 34)
    q = ops.QMatrix.from_gguf(data, O.Q8_0, 2, 32)
    assert ops.dequantize_row(q, 0).tolist() == [float(v) for v in range(32)]
    assert ops.dequantize_row(q, 1).tolist() == [0.5 * v for v in range(32)]
    assert q.matvec(np.ones(32, np.float32), io_type=F32).tolist() == [496.0, 248.0]


def test_affine8_matches_oracle_both_conventions():
    from stark_b200 import ops
    from stark_b200._lib import F32
    rng = np.random.default_rng(8)
    rows, columns = 512, 2048
    w = S.affine8_matrix(rng, rows, columns)
    q = ops.QMatrix.from_affine(w["codes"], w["scales"], w["biases"], rows, columns, bits=8)
    assert np.array_equal(q.unpack_codes(), w["codes"])
    r = ops.dequantize_row(q, 7)
    assert np.array_equal(r.view(np.uint32),
                          O.affine_row_f32(w["codes"], w["scales"], w["biases"], 30, 7, columns, bits=8).view(np.uint32))
    x = rng.standard_normal(columns).astype(np.float32)
    got = q.matvec(x, io_type=F32)
    want = O.affine_matvec_f32(w["codes"], w["scales"], w["biases"], 30, x, rows, columns, bits=8)
    wf = np.stack([O.affine_row_f32(w["codes"], w["scales"], w["biases"], 30, i, columns, bits=8) for i in range(rows)])
    assert np.all(np.abs(got - want) <= 2e-5 * (np.abs(wf) * np.abs(x)).sum(axis=1))
    xb = S.bf16_normal(rng, columns)
    gotb = q.matvec(xb)
    wantb = O.affine_matvec_bf16(w["codes"], w["scales"], w["biases"], xb, rows, columns, bits=8)[0]
    g, t = O.bf16_to_f32(gotb).astype(np.float64), O.bf16_to_f32(wantb).astype(np.float64)
    assert (np.abs(g - t) / np.maximum(np.abs(t), np.abs(t).mean())).max() < 1e-2


def test_selected_experts_match_per_expert_matvecs():
    from stark_b200 import ops
    rng = np.random.default_rng(12)
    experts, rows, columns = 6, 96, 512
    bank = np.stack([S.q4_k_rows(rng, rows, columns) for _ in range(experts)])
    q = ops.QMatrix.from_gguf(bank, O.Q4_K, rows, columns, experts=experts)
    ids = [4, 0, 5, 4]
    x = rng.standard_normal((len(ids), columns)).astype(np.float32)
    got = ops.matvec_experts(q, ids, x, shared_input=False)
    shared = ops.matvec_experts(q, ids, x[0], shared_input=True)
    for i, e in enumerate(ids):
        want = O.gguf_matvec_f32(O.Q4_K, bank[e], x[i], rows, columns)
        assert np.all(np.abs(got[i] - want) <= _bound(O.Q4_K, bank[e], x[i], rows, columns))
        want0 = O.gguf_matvec_f32(O.Q4_K, bank[e], x[0], rows, columns)
        assert np.all(np.abs(shared[i] - want0) <= _bound(O.Q4_K, bank[e], x[0], rows, columns))
    from stark_b200._lib import StarkB200Error
    with pytest.raises(StarkB200Error):
        ops.matvec_experts(q, [experts], x[0], shared_input=True)  # expert index out of range


def test_routed_expert_feed_forward_matches_oracle():
    """Qwen3-30B-A3B-shaped block at reduced expert count: hidden 2048, expert width 768, top-8."""
    from stark_b200 import ops
    rng = np.random.default_rng(30)
    experts, active, hidden, inter = 16, 8, 2048, 768
    gate = np.stack([S.q4_k_rows(rng, inter, hidden, 0.02) for _ in range(experts)])
    up = np.stack([S.q4_k_rows(rng, inter, hidden, 0.02) for _ in range(experts)])
    down = np.stack([S.q4_k_rows(rng, hidden, inter, 0.02) for _ in range(experts)])
    router = rng.standard_normal((experts, hidden)).astype(np.float32) / np.sqrt(hidden)
    x = rng.standard_normal(hidden).astype(np.float32)
    scores = ops.dense_matvec_f32(router, x)
    np.testing.assert_allclose(scores, O.dense_matvec_f32(router, x), rtol=0, atol=2e-5 * np.abs(router @ x).max() + 1e-6)
    scores = O.dense_matvec_f32(router, x)  # same selection input for both sides
    scores[3] = scores[9]                   # a tie: the lower index is selected first
    want, wids, wprobs = O.moe_ffn_f32(O.Q4_K, gate, up, O.Q4_K, down, scores, x, experts, active, hidden, inter,
                                       threads=O.max_threads())
    gq = ops.QMatrix.from_gguf(gate, O.Q4_K, inter, hidden, experts=experts)
    uq = ops.QMatrix.from_gguf(up, O.Q4_K, inter, hidden, experts=experts)
    dq = ops.QMatrix.from_gguf(down, O.Q4_K, hidden, inter, experts=experts)
    got, gids, gprobs = ops.moe_ffn(gq, uq, dq, scores, x, active)
    assert np.array_equal(gids, wids)
    np.testing.assert_allclose(gprobs, wprobs, rtol=2e-6)
    scale = np.abs(want).mean()
    assert np.abs(got - want).max() <= 1e-3 * scale + 1e-6  # f32 path: far inside the 1e-2 per-op bar
