"""GPU parity of the small decode operators against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from oracle import oracle as O
from stark_b200 import synthetic as S

pytestmark = pytest.mark.gpu
REL_TOL = 1e-2  # per-op bar for bf16 outputs with f32 accumulation


def _rel(got_bits, want_bits):
    g, w = O.bf16_to_f32(got_bits).astype(np.float64), O.bf16_to_f32(want_bits).astype(np.float64)
    return np.abs(g - w) / np.maximum(np.abs(w), np.abs(w).mean() + 1e-30)


@pytest.mark.parametrize("count", [64, 1024, 4096])
def test_rmsnorm_with_residual(count):
    from stark_b200 import ops
    rng = np.random.default_rng(count)
    x = S.bf16_normal(rng, count, 3.0)
    sc = S.bf16_normal(rng, count, 2.0)
    w = (1.0 + 0.2 * rng.standard_normal(count)).astype(np.float32)
    for add in (False, True):
        got, got_sc = ops.rmsnorm(x, w, 1e-6, shortcut=sc, residual_add=add)
        want, want_sc = O.rmsnorm_bf16(x, w, 1e-6, shortcut=sc, residual_add=add)
        assert np.array_equal(got_sc, want_sc)  # bf16 add is exact arithmetic + one rounding
        assert _rel(got, want).max() < REL_TOL
        assert (got != want).mean() < 0.01
    got, none = ops.rmsnorm(x, w, 1e-6)
    assert none is None and _rel(got, O.rmsnorm_bf16(x, w, 1e-6)[0]).max() < REL_TOL


def test_rmsnorm_reference_boundary_vector():
    """The reference's RMS boundary case (normalization_test.rs:337-393): the probe element sits on a bf16 rounding
    midpoint, so its output bits depend on the order of the f32 sum of squares.  The oracle gives the bits of
    the reference's default policy; a parallel sum may land on either neighbour, never further."""
    import json
    from pathlib import Path
    from stark_b200 import ops
    from tests.test_oracle_kats import rms_boundary_input
    k = json.loads((Path(__file__).parent / "golden" / "reference_kats.json").read_text())["rms_boundary"]
    x = rms_boundary_input(k)
    ones = np.ones(k["count"], np.float32)
    got, _ = ops.rmsnorm(x, ones, k["epsilon"])
    want, _ = O.rmsnorm_bf16(x, ones, k["epsilon"])
    assert int(want[k["probe_index"]]) == k["expected_default_bits"]
    assert int(got[k["probe_index"]]) in (k["expected_default_bits"], k["expected_alternative_bits"])
    print("rms boundary probe bits on the GPU:", int(got[k["probe_index"]]))
    assert (got != want).mean() < 0.01 and _rel(got, want).max() < REL_TOL


def test_swiglu_matches_oracle():
    from stark_b200 import ops
    rng = np.random.default_rng(3)
    fused = S.bf16_normal(rng, 2 * 3072, 4.0)
    got, want = ops.swiglu(fused, 3072), O.swiglu_bf16(fused, 3072)
    assert _rel(got, want).max() < REL_TOL
    assert (got != want).mean() < 0.01  # expf may differ in the last bit between libm and the device


def test_fused_upgate_swiglu_matvec():
    from stark_b200 import ops
    rng = np.random.default_rng(4)
    inter, hidden = 1536, 1024
    w = S.affine4_matrix(rng, 2 * inter, hidden, 0.005 * 0.5, 0.02 * 0.5)
    x = S.bf16_normal(rng, hidden)
    q = ops.QMatrix.from_affine(w["codes"], w["scales"], w["biases"], 2 * inter, hidden, pair_halves=True)
    assert np.array_equal(q.unpack_codes(), O.unpack_codes(w["codes"], 4, 2 * inter * hidden).reshape(-1, hidden))
    fused = O.affine_matvec_bf16(w["codes"], w["scales"], w["biases"], x, 2 * inter, hidden)[0]
    assert _rel(q.matvec(x), fused).max() < REL_TOL  # plain matvec on the pair-ordered tiling
    want = O.swiglu_bf16(fused, inter)
    got = ops.qmv_swiglu(q, x)
    assert _rel(got, want).max() < 2 * REL_TOL


def test_argmax_first_index_and_non_finite():
    from stark_b200 import ops
    rng = np.random.default_rng(5)
    logits = S.bf16_normal(rng, 151936, 2.0)
    assert ops.argmax(logits) == O.argmax_bf16(logits)
    logits[[7, 100000]] = O.f32_to_bf16(np.array([50.0], np.float32))[0]
    assert ops.argmax(logits) == 7
    logits[5000] = 0x7FC0  # NaN
    assert ops.argmax(logits) == 0xFFFFFFFF == O.argmax_bf16(logits)


def test_log_softmax_f64():
    from stark_b200 import ops
    rng = np.random.default_rng(6)
    logits = (rng.standard_normal(151936) * 3).astype(np.float32)
    got, want = ops.log_softmax(logits), O.log_softmax_f64(logits)
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-9)
    assert abs(np.exp(got).sum() - 1.0) < 1e-9


def test_moe_route_matches_oracle():
    from stark_b200 import ops
    rng = np.random.default_rng(7)
    logits = rng.standard_normal((33, 128)).astype(np.float32)
    logits[3, 10] = logits[3, 90] = 9.0  # tie: the lower id wins
    for rw, rl in ((False, False), (True, True)):
        gi, gw = ops.moe_route(logits, 128, 8, rw, rl)
        wi, ww = O.moe_route(logits, 128, 8, rw, rl)
        assert np.array_equal(gi, wi)
        np.testing.assert_allclose(gw, ww, rtol=2e-6 if not rw else 8e-3)
    assert gi[3, 0] == 10 and gi[3, 1] == 90


@pytest.mark.parametrize("q_heads,kv_heads,position", [(4, 2, 0), (4, 2, 5), (16, 8, 63), (16, 8, 64), (32, 8, 700),
                                                       (32, 4, 1500)])
def test_attention_decode_matches_oracle(q_heads, kv_heads, position):
    from stark_b200 import ops
    rng = np.random.default_rng(position + q_heads)
    hd, eps, theta = 128, 1e-6, 1e6
    capacity = position + 1
    keys = S.bf16_normal(rng, capacity * kv_heads * hd).reshape(capacity, kv_heads, hd)
    values = S.bf16_normal(rng, capacity * kv_heads * hd).reshape(capacity, kv_heads, hd)
    qkv = S.bf16_normal(rng, (q_heads + 2 * kv_heads) * hd, 2.0)
    qn = (1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kn = (1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    # oracle: norm + rope the row, append, attend
    row = O.head_norm_bf16(qkv, qn, 0, q_heads, hd, eps)
    row = O.head_norm_bf16(row, kn, q_heads, kv_heads, hd, eps)
    cos, sin = O.rope_coeffs(position, hd, theta)
    for h in range(q_heads + kv_heads):
        row[h * hd:(h + 1) * hd] = O.rope_head_bf16(row[h * hd:(h + 1) * hd], cos, sin)
    ok, ov = keys.copy(), values.copy()
    ok[position] = row[q_heads * hd:(q_heads + kv_heads) * hd].reshape(kv_heads, hd)
    ov[position] = row[(q_heads + kv_heads) * hd:].reshape(kv_heads, hd)
    want = O.attention_decode_bf16(row[:q_heads * hd], ok, ov, q_heads, kv_heads, hd, position + 1,
                                   1.0 / np.sqrt(np.float32(hd)))
    gk, gv = keys.copy(), values.copy()
    got = ops.attention_decode(qkv, gk, gv, q_heads, kv_heads, position, eps, theta, qn, kn)
    assert ops.take_device_error() == 0
    # the appended K row (norm + RoPE) and V row (copy)
    assert np.array_equal(gv[position], ov[position])
    assert (gk[position] != ok[position]).mean() < 0.02 and _rel(gk[position].ravel(), ok[position].ravel()).max() < REL_TOL
    assert np.array_equal(gk[:position], keys[:position])
    assert _rel(got, want).max() < REL_TOL


def test_attention_split_count_does_not_change_the_result_beyond_rounding():
    from stark_b200 import ops
    rng = np.random.default_rng(11)
    hd, pos = 128, 900
    keys = S.bf16_normal(rng, (pos + 1) * 8 * hd).reshape(pos + 1, 8, hd)
    values = S.bf16_normal(rng, (pos + 1) * 8 * hd).reshape(pos + 1, 8, hd)
    qkv = S.bf16_normal(rng, (32 + 16) * hd)
    outs = [ops.attention_decode(qkv, keys.copy(), values.copy(), 32, 8, pos, splits=s) for s in (1, 4, 32)]
    for o in outs[1:]:
        assert _rel(o, outs[0]).max() < REL_TOL
