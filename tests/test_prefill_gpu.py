"""GPU parity of the batched prompt path: the tensor-core contraction over a 4-bit matrix against the CPU
oracle's matmul (crates/stark-engine/src/backends/cpu/kernel/matmul/kernel.rs:168-285, many input rows), then
the whole chunked prefill against row-by-row steps."""
import numpy as np
import pytest

from oracle import oracle as O
from stark_b200 import synthetic as S

pytestmark = pytest.mark.gpu
REL_TOL = 1e-2  # per-operator bar: bf16 outputs, f32 accumulation


def _rel(got_bits, want_bits):
    g, w = O.bf16_to_f32(got_bits).astype(np.float64), O.bf16_to_f32(want_bits).astype(np.float64)
    return np.abs(g - w) / np.maximum(np.abs(w), np.abs(w).mean() + 1e-30)


def _oracle_rows(w, x, rows, columns):
    return np.stack([O.affine_matvec_bf16(w["codes"], w["scales"], w["biases"], xr, rows, columns)[0] for xr in x])


@pytest.mark.parametrize("m,rows,columns", [(1, 128, 64), (5, 256, 256), (128, 128, 1024), (300, 384, 512),
                                            (257, 6144, 4096), (64, 4096, 12288)])
def test_gemm_matches_oracle_rows(m, rows, columns):
    """Row counts on and off the 128 / 256 row tiles, K from one quantization group to the widest layer."""
    from stark_b200 import ops
    rng = np.random.default_rng(m + rows)
    w = S.affine4_matrix(rng, rows, columns, 0.005 * 17.3 / np.sqrt(columns), 0.02 * 17.3 / np.sqrt(columns))
    x = S.bf16_normal(rng, m * columns).reshape(m, columns)
    q = ops.QMatrix.from_affine(w["codes"], w["scales"], w["biases"], rows, columns)
    got = q.gemm(x)
    assert ops.take_device_error() == 0
    check = np.unique(np.concatenate([[0, m - 1], rng.integers(0, m, size=min(m, 6))]))
    want = _oracle_rows(w, x[check], rows, columns)
    assert _rel(got[check], want).max() < REL_TOL
    # the same rows through the one-row kernel: both round the same f32 sums, up to the bf16 rounding of the
    # dequantized operand that the tiled contraction (like the reference's own) makes
    one = np.stack([q.matvec(x[i]) for i in check[:3]])
    assert _rel(got[check[:3]], one).max() < REL_TOL


def test_gemm_residual_and_swiglu_epilogues():
    from stark_b200 import ops
    rng = np.random.default_rng(17)
    m, hidden, inter = 70, 512, 768
    wd = S.affine4_matrix(rng, hidden, inter, 0.005 * 0.6, 0.02 * 0.6)
    x = S.bf16_normal(rng, m * inter).reshape(m, inter)
    resid = S.bf16_normal(rng, m * hidden, 2.0).reshape(m, hidden)
    q = ops.QMatrix.from_affine(wd["codes"], wd["scales"], wd["biases"], hidden, inter)
    got = q.gemm(x, epilogue=1, residual=resid)
    prod = _oracle_rows(wd, x, hidden, inter)
    want = O.f32_to_bf16(O.bf16_to_f32(prod) + O.bf16_to_f32(resid))
    # the tolerance belongs to the product; the sum with the residual can cancel, so it is not the yardstick
    p64 = np.abs(O.bf16_to_f32(prod).astype(np.float64))
    w64 = O.bf16_to_f32(want).astype(np.float64)
    bound = REL_TOL * np.maximum(p64, p64.mean()) + np.abs(w64) * 2.0 ** -7
    assert np.all(np.abs(O.bf16_to_f32(got).astype(np.float64) - w64) <= bound)
    # [up; gate] with the SwiGLU folded into the epilogue
    wu = S.affine4_matrix(rng, 2 * inter, hidden, 0.005 * 0.7, 0.02 * 0.7)
    xh = S.bf16_normal(rng, m * hidden).reshape(m, hidden)
    qu = ops.QMatrix.from_affine(wu["codes"], wu["scales"], wu["biases"], 2 * inter, hidden, pair_halves=True)
    got = qu.gemm(xh, epilogue=2)
    assert got.shape == (m, inter)
    # the epilogue alone: the gated product of the contraction's own [up; gate] rows (same weights, plain row order)
    plain = ops.QMatrix.from_affine(wu["codes"], wu["scales"], wu["biases"], 2 * inter, hidden).gemm(xh)
    own = np.stack([O.swiglu_bf16(f, inter) for f in plain])
    assert (got != own).mean() < 0.01 and _rel(got, own).max() < REL_TOL   # expf may differ in the last bit
    # and end to end against the oracle: two rounded factors multiply, so the bar is twice the per-operator one,
    # taken against the magnitude of the factors' product
    fused = _oracle_rows(wu, xh, 2 * inter, hidden)
    want = np.stack([O.swiglu_bf16(f, inter) for f in fused])
    g64, w64 = O.bf16_to_f32(got).astype(np.float64), O.bf16_to_f32(want).astype(np.float64)
    up = np.abs(O.bf16_to_f32(fused[:, :inter]).astype(np.float64))
    gate = O.bf16_to_f32(fused[:, inter:]).astype(np.float64)
    scale = np.maximum(up, up.mean()) * np.maximum(np.abs(gate / (1 + np.exp(-gate))), 0.25 * np.abs(gate).mean())
    assert np.all(np.abs(g64 - w64) <= 4 * REL_TOL * scale)


def test_gemm_properties_at_full_size():
    """Size-independent checks at the widest layer shape: zero input, exact power-of-two scaling of the input,
    and bitwise repeatability."""
    from stark_b200 import ops
    rng = np.random.default_rng(23)
    rows, columns, m = 4096, 12288, 512
    w = S.affine4_matrix(rng, rows, columns, 0.005 * 0.15, 0.02 * 0.15)
    q = ops.QMatrix.from_affine(w["codes"], w["scales"], w["biases"], rows, columns)
    x = S.bf16_normal(rng, m * columns).reshape(m, columns)
    y = q.gemm(x)
    assert np.array_equal(y, q.gemm(x))
    assert not q.gemm(np.zeros_like(x)).any()
    x4 = O.f32_to_bf16(O.bf16_to_f32(x) * 4.0)
    y4 = q.gemm(x4)
    assert np.array_equal(O.bf16_to_f32(y4), O.bf16_to_f32(y) * 4.0)
    assert ops.take_device_error() == 0


def _set(name, value):
    from stark_b200 import _lib
    _lib.check(_lib.load().stark_b200_set_tunable(name.encode(), int(value)), f"set_tunable {name}")


@pytest.mark.parametrize("name,prompt_len", [("tiny", 200), ("small", 96), ("small", 4300), ("qwen3-0.6b-layers", 300),
                                             ("qwen3-8b-layers", 1100)])
def test_chunked_prefill_equals_row_by_row(name, prompt_len):
    """A prompt ingested in chunks on the tensor cores must leave the model where row-by-row steps leave it: the
    last row's logits inside the logits acceptance, and a cache that later tokens extend to the same effect
    (positions past one pass of 4096 rows included): the greedy continuation of the chunked model, replayed
    through the row-by-row model, is that model's own pick at every step up to a bf16 near-tie."""
    from stark_b200.engine import DenseModel
    from stark_b200.ops import take_device_error
    from tests.test_model_gpu import assert_logits_accepted, assert_sequence_is_greedy
    cfg = S.CONFIGS[name]
    w = S.dense_weights(cfg, seed=4, zero_point=7.5)
    model = DenseModel.load(cfg, w, context_tokens=prompt_len + 64)
    prompt = S.prompt(cfg, prompt_len, seed=11)
    try:
        _set("prefill_batch", 0)
        model.prefill(prompt)
        rows_logits = model.logits_bf16().copy()
        model.reset()
        _set("prefill_batch", 1)
        launches = model.info().launches_issued
        model.prefill(prompt)
        issued = model.info().launches_issued - launches
        chunks = -(-(prompt_len - 1) // 4096)
        assert issued == chunks * (1 + 8 * cfg["layers"]) + model.info().launches_per_step   # the batched path ran
        assert take_device_error() == 0
        assert_logits_accepted(rows_logits, model.logits_bf16())
        got_next = model.generate_greedy(12).tolist()      # the prompt's pick and the 12 picks after it
        assert model.position == prompt_len + 12
        _set("prefill_batch", 0)
        # two paths whose logits agree within the acceptance above (rmse about one bf16 step of the maximum):
        # a pick is taken as the same when it lies within a few such steps
        assert_sequence_is_greedy(model, prompt, got_next, steps=6.0)
    finally:
        _set("prefill_batch", 1)
        model.close()


def test_chunked_prefill_against_the_oracle():
    """The chunked path against the CPU oracle directly (not only against the one-row kernels)."""
    from stark_b200.engine import DenseModel
    from tests.test_model_gpu import assert_logits_accepted, pick_near_top
    cfg = S.CONFIGS["small"]
    w = S.dense_weights(cfg, seed=1, zero_point=7.5)
    model = DenseModel.load(cfg, w, context_tokens=256)
    oracle = O.DenseOracle(cfg, w, capacity=256)
    prompt = S.prompt(cfg, 150, seed=4)
    model.prefill(prompt)
    for t in prompt[:-1]:
        oracle.ingest(int(t))
    assert_logits_accepted(oracle.step(int(prompt[-1])), model.logits_bf16())
    agree, near, steps = 0, 0, 60
    teacher = S.prompt(cfg, steps, seed=12)
    for t in teacher:
        model.step_async(int(t))
        want = oracle.step(int(t))
        agree += int(model.argmax() == O.argmax_bf16(want))
        # the engine's logits sit about one bf16 step (rmse) from the oracle's, so two near-tied tokens can trade
        # places when they are up to two steps apart
        near += int(pick_near_top(want, model.argmax(), steps=2.0))
    assert near / steps >= 0.99 and agree / steps >= 0.90, (agree, near)
    model.close()


@pytest.mark.parametrize("m,rows,columns", [(1, 200, 64), (2, 256, 1024), (5, 6144, 4096), (8, 1024, 4096),
                                            (5, 4096, 12288), (3, 768, 3072)])
def test_several_rows_matvec_matches_oracle(m, rows, columns):
    """The verify pass's matvec: up to 8 rows against one pass over the matrix; row counts 1..8, K from one group
    to the widest layer, a row count off the 16-row tiles."""
    from stark_b200 import ops
    rng = np.random.default_rng(7 * m + rows)
    w = S.affine4_matrix(rng, rows, columns, 0.005 * 17.3 / np.sqrt(columns), 0.02 * 17.3 / np.sqrt(columns),
                         zero_point=7.5)
    x = S.bf16_normal(rng, m * columns, 3.0).reshape(m, columns)
    q = ops.QMatrix.from_affine(w["codes"], w["scales"], w["biases"], rows, columns)
    got = q.matvec_rows(x)
    assert ops.take_device_error() == 0
    want = _oracle_rows(w, x, rows, columns)
    assert _rel(got, want).max() < REL_TOL
    assert np.array_equal(got, q.matvec_rows(x))                        # bitwise repeatable
    # each row alone gives the same bits as the row inside a batch: rows never mix
    assert np.array_equal(q.matvec_rows(x[m - 1:m])[0], got[m - 1])
    assert not q.matvec_rows(np.zeros_like(x)).any()
    # residual epilogue: bf16(bf16(product) + residual), exact given the kernel's own product
    resid = S.bf16_normal(rng, m * rows, 2.0).reshape(m, rows)
    with_resid = q.matvec_rows(x, epilogue=1, residual=resid)
    assert np.array_equal(with_resid, O.f32_to_bf16(O.bf16_to_f32(got) + O.bf16_to_f32(resid)))
    if columns <= 4096:
        # RMS norm in the prologue against the oracle's norm followed by the oracle's matvec
        nw = (1.0 + 0.1 * rng.standard_normal(columns)).astype(np.float32)
        h = S.bf16_normal(rng, m * columns, 5.0).reshape(m, columns)
        normed = O.rmsnorm_bf16(h, nw, 1e-6)[0]
        got_n = q.matvec_rows(h, norm_weight=nw, eps=1e-6)
        assert _rel(got_n, _oracle_rows(w, normed, rows, columns)).max() < REL_TOL
        # and bit for bit against the kernel's own plain path on the oracle-normalized rows, wherever the two
        # norms round alike (the f32 sum of squares is formed in a different order)
        assert (got_n != q.matvec_rows(normed)).mean() < 0.1


def test_several_rows_matvec_swiglu():
    from stark_b200 import ops
    rng = np.random.default_rng(31)
    m, hidden, inter = 5, 1024, 3072
    wu = S.affine4_matrix(rng, 2 * inter, hidden, 0.005 * 0.5, 0.02 * 0.5, zero_point=7.5)
    xh = S.bf16_normal(rng, m * hidden).reshape(m, hidden)
    qu = ops.QMatrix.from_affine(wu["codes"], wu["scales"], wu["biases"], 2 * inter, hidden, pair_halves=True)
    got = qu.matvec_rows(xh, epilogue=2)
    plain = ops.QMatrix.from_affine(wu["codes"], wu["scales"], wu["biases"], 2 * inter, hidden).matvec_rows(xh)
    own = np.stack([O.swiglu_bf16(f, inter) for f in plain])
    assert got.shape == (m, inter)
    assert (got != own).mean() < 0.01 and _rel(got, own).max() < REL_TOL
    assert ops.take_device_error() == 0
