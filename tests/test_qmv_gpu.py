"""GPU parity of the quantized matvec against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from oracle import oracle as O
from stark_b200 import synthetic as S

pytestmark = pytest.mark.gpu

# per-op bar: integer unpack bit-exact; outputs within 1e-2 relative (bf16 in, f32 accumulate)
REL_TOL = 1e-2


def _rel_err(got_bits, want_bits):
    got, want = O.bf16_to_f32(got_bits).astype(np.float64), O.bf16_to_f32(want_bits).astype(np.float64)
    scale = np.maximum(np.abs(want), np.abs(want).mean())
    return np.abs(got - want) / scale


@pytest.mark.parametrize("rows,columns", [(16, 64), (48, 128), (4096, 4096), (1000, 1024), (6144, 4096),
                                          (4096, 12288)])
def test_unpack_is_bit_exact(rows, columns):
    from stark_b200.ops import QMatrix
    w = S.matvec_case(seed=rows + columns, rows=rows, columns=columns)
    q = QMatrix.from_affine(w["codes"], w["scales"], w["biases"], rows, columns)
    want = O.unpack_codes(w["codes"], 4, rows * columns).reshape(rows, columns)
    assert np.array_equal(q.unpack_codes(), want)
    assert q.device_bytes() == ((rows + 15) // 16) * (columns // 64) * 576


@pytest.mark.parametrize("rows,columns", [(16, 64), (48, 128), (4096, 4096), (1000, 1024), (6144, 4096),
                                          (4096, 12288), (151936, 1024)])
def test_matvec_bf16_matches_oracle(rows, columns):
    from stark_b200.ops import QMatrix, take_device_error
    w = S.matvec_case(seed=7 + rows, rows=rows, columns=columns)
    q = QMatrix.from_affine(w["codes"], w["scales"], w["biases"], rows, columns)
    got = q.matvec(w["x"])
    assert take_device_error() == 0
    want = O.affine_matvec_bf16(w["codes"], w["scales"], w["biases"], w["x"], rows, columns,
                                threads=O.max_threads())[0]
    err = _rel_err(got, want)
    assert err.max() < REL_TOL
    # far tighter in practice: same products, f32 accumulation in a different order
    assert (got != want).mean() < 0.02


def test_matvec_group_output_plane_layout():
    from stark_b200.ops import QMatrix
    rows, columns = 100, 256
    w = S.matvec_case(seed=11, rows=rows, columns=columns)
    pitch = (rows + 3) // 4 * 4
    st = np.zeros((columns // 64, pitch), np.uint16)
    bt = np.zeros((columns // 64, pitch), np.uint16)
    st[:, :rows] = w["scales"].T
    bt[:, :rows] = w["biases"].T
    q = QMatrix.from_affine(w["codes"], st, bt, rows, columns, scale_layout=1, plane_pitch=pitch)
    want = O.affine_matvec_bf16(w["codes"], w["scales"], w["biases"], w["x"], rows, columns)[0]
    assert _rel_err(q.matvec(w["x"]), want).max() < REL_TOL


def test_matvec_f32_hybrid_conventions():
    from stark_b200._lib import F32
    from stark_b200.ops import QMatrix
    rows, columns = 512, 2048
    w = S.matvec_case(seed=13, rows=rows, columns=columns)
    x = np.random.default_rng(2).standard_normal(columns).astype(np.float32)
    q = QMatrix.from_affine(w["codes"], w["scales"], w["biases"], rows, columns)
    got = q.matvec(x, io_type=F32)
    want = O.affine_matvec_f32(w["codes"], w["scales"], w["biases"], 30, x, rows, columns)
    # the reference's own bound for this comparison: 2e-5 * sum |w x| (weights.rs:4218-4297)
    wf = np.stack([O.affine_row_f32(w["codes"], w["scales"], w["biases"], 30, r, columns) for r in range(rows)])
    bound = 2e-5 * (np.abs(wf) * np.abs(x)).sum(axis=1)
    assert np.all(np.abs(got - want) <= bound)


def test_linearity_and_scaling_at_full_size():
    """Size-independent properties at the 4096x4096 benchmark size."""
    from stark_b200._lib import F32
    from stark_b200.ops import QMatrix
    w = S.matvec_case(seed=0)
    q = QMatrix.from_affine(w["codes"], w["scales"], w["biases"], 4096, 4096)
    rng = np.random.default_rng(4)
    a = rng.standard_normal(4096).astype(np.float32)
    b = rng.standard_normal(4096).astype(np.float32)
    ya, yb, yab = q.matvec(a, io_type=F32), q.matvec(b, io_type=F32), q.matvec(a + b, io_type=F32)
    np.testing.assert_allclose(yab, ya + yb, rtol=0, atol=2e-4 * np.abs(ya).mean() + 1e-4)
    # exact power-of-two scaling of the input scales the output exactly (the kernel rescales by 2^k)
    y4 = q.matvec(O.f32_to_bf16(O.bf16_to_f32(w["x"]) * 4.0))
    y1 = q.matvec(w["x"])
    assert np.array_equal(O.bf16_to_f32(y4), O.bf16_to_f32(y1) * 4.0)
    # zero input -> sum(bias * 0) = 0 exactly
    assert not q.matvec(np.zeros(4096, np.uint16)).any()


def test_repeatability_bitwise():
    from stark_b200.ops import QMatrix
    w = S.matvec_case(seed=21, rows=2048, columns=4096)
    q = QMatrix.from_affine(w["codes"], w["scales"], w["biases"], 2048, 4096)
    first = q.matvec(w["x"])
    for _ in range(3):
        assert np.array_equal(q.matvec(w["x"]), first)


def test_invalid_arguments_are_rejected():
    from stark_b200._lib import StarkB200Error
    from stark_b200.ops import QMatrix
    w = S.matvec_case(seed=1, rows=16, columns=64)
    with pytest.raises(ValueError):
        QMatrix.from_affine(w["codes"], w["scales"], w["biases"], 16, 128)
    q = QMatrix.from_affine(w["codes"], w["scales"], w["biases"], 16, 64)
    with pytest.raises(ValueError):
        q.matvec(np.zeros(63, np.uint16))
    with pytest.raises(StarkB200Error):
        QMatrix.from_affine(w["codes"], w["scales"], w["biases"], 16, 64, group=32)
