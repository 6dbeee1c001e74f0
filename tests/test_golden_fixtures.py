"""The committed oracle outputs: the oracle must reproduce them exactly (CPU), and the CUDA path must
meet the parity bars against the stored values (GPU)."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle as O
from stark_b200 import synthetic as S

GOLDEN = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def stored():
    return dict(np.load(GOLDEN / "oracle_outputs.npz"))


def test_oracle_reproduces_the_stored_outputs(stored):
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    fresh = mod.build()
    assert sorted(fresh) == sorted(stored)
    for name, want in stored.items():
        got = np.asarray(fresh[name])
        assert got.dtype == want.dtype and np.array_equal(got.view(np.uint8), want.view(np.uint8)), name


@pytest.mark.gpu
def test_cuda_matvec_and_block_decode_against_stored_values(stored):
    from stark_b200 import ops
    w = S.matvec_case(seed=3, rows=512, columns=1024)
    q = ops.QMatrix.from_affine(w["codes"], w["scales"], w["biases"], 512, 1024)
    got = O.bf16_to_f32(q.matvec(w["x"])).astype(np.float64)
    want = O.bf16_to_f32(stored["matvec_y"]).astype(np.float64)
    assert (np.abs(got - want) / np.maximum(np.abs(want), np.abs(want).mean())).max() < 1e-2
    rng = np.random.default_rng(11)
    for kind, gen, name in ((O.Q8_0, S.q8_0_rows, "q8_0_row"), (O.Q4_K, S.q4_k_rows, "q4_k_row")):
        data = gen(rng, 4, 512)
        row = ops.dequantize_row(ops.QMatrix.from_gguf(data, kind, 4, 512), 1)
        assert np.array_equal(row.view(np.uint32), stored[name].view(np.uint32)), name  # bit-exact decode


@pytest.mark.gpu
def test_cuda_decoder_against_stored_logits_and_tokens(stored):
    from stark_b200.engine import DenseModel
    from tests.test_model_gpu import assert_logits_accepted
    cfg = S.CONFIGS["tiny"]
    model = DenseModel.load(cfg, S.dense_weights(cfg, seed=0), context_tokens=128)
    model.prefill(S.prompt(cfg, 70, seed=5))
    assert_logits_accepted(stored["tiny_logits"], model.logits_bf16())
    tokens = model.generate_greedy(7)
    # the stored continuation is the oracle's own; on a 1024-way vocabulary with bf16 logits the two
    # may part ways at a near-tie, after which they are not comparable: require the first tokens
    assert int(tokens[0]) == int(stored["tiny_greedy"][0])
    agree = int((tokens[:4] == stored["tiny_greedy"][:4]).sum())
    assert agree >= 3, (tokens, stored["tiny_greedy"])
