"""The stochastic sampler: the oracle against the published Philox4x32-10 known answers and the
reference's own unit-interval test, host-side seed derivation, and (GPU) the device sampler against
the oracle on seeded rows."""
import numpy as np
import pytest

from oracle import oracle as O
from stark_b200.engine import position_seed


def test_philox_known_answers():
    """The three known-answer vectors published with the Philox generator (Random123 `kat_vectors`,
    philox4x32 with 10 rounds): zeros, all ones, and the digits of pi."""
    assert O.philox4x32_10([0, 0, 0, 0], [0, 0]).tolist() == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert O.philox4x32_10([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2).tolist() == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert O.philox4x32_10([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0]).tolist() == [
        0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]


def test_unit_interval_stays_open():
    """crates/stark-engine/unit/encodable_block/sampling/gumbel_test.rs:8-12."""
    assert O.unit_interval(0xFFFFFFFF) == 1.0 - 2.0 ** -24
    assert O.unit_interval(0) == 2.0 ** -24
    assert O.unit_interval(255) == 2.0 ** -24


def test_counter_layout_and_seed_derivation():
    # revidx (gumbel.rs:66-80): 1024 threads, 4 words per counter, vocab rounded up to 4096 per thread
    assert O.revidx(0, 151936) == (0, 0)
    assert O.revidx(1023, 151936) == (1023 * 38, 0)
    assert O.revidx(1024, 151936) == (0, 1)
    assert O.revidx(4096 + 7, 151936) == (7 * 38 + 1, 0)
    for seed, pos in [(0, 0), (1, 2), (2 ** 64 - 1, 5), (123456789, 4096)]:
        assert position_seed(seed, pos) == O.prng_derive(seed, pos)
    assert position_seed(0, 0) == 0  # the finalizer fixes zero


def test_oracle_sampler_semantics():
    rng = np.random.default_rng(0)
    l = rng.standard_normal(1000).astype(np.float32)
    assert O.unified_sampling(l) == int(l.argmax())
    tie = l.copy()
    tie[[10, 700]] = tie.max() + 1
    assert O.unified_sampling(tie) == 10                       # first index of the maximum
    bad = l.copy()
    bad[5] = np.inf
    assert O.unified_sampling(bad) == 0xFFFFFFFF               # non-finite logit: invalid row
    assert O.unified_sampling(l, seed=3, top_k=1) == int(l.argmax())   # one candidate left: noise cannot matter
    order = np.argsort(-l, kind="stable")
    for seed in range(20):
        assert O.unified_sampling(l, seed=seed, top_k=5) in order[:5].tolist()
        assert O.unified_sampling(l, seed=seed, temperature=0.5, min_p=0.5) in np.flatnonzero(
            l / np.float32(0.5) >= (l / np.float32(0.5)).max() + np.log(np.float32(0.5))).tolist()
    draws = {O.unified_sampling(l, seed=s, temperature=1.0) for s in range(64)}
    assert len(draws) > 20                                     # the noise really spreads the choice
    huge = np.array([3e38, 1.0, -3e38], np.float32)            # 1/T overflows the product: centred, not invalid
    assert O.unified_sampling(huge, seed=1, temperature=0.01) == 0


@pytest.mark.gpu
def test_device_sampler_matches_oracle():
    from stark_b200 import ops
    rng = np.random.default_rng(5)
    vocab = 151936
    base = (rng.standard_normal(vocab) * 3.0).astype(np.float32)
    bf = O.bf16_to_f32(O.f32_to_bf16(base))  # bf16-valued logits: many exact ties, as in the engine
    cases = [dict(), dict(seed=11), dict(seed=12, temperature=0.7), dict(seed=13, temperature=0.8, top_k=40),
             dict(seed=14, temperature=1.3, top_p=0.9), dict(seed=15, min_p=0.05),
             dict(seed=16, temperature=0.6, top_k=50, top_p=0.95, min_p=0.02), dict(top_k=3), dict(seed=17, top_k=1)]
    agree = 0
    for i, kw in enumerate(cases):
        for row in (base, bf):
            want = O.unified_sampling(row, **kw)
            got = ops.sample(row, **kw)
            agree += int(got == want)
    # device expf / logf differ from the host libm in the last bit, which can flip a near-tie of noisy scores
    assert agree >= 2 * len(cases) - 1, agree
    assert ops.sample(O.f32_to_bf16(bf), seed=21, temperature=0.9, top_k=20) == O.unified_sampling(
        bf, seed=21, temperature=0.9, top_k=20)               # bf16 input
    bad = base.copy()
    bad[77] = np.nan
    assert ops.sample(bad, seed=1) == 0xFFFFFFFF
    from stark_b200._lib import StarkB200Error
    for kw in (dict(temperature=0.0), dict(temperature=101.0), dict(top_k=0), dict(top_k=vocab + 1), dict(top_p=0.0),
               dict(top_p=1.5), dict(min_p=-0.1)):
        with pytest.raises(StarkB200Error):
            ops.sample(base, seed=1, **kw)
    small = rng.standard_normal(1000).astype(np.float32)      # a short row: idle lanes in the sort
    for s in range(8):
        assert ops.sample(small, seed=s, temperature=0.7, top_k=10, top_p=0.9) == O.unified_sampling(
            small, seed=s, temperature=0.7, top_k=10, top_p=0.9)


@pytest.mark.gpu
def test_model_sampling_follows_the_last_row():
    from stark_b200 import synthetic as S
    from stark_b200.engine import DenseModel
    cfg = S.CONFIGS["tiny"]
    model = DenseModel.load(cfg, S.dense_weights(cfg, seed=0), context_tokens=64)
    model.prefill(S.prompt(cfg, 9, seed=1))
    logits = model.logits()
    assert model.sample() == model.argmax() == O.unified_sampling(logits)
    for pos in range(4):
        seed = position_seed(42, model.position)
        tok = model.sample(seed=seed, temperature=0.8, top_k=20)
        assert tok == O.unified_sampling(model.logits(), seed=seed, temperature=0.8, top_k=20)
        model.step_async(tok)


# ---- the generation worker's host sampler (sorted f64 probabilities, SplitMix64) ----

def _full_sort_sample(logits, rng, temperature, top_k=None, top_p=None, min_p=None):
    """An independent restatement in numpy/Python of the full-sort form of the sampler
    (crates/stark-generate/src/hybrid.rs:1773-1816 keeps the same form as its differential oracle)."""
    import math
    logits = np.asarray(logits, np.float32)
    order = sorted(range(logits.size), key=lambda i: (O.descending_sample_key(float(logits[i])), i))
    order = order[:min(top_k, logits.size) if top_k is not None else logits.size]
    top = logits[order[0]]
    p = [math.exp(float(np.float32(np.float32(logits[i] - top) / np.float32(temperature)))) for i in order]
    total = 0.0
    for v in p:
        total += v
    kept, cum = 0, 0.0
    for v in p:
        if kept > 0 and ((min_p is not None and v < float(np.float32(min_p)))
                         or (top_p is not None and cum / total >= float(np.float32(top_p)))):
            break
        cum += v
        kept += 1
    u, rng = O.splitmix64_uniform(rng)
    target, mass = u * cum, 0.0
    for n in range(kept):
        mass += p[n]
        if target < mass:
            return order[n], rng
    return order[kept - 1], rng


def test_splitmix64_known_answers():
    """The first outputs of SplitMix64 from state 0 (the vectors published with the generator), seen
    through `uniform` (hybrid.rs:1103-1111): the top 53 bits scaled by 2^-53, state advanced by the step."""
    state = 0
    for word in (0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F):
        u, state = O.splitmix64_uniform(state)
        assert u == (word >> 11) / 2.0 ** 53
    assert state == (3 * O.SPLITMIX64_STEP) % 2 ** 64


def test_host_sampler_reference_cases():
    """hybrid.rs:1653-1664, 1751-1769, 2032-2062 (the cases the reference's own tests assert) and the
    descending key's order (hybrid.rs:1320-1328)."""
    f = lambda *v: np.array(v, np.float32)
    assert O.host_sampling(f(-1000.0, 1000.0), 99, 1.0, top_k=1, top_p=0.5)[0] == 1
    for seed in range(100):
        assert O.host_sampling(f(0.0, -1.0), seed, 1.0, min_p=0.9)[0] == 0   # min-p is relative to the top one
    assert O.host_sampling(f(0.0, 0.0), 12) == O.host_sampling(f(0.0, 0.0), 12)
    for bad in (np.nan, np.inf, -np.inf):
        assert O.host_sampling(f(0.0, bad), 0) == (0xFFFFFFFF, 0)             # no draw: the state stays
    assert O.host_sampling(f(), 0)[0] == 0xFFFFFFFF
    keys = [O.descending_sample_key(v) for v in (np.inf, 3.0, 1e-45, 0.0, -0.0, -1e-45, -3.0, -np.inf)]
    assert keys == sorted(keys) and len(set(keys)) == len(keys)              # +0 sorts before -0
    tok, state = O.host_sampling(f(0.5, 0.25), 7)
    assert state == (7 + O.SPLITMIX64_STEP) % 2 ** 64


def test_host_sampler_matches_full_sort_form():
    rng = np.random.default_rng(31)
    for n in (1, 2, 33, 257, 2000):
        row = (rng.standard_normal(n) * 2.5).astype(np.float32)
        row[rng.integers(0, n, max(1, n // 8))] = row[0]                      # ties
        if n > 2:
            row[1], row[2] = 0.0, -0.0
        for kw in (dict(), dict(top_k=5), dict(top_p=0.8), dict(min_p=0.1), dict(top_k=40, top_p=0.95, min_p=0.01)):
            for seed in (0, 1, 2 ** 63 + 5):
                for t in (0.5, 1.0, 1.7):
                    assert O.host_sampling(row, seed, t, **kw) == _full_sort_sample(row, seed, t, **kw)


@pytest.mark.gpu
def test_device_ordered_sampler_matches_oracle():
    from stark_b200 import ops
    from stark_b200._lib import StarkB200Error
    rng = np.random.default_rng(6)
    vocab = 151936
    base = (rng.standard_normal(vocab) * 3.0).astype(np.float32)
    bf = O.bf16_to_f32(O.f32_to_bf16(base))
    peaked = base.copy()
    peaked[4242] = 60.0                                                       # the tail stops moving the sums early
    cases = [dict(), dict(temperature=0.7), dict(temperature=0.8, top_k=40), dict(temperature=1.3, top_p=0.9),
             dict(min_p=0.05), dict(temperature=0.6, top_k=50, top_p=0.95, min_p=0.02), dict(top_k=1),
             dict(top_p=1.0), dict(temperature=100.0, top_p=0.999), dict(temperature=0.05)]
    total = agree = 0
    for kw in cases:
        for row in (base, bf, peaked):
            for seed in (3, 2 ** 64 - 1, 0x1234_5678_9ABC_DEF0):
                want, _ = O.host_sampling(row, seed, kw.get("temperature", 1.0),
                                          **{k: v for k, v in kw.items() if k != "temperature"})
                got = ops.sample(row, seed=seed, ordered=True, **kw)
                total += 1
                agree += int(got == want)
    # the device's f64 exp is within 1 ulp of the host's, not identical: a target that lands within a few
    # ulps of a partial sum can resolve to the neighbouring candidate
    assert agree >= total - 2, (agree, total)
    assert ops.sample(O.f32_to_bf16(bf), seed=21, temperature=0.9, top_k=20, ordered=True) == O.host_sampling(
        bf, 21, 0.9, top_k=20)[0]                                             # bf16 input
    bad = base.copy()
    bad[77] = -np.inf
    assert ops.sample(bad, seed=1, ordered=True) == 0xFFFFFFFF
    with pytest.raises(StarkB200Error):
        ops.sample(base, ordered=True)                                        # the ordered sampler only draws
    zeros = np.zeros(70, np.float32)
    zeros[1::2] = -0.0                                                        # +0 candidates come first, by id
    small = rng.standard_normal(1000).astype(np.float32)
    for s in range(8):
        assert ops.sample(zeros, seed=s, top_k=35, ordered=True) == O.host_sampling(zeros, s, top_k=35)[0]
        assert ops.sample(zeros, seed=s, top_k=35, ordered=True) % 2 == 0
        assert ops.sample(small, seed=s, temperature=0.7, top_k=10, top_p=0.9, ordered=True) == O.host_sampling(
            small, s, 0.7, top_k=10, top_p=0.9)[0]
