"""The exact speculative sampler's restatement against the cases the reference's own tests assert
(crates/stark-generate/src/hybrid/mtp.rs:405-1121), against the oracle's host sampler for the ordinary draw, and
against the property that makes it exact: committed tokens are distributed as ordinary samples of the target."""
import numpy as np
import pytest

from oracle import oracle as O
from stark_b200 import mtp_sampler as M

OPTIONS = {"mode": "stochastic", "temperature": 1.0, "top_k": None, "top_p": None, "min_p": None}
GREEDY = {"mode": "greedy"}


def _weights(w):
    idx = [i for i, x in enumerate(w) if x > 0.0]
    return M.Distribution(idx, [w[i] for i in idx], sum(w[i] for i in idx))


def test_splitmix_and_ordinary_draws_match_the_pinned_host_sampler():
    state = 1234567
    for _ in range(5):
        want, want_state = O.splitmix64_uniform(state)
        got, state = M.splitmix64_uniform(state)
        assert got == want and state == want_state
    rng = np.random.default_rng(3)
    for case in range(60):
        logits = (rng.standard_normal(97) * 3).astype(np.float32)
        if case % 5 == 0:
            logits[rng.integers(0, 97, 6)] = logits[0]                     # ties keep index order
        s = dict(OPTIONS, temperature=float(rng.choice([0.5, 0.7, 1.0, 1.3])),
                 top_k=int(rng.integers(1, 60)) if case % 2 else None,
                 top_p=float(rng.uniform(0.3, 0.99)) if case % 3 else None,
                 min_p=float(rng.uniform(0.001, 0.2)) if case % 4 == 0 else None)
        seed = int(rng.integers(0, 2 ** 63))
        want, want_state = O.host_sampling(logits, seed, s["temperature"], s["top_k"], s["top_p"], s["min_p"])
        got, got_state = M.draw(M.sampling_distribution(logits, s), seed, False)
        assert got == want and got_state == want_state, case


def test_greedy_point_proposals_are_an_argmax_compare_without_randomness():
    logits = [0.5, 3.0, 1.0, -2.0]
    for proposal in range(4):
        s = M.ExactMtpSampler(GREEDY, 5)
        s.begin_round()
        s.draft_point_mass(proposal)
        s.draft_point_mass(2)
        assert s.target(logits, proposal) == 1
        if proposal == 1:
            assert s.phase == s.VERIFYING and len(s.proposals) == 1
            assert s.target(logits, 2) == 1
        else:
            assert s.phase == s.FINISHED and not s.proposals
        assert s.rng == 5


def test_point_proposals_mix_with_lifecycle_checks_and_fail_closed():
    s = M.ExactMtpSampler(OPTIONS, 0)
    s.begin_round()
    s.draft_point_mass(1)
    with pytest.raises(M.SamplerError):
        s.target([0.0, 1.0], 0)                                             # a mismatched verify token
    s = M.ExactMtpSampler(OPTIONS, 0)
    s.begin_round()
    s.target([0.0, 1.0], None)
    s.begin_round()
    with pytest.raises(M.SamplerError):
        s.draft_point_mass(2)                                               # outside the now known vocabulary
    s = M.ExactMtpSampler(OPTIONS, 0)
    s.begin_round()
    s.draft_point_mass(0)
    s.target([5.0, -5.0], 0)
    with pytest.raises(M.SamplerError):
        s.draft_point_mass(1)                                               # after verification began


def test_residual_excludes_rejected_token_and_honors_support_holes():
    target = _weights([0.1, 0.0, 0.4, 0.5])
    draft = {0: 0.8, 1: 0.2}
    r = M.residual_distribution(target, lambda i: draft.get(i, 0.0))
    assert r.indices == [2, 3] and r.probability(0) == 0.0 and r.probability(1) == 0.0
    assert abs(r.probability(2) - 4.0 / 9.0) < 1e-15
    assert M.acceptance_probability(0.0, 1.0) == 0.0
    with pytest.raises(M.SamplerError):
        M.acceptance_probability(1.0, 0.0)


def test_matching_distributions_accept_and_bonus_uses_target_stream():
    logits = [0.5, 1.5, -0.5]
    s = M.ExactMtpSampler(OPTIONS, 37)
    s.begin_round()
    first, second = s.draft(logits), s.draft(logits)
    assert s.target(logits, first) == first and s.target(logits, second) == second
    bonus = s.target(logits, None)
    want, want_state = O.host_sampling(np.float32(logits), 37, 1.0, None, None, None)
    assert bonus == want and s.rng == want_state


def test_prompt_draw_matches_ordinary_sampling_and_can_only_run_once():
    logits = np.float32([1.0, 1.75, 0.5, -1.0, 2.0, 1.5])
    opts = dict(OPTIONS, temperature=0.7, top_k=4, top_p=0.8)
    s = M.ExactMtpSampler(opts, 91)
    want, want_state = O.host_sampling(logits, 91, 0.7, 4, 0.8, None)
    assert s.sample_initial(logits) == want and s.rng == want_state
    with pytest.raises(M.SamplerError):
        s.sample_initial(logits)
    with pytest.raises(M.SamplerError):
        s.draft(logits)                                                     # failed closed


def test_tiny_residual_stays_normalized_and_excludes_the_rejection():
    delta = np.finfo(np.float64).eps
    target = _weights([0.5 + delta, 0.5 - delta])
    r = M.residual_distribution(target, lambda i: 0.5)
    assert M.acceptance_probability(target.probability(1), 0.5) < 1.0
    assert 0.0 < r.total < 1e-14 and r.probability(0) == 1.0 and r.probability(1) == 0.0


def test_underflowed_candidates_remain_impossible_when_rejecting():
    fmax = float(np.finfo(np.float32).max)
    for seed in range(256):
        s = M.ExactMtpSampler(OPTIONS, seed)
        s.begin_round()
        proposal = s.draft([-fmax, fmax, 0.0])
        assert proposal == 1
        assert s.target([fmax, -fmax, 0.0], proposal) == 0


def test_disjoint_greedy_support_rejects_and_discards_later_proposals():
    s = M.ExactMtpSampler(GREEDY, 11)
    s.begin_round()
    first = s.draft([2.0, 1.0])
    s.draft([2.0, 1.0])
    assert s.target([1.0, 2.0], first) == 1
    assert not s.proposals and s.rng == 11
    s.begin_round()
    assert s.target([1.0, 2.0], None) == 1


def _replay(seed):
    s, draws = M.ExactMtpSampler(OPTIONS, seed), []
    for _ in range(16):
        s.begin_round()
        first, second = s.draft([1.0, 2.0, 3.0]), s.draft([1.0, 2.0, 3.0])
        out = s.target([3.0, 2.0, 1.0], first)
        draws.append(out)
        if out == first:
            out = s.target([3.0, 2.0, 1.0], second)
            draws.append(out)
            if out == second:
                draws.append(s.target([3.0, 2.0, 1.0], None))
    return draws


def test_sampler_is_seeded_and_draft_randomness_does_not_advance_target_rng():
    assert _replay(27) == _replay(27) and _replay(27) != _replay(28)
    s = M.ExactMtpSampler(OPTIONS, 17)
    s.draft([0.0, 0.0])
    assert s.rng == 17


def test_dense_filters_keep_full_vocabulary_nucleus_mass_when_top_k_is_enabled():
    # four equal logits, k = 2 and p = 0.4: two ids under the full-vocabulary policy, one under the top-k-first one
    opts = dict(OPTIONS, top_k=2, top_p=0.4)
    assert len(M.dense_distribution(np.zeros(4, np.float32), opts).indices) == 2
    assert len(M.sampling_distribution(np.zeros(4, np.float32), opts).indices) == 1


def test_invalid_order_nonfinite_and_changed_geometry_fail_closed():
    s = M.ExactMtpSampler(OPTIONS, 1)
    s.begin_round()
    with pytest.raises(M.SamplerError):
        s.target([0.0, 1.0], 1)                                             # no proposal was made
    for bad in ([0.0, float("nan")], [float("inf"), 0.0], []):
        s = M.ExactMtpSampler(OPTIONS, 1)
        s.begin_round()
        with pytest.raises(M.SamplerError):
            s.draft(bad)
        with pytest.raises(M.SamplerError):
            s.draft([0.0, 1.0])                                             # stays failed
    s = M.ExactMtpSampler(OPTIONS, 1)
    s.begin_round()
    t = s.draft([0.0, 1.0])
    with pytest.raises(M.SamplerError):
        s.target([0.0, 1.0, 2.0], t)                                        # the vocabulary changed
    s = M.ExactMtpSampler(OPTIONS, 1)
    s.begin_round()
    s.target([0.0, 1.0], None)
    with pytest.raises(M.SamplerError):
        s.target([0.0, 1.0], None)                                          # the round is finished


def test_sampled_rejection_recovers_the_target_distribution():
    """The property that makes the sampler exact: whatever q is, the token committed for a verified row is
    distributed as p.  20 000 seeded rounds, each cell within five standard deviations."""
    target_logits, draft_logits = np.float32([1.0, 0.2, -0.5, 2.0, 0.0]), np.float32([-1.0, 2.0, 0.5, 0.0, 1.0])
    p = M.sampling_distribution(target_logits, OPTIONS)
    counts, rounds = np.zeros(5), 20000
    for seed in range(rounds):
        s = M.ExactMtpSampler(OPTIONS, seed * 7919 + 13)
        s.begin_round()
        counts[s.target(target_logits, s.draft(draft_logits))] += 1
    for token in range(5):
        prob = p.probability(token)
        assert abs(counts[token] / rounds - prob) < 5.0 * np.sqrt(prob * (1 - prob) / rounds), (token, counts)
    # and with a point-mass proposal
    counts = np.zeros(5)
    for seed in range(rounds):
        s = M.ExactMtpSampler(OPTIONS, seed * 104729 + 1)
        s.begin_round()
        s.draft_point_mass(1)
        counts[s.target(target_logits, 1)] += 1
    for token in range(5):
        prob = p.probability(token)
        assert abs(counts[token] / rounds - prob) < 5.0 * np.sqrt(prob * (1 - prob) / rounds), (token, counts)
