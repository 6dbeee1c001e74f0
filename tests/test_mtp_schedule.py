"""The round scheduler's restatement against the cases the reference's own tests assert
(crates/stark-engine/src/engine/hybrid/mtp_policy.rs:622-914, mtp_lookup.rs:137-243).  Those tests run on the
reference's cost table (measured on its hardware); the table is repeated here as test data so that the planner's
decisions can be checked value for value.  The engine's own table is checked for shape only."""
import pytest

from stark_b200 import mtp_schedule as M

# CostTable::LILY_Q4_XL_LILYMERGE_01 (mtp_policy.rs:91-122): known-answer data of the reference's tests
GREEDY = M.RoundCosts(serial_ms=13.75, verify_ms=(12.80, 17.83, 22.86, 28.44), verify_extra_row_ms=5.58,
                      draft_ms=(0.0, 1.27, 2.29, 3.31), draft_extra_ms=1.02, finish_ms=(0.58, 0.75, 0.92, 1.09),
                      finish_extra_draft_ms=0.17, host_ms=(0.04, 0.07, 0.10, 0.13), host_extra_draft_ms=0.03,
                      head_advance_ms=0.40, lookup_verify_extra_ms=0.44)
SAMPLED = M.RoundCosts(serial_ms=13.61, verify_ms=(12.66, 17.44, 22.22, 27.70), verify_extra_row_ms=5.48,
                       draft_ms=(0.0, 1.36, 2.67, 4.00), draft_extra_ms=1.33, finish_ms=(0.55, 0.74, 0.93, 1.21),
                       finish_extra_draft_ms=0.28, host_ms=(0.13, 0.18, 0.24, 0.26), host_extra_draft_ms=0.02,
                       head_advance_ms=0.40, lookup_verify_extra_ms=0.75)
NL = 10


def test_cost_table_reproduces_the_measured_rounds():
    for costs, measured, serial, lookup in ((GREEDY, (19.92, 26.17, 32.96), 13.75, ((2, 24.71), (3, 30.50))),
                                            (SAMPLED, (19.72, 26.05, 33.17), 13.61, ((2, 24.54),))):
        for drafts, ms in enumerate(measured):
            assert abs(costs.head_round_ms(drafts + 1) - ms) < 0.05
        assert costs.head_round_ms(0) == serial
        for drafts, ms in lookup:
            assert abs(costs.lookup_round_ms(drafts) - ms) < 0.05
        assert costs.lookup_round_ms(3) < costs.head_round_ms(3)
        slope = costs.head_round_ms(5) - costs.head_round_ms(4)     # past the table: the last measured slopes
        assert costs.verify_extra_row_ms < slope < costs.verify_extra_row_ms + 3.0


def test_expected_tokens_is_one_plus_prefix_products():
    for acceptance, drafts, want in (((0.5, 0.5, 0.5), 0, 1.0), ((0.5, 0.5, 0.5), 1, 1.5), ((0.5, 0.5, 0.5), 3, 1.875),
                                     ((1.0, 0.0, 1.0), 3, 2.0), ((0.9, 0.8), 4, 1.0 + 0.9 + 0.72)):
        assert abs(M.expected_tokens(acceptance, drafts) - want) < 1e-12


def test_planner_matches_the_measured_best_depth():
    for costs, acceptance, expected in ((GREEDY, [0.932, 0.907, 0.80], (2,)), (SAMPLED, [0.740, 0.726, 0.37], (1, 2)),
                                        (GREEDY, [0.977, 0.945, 0.98], (3,)), (GREEDY, [0.67, 0.51, 0.09], (1,)),
                                        (GREEDY, [0.58, 0.50, 0.10], (1,)), (GREEDY, [0.20, 0.20, 0.20], (0,)),
                                        (SAMPLED, [0.20, 0.20, 0.20], (0,)), (SAMPLED, [1.0, 1.0, 1.0], (3,))):
        planner = M.DepthPlanner(costs, 3)
        planner.head.acceptance = list(acceptance)
        assert planner.head_depth(3) in expected, acceptance


def test_prior_opens_at_two_drafts_and_respects_the_cap():
    for costs in (GREEDY, SAMPLED):
        planner = M.DepthPlanner(costs, 3)
        assert planner.head_depth(3) == 2
        assert planner.head_depth(1) == 1
        assert planner.head_depth(0) == 0
        assert planner.incumbent == 2                                # a capped round does not replace the incumbent


def test_hysteresis_keeps_the_incumbent_until_a_challenger_is_two_percent_better():
    planner = M.DepthPlanner(GREEDY, 3)
    planner.head.acceptance = [0.932, 0.907, 0.80]
    assert planner.head_depth(3) == 2
    planner.head.acceptance = [0.95, 0.95, 0.86]
    assert planner.head_rate(3) > planner.head_rate(2)
    assert planner.head_rate(3) <= planner.head_rate(2) * (1.0 + M.HYSTERESIS)
    assert planner.head_depth(3) == 2
    planner.head.acceptance = [0.98, 0.97, 0.98]
    assert planner.head_depth(3) == 3
    planner.head.acceptance = [0.75, 0.1, 0.1]
    assert planner.head_depth(3) == 1 and planner.incumbent == 1


def test_observations_weigh_the_prior_as_two_and_unseen_positions_follow_their_predecessor():
    planner = M.DepthPlanner(SAMPLED, 3)
    planner.observe(False, 3, 1)
    p, d, f = M.ACCEPTANCE_PRIOR, M.ACCEPTANCE_DECAY, M.ACCEPTANCE_FOLLOW
    first, second = p + (1.0 / 3.0) * (1.0 - p), p + (1.0 / 3.0) * (0.0 - p)
    assert planner.head.acceptance[0] == first and planner.head.acceptance[1] == second
    assert planner.head.acceptance[2] == p + f * (second - p)
    assert planner.head.observed == [1, 1, 0]
    assert planner.lookup.acceptance == [M.LOOKUP_PRIOR] * 3
    planner = M.DepthPlanner(SAMPLED, 3)
    expected = p
    for n in range(1, 17):
        planner.observe(False, 1, 0)
        expected += max(1.0 / (n + M.PRIOR_OBSERVATIONS), M.ACCEPTANCE_WEIGHT) * (0.0 - expected)
        assert planner.head.acceptance[0] == expected
    assert 1.0 / (14.0 + M.PRIOR_OBSERVATIONS) == M.ACCEPTANCE_WEIGHT
    for _ in range(64):
        planner.observe(False, 1, 0)
    assert planner.head.acceptance[0] < 0.01 and planner.head.acceptance[1] < 0.5
    low = list(planner.head.acceptance)
    planner.observe(True, 2, 2)
    head0 = low[0] + d * (p - low[0])
    assert planner.head.acceptance[0] == head0
    assert planner.head.acceptance[1] == low[1] + f * (head0 - low[1])
    q = M.LOOKUP_PRIOR
    assert planner.lookup.acceptance[0] > q and planner.lookup.acceptance[1] > q
    assert planner.lookup.acceptance[2] == q + f * (planner.lookup.acceptance[1] - q)


def _run_hard_stretch():
    planner, depths = M.DepthPlanner(SAMPLED, 3), []
    for r in range(300):
        depth = planner.head_depth(3)
        depths.append(depth)
        planner.observe(False, depth, 0 if 60 <= r < 160 else depth)
    return depths


def test_adaptive_falls_back_and_recovers_deterministically():
    depths = _run_hard_stretch()
    assert depths == _run_hard_stretch()
    assert max(depths[:60]) == 3
    assert depths[150] <= 1
    assert depths[299] == 3


def _simulate(costs, rounds, rate):
    """Bernoulli acceptance from the fixed LCG of the reference's test, so a run is a pure function of its inputs."""
    planner, depths, state = M.DepthPlanner(costs, 3), [], 0x2545F4914F6CDD1D
    mask = (1 << 64) - 1

    def uniform():
        nonlocal state
        state = (state * 6364136223846793005 + 1442695040888963407) & mask
        return (state >> 11) / float(1 << 53)

    for r in range(rounds):
        depth = planner.head_depth(3)
        accepted = 0
        for position in range(depth):
            if uniform() < rate(r, position):
                accepted += 1
            else:
                break
        planner.observe(False, depth, accepted)
        depths.append(depth)
    return depths


def test_low_acceptance_settles_at_serial_quickly_and_recovers():
    for costs in (GREEDY, SAMPLED):
        depths = _simulate(costs, 400, lambda r, _: 0.3 if r < 150 else 0.95)
        assert depths.index(0) <= 8
        assert sum(d == 0 for d in depths[20:150]) >= 100
        assert sum(d >= 2 for d in depths[250:]) >= 140


def test_prose_acceptance_leaves_the_opening_depth_within_a_few_rounds():
    for costs in (GREEDY, SAMPLED):
        depths = _simulate(costs, 200, lambda _, position: (0.67, 0.51, 0.09)[position])
        assert depths[0] == 2
        assert next(i for i, d in enumerate(depths) if d < 2) <= 6
        assert sum(d == 1 for d in depths[10:]) >= 150


def test_lookup_is_preferred_only_when_it_beats_the_head_plan():
    for costs in (GREEDY, SAMPLED):
        planner = M.DepthPlanner(costs, 3)
        head = planner.head_depth(3)
        assert planner.lookup_depth(3, head) == 3
        assert planner.lookup_depth(0, head) is None
        planner.head.acceptance = [0.98, 0.97, 0.98]
        assert planner.head_depth(3) == 3
        assert planner.lookup_depth(3, 3) == 3
        assert planner.lookup_depth(1, 3) is None
        planner.observe(True, 3, 0)
        assert planner.lookup_depth(3, 3) is None
        planner.lookup.acceptance = [0.1, 0.1, 0.1]
        assert planner.lookup_depth(3, head) is None


def test_schedule_counts_rounds_and_serializes_up_to_the_limit():
    scheduler = M.RoundScheduler(True, GREEDY, 3)
    assert scheduler.plan(3) == ("head", 2)
    scheduler.observe(("head", 2), 2, [1, 2, 3], 0.03)
    scheduler.observe(("head", 0), 0, [4], 0.02)
    scheduler.record_head_advance(0.5)
    value = scheduler.stats.as_json()
    assert scheduler.stats.head_rounds_by_depth[:4] == [1, 0, 1, 0]
    assert value["policy"] == "adaptive" and value["head_rounds_by_depth"] == [1, 0, 1, 0] and value["head_advances"] == 1
    assert "cost_table" not in value and len(value) == 11
    fixed = M.RoundScheduler(False, SAMPLED, 3)
    assert fixed.plan(3) == ("head", 3) and fixed.plan(1) == ("head", 1)
    adaptive = M.RoundScheduler(True, GREEDY, 2, cost_table_id="some-table")
    assert adaptive.stats.as_json()["cost_table"] == "some-table" and len(adaptive.stats.as_json()) == 12
    assert "cost_table" not in M.RoundScheduler(False, GREEDY, 2, cost_table_id="some-table").stats.as_json()


# ---- prompt lookup (mtp_lookup.rs:137-243)
def _newline():
    return M.NewlineTokens(1000, lambda i: i == NL)


def _lookup(tokens):
    return M.PromptLookup(tokens, _newline())


def test_newline_set_is_a_bitset_over_the_vocabulary():
    s = M.NewlineTokens(130, lambda i: i % 64 == 3 or i == 129)
    assert 3 in s and 67 in s and 129 in s
    assert 4 not in s and 130 not in s and 0xFFFFFFFF not in s
    assert s.count() == 3


def test_copies_after_eight_tokens_of_agreement_across_a_line_break():
    line = [100, 101, 102, NL, 103, 104, 105, 106, 107, 108, 109]
    tokens = line + line[:8]
    assert _lookup(tokens).propose(3) == [107, 108, 109]
    assert _lookup(tokens).propose(8) == [107, 108, 109, 100, 101, 102, NL, 103]
    assert _lookup(tokens).propose(1) == [107]
    assert _lookup(tokens).propose(0) == []
    short = line + [1] + line[1:8]
    assert _lookup(short).propose(3) == []


def test_without_a_line_break_thirty_two_tokens_are_required():
    run = list(range(200, 240))
    tokens = run + run[:31]
    assert _lookup(tokens).propose(3) == []
    tokens.append(run[31])
    assert _lookup(tokens).propose(3) == [232, 233, 234]


def test_latest_occurrence_wins_and_push_matches_rebuild():
    first = [NL, 1, 2, 3, 4, 5, 6, 7, 8, 50]
    second = [NL, 1, 2, 3, 4, 5, 6, 7, 8, 60]
    tokens = first + second + second[:9]
    assert _lookup(tokens).propose(2) == [60, NL]
    incremental = _lookup(tokens[:5])
    for t in tokens[5:]:
        incremental.push(t)
    rebuilt = _lookup(tokens)
    assert incremental.index == rebuilt.index
    assert incremental.propose(3) == rebuilt.propose(3) and len(incremental) == len(tokens)


def test_the_current_tail_never_matches_itself():
    assert _lookup([300 + i for i in range(64)]).propose(3) == []
    assert _lookup([1, 2, 3]).propose(3) == [] and _lookup([]).propose(3) == []
    grow = _lookup([])
    for t in (1, 2, 3, 4, 5):
        grow.push(t)
    assert grow.propose(3) == []


def test_the_engines_own_table_is_well_formed():
    t = M.B200_QWEN3_8B_V1
    for costs in (t.greedy, t.sampled):
        rounds = [costs.head_round_ms(d) for d in range(8)]
        assert all(b > a for a, b in zip(rounds[1:], rounds[2:]))       # every proposal costs something
        assert costs.lookup_round_ms(2) < costs.head_round_ms(2)         # a lookup round skips the head
    assert t.id and t.for_mode(True) is t.greedy
