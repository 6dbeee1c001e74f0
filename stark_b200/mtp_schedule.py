"""Per-round scheduling of speculative decoding: how many proposals a round makes, and whether they come from the
draft head or are copied from the request's own context.

Host logic of the reference restated (crates/stark-engine/src/engine/hybrid/mtp_policy.rs and mtp_lookup.rs): a plan
is a pure function of request-visible state -- the acceptance history of earlier rounds, the remaining budget, the
sampling mode and a static cost table -- so a seeded request reproduces its output on every run; no wall-clock
measurement enters a plan.  The constants of the estimator are the reference's; the cost table is this engine's
own (round times on a B200), because that is the one part the reference says to replace when kernels change.
"""
from __future__ import annotations

from dataclasses import dataclass, field

# ---- estimator constants (mtp_policy.rs:178-229)
ACCEPTANCE_WEIGHT = 0.0625       # exponential-average weight of an observation once a position is well observed
PRIOR_OBSERVATIONS = 2.0         # the n-th observation weighs max(1 / (n + 2), 1/16)
ACCEPTANCE_PRIOR = 0.85          # starting estimate of every head position
LOOKUP_PRIOR = 0.95              # starting estimate of every lookup position
ACCEPTANCE_DECAY = 1.0 / 96.0    # per-round pull of the first position, while unobserved, toward the prior
ACCEPTANCE_FOLLOW = 1.0 / 16.0   # per-round pull of a later unobserved position toward the one before it
HYSTERESIS = 0.02                # a challenger depth must promise this much more tokens per millisecond
DEPTH_SLOTS = 9

# ---- prompt lookup constants (mtp_lookup.rs:15-24)
GRAM = 4
MIN_AGREEMENT_ACROSS_LINE = 8
MIN_AGREEMENT = 32


def _extended(table, extra: float, index: int) -> float:
    """table[index], continued past its end by its last value plus `extra` per step (mtp_policy.rs:127-138)."""
    if index < len(table):
        return table[index]
    last = max(len(table) - 1, 0)
    return (table[last] if table else 0.0) + extra * (index - last)


@dataclass(frozen=True)
class RoundCosts:
    """Static per-round wall costs in milliseconds for one sampling mode (mtp_policy.rs:19-51, 140-176)."""
    serial_ms: float
    verify_ms: tuple
    verify_extra_row_ms: float
    draft_ms: tuple
    draft_extra_ms: float
    finish_ms: tuple
    finish_extra_draft_ms: float
    host_ms: tuple
    host_extra_draft_ms: float
    head_advance_ms: float
    lookup_verify_extra_ms: float

    def verify(self, rows: int) -> float:
        return _extended(self.verify_ms, self.verify_extra_row_ms, max(rows - 1, 0))

    def tail(self, drafts: int) -> float:
        return (self.verify(drafts + 1) + _extended(self.finish_ms, self.finish_extra_draft_ms, drafts)
                + _extended(self.host_ms, self.host_extra_draft_ms, drafts))

    def head_round_ms(self, drafts: int) -> float:
        if drafts == 0:
            return self.serial_ms
        return _extended(self.draft_ms, self.draft_extra_ms, drafts) + self.tail(drafts)

    def lookup_round_ms(self, drafts: int) -> float:
        return self.head_advance_ms + self.lookup_verify_extra_ms + self.tail(drafts)


@dataclass(frozen=True)
class CostTable:
    id: str
    greedy: RoundCosts
    sampled: RoundCosts

    def for_mode(self, greedy: bool) -> RoundCosts:
        return self.greedy if greedy else self.sampled


def _b200_costs() -> RoundCosts:
    # Qwen3-8B shape + one-layer head on one B200, 8 192 rows of cache, milliseconds per round measured with
    # `bench.py --workload qwen3-8b-mtp --drafts d --accept 1.0` for d = 0 .. 4: 1.97 (a round without proposals is
    # the recorded one-token sequence), 3.50, 3.80, 4.05, 4.33.  The verify pass streams every matrix once whatever
    # the row count, so a further row costs about 0.15 ms; a proposal costs the head's layer and one pass over the
    # read-out table, 0.11 ms (12 launches in the launch list).  What a round costs beyond those and the small
    # finish and host terms is booked as its verify pass.
    return RoundCosts(
        serial_ms=1.97,
        verify_ms=(3.28, 3.30, 3.48, 3.61, 3.77), verify_extra_row_ms=0.16,
        draft_ms=(0.0, 0.11, 0.22, 0.33, 0.44), draft_extra_ms=0.11,
        finish_ms=(0.05, 0.06, 0.07, 0.08, 0.09), finish_extra_draft_ms=0.01,
        host_ms=(0.03, 0.03, 0.03, 0.03, 0.03), host_extra_draft_ms=0.0,
        head_advance_ms=0.02, lookup_verify_extra_ms=0.0)


# Greedy only: acceptance under sampling runs on the host side of the boundary and is not timed here; the sampled
# table repeats the greedy one until it is.
B200_QWEN3_8B_V1 = CostTable("b200-qwen3-8b-4bit-v1", _b200_costs(), _b200_costs())


def expected_tokens(acceptance, drafts: int) -> float:
    """Expected committed tokens of a round: 1 + sum over k of the product of the conditional acceptances a[0..k]
    (mtp_policy.rs:231-244)."""
    expected, reach = 1.0, 1.0
    for i in range(drafts):
        reach *= acceptance[i] if i < len(acceptance) else 0.0
        expected += reach
    return expected


class Estimates:
    """Per-position conditional acceptance estimates and observation counts (mtp_policy.rs:246-292)."""

    def __init__(self, limit: int, prior: float):
        self.prior = prior
        self.acceptance = [prior] * limit
        self.observed = [0] * limit

    def update(self, proposed: int, accepted: int) -> None:
        # positions in order: an unobserved position drifts toward the already updated estimate before it
        for i in range(len(self.acceptance)):
            if i < proposed and i <= accepted:
                outcome = 1.0 if i < accepted else 0.0
                self.observed[i] = min(self.observed[i] + 1, 0xFFFFFFFF)
                weight = max(1.0 / (self.observed[i] + PRIOR_OBSERVATIONS), ACCEPTANCE_WEIGHT)
                self.acceptance[i] += weight * (outcome - self.acceptance[i])
            else:
                target, pull = (self.prior, ACCEPTANCE_DECAY) if i == 0 else (self.acceptance[i - 1], ACCEPTANCE_FOLLOW)
                self.acceptance[i] += pull * (target - self.acceptance[i])


class DepthPlanner:
    """Request-scoped depth planner; its state changes only through ``observe`` (mtp_policy.rs:318-419)."""

    def __init__(self, costs: RoundCosts, limit: int):
        self.costs, self.limit = costs, limit
        self.head = Estimates(limit, ACCEPTANCE_PRIOR)
        self.lookup = Estimates(limit, LOOKUP_PRIOR)
        self.incumbent = None

    def head_rate(self, drafts: int) -> float:
        return expected_tokens(self.head.acceptance, drafts) / self.costs.head_round_ms(drafts)

    def lookup_rate(self, drafts: int) -> float:
        return expected_tokens(self.lookup.acceptance, drafts) / self.costs.lookup_round_ms(drafts)

    def head_depth(self, cap: int) -> int:
        """Head depth in 0..=cap with the best expected tokens per millisecond; the incumbent stays unless a
        challenger beats it by HYSTERESIS; ties go to the smaller depth; the depth rises one step per round; a cap
        below the limit (the end of the budget) does not replace the incumbent."""
        cap = min(cap, self.limit)
        reach = cap if self.incumbent is None else min(cap, self.incumbent + 1)
        best = 0
        for drafts in range(1, reach + 1):
            if self.head_rate(drafts) > self.head_rate(best):
                best = drafts
        chosen = best
        if self.incumbent is not None:
            incumbent = min(self.incumbent, cap)
            if self.head_rate(best) <= self.head_rate(incumbent) * (1.0 + HYSTERESIS):
                chosen = incumbent
        if cap == self.limit:
            self.incumbent = chosen
        return chosen

    def lookup_depth(self, available: int, head: int):
        """Lookup depth in 1..=available that is at least as fast as `head` head drafts, if any."""
        available = min(available, self.limit)
        best = None
        for drafts in range(1, available + 1):
            if best is None or self.lookup_rate(drafts) > self.lookup_rate(best):
                best = drafts
        if best is not None and self.lookup_rate(best) >= self.head_rate(head):
            return best
        return None

    def observe(self, lookup: bool, proposed: int, accepted: int) -> None:
        ran, idle = (self.lookup, self.head) if lookup else (self.head, self.lookup)
        ran.update(proposed, accepted)
        idle.update(0, 0)


class NewlineTokens:
    """Which token ids decode to text with a line break, as a bitset over the vocabulary (mtp_lookup.rs:26-68)."""

    def __init__(self, vocabulary: int, contains_newline):
        self.bits = bytearray((vocabulary + 7) // 8)
        self.vocabulary = vocabulary
        for i in range(vocabulary):
            if contains_newline(i):
                self.bits[i >> 3] |= 1 << (i & 7)

    def __contains__(self, token: int) -> bool:
        return 0 <= token < self.vocabulary and bool(self.bits[token >> 3] & (1 << (token & 7)))

    def count(self) -> int:
        return sum(bin(b).count("1") for b in self.bits)


class PromptLookup:
    """Copies what followed the latest earlier occurrence of the context's last GRAM tokens, once the match is long
    enough backwards: 32 tokens, or 8 when it crosses a line break (mtp_lookup.rs:70-135)."""

    def __init__(self, context, newline: NewlineTokens):
        self.tokens = [int(t) for t in context]
        self.newline = newline
        self.index = {}
        for end in range(GRAM - 1, max(len(self.tokens) - 1, 0)):
            self.index[tuple(self.tokens[end + 1 - GRAM:end + 1])] = end + 1

    def push(self, token: int) -> None:
        end = len(self.tokens) - 1
        self.tokens.append(int(token))
        if len(self.tokens) > GRAM:
            self.index[tuple(self.tokens[end + 1 - GRAM:end + 1])] = end + 1

    def propose(self, limit: int) -> list:
        n = len(self.tokens)
        if limit == 0 or n < GRAM:
            return []
        nxt = self.index.get(tuple(self.tokens[n - GRAM:n]))
        if nxt is None:
            return []
        agreement, line = 0, False
        while agreement < MIN_AGREEMENT and agreement < nxt and self.tokens[nxt - 1 - agreement] == self.tokens[n - 1 - agreement]:
            line = line or (self.tokens[n - 1 - agreement] in self.newline)
            agreement += 1
        if agreement < MIN_AGREEMENT and not (line and agreement >= MIN_AGREEMENT_ACROSS_LINE):
            return []
        return self.tokens[nxt:min(n, nxt + limit)]

    def __len__(self) -> int:
        return len(self.tokens)


@dataclass
class ScheduleStats:
    """Aggregate scheduling counters; no token, logit or probability data (mtp_policy.rs:444-493)."""
    policy: str = "fixed"
    lookup: bool = False
    limit: int = 0
    head_rounds_by_depth: list = field(default_factory=lambda: [0] * DEPTH_SLOTS)
    head_round_seconds_by_depth: list = field(default_factory=lambda: [0.0] * DEPTH_SLOTS)
    lookup_round_seconds: float = 0.0
    lookup_rounds: int = 0
    lookup_proposed: int = 0
    lookup_accepted: int = 0
    head_advances: int = 0
    head_advance_seconds: float = 0.0
    cost_table: str | None = None

    def as_json(self) -> dict:
        slots = min(self.limit + 1, DEPTH_SLOTS)
        out = {"policy": self.policy}
        if self.cost_table is not None:
            out["cost_table"] = self.cost_table
        out.update(lookup=self.lookup, limit=self.limit, head_rounds_by_depth=self.head_rounds_by_depth[:slots],
                   head_round_seconds_by_depth=self.head_round_seconds_by_depth[:slots],
                   lookup_round_seconds=self.lookup_round_seconds, lookup_rounds=self.lookup_rounds,
                   lookup_proposed=self.lookup_proposed, lookup_accepted=self.lookup_accepted,
                   head_advances=self.head_advances, head_advance_seconds=self.head_advance_seconds)
        return out


class RoundScheduler:
    """Request-scoped round scheduler: the planner, the optional prompt-lookup index and their counters
    (mtp_policy.rs:495-620).  ``plan(cap)`` returns ("head", drafts) or ("lookup", [tokens])."""

    def __init__(self, adaptive: bool, costs: RoundCosts, limit: int, lookup: PromptLookup | None = None,
                 cost_table_id: str | None = None):
        self.adaptive = adaptive
        self.planner = DepthPlanner(costs, limit)
        self.lookup = lookup
        self.stats = ScheduleStats(policy="adaptive" if adaptive else "fixed", lookup=lookup is not None, limit=limit,
                                   cost_table=cost_table_id if adaptive else None)

    def plan(self, cap: int):
        head = self.planner.head_depth(cap) if self.adaptive else cap
        if cap == 0 or self.lookup is None:
            return ("head", head)
        proposal = self.lookup.propose(cap)
        if not proposal:
            return ("head", head)
        if self.adaptive:
            drafts = self.planner.lookup_depth(len(proposal), head)
            if drafts is None:
                return ("head", head)
            proposal = proposal[:drafts]
        return ("lookup", proposal)

    def observe(self, plan, accepted: int, committed, seconds: float) -> None:
        kind, what = plan
        proposed = what if kind == "head" else len(what)
        if kind == "head":
            if proposed < DEPTH_SLOTS:
                self.stats.head_rounds_by_depth[proposed] += 1
                self.stats.head_round_seconds_by_depth[proposed] += seconds
        else:
            self.stats.lookup_round_seconds += seconds
            self.stats.lookup_rounds += 1
            self.stats.lookup_proposed += proposed
            self.stats.lookup_accepted += accepted
        self.planner.observe(kind == "lookup", proposed, accepted)
        if self.lookup is not None:
            for token in committed:
                self.lookup.push(token)

    def record_head_advance(self, seconds: float) -> None:
        self.stats.head_advances += 1
        self.stats.head_advance_seconds += seconds
