"""Exact speculative sampling on the host side of the boundary.

The reference's `ExactMtpSampler` restated (crates/stark-generate/src/hybrid/mtp.rs:72-403): proposals are drawn
from the draft distribution q, accepted with probability min(1, p/q) against the target distribution p, and a
rejection draws from the normalized positive part of p - q, so that the committed text is distributed exactly as
ordinary sampling from p.  Distributions are the worker's own (`sampling_distribution`,
crates/stark-generate/src/hybrid.rs:1153-1212: candidates in descending order of logit, f64 weights
exp((l - max) / T), top-k, then the min-p / top-p prefix); draws use SplitMix64 with a separate stream for the
proposals, so draft randomness never advances the target stream.  A point-mass proposal (a token copied from the
context, q = 1) needs no randomness.

The engine hands this sampler the rows it needs: `stark_b200_readout_f32` for the prompt's last row and the head's
rows, `stark_b200_mtp_readout_row_f32` for the rows of a verify pass.  Nothing here touches the device.
"""
from __future__ import annotations

import math

import numpy as np

MASK64 = (1 << 64) - 1
DRAFT_SEED_DOMAIN = 0x4D54505F44524146   # mtp.rs:19
SPLITMIX64_STEP = 0x9E3779B97F4A7C15


class SamplerError(Exception):
    pass


def splitmix64_uniform(state: int) -> tuple[float, int]:
    """One SplitMix64 step and its output as a double in [0, 1) (hybrid.rs `uniform`)."""
    state = (state + SPLITMIX64_STEP) & MASK64
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    z ^= z >> 31
    return (z >> 11) * (1.0 / (1 << 53)), state


class Distribution:
    __slots__ = ("indices", "weights", "total")

    def __init__(self, indices, weights, total):
        self.indices, self.weights, self.total = list(indices), list(weights), float(total)

    def probability(self, token: int) -> float:
        for i, w in zip(self.indices, self.weights):
            if i == token:
                return w / self.total
        return 0.0


def greedy_index(logits: np.ndarray) -> int:
    """First index whose logit no other exceeds; a non-finite row is refused (hybrid.rs:1214-1260)."""
    if logits.size == 0 or not np.isfinite(logits).all():
        raise SamplerError("native_generation_failed")
    return int(np.argmax(logits))


def sampling_distribution(logits, sampling: dict) -> Distribution:
    """hybrid.rs:1153-1212.  `sampling`: {"mode": "greedy"} or {"mode": "stochastic", "temperature", "top_k",
    "top_p", "min_p"} with None for an absent filter."""
    logits = np.asarray(logits, np.float32)
    if sampling["mode"] != "stochastic":
        return Distribution([greedy_index(logits)], [1.0], 1.0)
    if logits.size == 0 or not np.isfinite(logits).all():
        raise SamplerError("native_generation_failed")
    top_k, top_p, min_p = sampling.get("top_k"), sampling.get("top_p"), sampling.get("min_p")
    k = logits.size if top_k is None else min(int(top_k), logits.size)
    if k == 0:
        raise SamplerError("native_generation_failed")
    # descending by value, ties by ascending index; -0.0 sorts below +0.0 as under total_cmp
    keys = logits.view(np.int32).astype(np.int64)
    keys = np.where(keys < 0, -(keys & 0x7FFFFFFF) - 1, keys)
    order = np.lexsort((np.arange(logits.size), -keys))[:k]
    top = logits[order[0]]
    with np.errstate(over="ignore"):   # a difference of extreme logits overflows to -inf, whose weight is 0
        args = ((logits[order] - top) / np.float32(sampling["temperature"])).astype(np.float32)
    weights = [math.exp(float(a)) for a in args]
    total = 0.0
    for w in weights:
        total += w
    kept, cumulative = 0, 0.0
    for w in weights:
        if kept > 0 and ((min_p is not None and w < float(np.float32(min_p)))
                         or (top_p is not None and cumulative / total >= float(np.float32(top_p)))):
            break
        cumulative += w
        kept += 1
    return Distribution([int(i) for i in order[:kept]], weights[:kept], cumulative)


def dense_distribution(logits, sampling: dict) -> Distribution:
    """The converted-model path's filter order: nucleus mass measured against the full vocabulary, then top-k
    (mtp.rs:263-291)."""
    if sampling["mode"] != "stochastic" or sampling.get("top_k") is None:
        return sampling_distribution(logits, sampling)
    d = sampling_distribution(logits, dict(sampling, top_k=None))
    k = int(sampling["top_k"])
    d.indices, d.weights = d.indices[:k], d.weights[:k]
    d.total = float(sum(d.weights))
    return d


def acceptance_probability(p: float, q: float) -> float:
    if not math.isfinite(p) or not math.isfinite(q) or p < 0.0 or q <= 0.0:
        raise SamplerError("MTP proposal probability")
    return min(p / q, 1.0)


def residual_distribution(target: Distribution, draft) -> Distribution:
    """Normalized positive part of p - q over the target's support, in the target's order (mtp.rs:350-375).
    `draft` maps a token to its proposal probability (0 outside the proposal's support)."""
    indices, weights, total = [], [], 0.0
    for i, w in zip(target.indices, target.weights):
        r = max(w / target.total - draft(i), 0.0)
        if r > 0.0:
            indices.append(i)
            weights.append(r)
            total += r
    if not math.isfinite(total) or total <= 0.0 or not indices:
        raise SamplerError("MTP rejection residual")
    return Distribution(indices, weights, total)


def draw(d: Distribution, rng: int, greedy: bool) -> tuple[int, int]:
    """(token, advanced state); greedy takes the first candidate and leaves the state alone (mtp.rs:377-401)."""
    if not d.indices or not math.isfinite(d.total) or d.total <= 0.0:
        raise SamplerError("MTP draw distribution")
    if greedy:
        return d.indices[0], rng
    u, rng = splitmix64_uniform(rng)
    target, mass = u * d.total, 0.0
    for i, w in zip(d.indices, d.weights):
        mass += w
        if target < mass:
            return i, rng
    return d.indices[-1], rng


class ExactMtpSampler:
    """One request's sampler: `begin_round`, then `draft` / `draft_point_mass` for each proposal, then `target` for
    each verified row in order (with the proposal it verifies, or None for the bonus row after the last one).
    Any misuse fails closed: every later call raises."""
    DRAFTING, VERIFYING, FINISHED = range(3)

    def __init__(self, sampling: dict, rng: int, dense_filters: bool = False):
        self.sampling, self.rng = sampling, rng & MASK64
        self.draft_rng = (rng ^ DRAFT_SEED_DOMAIN) & MASK64
        self.greedy = sampling["mode"] != "stochastic"
        self.dense = bool(dense_filters) and not self.greedy and sampling.get("top_k") is not None \
            and sampling.get("top_p") is not None
        self.proposals, self.phase, self.vocabulary, self.failed = [], self.DRAFTING, None, False

    def _guarded(self, fn, *a):
        try:
            return fn(*a)
        except SamplerError:
            self.failed = True
            raise

    def _distribution(self, logits) -> Distribution:
        logits = np.asarray(logits, np.float32)
        if self.failed or (self.vocabulary is not None and self.vocabulary != logits.size):
            raise SamplerError("MTP sampler vocabulary or state")
        try:
            d = dense_distribution(logits, self.sampling) if self.dense else sampling_distribution(logits, self.sampling)
        except SamplerError:
            raise SamplerError("MTP sampling distribution") from None
        self.vocabulary = logits.size
        return d

    def sample_initial(self, logits) -> int:
        """The prompt's first draw: exactly the ordinary sampler, once, before the first round (mtp.rs:131-152)."""
        def run():
            if self.failed or self.phase != self.DRAFTING or self.proposals or self.vocabulary is not None:
                raise SamplerError("native_generation_failed")
            token, self.rng = draw(self._distribution(logits), self.rng, self.greedy)
            return token
        return self._guarded(run)

    def begin_round(self) -> None:
        self.proposals, self.phase = [], self.DRAFTING

    def draft(self, logits) -> int:
        def run():
            if self.phase != self.DRAFTING:
                raise SamplerError("MTP draft after verification")
            d = self._distribution(logits)
            token, self.draft_rng = draw(d, self.draft_rng, self.greedy)
            lookup = {i: w / d.total for i, w in zip(d.indices, d.weights)}
            self.proposals.append((token, lookup))
            return token
        return self._guarded(run)

    def draft_point_mass(self, token: int) -> None:
        def run():
            if self.failed or self.phase != self.DRAFTING:
                raise SamplerError("MTP draft after verification")
            if self.vocabulary is not None and token >= self.vocabulary:
                raise SamplerError("MTP sampler vocabulary or state")
            self.proposals.append((int(token), {int(token): 1.0}))
        return self._guarded(run)

    def target(self, logits, proposal: int | None) -> int:
        def run():
            if self.phase == self.FINISHED:
                raise SamplerError("MTP verify after round completion")
            d = self._distribution(logits)
            self.phase = self.VERIFYING
            if proposal is None:
                if self.proposals:
                    raise SamplerError("MTP bonus before proposal verification")
                self.phase = self.FINISHED
                token, self.rng = draw(d, self.rng, self.greedy)
                return token
            if not self.proposals:
                raise SamplerError("MTP proposal distribution missing")
            drafted, lookup = self.proposals.pop(0)
            if proposal != drafted:
                raise SamplerError("MTP proposal distribution mismatch")
            accept = acceptance_probability(d.probability(proposal), lookup.get(proposal, 0.0))
            if accept == 1.0:
                return proposal
            if not self.greedy:
                u, self.rng = splitmix64_uniform(self.rng)
                if u < accept:
                    return proposal
            self.proposals = []          # later proposals were conditioned on the rejected prefix
            self.phase = self.FINISHED
            token, self.rng = draw(residual_distribution(d, lambda i: lookup.get(i, 0.0)), self.rng, self.greedy)
            return token
        return self._guarded(run)

    def device_greedy_drafts(self) -> bool:
        return self.greedy and not self.dense and not self.failed
