"""The worker processes on the reference's wire: command lines, readiness, strict requests, fixed error strings,
the token loop's finish reasons, streaming frames, prefix reuse, fencing, the scorer's f64 read-out and cache.
Model-free cases run the request layer against a scripted backend (the style of the reference's own
`scripts/test_generation_process.py` and the `FakeBackend` tests in crates/stark-generate/src/generation.rs);
one GPU case drives the real process end to end on a small synthetic artifact."""
import io
import json
import math
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from stark_b200 import worker as W

ROOT = Path(__file__).resolve().parent.parent


# ----------------------------------------------------------------------------------------------- process boundary

def _run(args, stdin=b"", env=None):
    e = dict(os.environ, PYTHONPATH=str(ROOT))
    e.update(env or {})
    return subprocess.run([sys.executable, "-m", "stark_b200.worker", *args], input=stdin, capture_output=True,
                          env=e, timeout=120, check=False, cwd=str(ROOT))


def test_startup_refusals_are_one_line_and_leak_nothing(tmp_path):
    missing = str(tmp_path / "private-marker-no-model")
    cases = [([], "invalid_arguments"), (["--model-path"], "invalid_arguments"), (["--model-path", ""], "invalid_arguments"),
             (["--unknown-private-marker", missing], "invalid_arguments"),
             (["--model-path", missing, "--unknown-private-marker"], "invalid_arguments"),
             (["--model-path", missing, "--prefix-cache", "--prefix-cache"], "invalid_arguments"),
             (["--model-path", missing], "model_config_unavailable"),
             (["--score-model-path", missing, "--consecutive-cache", "x"], "invalid_arguments"),
             (["--score-model-path", missing, "--prefix-cache"], "invalid_arguments"),
             (["--score-model-path", missing], "model_config_unavailable")]
    for args, error in cases:
        r = _run(args, env={"STARK_CAPTURE_TEST_SECRET": "private-marker"})
        assert r.returncode == 1 and not r.stderr and len(r.stdout.splitlines()) == 1, (args, r)
        assert json.loads(r.stdout) == {"ready": False, "error": error}
        assert b"private-marker" not in r.stdout
    r = _run(["--model-path", missing], env={"STARK_REQUEST_BUDGET_MIB": "1x"})
    assert json.loads(r.stdout) == {"ready": False, "error": "invalid_resource_budget"}


# ----------------------------------------------------------------------------------------------- scripted backend

class ScriptedBackend:
    """Returns a scripted token stream; records what it was asked."""

    def __init__(self, tokens, vocab=100, eos=(7,), max_context=5000):
        self.script, self.vocab, self.eos, self.max_context = list(tokens), vocab, list(eos), max_context
        self.key, self.calls, self.is_fenced, self.cursor = "k", [], False, 0

    def vocab_size(self):
        return self.vocab

    def max_context_length(self):
        return self.max_context

    def eos_token_ids(self):
        return self.eos

    def tokenize(self, text, special):
        return [ord(c) % self.vocab for c in text]

    def decode(self, ids, skip):
        return "".join(chr(97 + t % 26) for t in ids)

    def begin(self, ids, reuse, sampling, seed):
        self.calls.append(("begin", len(ids), reuse, sampling["mode"], seed))
        self.cursor = 0

    def next_token(self):
        t = self.script[self.cursor]
        self.cursor += 1
        if isinstance(t, str):
            raise W.Refusal(t)
        return t

    def advance(self, token):
        self.calls.append(("advance", token))

    def fenced(self):
        return self.is_fenced

    def forget(self):
        self.calls.append(("forget",))


def _worker(tokens, prefix_cache=False, **kw):
    return W.GenerationWorker(ScriptedBackend(tokens, **kw), W.Budget(16), prefix_cache)


def _ask(worker, request):
    out = io.BytesIO()
    data = request if isinstance(request, bytes) else json.dumps(request).encode()
    worker.process_line(data + b"\n", out)
    return [json.loads(line) for line in out.getvalue().splitlines()]


GEN = {"operation": "generate", "input_token_ids": [1, 2, 3], "context_tokens": 64, "max_new_tokens": 4}


def test_readiness_carries_the_reference_fields():
    r = _worker([1]).readiness()
    for key in ("ready", "engine", "version", "mode", "operations", "state_policy", "vocab_size", "max_context_tokens",
                "max_new_tokens", "max_request_bytes", "request_budget_bytes", "eos_token_ids", "sampling_modes",
                "streaming", "generation_progress", "stop_sequences", "cancellation", "mtp", "prefix_cache"):
        assert key in r, key
    assert r["ready"] is True and r["engine"] == "stark" and r["mode"] == "text-generation-v1"
    assert r["state_policy"] == "fresh-per-request" and r["operations"] == ["tokenize", "decode", "generate"]
    assert r["max_request_bytes"] == 6 * 16 * 2 ** 20 + 2 * 2 ** 20 and r["request_budget_bytes"] == 16 * 2 ** 20
    assert r["mtp"] == {"supported": False, "max_drafts": 0, "recommended_drafts": 0, "default_drafts": 0, "operations": []}
    p = _worker([1], prefix_cache=True).readiness()
    assert p["state_policy"] == "consecutive-prefix-v1" and "reset_cache" in p["operations"]
    assert p["prefix_cache"]["chunk_tokens"] == 1024 and p["prefix_cache"]["idle_seconds"] == 600


def test_requests_are_parsed_strictly():
    w = _worker([1, 2, 3, 4])
    assert _ask(w, b"not json") == [{"error": "invalid_request"}]
    assert _ask(w, {"operation": "dance"}) == [{"error": "invalid_request"}]
    assert _ask(w, dict(GEN, surprise=1)) == [{"error": "invalid_request"}]                 # deny_unknown_fields
    assert _ask(w, dict(GEN, mtp=None)) == [{"error": "invalid_request"}]                   # present_value: null is not absent
    assert _ask(w, dict(GEN, cache_scope=None)) == [{"error": "invalid_request"}]
    assert _ask(w, dict(GEN, context_tokens=64.0)) == [{"error": "invalid_request"}]        # u32 takes integers only
    assert _ask(w, dict(GEN, context_tokens=-1)) == [{"error": "invalid_request"}]
    assert _ask(w, dict(GEN, stream="yes")) == [{"error": "invalid_request"}]
    assert _ask(w, b'{"operation":"generate","operation":"generate"}') == [{"error": "invalid_request"}]
    assert _ask(w, dict(GEN, sampling={"mode": "greedy", "temperature": 1})) == [{"error": "invalid_request"}]
    assert _ask(w, dict(GEN, sampling={"mode": "stochastic"})) == [{"error": "invalid_request"}]   # temperature is required
    assert "generated_token_ids" in _ask(w, dict(GEN, rendered_prompt=None))[0]            # Option<String>: null is absent
    deep = b'{"operation":"decode","token_ids":' + b"[" * 70 + b"]" * 70 + b"}"
    assert _ask(w, deep) == [{"error": "resource_budget_exceeded"}]                         # depth > 64, before parsing


def test_validation_order_and_codes():
    w = _worker([1, 2, 3, 4])
    assert _ask(w, dict(GEN, max_new_tokens=0))[0]["error"] == "invalid_generation_request"
    assert _ask(w, dict(GEN, stop=[""]))[0]["error"] == "invalid_generation_request"
    assert _ask(w, dict(GEN, stop_token_ids=[5, 5]))[0]["error"] == "invalid_generation_request"
    assert _ask(w, dict(GEN, stop_token_ids=[100]))[0]["error"] == "invalid_generation_request"
    assert _ask(w, dict(GEN, context_tokens=5001))[0]["error"] == "context_overflow"        # above the backend maximum
    assert _ask(w, dict(GEN, max_new_tokens=2 ** 23))[0]["error"] == "resource_budget_exceeded"
    assert _ask(w, dict(GEN, sampling={"mode": "stochastic", "temperature": 0}))[0]["error"] == "invalid_sampling_request"
    assert _ask(w, dict(GEN, sampling={"mode": "stochastic", "temperature": 1, "top_k": 101}))[0]["error"] == "invalid_sampling_request"
    assert _ask(w, dict(GEN, sampling={"mode": "stochastic", "temperature": 1, "top_p": 0}))[0]["error"] == "invalid_sampling_request"
    assert _ask(w, dict(GEN, input_token_ids=[]))[0]["error"] == "invalid_generation_request"
    assert _ask(w, dict(GEN, input_token_ids=[100]))[0]["error"] == "invalid_generation_request"
    assert _ask(w, dict(GEN, rendered_prompt="x"))[0]["error"] == "invalid_generation_request"   # both inputs
    g = dict(GEN)
    del g["input_token_ids"]
    assert _ask(w, g)[0]["error"] == "invalid_generation_request"                           # neither input
    assert _ask(w, dict(GEN, context_tokens=3))[0]["error"] == "context_overflow"           # len >= context
    assert _ask(w, dict(GEN, context_tokens=6))[0]["error"] == "context_overflow"           # len + max_new > context
    assert _ask(w, dict(GEN, mtp=True))[0]["error"] == "mtp_not_supported"
    assert _ask(w, dict(GEN, mtp=True, mtp_drafts=1))[0]["error"] == "invalid_generation_request"
    assert _ask(w, dict(GEN, cache_scope="00" * 16))[0]["error"] == "invalid_generation_request"  # cache not enabled
    assert _ask(w, {"operation": "reset_cache"})[0]["error"] == "invalid_request"
    assert _ask(w, {"operation": "decode", "token_ids": [100]})[0]["error"] == "invalid_decoding_request"
    assert _ask(w, {"operation": "decode", "token_ids": [0, 1]}) == [{"text": "ab", "token_count": 2}]
    assert _ask(w, {"operation": "tokenize", "text": "ab"}) == [{"token_ids": [97, 98], "token_count": 2}]
    assert _ask(w, {"operation": "plan_generation", "input_tokens": 3, "context_tokens": 9})[0]["error"] == "context_planning_unavailable"


def test_finish_reasons_and_token_accounting():
    r = _ask(_worker([10, 11, 12, 13, 14]), GEN)[0]
    assert r["generated_token_ids"] == [10, 11, 12, 13] and r["finish_reason"] == "length" and r["sampled_tokens"] == 4
    assert r["stop_token_id"] is None and r["input_tokens"] == 3 and r["output_tokens"] == 4 and r["text"] == "klmn"
    assert r["timing_method"] == "first-token-wall-clock-v1" and r["prefill_seconds"] is not None
    r = _ask(_worker([10, 11, 12, 13]), dict(GEN, context_tokens=5, max_new_tokens=2))[0]
    assert r["finish_reason"] == "length" and r["sampled_tokens"] == 2
    r = _ask(_worker([10, 7, 12]), GEN)[0]                                                   # 7 is the end-of-sequence id
    assert r["finish_reason"] == "eos" and r["stop_token_id"] == 7 and r["generated_token_ids"] == [10]
    assert r["sampled_tokens"] == 2 and r["output_tokens"] == 1
    r = _ask(_worker([10, 11, 12]), dict(GEN, stop_token_ids=[11]))[0]
    assert r["finish_reason"] == "stop_token" and r["stop_token_id"] == 11 and r["sampled_tokens"] == 2
    r = _ask(_worker([0, 1, 2, 3]), dict(GEN, stop=["bc"]))[0]                               # text "abc..." stops at "bc"
    assert r["finish_reason"] == "stop_sequence" and r["text"] == "a" and r["generated_token_ids"] == [0, 1, 2]
    r = _ask(_worker([7]), GEN)[0]                                                           # a first sample that ends the request
    assert r["sampled_tokens"] == 1 and r["decode_seconds"] is None and r["output_tokens_per_second"] is None
    w = _worker([10, 11, 12, 13])
    _ask(w, dict(GEN, seed=9, sampling={"mode": "stochastic", "temperature": 0.5}))
    assert w.backend.calls[0] == ("begin", 3, 0, "stochastic", 9)
    assert [c for c in w.backend.calls if c[0] == "advance"] == [("advance", 10), ("advance", 11), ("advance", 12)]


def test_streaming_frames_concatenate_to_the_text():
    frames = _ask(_worker([0, 1, 2, 3]), dict(GEN, stream=True))
    assert frames[0]["event"] == "progress" and frames[0]["sampled_tokens"] == 0 and frames[0]["output_token_budget"] == 4
    final = frames[-1]
    deltas = "".join(f["text"] for f in frames[:-1] if f.get("event") == "delta")
    assert deltas == final["text"] == "abcd"
    assert [f["sampled_tokens"] for f in frames[:-1] if f.get("event") == "progress"] == [0, 1, 2, 3, 4]
    frames = _ask(_worker([0, 1, 2, 3]), dict(GEN, stream=True, stop=["cd"]))                # held-back text never leaks the stop
    assert "".join(f["text"] for f in frames[:-1] if f.get("event") == "delta") == frames[-1]["text"] == "ab"


def test_fencing_errors_end_the_process_others_do_not():
    w = _worker(["native_generation_failed"])
    out = io.BytesIO()
    with pytest.raises(W.Refusal) as stop:
        w.process_line(json.dumps(GEN).encode() + b"\n", out)
    assert stop.value.code == "native_operation_failed"
    assert json.loads(out.getvalue()) == {"error": "native_generation_failed"}
    with pytest.raises(W.Refusal):
        _worker([100]).process_line(json.dumps(GEN).encode() + b"\n", io.BytesIO())          # a token outside the vocabulary
    w = _worker([1, 2, 3, 4])
    w.backend.is_fenced = True
    with pytest.raises(W.Refusal):
        w.process_line(json.dumps(GEN).encode() + b"\n", io.BytesIO())                       # the model fenced itself meanwhile


def test_serve_loop_handles_oversize_frames_and_end_of_input():
    w = W.GenerationWorker(ScriptedBackend([1, 2, 3, 4]), W.Budget(1), False)
    big = b'{"operation":"decode","token_ids":[' + b"1," * (w.budget.wire_bytes // 2 + 8) + b"1]}\n"
    stdin = io.BytesIO(big + json.dumps({"operation": "decode", "token_ids": [0]}).encode() + b"\n")
    out = io.BytesIO()
    assert W.serve_generation(w, stdin, out) == 0
    lines = [json.loads(x) for x in out.getvalue().splitlines()]
    assert lines[0]["ready"] is True and lines[1] == {"error": "request_too_large"} and lines[2] == {"text": "a", "token_count": 1}


def test_prefix_reuse_is_chunk_aligned_and_published_after_the_reply():
    scope = "000102030405060708090a0b0c0d0e0f"
    w = _worker(list(range(10, 60)) * 4, prefix_cache=True)
    first = [int(t) for t in np.arange(2500) % 90]
    base = dict(operation="generate", context_tokens=4096, max_new_tokens=2, cache_scope=scope)
    r = _ask(w, dict(base, input_token_ids=first))[0]
    assert r["reused_input_tokens"] == 0 and w.retained[2] == first[:2048]                   # whole chunks below the final one
    second = first[:2300] + [91] * 300
    r = _ask(w, dict(base, input_token_ids=second))[0]
    assert r["reused_input_tokens"] == 2048
    assert ("begin", 2600, 2048, "greedy", 0) in w.backend.calls
    diverged = list(second)
    diverged[1500] = 93
    assert _ask(w, dict(base, input_token_ids=diverged))[0]["reused_input_tokens"] == 1024   # down to the chunk before the change
    assert _ask(w, dict(base, input_token_ids=diverged, context_tokens=4000))[0]["reused_input_tokens"] == 0   # other context
    assert _ask(w, dict(base, input_token_ids=diverged, cache_scope="ff" * 16))[0]["reused_input_tokens"] == 0  # other scope
    assert _ask(w, dict(base, input_token_ids=diverged, cache_scope="FF" * 16))[0]["error"] == "invalid_generation_request"
    assert w.retained is None                                                               # every error clears the cache
    _ask(w, dict(base, input_token_ids=first))
    assert _ask(w, {"operation": "reset_cache"}) == [{"cache_reset": True}] and w.retained is None
    assert W.reusable_prefill_rows(0) == 0 and W.reusable_prefill_rows(1024) == 0 and W.reusable_prefill_rows(1025) == 1024
    assert W.reusable_prefill_rows(18_544) == 18 * 1024


def test_cancellation_over_the_pipe():
    r, wr = os.pipe()
    os.set_blocking(r, False)
    signal = W.CancelSignal(r)
    assert signal.check(5) is False
    os.write(wr, (4).to_bytes(8, "little") + (5).to_bytes(8, "little")[:3])
    assert signal.check(5) is False                                                          # another id, then a partial frame
    os.write(wr, (5).to_bytes(8, "little")[3:])
    assert signal.check(5) is True
    w = W.GenerationWorker(ScriptedBackend([1, 2, 3, 4]), W.Budget(16), False, cancel=signal)
    os.write(wr, (77).to_bytes(8, "little"))
    assert _ask(w, dict(GEN, request_id=77)) == [{"error": "generation_cancelled"}]
    os.close(wr)
    assert signal.check(1) is True                                                           # the owner vanished


# ----------------------------------------------------------------------------------------------- scorer

class ScoringBackend(ScriptedBackend):
    def __init__(self):
        super().__init__([], vocab=50)
        self.scored = 0

    def score(self, ids):
        self.scored += 1
        rng = np.random.default_rng(sum(ids))
        return rng.standard_normal(50).astype(np.float32) * 3, (0.001, 0.002, 0.003)


SCORE = {"operation": "score", "input_token_ids": [1, 2, 3], "candidate_token_ids": [4, 9, 20], "context_tokens": 16,
         "temperature": 0.7}


def _score(worker, request):
    out = io.BytesIO()
    worker.process_line(json.dumps(request).encode() + b"\n", out)
    return json.loads(out.getvalue())


def test_scorer_readout_is_the_f64_formula():
    w = W.ScoreWorker(ScoringBackend(), W.Budget(16), False)
    r = _score(w, SCORE)
    logits, _ = ScoringBackend().score([1, 2, 3])
    l64 = logits.astype(np.float64)
    log_partition = l64.max() + math.log(np.exp(l64 - l64.max()).sum())
    assert r["logits"] == [float(logits[c]) for c in SCORE["candidate_token_ids"]]
    np.testing.assert_allclose(r["log_probabilities"], [float(logits[c]) - log_partition for c in (4, 9, 20)], rtol=0, atol=1e-12)
    c = np.array(r["logits"])
    want = np.exp((c - c.max()) / 0.7)
    np.testing.assert_allclose(r["candidate_probabilities"], want / want.sum(), rtol=1e-14)
    assert abs(sum(r["candidate_probabilities"]) - 1.0) < 1e-12
    assert r["input_tokens"] == 3 and r["cache_hit"] is False and r["truncated"] is False
    assert r["prompt_tokens_sha256"] == W.token_hash([1, 2, 3]) and r["cache"] == {"enabled": False, "hits": 0, "native_score_calls": 1}
    ready = w.readiness(0.5)
    assert ready["mode"] == "exact-token-scoring-cache-v1" and ready["cache_policy"] == "fresh-state"


def test_scorer_validation_and_cache():
    w = W.ScoreWorker(ScoringBackend(), W.Budget(16), True)
    assert w.readiness(0.0)["cache_policy"] == "consecutive-full-vocabulary-logits-v1"
    for bad in (dict(SCORE, candidate_token_ids=[4]), dict(SCORE, candidate_token_ids=[4, 4]),
                dict(SCORE, candidate_token_ids=list(range(17))), dict(SCORE, temperature=0), dict(SCORE, input_token_ids=[]),
                dict(SCORE, input_token_ids=[50]), dict(SCORE, context_tokens=0)):
        assert _score(w, bad)["error"] == "invalid_scoring_request", bad
    assert _score(w, dict(SCORE, context_tokens=2))["error"] == "context_overflow"
    assert _score(w, dict(SCORE, extra=1))["error"] == "invalid_request"
    a = _score(w, SCORE)
    b = _score(w, SCORE)
    assert a["cache_hit"] is False and b["cache_hit"] is True and b["logits"] == a["logits"]
    assert b["cache"]["hits"] == 1 and w.backend.scored == 1
    other = dict(SCORE, input_token_ids=[3, 2, 1])
    assert _score(w, other)["cache_hit"] is False and _score(w, SCORE)["cache_hit"] is False   # A / B / A cannot hit
    assert _score(w, dict(SCORE, candidate_token_ids=[4]))["error"] == "invalid_scoring_request"
    assert _score(w, SCORE)["cache_hit"] is False                                             # every error clears the cache
    assert _score(w, {"operation": "reset_cache"})["cache_reset"] is True
    out = io.BytesIO()
    big = b"x" * (w.budget.wire_bytes + 10) + b"\n" + json.dumps(SCORE).encode() + b"\n"
    assert W.serve_scoring(w, 0.0, io.BytesIO(big), out) == 0
    lines = [json.loads(x) for x in out.getvalue().splitlines()]
    assert len(lines) == 2 and lines[1]["error"] == "request_too_large"                     # the scorer ends after an oversize frame


# ----------------------------------------------------------------------------------------------- the real process

@pytest.mark.gpu
def test_worker_process_round_trip_on_a_small_artifact(tmp_path):
    from stark_b200 import synthetic as S
    from stark_b200.artifact import row_major_planes, write_artifact
    from stark_b200.engine import DenseModel
    cfg = S.CONFIGS["tiny"]
    w = S.dense_weights(cfg, seed=0, zero_point=7.5)
    write_artifact(tmp_path / "model", cfg, w)
    prompt = [int(t) for t in S.prompt(cfg, 1100, seed=3)]                                   # more than one prefill chunk
    longer = prompt[:1060] + [5, 6, 7]
    scope = "ab" * 16
    requests = [dict(operation="generate", input_token_ids=prompt, context_tokens=2048, max_new_tokens=6, cache_scope=scope),
                dict(operation="generate", input_token_ids=longer, context_tokens=2048, max_new_tokens=3, cache_scope=scope),
                dict(operation="generate", input_token_ids=prompt[:9], context_tokens=64, max_new_tokens=5, seed=4,
                     sampling=dict(mode="stochastic", temperature=0.8, top_k=50)),
                dict(operation="bogus"),
                dict(operation="plan_generation", input_tokens=40, context_tokens=100000)]
    r = _run(["--model-path", str(tmp_path / "model"), "--prefix-cache"],
             stdin="".join(json.dumps(q) + "\n" for q in requests).encode(), env={"STARK_B200_WORKER_CONTEXT": "2048"})
    assert r.returncode == 0 and not r.stderr, r
    lines = [json.loads(x) for x in r.stdout.splitlines()]
    assert len(lines) == 6 and lines[0]["ready"] is True and lines[0]["vocab_size"] == cfg["vocab"]
    assert lines[5] == {"context_tokens": 2048, "max_new_tokens": 2008, "context_capacity_known": True, "budget_kind": "memory"}
    assert lines[0]["max_context_tokens"] == 2048 and lines[0]["state_policy"] == "consecutive-prefix-v1"
    model = DenseModel.load(cfg, w, context_tokens=2048)
    model.prefill(np.asarray(prompt, np.uint32))
    assert lines[1]["generated_token_ids"] == model.generate_greedy(5).tolist()
    assert lines[1]["finish_reason"] == "length" and lines[1]["reused_input_tokens"] == 0 and lines[1]["sampled_tokens"] == 6
    model.reset()
    model.prefill(np.asarray(longer, np.uint32))
    assert lines[2]["generated_token_ids"] == model.generate_greedy(2).tolist()              # reuse changes nothing
    assert lines[2]["reused_input_tokens"] == 1024
    assert len(lines[3]["generated_token_ids"]) == 5 and all(0 <= t < cfg["vocab"] for t in lines[3]["generated_token_ids"])
    assert lines[4] == {"error": "invalid_request"}
    # the scorer on the same artifact
    score = dict(operation="score", input_token_ids=prompt[:40], candidate_token_ids=[1, 2, 3], context_tokens=64, temperature=1.0)
    r = _run(["--score-model-path", str(tmp_path / "model"), "--consecutive-cache"],
             stdin=(json.dumps(score) + "\n" + json.dumps(score) + "\n").encode(), env={"STARK_B200_WORKER_CONTEXT": "256"})
    assert r.returncode == 0 and not r.stderr, r
    lines = [json.loads(x) for x in r.stdout.splitlines()]
    assert lines[0]["ready"] is True and lines[1]["cache_hit"] is False and lines[2]["cache_hit"] is True
    model.reset()
    model.prefill(np.asarray(prompt[:40], np.uint32))
    logits = model.logits()
    l64 = logits.astype(np.float64)
    want = l64[[1, 2, 3]] - (l64.max() + math.log(np.exp(l64 - l64.max()).sum()))
    np.testing.assert_allclose(lines[1]["log_probabilities"], want, rtol=0, atol=1e-9)
    assert lines[1]["logits"] == [float(logits[c]) for c in (1, 2, 3)]
    model.close()


# ----------------------------------------------------------------------------------------------- speculative rounds

class SpeculativeBackend(ScriptedBackend):
    """A scripted backend that declares a draft head (generation.rs:1706-1830 does the same with its FakeBackend)."""
    CAPS = {"max_drafts": 3, "recommended_drafts": 2, "sampling": "greedy-exact-v1", "verification": "v"}

    def __init__(self, tokens, scheduling=True, **kw):
        super().__init__(tokens, **kw)
        self.scheduling, self.begun = scheduling, []

    def mtp_capabilities(self):
        return dict(self.CAPS)

    def supports_mtp_scheduling(self):
        return self.scheduling

    def effective_mtp_drafts(self, drafts, sampling):
        return drafts if sampling["mode"] == "greedy" else 0

    def begin(self, ids, reuse, sampling, seed, mtp=None, budget_tokens=0):
        self.begun.append((mtp, budget_tokens))
        super().begin(ids, reuse, sampling, seed)

    def mtp_metadata(self):
        return {"rounds": 1}


def _spec(tokens, **kw):
    return W.GenerationWorker(SpeculativeBackend(tokens, **kw), W.Budget(16), False)


def test_speculative_selectors_resolve_as_the_reference_does():
    # without a draft head every way of asking for proposals is refused, and a schedule without proposals is malformed
    plain = _worker([1, 2, 3, 4])
    assert plain.readiness()["mtp"] == {"supported": False, "max_drafts": 0, "recommended_drafts": 0, "default_drafts": 0,
                                        "operations": []}
    assert _ask(plain, dict(GEN, mtp=True)) == [{"error": "mtp_not_supported"}]
    assert _ask(plain, dict(GEN, mtp_drafts=1)) == [{"error": "mtp_not_supported"}]
    assert "error" not in _ask(plain, dict(GEN, mtp=False))[0] and "mtp" not in _ask(plain, dict(GEN, mtp_drafts=0))[0]
    assert _ask(plain, dict(GEN, mtp_policy="adaptive")) == [{"error": "invalid_generation_request"}]
    # with one
    w = _spec([1, 2, 3, 4])
    ready = w.readiness()["mtp"]
    assert ready["supported"] and ready["max_drafts"] == 3 and ready["recommended_drafts"] == 2 and ready["operations"] == ["generate"]
    assert ready["policies"] == ["fixed", "adaptive"] and ready["default_policy"] == "fixed" and ready["lookup"] is True
    assert _ask(w, dict(GEN, mtp=True, mtp_drafts=2)) == [{"error": "invalid_generation_request"}]   # both selectors
    assert _ask(w, dict(GEN, mtp_drafts=4)) == [{"error": "invalid_generation_request"}]              # past the limit
    assert _ask(w, dict(GEN, mtp=None)) == [{"error": "invalid_request"}]                              # an explicit null
    assert _ask(w, dict(GEN, mtp_policy="eager", mtp_drafts=1)) == [{"error": "invalid_generation_request"}]
    assert _ask(w, dict(GEN, mtp_lookup=True)) == [{"error": "invalid_generation_request"}]            # a schedule, no proposals
    reply = _ask(w, dict(GEN, mtp=True))[0]
    assert reply["mtp"] == {"rounds": 1, "enabled": True, "drafts": 2, "sampling": "greedy-exact-v1", "verification": "v"}
    assert w.backend.begun[-1] == ({"drafts": 2, "adaptive": False, "lookup": False}, 4)
    reply = _ask(w, dict(GEN, mtp=True, mtp_policy="adaptive", mtp_lookup=True))[0]
    assert reply["mtp"]["drafts"] == 3 and reply["mtp"]["policy"] == "adaptive" and reply["mtp"]["lookup"] is True
    assert w.backend.begun[-1][0] == {"drafts": 3, "adaptive": True, "lookup": True}                 # adaptive plans up to the limit
    reply = _ask(w, dict(GEN, mtp_drafts=1, mtp_policy="adaptive"))[0]
    assert reply["mtp"]["drafts"] == 1                                                                # an explicit count wins
    reply = _ask(w, dict(GEN, mtp_drafts=0))[0]
    assert reply["mtp"]["enabled"] is False and reply["mtp"]["drafts"] == 0 and w.backend.begun[-1][0] is None
    # a stochastic request runs without proposals and says so
    reply = _ask(w, dict(GEN, mtp=True, sampling=dict(mode="stochastic", temperature=1.0)))[0]
    assert reply["mtp"]["enabled"] is False and reply["mtp"]["requested_drafts"] == 2
    assert reply["mtp"]["fallback_reason"] == "unsupported_sampling" and w.backend.begun[-1][0] is None
    # a backend without scheduling support
    w = _spec([1, 2, 3, 4], scheduling=False)
    assert "policies" not in w.readiness()["mtp"]
    assert _ask(w, dict(GEN, mtp=True, mtp_policy="adaptive")) == [{"error": "mtp_not_supported"}]


@pytest.mark.gpu
def test_speculative_generation_equals_plain_greedy_through_the_worker():
    """The engine behind the worker with a draft head: fixed, adaptive and prompt-lookup schedules must all emit the
    target's own greedy text (replayed through the one-row path, up to bf16 near-ties), whatever the rounds accept."""
    from stark_b200 import synthetic as S
    from stark_b200.engine import DenseModel
    from tests.test_model_gpu import assert_sequence_is_greedy
    cfg = S.CONFIGS["small"]
    w = S.dense_weights(cfg, seed=3, zero_point=7.5)
    backend = object.__new__(W.B200Backend)      # the engine without an artifact directory
    backend.cfg, backend.capacity, backend.eos, backend.tokenizer, backend.key = dict(cfg, mtp=True), 1024, [], None, "k"
    backend.model = DenseModel.load(dict(cfg, mtp=True), dict(w, mtp=S.mtp_weights(cfg, seed=3, zero_point=7.5)), 1024)
    backend.has_head, backend.rounds, backend._newline, backend.position_tokens = True, None, None, []
    worker = W.GenerationWorker(backend, W.Budget(16), False)
    block = [int(t) for t in S.prompt(cfg, 48, seed=8)]
    prompt = [int(t) for t in S.prompt(cfg, 90, seed=9)] + block + block[:40]       # the tail repeats: lookup proposes
    plain = DenseModel.load(cfg, w, context_tokens=1024)
    base = dict(operation="generate", input_token_ids=prompt, context_tokens=512, max_new_tokens=40)
    seen = {}
    for name, extra in (("fixed", dict(mtp_drafts=3)), ("adaptive", dict(mtp=True, mtp_policy="adaptive")),
                        ("lookup", dict(mtp_drafts=3, mtp_lookup=True)), ("off", dict(mtp_drafts=0))):
        reply = _ask(worker, dict(base, **extra))[0]
        assert "error" not in reply, (name, reply)
        assert reply["sampled_tokens"] == 40 and reply["finish_reason"] == "length"
        assert_sequence_is_greedy(plain, prompt, reply["generated_token_ids"])
        seen[name] = reply
        if name != "off":
            m = reply["mtp"]
            assert m["enabled"] and m["verified_rows"] >= m["rounds"] >= 1 and m["accepted"] <= m["proposed"]
            assert sum(m["rounds_by_accepted_drafts"]) == m["rounds"]
    assert seen["adaptive"]["mtp"]["drafts"] == 4 and seen["adaptive"]["mtp"]["schedule"]["cost_table"]
    assert seen["lookup"]["mtp"]["schedule"]["lookup_rounds"] >= 1                  # the repeated tail was tried
    assert seen["off"]["mtp"]["enabled"] is False
    # stochastic requests: acceptance by the exact rejection sampler on the host over the rows of held rounds.  At a
    # temperature near zero the target distribution is its arg-max, so the text must again be the greedy one --
    # which checks the row order, the commit and the next-token hand-over end to end
    cold = dict(mode="stochastic", temperature=0.01, top_k=None, top_p=None, min_p=None)
    reply = _ask(worker, dict(base, mtp_drafts=3, sampling=cold, seed=5, max_new_tokens=24))[0]
    assert "error" not in reply and reply["mtp"]["enabled"] and reply["mtp"]["sampling"] == "exact-rejection-v1"
    assert_sequence_is_greedy(plain, prompt, reply["generated_token_ids"])
    warm = dict(mode="stochastic", temperature=1.0, top_k=40, top_p=0.95, min_p=None)
    a = _ask(worker, dict(base, mtp_drafts=2, sampling=warm, seed=11, max_new_tokens=16))[0]
    b = _ask(worker, dict(base, mtp_drafts=2, sampling=warm, seed=11, max_new_tokens=16))[0]
    c = _ask(worker, dict(base, mtp_drafts=2, sampling=warm, seed=12, max_new_tokens=16))[0]
    assert a["generated_token_ids"] == b["generated_token_ids"] != c["generated_token_ids"]     # seeded
    assert len(a["generated_token_ids"]) == 16 and all(0 <= t < cfg["vocab"] for t in a["generated_token_ids"])
    assert a["mtp"]["verified_rows"] == a["mtp"]["proposed"] + a["mtp"]["rounds"]
    plain.close()
    backend.model.close()


def test_plan_generation_answers_the_largest_context_that_fits():
    """generation.rs:1114-1182 with a scripted planner: limits, validation order and the reply's fields."""
    class Planning(ScriptedBackend):
        def __init__(self, *a, fits=None, **kw):
            super().__init__(*a, **kw)
            self.fits, self.asked = fits, []

        def plan_context_length(self, input_tokens, maximum, drafts):
            self.asked.append((input_tokens, maximum, drafts))
            return self.fits if self.fits is not None else maximum

    plan = {"operation": "plan_generation", "input_tokens": 100, "context_tokens": 4000}
    w = W.GenerationWorker(Planning([1], max_context=3000), W.Budget(16), False)
    assert _ask(w, plan) == [{"context_tokens": 3000, "max_new_tokens": 2900, "context_capacity_known": True, "budget_kind": "memory"}]
    assert w.backend.asked == [(100, 3000, 0)]                                   # capped by the model's limit
    assert _ask(w, dict(plan, context_tokens=500))[0]["context_tokens"] == 500   # and by the request's
    for bad in (dict(plan, input_tokens=0), dict(plan, context_tokens=100), dict(plan, input_token_ids=[1, 2]),
                dict(plan, input_tokens=2, input_token_ids=[1, 100]), dict(plan, cache_scope="ab" * 16),
                dict(plan, mtp=True, mtp_drafts=1)):
        assert _ask(w, bad) == [{"error": "invalid_generation_request"}], bad
    assert _ask(w, dict(plan, mtp=True)) == [{"error": "mtp_not_supported"}]
    assert _ask(w, dict(plan, extra=1)) == [{"error": "invalid_request"}]
    assert _ask(w, dict(plan, input_tokens=2, input_token_ids=[1, 2]))[0]["max_new_tokens"] == 2998
    # the planner's answer is checked: nothing fits, or an answer outside (input, maximum]
    for fits in (0, 100, 3001):
        w = W.GenerationWorker(Planning([1], max_context=3000, fits=fits), W.Budget(16), False)
        assert _ask(w, plan) == [{"error": "resource_budget_exceeded"}]
    w = W.GenerationWorker(Planning([1], max_context=3000, fits=1200), W.Budget(16), False)
    assert _ask(w, plan)[0] == {"context_tokens": 1200, "max_new_tokens": 1100, "context_capacity_known": True,
                                "budget_kind": "memory"}
    # a planning request does not disturb a retained prefix, anything unknown does
    assert _ask(_worker([1]), plan) == [{"error": "context_planning_unavailable"}]
