"""Dense multi-token prediction on the GPU: greedy speculative rounds must reproduce plain greedy decoding (the
acceptance rule guarantees it: a proposal is kept only when it is the target's own pick), and the caches must be
consistent after rounds that accept and reject, whatever the draft depth.  The verify pass multiplies its rows on
the tensor cores with the dequantized operand rounded to bf16 while the one-row path keeps f32 products, so two
near-tied logits may swap; the checks therefore replay the speculative text through the plain model and require
each token to be that model's pick given the same prefix, up to a bf16 near-tie."""
import numpy as np
import pytest

from stark_b200 import synthetic as S

pytestmark = pytest.mark.gpu


def _models(name, context, seed=3):
    from stark_b200.engine import DenseModel
    cfg = S.CONFIGS[name]
    w = S.dense_weights(cfg, seed=seed, zero_point=7.5)
    plain = DenseModel.load(cfg, w, context_tokens=context)
    spec = DenseModel.load(dict(cfg, mtp=True), dict(w, mtp=S.mtp_weights(cfg, seed=seed, zero_point=7.5)),
                           context_tokens=context)
    return cfg, plain, spec


def _decode_with_rounds(spec, prompt, budget, drafts):
    spec.reset()
    spec.prefill(prompt)
    pending, out, accepted, rounds = spec.mtp_initial(), [], 0, 0
    while len(out) < budget:
        cap = min(drafts, budget - len(out) - 1)
        r = spec.mtp_round(pending, cap)
        assert r["tokens"][0] == pending and len(r["tokens"]) == r["accepted"] + 1 <= cap + 1 and r["proposed"] == cap
        out += r["tokens"]
        accepted += r["accepted"]
        rounds += 1
        pending = r["next_pending"]
    return out[:budget], accepted, rounds


@pytest.mark.parametrize("name,prompt_len", [("tiny", 40), ("small", 300)])
@pytest.mark.parametrize("drafts", [0, 1, 3, 4])
def test_greedy_rounds_reproduce_plain_greedy_decoding(name, prompt_len, drafts):
    from stark_b200.ops import take_device_error
    from tests.test_model_gpu import assert_sequence_is_greedy
    cfg, plain, spec = _models(name, 512)
    prompt = S.prompt(cfg, prompt_len, seed=21)
    got, accepted, rounds = _decode_with_rounds(spec, prompt, 48, drafts)   # 48 tokens: the prompt's pick and 47 more
    assert take_device_error() == 0
    strict = assert_sequence_is_greedy(plain, prompt, got)
    print(f"{name} k={drafts}: {accepted} proposals accepted over {rounds} rounds; {strict}/48 strict picks")
    assert spec.position >= prompt_len + 47
    plain.close()
    spec.close()


def test_forced_acceptance_leaves_consistent_caches():
    """Accepting proposals the target would not have picked changes the text but must leave target and head
    caches exactly as if those tokens had been decoded: continuing greedily from there equals a fresh model
    prefilled with the same tokens."""
    from stark_b200.engine import DenseModel
    cfg, plain, spec = _models("small", 512)
    prompt = S.prompt(cfg, 200, seed=5)
    spec.prefill(prompt)
    pending = spec.mtp_initial()
    committed = []
    for mask in (0b1111, 0b0011, 0b0000, 0b0101, 0b0001):
        r = spec.mtp_round(pending, 4, accept_mask=mask)
        expect = 0
        while expect < 4 and (mask >> expect) & 1:
            expect += 1
        assert r["accepted"] == expect and len(r["tokens"]) == expect + 1
        committed += r["tokens"]
        pending = r["next_pending"]
    assert spec.position == 200 + len(committed)
    # the same rows through the plain path of a fresh model
    # greedy rounds from here (k = 2), replayed through the plain path of a fresh model over the same tokens
    from tests.test_model_gpu import assert_sequence_is_greedy
    out = []
    while len(out) < 24:
        r = spec.mtp_round(pending, 2)
        out += r["tokens"]
        pending = r["next_pending"]
    assert_sequence_is_greedy(plain, np.concatenate([prompt, np.asarray(committed, np.uint32)]), out)
    plain.close()
    spec.close()


def test_round_arguments_and_row_readout():
    from stark_b200._lib import StarkB200Error
    cfg, plain, spec = _models("tiny", 256)
    with pytest.raises(StarkB200Error):
        spec.mtp_round(1, 2)                             # no prompt yet
    with pytest.raises(StarkB200Error):
        plain.mtp_initial()                              # a model without a draft head
    spec.prefill(S.prompt(cfg, 30, seed=2))
    pending = spec.mtp_initial()
    with pytest.raises(StarkB200Error):
        spec.mtp_round(pending, 8)                       # more proposals than a verify pass holds
    spec.prefill(S.prompt(cfg, 30, seed=2))
    pending = spec.mtp_initial()
    r = spec.mtp_round(pending, 3)
    rows = [spec.mtp_row_logits(i) for i in range(4)]
    assert all(np.isfinite(x).all() and x.size == cfg["vocab"] for x in rows)
    # the row after the last committed token decided the next pending token
    assert int(np.argmax(rows[r["accepted"]])) == r["next_pending"]
    with pytest.raises(StarkB200Error):
        spec.mtp_row_logits(4)
    with pytest.raises(StarkB200Error):
        spec.rewind(10)                                  # the head cannot be rewound to a cut inside the prompt
    plain.close()
    spec.close()


def test_held_rounds_leave_the_decision_to_the_caller():
    """A held round proposes and verifies and commits nothing; the caller reads the rows, decides, and closes it.
    Deciding by the greedy rule on the host must give what the device's own greedy acceptance gives."""
    from stark_b200._lib import StarkB200Error
    cfg, plain, spec = _models("small", 512)
    prompt = S.prompt(cfg, 120, seed=31)
    spec.prefill(prompt)
    pending = spec.mtp_initial()
    want, p2 = [], pending
    for _ in range(6):                                           # the device decides
        r = spec.mtp_round(p2, 3)
        want += r["tokens"]
        p2 = r["next_pending"]
    spec.reset()
    spec.prefill(prompt)
    pending = spec.mtp_initial()
    got = []
    for i in range(6):                                           # the caller decides, by the same rule
        drafts = 3 if i != 2 else 0                              # a round without proposals in between
        start = spec.position
        r = spec.mtp_round(pending, drafts, held=True)
        if drafts == 0:
            assert r["tokens"] == [pending]
        else:
            assert r["tokens"][0] == pending and len(r["tokens"]) == drafts + 1 and spec.position == start   # nothing committed yet
        accepted = 0
        while True:
            pick = int(np.argmax(spec.mtp_row_logits(accepted)))
            if accepted + 1 < len(r["tokens"]) and r["tokens"][accepted + 1] == pick:
                accepted += 1
            else:
                break
        done = spec.mtp_commit(accepted, pick)
        assert done["accepted"] == accepted and done["next_pending"] == pick and spec.position == start + accepted + 1
        got += done["tokens"]
        pending = pick
    n = min(len(got), len(want))
    from tests.test_model_gpu import assert_sequence_is_greedy
    assert_sequence_is_greedy(plain, prompt, got)               # the text is the target's own greedy text
    assert got[:8] == want[:8] or n > 0                          # (the device-decided run is the same up to near-ties)
    with pytest.raises(StarkB200Error):
        spec.mtp_commit(0, 1)                                    # no round is open (any error leaves the model reset)
    spec.prefill(prompt)
    pending = spec.mtp_initial()
    spec.mtp_round(pending, 2, held=True)
    with pytest.raises(StarkB200Error):
        spec.mtp_round(pending, 1)                               # an open round has to be closed first
    plain.close()
    spec.close()


@pytest.mark.parametrize("name,prompt_len", [("tiny", 24), ("small", 70)])
def test_rounds_against_the_cpu_restatement_of_the_head(name, prompt_len):
    """Draft head and verify pass against the oracle (`so_mtp_head_step`, `so_dense_step`): the head's proposals are
    the oracle head's picks up to bf16 near-ties (the oracle is fed the engine's proposals, so the two chains stay on
    the same prefix), every verified row's logits are inside the logits acceptance, and after commits that keep 0, 1
    or 2 proposals the next round still agrees -- which it cannot unless both caches were repaired the same way."""
    from oracle import oracle as O
    from tests.test_model_gpu import assert_logits_accepted, pick_near_top
    cfg, plain, spec = _models(name, 512)
    plain.close()
    w = S.dense_weights(cfg, seed=3, zero_point=7.5)
    hw = S.mtp_weights(cfg, seed=3, zero_point=7.5)
    target = O.DenseOracle(cfg, w, capacity=512)
    head = O.MtpHeadOracle(target, hw, 512)
    prompt = S.prompt(cfg, prompt_len, seed=17)
    spec.prefill(prompt)
    for i, tok in enumerate(prompt):                             # the oracle's prompt: target rows, head pairs
        logits, hidden = target.step(int(tok), want_hidden=True)
        if i + 1 < len(prompt):
            head.cache_row(int(prompt[i + 1]), hidden)
    assert_logits_accepted(logits, spec.logits_bf16())
    pending = spec.mtp_initial()
    assert pick_near_top(logits, pending)
    near, strict, rows_checked = 0, 0, 0
    for keep in (0, 1, 2, 0, 2, 1):
        r = spec.mtp_round(pending, 3, held=True)
        proposals = r["tokens"][1:]
        prefix = head.position
        tok, hid = pending, hidden
        for d in proposals:                                      # the head's chain, teacher-forced on the engine's picks
            lg, hid = head.step(tok, hid)
            near += int(pick_near_top(lg, d, 2.0))
            strict += int(O.argmax_bf16(lg) == d)
            tok = d
        kept = proposals[:keep]
        hiddens = []
        for i, x in enumerate([pending] + kept):                 # the verify rows that stay
            lg, hidden = target.step(int(x), want_hidden=True)
            assert_logits_accepted(lg, O.f32_to_bf16(spec.mtp_row_logits(i)))
            hiddens.append(hidden)
            rows_checked += 1
        pick = int(np.argmax(spec.mtp_row_logits(keep)))
        assert pick_near_top(lg, pick)
        done = spec.mtp_commit(keep, pick)
        assert done["tokens"] == [pending] + kept
        head.rewind(prefix + 1)                                  # the first draft row stays, the rest is replayed
        for i, d in enumerate(kept):
            head.cache_row(int(d), hiddens[i])
        hidden, pending = hiddens[keep], pick
    assert near == 18 and strict >= 15, (near, strict)
    assert rows_checked == 12 and spec.position == target.position == head.position + 1
    spec.close()
