"""Regenerates `oracle_outputs.npz`: outputs of the CPU oracle on seeded inputs, committed so that the GPU
parity tests can also be checked against values that were produced once and never move.

    python tests/golden/make_golden.py

    python tests/golden/make_golden.py --full     # also the long continuations (minutes of CPU time)

Inputs come from `stark_b200.synthetic` (seeded), outputs from `oracle/` only.  The arrays:
  matvec_y        bf16 bits, the 4-bit affine matvec of `matvec_case(seed=3, rows=512, columns=1024)`
  tiny_logits     bf16 bits, last-row logits of the `tiny` decoder (weights seed 0) after `prompt(tiny, 70, seed=5)`
  tiny_greedy     the oracle's own greedy continuation of that prompt, 8 tokens
  q8_0_row / q4_k_row   f32, row 1 of `q8_0_rows` / `q4_k_rows` (default_rng(11), 4 x 512) decoded
  <shape>_logits        bf16 bits, last-row logits of the two-layer `qwen3-8b-layers` / `qwen3-0.6b-layers`
                        decoders (weights seed 2, zero point 7.5: zero-mean weights, so that the arg-max depends on the
                        input) after `prompt(cfg, 24, seed=6)`
  <shape>_teacher       (--full) LAYERS_STEPS seeded random tokens fed after that prompt (`prompt(cfg, 100, seed=7)`)
  <shape>_top1          (--full) the oracle's pick (first index of the maximum) after each of those tokens
  <shape>_lead_ids / _lead_bits   (--full) the oracle's eight largest logits at each of those steps (token ids and
                        bf16 bits), so that a test can tell a different pick at a near-tie from a different pick
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import oracle as O  # noqa: E402
from stark_b200 import synthetic as S  # noqa: E402


LAYERS_STEPS = 100
LEADERS = 8  # largest logits kept per step
LAYERS_SHAPES = {"q8b": "qwen3-8b-layers", "q06b": "qwen3-0.6b-layers"}


def layers_case(shape: str, steps: int) -> dict:
    cfg = S.CONFIGS[LAYERS_SHAPES[shape]]
    weights = S.dense_weights(cfg, seed=2, zero_point=7.5)
    prompt = S.prompt(cfg, 24, seed=6)
    orc = O.DenseOracle(cfg, weights, capacity=24 + steps + 1)
    for t in prompt[:-1]:
        orc.ingest(int(t))
    logits = np.asarray(orc.step(int(prompt[-1])), np.uint16)
    out = {f"{shape}_logits": logits.copy()}
    if steps:
        # A random-init decoder decoded greedily falls into repeating one token, which would make agreement
        # trivial; the continuation is therefore a seeded random token sequence fed to both sides.
        teacher = S.prompt(cfg, steps, seed=7)
        top1, lead_ids, lead_bits = [], [], []
        for t in teacher:
            logits = np.asarray(orc.step(int(t)), np.uint16)
            values = O.bf16_to_f32(logits)
            lead = np.argsort(-values, kind="stable")[:LEADERS]      # equal values: lower index first
            lead_ids.append(lead.astype(np.uint32))
            lead_bits.append(logits[lead])
            top1.append(O.argmax_bf16(logits))
        out[f"{shape}_teacher"] = np.asarray(teacher, np.uint32)
        out[f"{shape}_top1"] = np.asarray(top1, np.uint32)
        out[f"{shape}_lead_ids"] = np.asarray(lead_ids, np.uint32)
        out[f"{shape}_lead_bits"] = np.asarray(lead_bits, np.uint16)
    return out


def build(full: bool = False) -> dict:
    out = {}
    for shape in LAYERS_SHAPES:
        out.update(layers_case(shape, LAYERS_STEPS if full else 0))
    w = S.matvec_case(seed=3, rows=512, columns=1024)
    out["matvec_y"] = O.affine_matvec_bf16(w["codes"], w["scales"], w["biases"], w["x"], 512, 1024)[0]
    cfg = S.CONFIGS["tiny"]
    weights = S.dense_weights(cfg, seed=0)
    prompt = S.prompt(cfg, 70, seed=5)
    orc = O.DenseOracle(cfg, weights, capacity=128)
    for t in prompt[:-1]:
        orc.ingest(int(t))
    logits = orc.step(int(prompt[-1]))
    out["tiny_logits"] = np.asarray(logits, np.uint16)
    toks, tok = [], O.argmax_bf16(logits)
    for _ in range(8):
        toks.append(tok)
        tok = O.argmax_bf16(orc.step(tok))
    out["tiny_greedy"] = np.asarray(toks, np.uint32)
    # the draft head of the dense multi-token-prediction path after a 24-token prompt: two chained draft steps
    weights = S.dense_weights(cfg, seed=3, zero_point=7.5)
    head_w = S.mtp_weights(cfg, seed=3, zero_point=7.5)
    target = O.DenseOracle(cfg, weights, capacity=64)
    head = O.MtpHeadOracle(target, head_w, 64)
    prompt = S.prompt(cfg, 24, seed=17)
    for i, t in enumerate(prompt):
        logits, hidden = target.step(int(t), want_hidden=True)
        if i + 1 < len(prompt):
            head.cache_row(int(prompt[i + 1]), hidden)
    first, out_hidden = head.step(O.argmax_bf16(logits), hidden)
    second, _ = head.step(O.argmax_bf16(first), out_hidden)
    out["tiny_mtp_draft_logits"] = np.stack([first, second]).astype(np.uint16)
    out["tiny_mtp_draft_hidden"] = np.asarray(out_hidden, np.uint16)
    rng = np.random.default_rng(11)
    out["q8_0_row"] = O.gguf_decode_row(O.Q8_0, S.q8_0_rows(rng, 4, 512)[1], 512)
    out["q4_k_row"] = O.gguf_decode_row(O.Q4_K, S.q4_k_rows(rng, 4, 512)[1], 512)
    return out


if __name__ == "__main__":
    np.savez_compressed(Path(__file__).with_name("oracle_outputs.npz"), **build(full="--full" in sys.argv))
    print("wrote", Path(__file__).with_name("oracle_outputs.npz"))
