"""The opt-in persistent decode kernel (STARK_B200_MEGA=1: one launch per token) against the oracle.  The
switch is read when the library loads, so the check runs in a child process."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

CHILD = r"""
import sys
sys.path.insert(0, %r)
import numpy as np
from oracle import oracle as O
from stark_b200 import synthetic as S
from stark_b200.engine import DenseModel
from stark_b200.ops import take_device_error
from tests.test_model_gpu import assert_logits_accepted
cfg = S.CONFIGS["small"]
w = S.dense_weights(cfg, seed=1)
model = DenseModel.load(cfg, w, context_tokens=256)
info = model.info()
assert info.persistent == 1 and info.launches_per_step == 1, (info.persistent, info.launches_per_step)
oracle = O.DenseOracle(cfg, w, capacity=256)
prompt = S.prompt(cfg, 70, seed=5)
model.prefill(prompt)
for t in prompt[:-1]:
    oracle.ingest(int(t))
assert_logits_accepted(oracle.step(int(prompt[-1])), model.logits_bf16())
tokens = model.generate_greedy(12)
model.drain()
assert take_device_error() == 0
agree, tok = 0, int(tokens[0])
for i in range(12):
    agree += int(O.argmax_bf16(oracle.step(tok)) == int(tokens[i + 1]))
    tok = int(tokens[i + 1])
assert agree >= 11, agree
print("PERSISTENT-OK")
""" % str(ROOT)


@pytest.mark.gpu
def test_persistent_kernel_matches_oracle():
    env = dict(os.environ, STARK_B200_MEGA="1")
    res = subprocess.run([sys.executable, "-c", CHILD], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "PERSISTENT-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
