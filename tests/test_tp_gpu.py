"""Tensor-parallel decode on 2, 4 and 8 GPUs against the CPU oracle and against the single-GPU engine.

The test launches one process per GPU (this file is also the rank program); a case is skipped on a box
with fewer GPUs than it needs.  Ranks rendezvous over gloo on 127.0.0.1: the host side only moves the
64-byte buffer handles and read-out shards, the per-token exchange happens on the device.
"""
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _gpu_count() -> int:
    import ctypes as C
    from stark_b200 import _lib
    n = C.c_int32(0)
    return n.value if _lib.load().stark_b200_device_count(C.byref(n)) == 0 else 0


@pytest.mark.gpu
@pytest.mark.parametrize("config,ranks,mode", [("tiny", 2, ""), ("small", 2, ""), ("small", 2, "staged"),
                                               ("small", 2, "token-rows"), ("small", 2, "copy-rows"), ("small", 2, "push-rows"),
                                               ("small", 4, "push-rows"), ("small", 4, ""),
                                               ("small", 8, "")])
def test_ranks_match_oracle_and_single_gpu(config, ranks, mode):
    """Modes: "staged", the reduction kernel also normalizes and scales the row for the matvec behind it (off by
    default); "token-rows", prompt rows take the token path instead of batched passes across the ranks; "copy-rows",
    a copy kernel moves every column slice of a batched pass; "push-rows", every contraction's own epilogue does (the
    default between two ranks; more ranks use the copy kernel unless told otherwise)."""
    if _gpu_count() < ranks:
        pytest.skip(f"needs {ranks} GPUs")
    env = dict(os.environ, STARK_B200_TP_STAGE=str(int(mode == "staged")), STARK_B200_TEST_TP_MODE=mode,
               STARK_B200_TP_ROWS_PUSH={"copy-rows": "0", "push-rows": "1"}.get(mode, "2"))
    for attempt in range(2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(ranks), "--master-addr",
               "127.0.0.1", "--master-port", str(port), str(Path(__file__).resolve()), config]
        res = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=900, env=env)
        # A rank that fails says so itself (RANK-FAILED).  A launch that dies without any rank's word -- the port
        # found above taken by someone else before the launcher bound it -- is tried once more on another port.
        if res.returncode == 0 or "RANK-FAILED" in res.stdout:
            break
    failed = [line for line in res.stdout.splitlines() if "RANK-FAILED" in line]
    assert res.returncode == 0, "\n".join(failed) + res.stdout[-3000:] + res.stderr[-1500:]
    assert "TP-OK" in res.stdout


def _rank_main(config: str) -> None:
    sys.path.insert(0, str(ROOT))
    import ctypes as C
    import torch.distributed as dist
    from oracle import oracle as O
    from stark_b200 import _lib, synthetic as S
    from stark_b200.engine import DenseModel, TensorParallel
    from stark_b200.ops import take_device_error
    from tests.test_model_gpu import assert_logits_accepted

    rank, ranks = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=ranks)
    _lib.check(_lib.load().stark_b200_set_device(int(os.environ.get("LOCAL_RANK", rank))), "set_device")

    def all_gather(blob: bytes):
        out = [None] * ranks
        dist.all_gather_object(out, blob)
        return out

    cfg = S.CONFIGS[config]
    w = S.dense_weights(cfg, seed=0)
    context = 256
    batched = os.environ.get("STARK_B200_TEST_TP_MODE", "") != "token-rows"
    model = DenseModel.load(cfg, w, context, tp=TensorParallel(rank, ranks, all_gather, rows=batched))
    info = model.info()
    # 5 launches per layer, plus one small reduction kernel per exchange unless the exchanges are fused
    assert info.launches_per_step in (1 + 5 * cfg["layers"] + 2, 1 + 7 * cfg["layers"] + 2)

    prompt = S.prompt(cfg, 70, seed=5)  # crosses a KV page boundary
    before = model.info().launches_issued
    model.prefill(prompt)
    issued = model.info().launches_issued - before
    if batched:  # one pass over 69 rows (8 kernels and 4 gathers a layer) and one token, not 70 tokens
        assert issued == 1 + 12 * cfg["layers"] + info.launches_per_step, issued
    else:
        assert issued >= 69 * 5 * cfg["layers"]
    logits = model.logits_bf16()        # gathered from the ranks' vocabulary shards
    assert logits.size == cfg["vocab"]
    first = model.argmax()
    assert first == O.argmax_bf16(logits)  # the cross-shard pick is the first index of the global maximum
    steps = 100
    tokens = model.generate_greedy(steps)
    model.drain()
    assert take_device_error() == 0
    assert int(tokens[0]) == first
    everyone = all_gather(tokens.tobytes())
    assert all(t == everyone[0] for t in everyone)  # all ranks chose the same tokens

    if rank == 0:
        oracle = O.DenseOracle(cfg, w, capacity=context)
        for t in prompt[:-1]:
            oracle.ingest(int(t))
        assert_logits_accepted(oracle.step(int(prompt[-1])), logits)
        agree, tok = 0, int(tokens[0])
        for i in range(steps):  # teacher-forced on the engine's tokens
            agree += int(O.argmax_bf16(oracle.step(tok)) == int(tokens[i + 1]))
            tok = int(tokens[i + 1])
        assert agree / steps >= 0.99, agree
        # the same model on one GPU: logits within the acceptance, and the same first token
        single = DenseModel.load(cfg, w, context)
        single.prefill(prompt)
        assert_logits_accepted(single.logits_bf16(), logits)
        single.close()
    # host-fed steps follow the same path as the device-chained ones (prefill lines the ranks up
    # again after rank 0's checks)
    model.reset()
    model.prefill(prompt)
    tok, fed = model.argmax(), []
    for _ in range(4):
        fed.append(tok)
        model.step_async(tok)
        tok = model.argmax()
    assert fed == tokens[:4].tolist()
    # a longer prompt in two calls (several row tiles; the second call continues at a position that is not a page
    # boundary), against the same calls on one GPU: the batched rows are the same bits there, the last row differs
    # by the token path's summation order
    model.reset()
    longer = S.prompt(cfg, 230, seed=8)
    model.prefill(longer[:150])
    model.prefill(longer[150:])
    logits = model.logits_bf16()
    assert take_device_error() == 0
    if rank == 0:
        single = DenseModel.load(cfg, w, context)
        single.prefill(longer[:150])
        single.prefill(longer[150:])
        assert_logits_accepted(single.logits_bf16(), logits)
        single.close()
    model.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("TP-OK", config, flush=True)


if __name__ == "__main__":
    try:
        _rank_main(sys.argv[1])
    except BaseException:
        import traceback
        print("RANK-FAILED", os.environ.get("RANK"), traceback.format_exc()[-1500:], flush=True)
        raise
