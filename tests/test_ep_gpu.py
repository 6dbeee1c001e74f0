"""Expert-parallel routed-expert decoding on 2, 4 and 8 GPUs against the single-GPU decoder and the CPU oracle.

The test launches one process per GPU (this file is also the rank program); a case is skipped on a box with
fewer GPUs than it needs.  Ranks rendezvous over gloo on 127.0.0.1: the host side only moves the 64-byte buffer
handles, the per-layer exchange of expert rows happens on the device.  The mixture is formed in selection order
from the same rows on every rank, so logits and tokens must be the same BITS as on one GPU.
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
@pytest.mark.parametrize("config,ranks", [("moe-tiny", 2), ("moe-small", 2), ("moe-small", 4), ("moe-small", 8)])
def test_ranks_match_single_gpu_and_oracle(config, ranks):
    if _gpu_count() < ranks:
        pytest.skip(f"needs {ranks} GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(ranks), "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(Path(__file__).resolve()), config]
    res = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=900)
    failed = [line for line in res.stdout.splitlines() if "RANK-FAILED" in line]
    assert res.returncode == 0, "\n".join(failed) + res.stdout[-3000:] + res.stderr[-1500:]
    assert "EP-OK" in res.stdout


def _rank_main(config: str) -> None:
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    from oracle import oracle as O
    from stark_b200 import _lib, synthetic as S
    from stark_b200.engine import ExpertParallel, MoEModel

    rank, ranks = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=ranks)
    _lib.check(_lib.load().stark_b200_set_device(int(os.environ.get("LOCAL_RANK", rank))), "set_device")

    def all_gather(blob: bytes):
        out = [None] * ranks
        dist.all_gather_object(out, blob)
        return out

    cfg = S.MOE_CONFIGS[config]
    w = S.moe_weights(cfg, seed=0)
    context = 128
    model = MoEModel.load(cfg, w, context, ep=ExpertParallel(rank, ranks, all_gather))
    assert model.launches_per_token == 4 + 10 * cfg["layers"] + cfg["layers"] + 1
    prompt = S.prompt(cfg, 20, seed=5)
    model.ingest(prompt[:-1])
    logits = model.step(int(prompt[-1]))
    experts = model.last_experts()
    assert model.position == len(prompt)
    first = int(np.argmax(logits))
    steps = 24
    tokens = model.generate_greedy(first, steps)
    everyone = all_gather(logits.tobytes() + tokens.tobytes() + experts.tobytes())
    assert all(b == everyone[0] for b in everyone)          # every rank: the same bits

    if rank == 0:
        # one GPU, same weights: the exchange must not change a bit
        single = MoEModel.load(cfg, w, context)
        single.ingest(prompt[:-1])
        want = single.step(int(prompt[-1]))
        assert np.array_equal(single.last_experts(), experts)
        assert np.array_equal(want.view(np.uint32), logits.view(np.uint32))
        assert np.array_equal(single.generate_greedy(first, steps), tokens)
        single.close()
        # and the CPU oracle, to the bar of the single-GPU decoder's own test
        oracle = O.MoEDecoder(cfg, w, context)
        oracle.ingest(prompt[:-1])
        ref = oracle.step(int(prompt[-1]))
        assert np.asarray(oracle.last_experts).reshape(experts.shape).tolist() == experts.tolist()
        assert np.abs(logits - ref).max() <= 1e-3 * np.abs(ref).max()
    # a second request after a reset: tickets keep counting, buffers are reused
    model.reset()
    model.ingest(prompt[:5])
    again = model.step(int(prompt[5]))
    if rank == 0:
        single = MoEModel.load(cfg, w, context)
        single.ingest(prompt[:5])
        assert np.array_equal(single.step(int(prompt[5])).view(np.uint32), again.view(np.uint32))
        single.close()
    model.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("EP-OK", config, flush=True)


if __name__ == "__main__":
    try:
        _rank_main(sys.argv[1])
    except BaseException:
        import traceback
        print("RANK-FAILED", os.environ.get("RANK"), traceback.format_exc()[-1500:], flush=True)
        sys.exit(1)
