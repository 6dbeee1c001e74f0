"""Host side of the expert-parallel path on CPU: the banks' shards tile the experts, and two gloo ranks that
each compute only the selected experts they own, exchange the rows and mix them in selection order reproduce the
oracle's unsharded routed feed-forward bit for bit (the property the device path is built on: the mixture does
not depend on the rank count)."""
import os
import socket

import numpy as np
import pytest

from oracle import oracle as O
from stark_b200 import synthetic as S
from stark_b200.engine import ExpertParallel, expert_owner, expert_shard

Q4_K = 12


def test_expert_shards_tile_the_bank():
    bank = np.arange(128 * 6, dtype=np.uint8).reshape(128, 6)
    for ranks in (2, 4, 8):
        parts = [expert_shard(bank, r, ranks) for r in range(ranks)]
        assert np.array_equal(np.concatenate(parts), bank)
        per = 128 // ranks
        assert all(expert_owner(e, 128, ranks) == e // per for e in (0, per - 1, per, 127))
    with pytest.raises(ValueError):
        expert_shard(bank, 0, 3)


def _expert_row(w, cfg, expert, x, bank_first=0):
    """down_e (silu(gate_e x) * up_e x) through the oracle's block kernels, experts numbered from bank_first."""
    H, I = cfg["hidden"], cfg["inter"]
    local = expert - bank_first
    gate = O.gguf_matvec_f32(Q4_K, w["gate"][local], x, I, H)
    up = O.gguf_matvec_f32(Q4_K, w["up"][local], x, I, H)
    act = np.array([np.float32(O.silu_f32(float(g))) * u for g, u in zip(gate, up)], np.float32)
    return O.gguf_matvec_f32(Q4_K, w["down"][local], act, H, I)


def _worker(rank: int, ranks: int, port: int, failures):
    try:
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=ranks)

        def all_gather(blob: bytes):
            out = [None] * ranks
            dist.all_gather_object(out, blob)
            return out

        ep = ExpertParallel(rank, ranks, all_gather)
        cfg = S.MOE_CONFIGS["moe-tiny"]
        E, A, H, I = cfg["experts"], cfg["active"], cfg["hidden"], cfg["inter"]
        layer = S.moe_layer_weights(cfg, np.random.default_rng(3))      # every rank draws the same whole layer
        rng = np.random.default_rng(11)
        x = rng.standard_normal(H).astype(np.float32)
        scores = rng.standard_normal(E).astype(np.float32)
        want, ids, probs = O.moe_ffn_f32(Q4_K, layer["gate"], layer["up"], Q4_K, layer["down"], scores, x, E, A, H, I)
        banks = {k: np.asarray(layer[k], np.uint8).reshape(E, -1) for k in ("gate", "up", "down")}
        mine = {k: expert_shard(v, rank, ranks) for k, v in banks.items()}
        first = rank * (E // ranks)
        # the rows of the selection slots this rank owns, empty for the others; then everyone has every row
        rows = [(_expert_row(mine, cfg, int(e), x, first).tobytes() if expert_owner(e, E, ranks) == rank else b"")
                for e in ids]
        gathered = ep.all_gather(b"".join(len(r).to_bytes(4, "little") + r for r in rows))
        full = [None] * A
        for blob in gathered:
            at = 0
            for slot in range(A):
                n = int.from_bytes(blob[at:at + 4], "little")
                if n:
                    assert full[slot] is None                           # exactly one owner per slot
                    full[slot] = np.frombuffer(blob[at + 4:at + 4 + n], np.float32)
                at += 4 + n
        assert all(r is not None for r in full)
        out = np.zeros(H, np.float32)
        for slot in range(A):                                           # selection order, f32, as qwen.rs:894-899
            out = out + np.float32(probs[slot]) * full[slot]
        assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
        dist.barrier()
        dist.destroy_process_group()
    except BaseException as e:  # surfaced by the parent
        failures.put(f"rank {rank}: {type(e).__name__}: {e}")
        raise


def test_two_gloo_ranks_reproduce_the_unsharded_mixture():
    import torch.multiprocessing as mp
    O.lib()  # build the oracle once, before the ranks race for it
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, failures)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    msgs = []
    while not failures.empty():
        msgs.append(failures.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            msgs.append("a rank did not finish")
    assert not msgs and all(p.exitcode == 0 for p in procs), msgs
