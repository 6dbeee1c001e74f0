"""Host side of the tensor-parallel path on CPU: two gloo ranks shard the same model, and the oracle's
matvecs over the shards must reassemble the unsharded results (row splits exactly, column splits up to
f32 summation order, the vocabulary split to the same first index of the maximum)."""
import os
import socket

import numpy as np
import pytest

from oracle import oracle as O
from stark_b200 import synthetic as S
from stark_b200.engine import TensorParallel, shard_dense, vocab_shard


def test_vocab_shards_tile_the_vocabulary():
    for vocab, ranks in [(151936, 8), (151936, 2), (1024, 2), (1000, 4), (48, 4)]:
        spans = [vocab_shard(vocab, r, ranks) for r in range(ranks)]
        assert spans[0][0] == 0 and spans[-1][1] == vocab
        for (a, b), (c, d) in zip(spans, spans[1:]):
            assert b == c and a % 16 == 0 and c % 16 == 0


def test_indivisible_shapes_are_refused():
    cfg = S.CONFIGS["tiny"]
    w = S.dense_weights(cfg, seed=0)
    with pytest.raises(ValueError):
        shard_dense(cfg, w, 0, 4)  # 2 KV heads over 4 ranks
    with pytest.raises(ValueError):
        shard_dense(dict(cfg, inter=320), w, 0, 2)  # 160 columns: not whole 64-wide groups


def _mv(t, x):
    return O.affine_matvec_f32(t["codes"], t["scales"], t["biases"], 30, x, t["n"], t["k"])


@pytest.mark.parametrize("ranks", [2, 8])
def test_row_cuts_for_prompt_passes_gather_to_the_unsharded_products(ranks):
    """The second cut of o and down (output rows over ALL columns, for batched prompt passes): each rank's product
    is a slice of the unsharded one, bit for bit, so gathering the slices needs no arithmetic."""
    cfg = S.CONFIGS["small"]
    w = S.dense_weights(cfg, seed=2)
    rng = np.random.default_rng(11)
    a = rng.standard_normal(cfg["q_heads"] * cfg["head_dim"]).astype(np.float32)
    g = rng.standard_normal(cfg["inter"]).astype(np.float32)
    F = w["layers"][2]
    parts_o, parts_d = [], []
    for rank in range(ranks):
        _, lw, _ = shard_dense(cfg, w, rank, ranks)
        L = lw["layers"][2]
        assert L["o_rows"]["n"] == L["down_rows"]["n"] == cfg["hidden"] // ranks
        assert L["o_rows"]["k"] == cfg["q_heads"] * cfg["head_dim"] and L["down_rows"]["k"] == cfg["inter"]
        parts_o.append(_mv(L["o_rows"], a))
        parts_d.append(_mv(L["down_rows"], g))
    assert np.array_equal(np.concatenate(parts_o), _mv(F["o"], a))
    assert np.array_equal(np.concatenate(parts_d), _mv(F["down"], g))
    # the smallest width that still fills a whole 128-row tile per rank
    _, lw, _ = shard_dense(S.CONFIGS["tiny"], S.dense_weights(S.CONFIGS["tiny"], seed=0), 0, 2)
    assert "o_rows" in lw["layers"][0]           # 256 / 2 = 128 rows


@pytest.mark.parametrize("ranks", [4, 8])
def test_four_and_eight_rank_shards_cover_the_model(ranks):
    """Every rank's shard of the `small` shape (8 KV heads): whole heads, whole quantization groups, and over
    all ranks the column splits of o and down sum to the unsharded products."""
    cfg = S.CONFIGS["small"]
    w = S.dense_weights(cfg, seed=2)
    rng = np.random.default_rng(9)
    F = w["layers"][1]
    a = rng.standard_normal(cfg["q_heads"] * cfg["head_dim"]).astype(np.float32)
    g = rng.standard_normal(cfg["inter"]).astype(np.float32)
    o_sum, d_sum, rows = 0.0, 0.0, 0
    for rank in range(ranks):
        local, lw, vocab_offset = shard_dense(cfg, w, rank, ranks)
        L = lw["layers"][1]
        assert local["q_heads"] * ranks == cfg["q_heads"] and local["kv_heads"] * ranks == cfg["kv_heads"]
        assert local["inter"] * ranks == cfg["inter"] and local["inter"] % 64 == 0
        assert L["qkv"]["n"] == (local["q_heads"] + 2 * local["kv_heads"]) * cfg["head_dim"]
        ql, il = local["q_heads"] * cfg["head_dim"], local["inter"]
        o_sum = o_sum + _mv(L["o"], a[rank * ql:(rank + 1) * ql]).astype(np.float64)
        d_sum = d_sum + _mv(L["down"], g[rank * il:(rank + 1) * il]).astype(np.float64)
        lo, hi = vocab_shard(cfg["vocab"], rank, ranks)
        assert vocab_offset == lo and lw["lm_head"]["n"] == hi - lo
        rows += hi - lo
    assert rows == cfg["vocab"]
    for got, t, x in ((o_sum, F["o"], a), (d_sum, F["down"], g)):
        want = _mv(t, x).astype(np.float64)
        assert np.abs(got - want).max() <= 1e-4 * max(1.0, np.abs(want).max())


def _worker(rank: int, ranks: int, port: int, failures):
    import torch.distributed as dist
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=ranks)

        def all_gather(blob: bytes):
            out = [None] * ranks
            dist.all_gather_object(out, blob)
            return out

        tp = TensorParallel(rank, ranks, all_gather)
        cfg = S.CONFIGS["tiny"]
        w = S.dense_weights(cfg, seed=0)  # every rank draws the same whole model
        local, lw, vocab_offset = shard_dense(cfg, w, rank, ranks)
        rng = np.random.default_rng(7)
        hd, hq, hkv, inter = cfg["head_dim"], cfg["q_heads"], cfg["kv_heads"], cfg["inter"]
        L, F = lw["layers"][0], w["layers"][0]
        x = rng.standard_normal(cfg["hidden"]).astype(np.float32)

        # row splits: each rank's outputs are a subset of the unsharded outputs, bit for bit
        full = _mv(F["qkv"], x)
        mine = _mv(L["qkv"], x)
        ql, kl = local["q_heads"] * hd, local["kv_heads"] * hd
        want = np.concatenate([full[rank * ql:(rank + 1) * ql], full[hq * hd + rank * kl:hq * hd + (rank + 1) * kl],
                               full[(hq + hkv) * hd + rank * kl:(hq + hkv) * hd + (rank + 1) * kl]])
        assert np.array_equal(mine.view(np.uint32), want.view(np.uint32))
        full = _mv(F["upgate"], x)
        mine = _mv(L["upgate"], x)
        il = local["inter"]
        want = np.concatenate([full[rank * il:(rank + 1) * il], full[inter + rank * il:inter + (rank + 1) * il]])
        assert np.array_equal(mine.view(np.uint32), want.view(np.uint32))

        # column splits: the ranks' partial products sum to the unsharded product
        for name, width, lo in (("o", hq * hd, rank * ql), ("down", inter, rank * il)):
            a = rng.standard_normal(width).astype(np.float32)
            part = _mv(L[name], a[lo:lo + L[name]["k"]])
            parts = [np.frombuffer(b, np.float32) for b in tp.all_gather(part.tobytes())]
            total = np.sum(parts, axis=0, dtype=np.float32)
            full = _mv(F[name], a)
            np.testing.assert_allclose(total, full, rtol=0, atol=2e-5 * np.abs(full).max() + 1e-6)

        # prompt passes: the row cuts of o and down produce whole output elements over the full width, so the
        # ranks' slices of several rows only have to be gathered -- no sum, the same bits as unsharded
        rows = rng.standard_normal((3, hq * hd)).astype(np.float32)
        for name, inputs in (("o", rows), ("down", rng.standard_normal((3, inter)).astype(np.float32))):
            mine = np.stack([_mv(L[name + "_rows"], a) for a in inputs])          # [3, hidden / ranks]
            slices = [np.frombuffer(b, np.float32).reshape(3, -1) for b in tp.all_gather(mine.tobytes())]
            gathered = np.concatenate(slices, axis=1)
            full = np.stack([_mv(F[name], a) for a in inputs])
            assert np.array_equal(gathered.view(np.uint32), full.view(np.uint32))

        # vocabulary split: (max, first index) per shard reduces to the unsharded greedy token
        h = rng.standard_normal(cfg["hidden"]).astype(np.float32)
        full = O.f32_to_bf16(_mv(w["lm_head"], h))
        full[[5, 900]] = O.f32_to_bf16(np.float32([abs(O.bf16_to_f32(full)).max() * 2 + 1]))[0]  # a tie across shards
        lo, hi = vocab_shard(cfg["vocab"], rank, ranks)
        assert lo == vocab_offset and local["vocab"] == hi - lo and local["vocab_total"] == cfg["vocab"]
        shard = full[lo:hi]
        cand = (float(O.bf16_to_f32(shard).max()), lo + O.argmax_bf16(shard))
        cands = [tuple(np.frombuffer(b, np.float64)) for b in tp.all_gather(np.array(cand, np.float64).tobytes())]
        best = max(cands, key=lambda c: (c[0], -c[1]))
        assert int(best[1]) == O.argmax_bf16(full) == 5
        dist.barrier()
        dist.destroy_process_group()
    except BaseException as e:  # surfaced by the parent
        failures.put(f"rank {rank}: {type(e).__name__}: {e}")
        raise


def test_two_gloo_ranks_reassemble_the_unsharded_results():
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


def _leaver(rank: int, port: int, results):
    """Rank 1 leaves between two requests; rank 0 must learn of it on the host, at the rendezvous that opens its
    next request (`DenseModel.prefill` starts with one), before it would launch anything."""
    import datetime
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2, timeout=datetime.timedelta(seconds=6))

    def all_gather(blob: bytes):
        out = [None, None]
        dist.all_gather_object(out, blob)
        return out

    def report_and_leave(message: str):
        results.put(message)
        results.close()
        results.join_thread()  # the queue's feeder thread has written the message: an abrupt exit cannot lose it
        os._exit(0)

    tp = TensorParallel(rank, 2, all_gather)
    assert tp.all_gather(b"request 1") == [b"request 1", b"request 1"]   # both ranks open the first request
    if rank == 1:
        report_and_leave("rank 1 left between requests")                # no kernel in flight: a host-side leave
    try:
        tp.all_gather(b"request 2")
        report_and_leave("rank 0 was not told")
    except Exception as e:  # noqa: BLE001 - gloo reports a closed connection or a timeout
        report_and_leave(f"rank 0 learned of it on the host: {type(e).__name__}")


def test_a_rank_that_leaves_between_requests_is_noticed_on_the_host():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    procs = [ctx.Process(target=_leaver, args=(r, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    msgs = []
    while not results.empty():
        msgs.append(results.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            msgs.append("a rank hung")
    assert any(m.startswith("rank 0 learned of it on the host") for m in msgs), msgs
    assert not any("hung" in m or "not told" in m for m in msgs), msgs
