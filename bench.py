#!/usr/bin/env python
"""Batch-1 decode benchmark of the token loop on synthetic random-init weights.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload qwen3-8b|qwen3-0.6b]
    python bench.py --impl reference ...      # the reference's CPU path (oracle port), bounded sample

A "step" is one greedy decode token at batch 1.  The default workload is the 4-bit Qwen3-8B-shaped
dense decoder (36 layers, hidden 4096, 32 Q / 8 KV heads, intermediate 12288, vocab 151936) with a
4096-token random prompt, the configuration the headline target is stated on.  Prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from stark_b200 import synthetic as S  # noqa: E402

WORKLOADS = {
    "qwen3-8b": dict(cfg="qwen3-8b", prompt=4096, context=4096 + 1024),
    "qwen3-0.6b": dict(cfg="qwen3-0.6b", prompt=512, context=512 + 512),
    "small": dict(cfg="small", prompt=96, context=512),
    # speculative rounds on the dense model plus a one-layer draft head: 4 proposals, a 5-row verify pass
    # against 8192 cache rows, acceptance forced to a seeded Bernoulli(0.6) per proposal
    "qwen3-8b-mtp": dict(cfg="qwen3-8b", prompt=8192, context=8192, mtp=True, drafts=4, accept=0.6),
    "small-mtp": dict(cfg="small", prompt=96, context=96, mtp=True, drafts=4, accept=0.6),
    # two layers at the 8B shape's dimensions: the same kernels on a gigabyte of weights (what the ncu captures run)
    "qwen3-8b-layers-mtp": dict(cfg="qwen3-8b-layers", prompt=8192, context=8192, mtp=True, drafts=4, accept=0.6),
    "qwen3-8b-layers": dict(cfg="qwen3-8b-layers", prompt=4096, context=4096 + 1024),
    # routed-expert decoders (f32 host-path conventions, GGUF Q8_0 attention + Q4_K experts)
    "qwen3-30b-a3b": dict(cfg="qwen3-30b-a3b", prompt=2048, context=2048 + 512, moe=True),
    "moe-small": dict(cfg="moe-small", prompt=64, context=256, moe=True),
    # a single quantized matvec (BASELINE config 1 by default): micro-benchmark / profiling target
    "matvec": dict(cfg=None, prompt=0, context=0),
    # the prompt-chunk contraction alone (tensor-core GEMM over a 4-bit matrix): profiling target
    "gemm": dict(cfg=None, prompt=0, context=0),
}
BYTES_PER_WEIGHT = 0.5625  # 4-bit codes + bf16 scale and bias per 64 columns
DRAM_TRAFFIC_RATIO = 1.011  # measured dram bytes / algorithmic bytes of the 4-bit matvec (ncu, 151936x4096)


def host_threads() -> int:
    """Host cores this process may run on.  Passed to the CPU arm explicitly: launchers such as
    torch.distributed.run export OMP_NUM_THREADS=1, which would otherwise pin it to one core."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def weight_count(cfg: dict) -> tuple[int, int]:
    """(weights read by one decode step, of which read-out table)."""
    D, hd, I, V = cfg["hidden"], cfg["head_dim"], cfg["inter"], cfg["vocab"]
    per_layer = (cfg["q_heads"] + 2 * cfg["kv_heads"]) * hd * D + D * cfg["q_heads"] * hd + 2 * I * D + D * I
    return cfg["layers"] * per_layer + V * D, V * D


def prefill_flops(cfg: dict, prompt_rows: int) -> float:
    """Multiply-add work of ingesting a prompt: 2 M N K per layer matrix over the cache-only rows, plus attention
    4 * rows * context * q_heads * head_dim with the causal mean context (the last row is a decode step)."""
    rows = prompt_rows - 1
    per_layer_weights = (weight_count(cfg)[0] - weight_count(cfg)[1]) / cfg["layers"]
    gemm = 2.0 * rows * per_layer_weights * cfg["layers"]
    attention = 4.0 * rows * (rows / 2.0) * cfg["q_heads"] * cfg["head_dim"] * cfg["layers"]
    return gemm + attention


def tensor_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["bf16_tflops_sustained"]), "measured sustained"
    return 1400.0, "fallback"


def step_bytes(cfg: dict, context_rows: float) -> float:
    """Algorithmic bytes of one decode step: every quantized matrix once, the KV rows of the
    context, one embedding row, and the activation vectors."""
    n, _ = weight_count(cfg)
    kv = cfg["layers"] * 2 * cfg["kv_heads"] * cfg["head_dim"] * 2 * context_rows
    D, I = cfg["hidden"], cfg["inter"]
    vectors = cfg["layers"] * 2 * (4 * D + (cfg["q_heads"] + 2 * cfg["kv_heads"]) * 128 + cfg["q_heads"] * 128 + I) \
        + 2 * cfg["vocab"]
    return n * BYTES_PER_WEIGHT + kv + cfg["hidden"] * BYTES_PER_WEIGHT + vectors


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 7 and r[3 + i] == "Active" for r in self.rows)]
        out = {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
               "reasons": reasons, "samples": len(sm)}
        if not sm:
            out["note"] = "unavailable: nvidia-smi returned no sample during the timed region"
        return out


def cpu_sample(cfg: dict, weights: dict, prompt: np.ndarray, prompt_rows: int, steps: int, threads: int) -> dict:
    """Times the CPU oracle (a port of the reference's CPU kernels) on a bounded sample."""
    from oracle import oracle as O
    orc = O.DenseOracle(cfg, weights, capacity=prompt_rows + steps + 1, threads=threads)
    for t in prompt[:prompt_rows - 1]:
        orc.ingest(int(t))
    logits = orc.step(int(prompt[prompt_rows - 1]))
    tok = O.argmax_bf16(logits)
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = O.argmax_bf16(orc.step(tok))
    dt = time.perf_counter() - t0
    return {"value": steps / dt, "unit": "tok/s", "cores": threads, "kind": "port",
            "sample": f"{steps} greedy decode steps after a {prompt_rows}-token prompt, same weights"}


def run_matvec(args) -> None:
    """One y = W x per step over a pool of matrices larger than L2, recorded as a CUDA graph."""
    import torch

    from stark_b200.ops import Graph, QMatrix, take_device_error
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    rows, cols = args.rows, args.columns
    w = S.matvec_case(seed=args.seed, rows=rows, columns=cols)
    rng = np.random.default_rng(args.seed)
    bytes_per_weight = {"affine4": 0.5625, "affine8": 1.0625, "q8_0": 34 / 32, "q4_k": 144 / 256}[args.format]
    per = rows * cols * bytes_per_weight + 2 * (rows + cols)
    pool_n = min(40, max(2, int(300e6 // per) + 1))
    if args.format == "affine4":
        make = lambda: QMatrix.from_affine(w["codes"], w["scales"], w["biases"], rows, cols)
    elif args.format == "affine8":
        w8 = S.affine8_matrix(rng, rows, cols)
        make = lambda: QMatrix.from_affine(w8["codes"], w8["scales"], w8["biases"], rows, cols, bits=8)
    else:
        kind = 8 if args.format == "q8_0" else 12
        data = (S.q8_0_rows if kind == 8 else S.q4_k_rows)(rng, rows, cols)
        make = lambda: QMatrix.from_gguf(data, kind, rows, cols)
    pool = [make() for _ in range(pool_n)]
    x = torch.from_numpy(w["x"].view(np.int16)).cuda()
    y = torch.empty(rows, dtype=torch.int16, device="cuda")
    stream = torch.cuda.Stream()
    steps, warmup = args.steps, max(args.warmup, 3)
    with torch.cuda.stream(stream):
        st = stream.cuda_stream
        pool[0].matvec_device(x.data_ptr(), y.data_ptr(), stream=st)
        stream.synchronize()
        with Graph(st) as graph:
            for q in pool:
                q.matvec_device(x.data_ptr(), y.data_ptr(), stream=st)
        reps = max(1, (steps + pool_n - 1) // pool_n)
        for _ in range(max(1, (warmup + pool_n - 1) // pool_n)):
            graph.launch()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            graph.launch()
        e1.record(stream)
        stream.synchronize()
    n = reps * pool_n
    us = e0.elapsed_time(e1) * 1e3 / n
    assert take_device_error() == 0
    peak, kind = peaks()
    # end to end: host vectors in and out through the operator call, every step
    t0 = time.perf_counter()
    for i in range(min(n, 64)):
        pool[i % pool_n].matvec(w["x"])
    e2e = (time.perf_counter() - t0) / min(n, 64)
    graph.destroy()
    print(json.dumps({
        "metric": f"{args.format} matvec GB/s", "value": per / us / 1e3, "unit": "GB/s", "n_gpus": 1, "steps": n,
        "warmup": warmup, "ms_per_step": us / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"matvec {rows}x{cols} {args.format}, batch 1",
                   "l2": f"pool of {pool_n} matrices ({pool_n * per / 1e6:.0f} MB) cycled, larger than L2"},
        "e2e": {"value": per / e2e / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 2 * cols, "d2h_bytes_per_step": 2 * rows},
        "gpu_launches": n,
        "roofline": {"bound": "hbm", "achieved": per / us / 1e3, "peak": peak, "unit": "GB/s",
                     "frac": per / us / 1e3 / peak,
                     "traffic": DRAM_TRAFFIC_RATIO * per if args.format == "affine4" else None, "peak_kind": kind},
    }))


def run_gemm(args) -> None:
    """One Y[M, N] = X[M, K] W^T per step (the prompt-chunk contraction) over a pool of matrices larger than L2."""
    import torch

    from stark_b200 import _lib
    from stark_b200.ops import QMatrix, take_device_error
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    rows, cols, m = args.rows, args.columns, args.m
    rng = np.random.default_rng(args.seed)
    c = 17.3 / np.sqrt(cols)
    per = rows * cols * BYTES_PER_WEIGHT
    pool_n = min(24, max(2, int(300e6 // per) + 1))
    pool = []
    for _ in range(pool_n):
        w = S.affine4_matrix(rng, rows, cols, 0.005 * c, 0.02 * c)
        pool.append(QMatrix.from_affine(w["codes"], w["scales"], w["biases"], rows, cols))
    x = torch.from_numpy(S.bf16_normal(rng, m * cols).view(np.int16)).cuda()
    y = torch.empty(m * rows, dtype=torch.int16, device="cuda")
    lib = _lib.load()
    stream = torch.cuda.Stream()
    st = stream.cuda_stream
    steps, warmup = args.steps, max(args.warmup, 3)

    def one(q):
        _lib.check(lib.stark_b200_op_qgemm(q._h, x.data_ptr(), y.data_ptr(), m, 0, _lib.DEVICE, st), "op_qgemm")
    with torch.cuda.stream(stream):
        for i in range(warmup):
            one(pool[i % pool_n])
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            one(pool[i % pool_n])
        e1.record(stream)
        stream.synchronize()
    assert take_device_error() == 0
    us = e0.elapsed_time(e1) * 1e3 / steps
    flops = 2.0 * m * rows * cols
    tpeak, tkind = tensor_peak()
    tf = flops / us / 1e6
    # end to end: host rows in and out through the operator call
    xh = S.bf16_normal(rng, m * cols).reshape(m, cols)
    t0 = time.perf_counter()
    for i in range(min(steps, 8)):
        pool[i % pool_n].gemm(xh)
    e2e = (time.perf_counter() - t0) / min(steps, 8)
    print(json.dumps({
        "metric": "4-bit affine GEMM TFLOP/s", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": us / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"gemm {m} rows x [{rows} x {cols}] 4-bit affine g64, bf16 in/out",
                   "l2": f"pool of {pool_n} matrices ({pool_n * per / 1e6:.0f} MB) cycled, larger than L2"},
        "e2e": {"value": flops / e2e / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * m * cols,
                "d2h_bytes_per_step": 2 * m * rows},
        "gpu_launches": steps,
        "roofline": {"bound": "tensor", "achieved": tf, "peak": tpeak, "unit": "TFLOP/s", "frac": tf / tpeak,
                     "traffic": None, "peak_kind": tkind},
    }))


def moe_weights_cycled(cfg: dict, seed: int, distinct: int = 4) -> dict:
    """Weights of a routed-expert decoder with `distinct` independently drawn layers repeated in turn: the
    full shape has 16 GB of expert banks, and drawing every layer separately would take minutes of host time
    without changing what a step reads (each layer still gets its own device copy)."""
    rng = np.random.default_rng(seed)
    g = dict(token_table=S.q8_0_rows(rng, cfg["vocab"], cfg["hidden"], scale=3e-4),
             output=S.q8_0_rows(rng, cfg["vocab"], cfg["hidden"], scale=3e-4),
             final_norm=(1.0 + 0.1 * rng.standard_normal(cfg["hidden"])).astype(np.float32))
    drawn = [S.moe_layer_weights(cfg, rng) for _ in range(min(distinct, cfg["layers"]))]
    g["layers"] = [drawn[i % len(drawn)] for i in range(cfg["layers"])]
    return g


def moe_step_bytes(model, cfg: dict, context_rows: float) -> float:
    """Algorithmic bytes of one decode token: the weights it reads plus the f32 key/value rows."""
    kv = cfg["layers"] * 2 * cfg["kv_heads"] * cfg["head_dim"] * 4 * context_rows
    return model.weight_bytes_per_token() + kv


def moe_cpu_sample(cfg: dict, weights: dict, prompt: np.ndarray, prompt_rows: int, steps: int, threads: int) -> dict:
    from oracle import oracle as O
    orc = O.MoEDecoder(cfg, weights, prompt_rows + steps + 1, threads=threads)
    orc.ingest(prompt[:prompt_rows - 1])
    tok = int(orc.step(int(prompt[prompt_rows - 1])).argmax())
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = int(orc.step(tok).argmax())
    dt = time.perf_counter() - t0
    return {"value": steps / dt, "unit": "tok/s", "cores": threads, "kind": "port",
            "sample": f"{steps} greedy decode steps after a {prompt_rows}-token prompt, same weights"}


def run_moe(args, wl) -> None:
    """Greedy decode of a routed-expert decoder: one GPU, or expert parallel over the ranks of the launch (one
    token stream; every rank runs attention, router and read-out, the experts are divided: strong scaling)."""
    import torch

    from stark_b200.engine import ExpertParallel, MoEModel
    cfg = S.MOE_CONFIGS[wl["cfg"]]
    steps, warmup = args.steps, max(args.warmup, 3)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference" and rank != 0:
        return
    weights = moe_weights_cycled(cfg, args.seed)
    prompt = S.prompt(cfg, wl["prompt"], seed=args.seed + 1)
    threads = host_threads()
    if args.impl == "reference":
        sample_steps = max(1, min(args.steps, 4))
        rows = min(wl["prompt"], 16)
        for _ in range(max(args.warmup, 0) and 1):
            moe_cpu_sample(cfg, weights, prompt, rows, 1, threads)
        base = moe_cpu_sample(cfg, weights, prompt, rows, sample_steps, threads)
        print(json.dumps({
            "impl": "reference", "metric": "decode tokens/s", "value": base["value"], "unit": "tok/s",
            "n_gpus": args.gpus, "steps": sample_steps, "warmup": args.warmup, "ms_per_step": 1e3 / base["value"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{wl['cfg']} routed-expert decoder, GGUF Q8_0 attention + Q4_K experts, batch 1"},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    torch.cuda.set_device(local)
    ep = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        host_group = dist.new_group(backend="gloo")  # moves the 64-byte buffer handles and lines requests up

        def all_gather(blob: bytes):
            out = [None] * world
            dist.all_gather_object(out, blob, group=host_group)
            return out
        ep = ExpertParallel(rank, world, all_gather)
    # rows of cache: the prompt, the warm-up and timed steps, and the end-to-end loop after them
    model = MoEModel.load(cfg, weights, max(wl["context"], wl["prompt"] + warmup + steps + min(steps, 64) + 8), ep=ep)
    model.ingest(prompt[:-1])
    first = int(model.step(int(prompt[-1])).argmax())
    picks = model.generate_greedy(first, warmup)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream = torch.cuda.ExternalStream(model.stream)  # events go on the stream the decoder launches on
    with ClockSampler(local) as clocks:
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0.record(stream)
        out = model.generate_greedy(int(picks[-1]), steps)
        e1.record(stream)
        torch.cuda.synchronize()
        # end to end: the token goes in from the host, the full logits come back, the host picks
        tok = int(out[-1])
        t0 = time.perf_counter()
        e2e_steps = min(steps, 64)
        for _ in range(e2e_steps):
            tok = int(model.step(tok).argmax())
        e2e = (time.perf_counter() - t0) / e2e_steps
    ms = e0.elapsed_time(e1) / steps
    if world > 1:  # a token is done when the slowest rank is
        t = torch.tensor([ms, e2e], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e = t.tolist()
    rows = wl["prompt"] + warmup + steps / 2
    per = moe_step_bytes(model, cfg, rows)
    peak, kind = peaks()
    line = {
        "metric": "decode tokens/s", "value": 1e3 / ms, "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"{wl['cfg']} routed-expert decoder, GGUF Q8_0 attention + Q4_K experts, batch 1, "
                               f"{wl['prompt']}-token prompt, greedy decode",
                   "parallelism": "one GPU" if world == 1 else f"ep{world}: experts divided over the ranks, attention, "
                                                               "router and read-out on every rank, rows exchanged over peer memory",
                   "l2": f"{per / 1e6:.0f} MB read per step, larger than L2" if per > 126e6 else
                         f"{per / 1e6:.0f} MB read per step (fits in L2: a test shape, not a bench line)"},
        "e2e": {"value": 1.0 / e2e, "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4 * cfg["vocab"]},
        "gpu_launches": steps * model.launches_per_token, "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "achieved": per / ms / 1e6, "peak": peak, "unit": "GB/s",
                     "frac": per / ms / 1e6 / peak, "traffic": None, "peak_kind": kind},
    }
    if world > 1:
        line["roofline"]["note"] = "per GPU: replicated matrices and cache plus the rank's mean share of the selected experts"
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = moe_cpu_sample(cfg, weights, prompt, min(wl["prompt"], 16), 2, threads)
    model.close()
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def mtp_round_bytes(cfg: dict, drafts: int, context_rows: float) -> float:
    """Algorithmic bytes of one speculative round: the target's matrices once (the verify pass reads each record
    once for all rows), its KV rows once, and per proposal the head's fusion matrix, its one layer, the read-out
    table and the head's own KV rows."""
    n, table = weight_count(cfg)
    D = cfg["hidden"]
    layer = (n - table) / cfg["layers"]
    kv_layer = 2 * cfg["kv_heads"] * cfg["head_dim"] * 2 * context_rows
    target = n * BYTES_PER_WEIGHT + cfg["layers"] * kv_layer
    head = (2 * D * D + layer + table) * BYTES_PER_WEIGHT + kv_layer
    return target + drafts * head


def run_mtp(args, wl) -> None:
    """Speculative rounds: `--steps` counts rounds; the value is committed tokens per second."""
    import torch
    from stark_b200.engine import DenseModel
    from stark_b200.ops import take_device_error
    assert int(os.environ.get("WORLD_SIZE", "1")) == 1, "the speculative workload runs on one GPU"
    cfg = S.CONFIGS[wl["cfg"]]
    drafts = wl["drafts"] if args.drafts < 0 else min(args.drafts, 7)
    p_accept = wl["accept"] if args.accept < 0 else min(args.accept, 1.0)
    rounds, warmup = args.steps, max(args.warmup, 3)
    repeats = args.repeats if args.repeats > 0 else max(5, min(64, -(-160 // max(rounds, 1))))
    weights = S.dense_weights(cfg, seed=args.seed)
    weights_mtp = dict(weights, mtp=S.mtp_weights(cfg, seed=args.seed))
    prompt = S.prompt(cfg, wl["prompt"], seed=args.seed + 1)
    context = wl["prompt"] + (drafts + 1) * (warmup + 2 * repeats * rounds + 4) + 64
    model = DenseModel.load(dict(cfg, mtp=True), weights_mtp, context_tokens=context)
    info = model.info()
    stream = torch.cuda.ExternalStream(model.stream())
    rng = np.random.default_rng(args.seed + 5)

    def mask() -> int:
        m = 0
        for i in range(drafts):
            if rng.random() < p_accept:
                m |= 1 << i
        return m

    model.prefill(prompt)
    model.drain()
    model.reset()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record(stream)
    model.prefill(prompt)
    p1.record(stream)
    model.drain()
    prefill_ms = p0.elapsed_time(p1)
    pending = model.mtp_initial()
    launches0 = model.info().launches_issued
    for _ in range(warmup):
        pending = model.mtp_round(pending, drafts, accept_mask=mask())["next_pending"]
    launches_per_round = (model.info().launches_issued - launches0) / warmup
    torch.cuda.synchronize()
    # A round ends with the host reading the accepted tokens (the acceptance decision is the caller's in the
    # reference: its sampler runs on the host), so the device-timed and the end-to-end figure cover the same
    # calls; the first is taken with CUDA events on the model's stream, the second with the host clock.
    events = [torch.cuda.Event(enable_timing=True) for _ in range(repeats + 1)]
    regions, host_regions, committed = [], [], []
    with ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) as clocks:
        events[0].record(stream)
        for r in range(repeats):
            t0, n = time.perf_counter(), 0
            for _ in range(rounds):
                out = model.mtp_round(pending, drafts, accept_mask=mask())
                pending, n = out["next_pending"], n + len(out["tokens"])
            events[r + 1].record(stream)
            torch.cuda.synchronize()
            host_regions.append(time.perf_counter() - t0)
            committed.append(n)
        regions = [events[r].elapsed_time(events[r + 1]) for r in range(repeats)]
    assert take_device_error() == 0, "a kernel reported a timed-out wait"
    tok_s = [c / (ms * 1e-3) for c, ms in zip(committed, regions)]
    e2e_tok_s = [c / s for c, s in zip(committed, host_regions)]
    mid = int(np.argsort(tok_s)[len(tok_s) // 2])
    ms_round = regions[mid] / rounds
    mean_context = wl["prompt"] + (warmup + repeats * rounds / 2.0) * (1 + sum(p_accept ** (i + 1) for i in range(drafts)))
    peak, peak_kind = peaks()
    algo = mtp_round_bytes(cfg, drafts, mean_context)
    achieved = algo / (ms_round * 1e-3) / 1e9
    line = {
        "metric": "batch-1 decode tok/s", "value": tok_s[mid], "unit": "tok/s", "n_gpus": 1, "steps": rounds,
        "warmup": warmup, "ms_per_step": ms_round, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{wl['cfg']} 4-bit MLX-affine g64 + one-layer draft head, batch 1, speculative rounds "
                               f"of {drafts} proposals and a {drafts + 1}-row verify pass over a {wl['prompt']}-row cache, "
                               f"acceptance forced Bernoulli({p_accept}) per proposal (seeded host generator)",
                   "step": "one speculative round",
                   "tokens_per_round": float(np.mean(committed)) / rounds,
                   "l2": "per-round inputs (weights %.2f GB + KV) exceed the 126 MB L2" % (info.weight_bytes / 1e9),
                   "mean_context_rows": mean_context, "prompt_ingest_ms": prefill_ms,
                   "timed_regions": {"repeats": repeats, "rounds_each": rounds, "value_from": "median region",
                                     "tok_s_min": min(tok_s), "tok_s_max": max(tok_s)}},
        "e2e": {"value": float(np.median(e2e_tok_s)), "unit": "tok/s", "h2d_bytes_per_step": 4 + 16 + 4,   # pending token, head state words, position
                "d2h_bytes_per_step": 4 * (2 * (drafts + 1) + 1),   # verify inputs, row picks, error word
                "note": "host clock around the same rounds: pending token and acceptance pattern in, committed tokens out"},
        "gpu_launches": int(round(repeats * rounds * launches_per_round)),
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_kind": peak_kind, "algorithmic_bytes_per_step": algo,
                     "note": "whole round (draft chain, verify pass, commit and head repair) over the round's "
                             "algorithmic bytes: target matrices and KV once, head matrices, read-out table and head KV "
                             "once per proposal"},
    }
    if not args.no_cpu_baseline:
        n = 2 if cfg["layers"] >= 28 else 8
        base = cpu_sample(cfg, weights, prompt, 8, n, host_threads())
        base["sample"] += "; plain one-token steps (the CPU arm has no draft head: one committed token per pass)"
        line["cpu_baseline"] = base
    print(json.dumps(line))
    model.close()


def run_reference(args, wl, cfg) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    from oracle import oracle as O
    weights = S.dense_weights(cfg, seed=args.seed)
    prompt = S.prompt(cfg, wl["prompt"], seed=args.seed + 1)
    # bounded sample: a short prompt, then `warmup` untimed and `steps` timed decode steps
    steps = max(1, min(args.steps, 4 if cfg["layers"] >= 28 else 16))
    warm = min(args.warmup, 1)
    orc = O.DenseOracle(cfg, weights, capacity=8 + warm + steps + 1, threads=threads)
    for t in prompt[:7]:
        orc.ingest(int(t))
    tok = O.argmax_bf16(orc.step(int(prompt[7])))
    for _ in range(warm):
        tok = O.argmax_bf16(orc.step(tok))
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = O.argmax_bf16(orc.step(tok))
    dt = time.perf_counter() - t0
    value = steps / dt
    sample = (f"{steps} greedy decode steps at 8 to {8 + warm + steps} rows of context (CPU oracle port, OpenMP over "
              f"rows, {threads} threads)")
    print(json.dumps({
        "impl": "reference", "metric": "batch-1 decode tok/s", "value": value, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": 1e3 * dt / steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{wl['cfg']} 4-bit MLX-affine g64, batch 1, greedy decode; CPU arm: {sample}"},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qwen3-8b", choices=sorted(WORKLOADS))
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--repeats", type=int, default=0,
                    help="timed regions of --steps tokens each (0: at least 5, enough for 0.3 s of load)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parallel", default="tp", choices=["tp", "replicas"],
                    help="N > 1: shard the one token stream over the GPUs (tensor parallel, strong scaling) or "
                         "run N independent streams (weak scaling)")
    ap.add_argument("--rows", type=int, default=4096, help="matvec workload only")
    ap.add_argument("--columns", type=int, default=4096, help="matvec workload only")
    ap.add_argument("--m", type=int, default=1024, help="gemm workload only: rows of activations")
    ap.add_argument("--drafts", type=int, default=-1, help="speculative workloads only: proposals per round (0..7)")
    ap.add_argument("--accept", type=float, default=-1.0, help="speculative workloads only: acceptance probability")
    ap.add_argument("--format", default="affine4", choices=["affine4", "affine8", "q8_0", "q4_k"],
                    help="matvec workload only")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if wl.get("moe"):
        run_moe(args, wl)
        return
    if args.workload == "matvec":
        run_matvec(args)
        return
    if args.workload == "gemm":
        run_gemm(args)
        return
    cfg = S.CONFIGS[wl["cfg"]]
    if args.impl == "reference":
        run_reference(args, wl, cfg)
        return
    if wl.get("mtp"):
        run_mtp(args, wl)
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    from stark_b200.engine import DenseModel, TensorParallel
    from stark_b200.ops import take_device_error

    tp = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        if args.parallel == "tp":
            host_group = dist.new_group(backend="gloo")  # moves buffer handles and read-out shards, not tokens

            def all_gather(blob: bytes):
                out = [None] * world
                dist.all_gather_object(out, blob, group=host_group)
                return out
            tp = TensorParallel(rank, world, all_gather)

    steps, warmup = args.steps, max(args.warmup, 3)
    # The timed region is `steps` tokens; it is taken `repeats` times back to back (the cache keeps growing)
    # and the median region is the value, so that a 20-step region of 30 ms does not decide the line alone
    # and the clock sampler sees at least 0.3 s of load.
    repeats = args.repeats if args.repeats > 0 else max(5, min(64, -(-320 // max(steps, 1))))
    e2e_steps = min(steps, 256)
    context = max(wl["context"], wl["prompt"] + warmup + repeats * steps + 8, wl["prompt"] + warmup + repeats * e2e_steps + 8)
    weights = S.dense_weights(cfg, seed=args.seed)
    prompt = S.prompt(cfg, wl["prompt"], seed=args.seed + 1)
    model = DenseModel.load(cfg, weights, context_tokens=context, tp=tp)
    info = model.info()
    stream = torch.cuda.ExternalStream(model.stream())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed decode: tokens chained on the device, inputs resident in HBM ------------
    model.prefill(prompt)   # untimed first pass: allocates the chunk buffers, touches every weight
    model.drain()
    model.reset()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    p0.record(stream)
    model.prefill(prompt)
    p1.record(stream)
    model.drain()
    prefill_ms = p0.elapsed_time(p1)
    model.generate_greedy(warmup)
    barrier()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(repeats + 1)]
    with ClockSampler(local) as clocks:
        events[0].record(stream)
        for r in range(repeats):
            model.generate_greedy(steps)
            events[r + 1].record(stream)
        barrier()
        regions = [events[r].elapsed_time(events[r + 1]) for r in range(repeats)]
        assert take_device_error() == 0, "a kernel reported a timed-out wait"
        mean_context = wl["prompt"] + warmup + repeats * steps / 2.0

        # ---- end to end through the public API: host token in, host result out, every step --------
        model.reset()
        model.prefill(prompt)
        tok = model.argmax()
        for _ in range(warmup):
            model.step_async(tok)
            tok = model.argmax()
        barrier()
        e2e_regions = []
        for r in range(repeats):
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                model.step_async(tok)   # 4-byte host->device token copy
                tok = model.argmax()    # 16-byte device->host read of the step result
            torch.cuda.synchronize()
            e2e_regions.append(time.perf_counter() - t0)

    # ---- the second request of the workload: shares a prefix with the first, reuses its KV rows ----
    reuse = None
    if wl["prompt"] >= 2048:
        from stark_b200.engine import reusable_prefix_rows
        shared = wl["prompt"] - 512
        second = np.concatenate([prompt[:shared], S.prompt(cfg, 512, seed=args.seed + 2)])
        model.reset()
        model.prefill(prompt)
        model.drain()
        rows = reusable_prefix_rows(len(prompt), shared, len(second))
        barrier()
        t0 = time.perf_counter()
        model.rewind(rows)
        model.prefill(second[rows:])
        model.drain()
        reuse = {"shared_prefix_tokens": int(shared), "rows_reused": int(rows),
                 "rows_recomputed": int(len(second) - rows), "prefill_ms": 1e3 * (time.perf_counter() - t0)}

    # every region is the max over ranks (a token is done when the slowest rank is); then the median region
    t = torch.tensor(regions + e2e_regions + [prefill_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    regions, e2e_regions, prefill_ms = t[:repeats].tolist(), t[repeats:2 * repeats].tolist(), float(t[-1])
    ms, e2e_s = float(np.median(regions)), float(np.median(e2e_regions))
    streams = 1 if (tp is not None or world == 1) else world  # tensor parallel: all GPUs work on the one token stream
    value = streams * steps / (ms / 1e3)
    e2e_value = streams * e2e_steps / e2e_s

    peak, peak_kind = peaks()
    algo = step_bytes(cfg, mean_context)
    # per GPU: a rank of a tensor-parallel group streams 1/N of the step's bytes (plus the whole
    # embedding row and vectors, which are negligible)
    achieved = algo / (world if tp is not None else 1) / (ms / steps * 1e-3) / 1e9
    line = {
        "metric": "batch-1 decode tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True,
        # one token stream however many GPUs work on it (tensor parallel): strong scaling at every N, N = 1
        # included; independent replicas are the weak-scaling alternative
        "scaling": "weak" if (world > 1 and tp is None) else "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{wl['cfg']} 4-bit MLX-affine g64, batch 1, {wl['prompt']}-token prompt, greedy decode",
                   "parallelism": "tp1" if world == 1 else (f"tp{world}" if tp is not None
                                                            else f"{world} independent replicas"),
                   "l2": "per-step inputs (weights %.2f GB + KV) exceed the 126 MB L2" % (info.weight_bytes / 1e9),
                   "mean_context_rows": mean_context, "prefix_reuse": reuse,
                   "timed_regions": {"repeats": repeats, "steps_each": steps, "value_from": "median region",
                                     "ms_per_step_min": min(regions) / steps, "ms_per_step_max": max(regions) / steps,
                                     "e2e_tok_s_min": streams * e2e_steps / max(e2e_regions),
                                     "e2e_tok_s_max": streams * e2e_steps / min(e2e_regions)},
                   "prompt_ingest_ms": prefill_ms},
        "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 16,
                "steps": e2e_steps},
        "gpu_launches": int(repeats * steps * info.launches_per_step),
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": DRAM_TRAFFIC_RATIO * algo / (world if tp is not None else 1),
                     "traffic_note": "algorithmic bytes x 1.011, the dram read+write / algorithmic ratio of one ncu "
                                     "capture of the dominant matvec kernel (profiles/), scaled to the step",
                     "peak_kind": peak_kind, "frac_of_8tbs": achieved / 8000.0,
                     "algorithmic_bytes_per_step": algo,
                     "note": "whole decode step (all kernels of the token) over the step's algorithmic bytes"
                             + (", per GPU" if world > 1 else "")},
    }
    if tp is None or world == 1 or tp.rows:
        # Prompt ingest (passes of up to 4096 rows through the tcgen05 contraction): a dense contraction, so it is
        # set against the tensor-pipe peak, not the HBM one.  Tensor parallel: a rank contracts 1/N of every matrix
        # and the ranks gather column slices over NVLink; FLOP/s are per GPU.
        tpeak, tkind = tensor_peak()
        share = world if tp is not None else 1
        tflops = prefill_flops(cfg, wl["prompt"]) / share / (prefill_ms * 1e-3) / 1e12
        line["prefill"] = {"prefill_tok_s": wl["prompt"] / (prefill_ms * 1e-3), "ms": prefill_ms,
                           "prompt_tokens": wl["prompt"], "achieved_tflops": tflops, "peak_tflops": tpeak,
                           "frac": tflops / tpeak, "peak_kind": tkind, "bound": "tensor",
                           "note": "device time (CUDA events, max over ranks) of ingesting the prompt, last row included"
                                   + (", FLOP/s per GPU" if share > 1 else "")}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import oracle as O
        n = 2 if cfg["layers"] >= 28 else 8
        line["cpu_baseline"] = cpu_sample(cfg, weights, prompt, 8, n, host_threads())
    if rank == 0:
        print(json.dumps(line))
    model.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
