"""``stark-b200-worker``: the reference's two worker processes over the B200 engine, on the same wire.

    python -m stark_b200.worker --model-path PATH [--prefix-cache]
    python -m stark_b200.worker --score-model-path PATH [--consecutive-cache]

One UTF-8 JSON object per ``\\n``-terminated line on stdin and stdout; the first output line is the readiness
object; every request gets exactly one terminal reply, in order; a fencing error is followed by
``{"ready":false,"error":"native_operation_failed"}`` and exit 1.  What each piece follows:

* command lines          crates/stark-generate/src/protocol.rs:18-53, crates/stark-score/src/protocol.rs:10-26
* output redirection     protocol.rs:55-70 (replies on a duplicate of stdout, the process' own stdout / stderr to /dev/null)
* request budget         crates/stark-resource-budget/src/lib.rs:44-166
* generation requests    crates/stark-generate/src/generation.rs:113-200 (strict fields), :861-887 and :1218-1243
                         (validation order and codes), :452-526 (token loop and finish reasons), :1015-1025 (reply)
* readiness              generation.rs:1529-1575, crates/stark-score/src/scoring.rs:736-751
* prefix reuse           crates/stark-generate/src/prefix_cache.rs:44-99
* cancellation           crates/stark-generate/src/cancel.rs:14-70
* scoring                crates/stark-score/src/scoring.rs:25-40, 274-336, 545-714, cache.rs

The request layer talks to a backend object (``vocab_size``, ``max_context_length``, ``eos_token_ids``,
``tokenize``, ``decode``, ``begin`` / ``next_token``, ``score``), the image of the reference's crate-private
``GenerationBackend`` / ``ScoringBackend`` traits; ``B200Backend`` implements it over ``DenseModel``.  The
``mtp`` / ``mtp_drafts`` / ``mtp_policy`` / ``mtp_lookup`` selectors are resolved as the reference resolves them and
served when the model carries a draft head (``mtp_not_supported`` otherwise); images and chat templates belong to
the reference's product shell and are answered with its own refusals (``images_not_supported``).
"""
from __future__ import annotations

import hashlib
import json
import math
import os
import stat
import struct
import sys
import time
from pathlib import Path

MIB = 1024 * 1024
U32_MAX = (1 << 32) - 1
U64_MAX = (1 << 64) - 1
PREFIX_CHUNK = 1024          # prefix_cache.rs:14
PREFIX_IDLE_SECONDS = 600    # prefix_cache.rs:16
PREFIX_POLICY = "consecutive-prefix-v1"
MAX_EXTRA_STOPS = 256        # generation.rs:21
VERSION = "0.1.0"
FENCING_GENERATION = {"native_generation_failed", "invalid_generation_output", "invalid_tokenization_output",
                      "invalid_image_preparation_output", "decoding_failed", "cancel_channel_failed"}
FENCING_SCORING = {"native_scoring_failed", "invalid_score_values", "mma_score_probe_failed"}


class Refusal(Exception):
    """A request-level error code (the reference's ``&'static str`` errors)."""

    def __init__(self, code: str):
        super().__init__(code)
        self.code = code


# ----------------------------------------------------------------------------------------------- budget

class Budget:
    """stark-resource-budget: the logical input budget B and what derives from it."""

    def __init__(self, mib: int):
        self.mib = mib
        self.input_bytes = mib * MIB
        self.wire_bytes = self.input_bytes * 6 + 2 * MIB

    @staticmethod
    def available_memory_bytes() -> int:
        try:
            for line in Path("/proc/meminfo").read_text().splitlines():
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) * 1024
        except (OSError, ValueError, IndexError):
            pass
        return 0

    @classmethod
    def from_environment(cls) -> "Budget":
        value = os.environ.get("STARK_REQUEST_BUDGET_MIB")
        max_mib = ((1 << 63) - 1 - 32 * MIB) // (32 * MIB)
        if value is None:
            return cls(min(max(cls.available_memory_bytes() // (128 * MIB), 16), max_mib))
        if not value or len(value) > len(str(max_mib)) or not all(c in "0123456789" for c in value):
            raise Refusal("invalid_resource_budget")
        mib = int(value)
        if not 1 <= mib <= max_mib:
            raise Refusal("invalid_resource_budget")
        return cls(mib)


def check_json_structure(data: bytes, budget: Budget) -> None:
    """Bounds container depth, node count and numeric leaves before the request is parsed (lib.rs:104-166)."""
    offset, depth, nodes, numeric, n = 0, 0, 0, 0, len(data)
    separators = b" \n\r\t,:"
    enders = b" \n\r\t,:[]{}\""
    numeric_limit = budget.input_bytes // 4 + 65_536
    while offset < n:
        byte = data[offset]
        offset += 1
        if byte in separators:
            continue
        if byte in b"}]":
            depth = max(depth - 1, 0)
            continue
        if byte in b"{[":
            depth += 1
            if depth > 64:
                raise Refusal("resource_budget_exceeded")
        elif byte == 0x22:
            while offset < n:
                ch = data[offset]
                offset += 1
                if ch == 0x5C:
                    offset += 1
                elif ch == 0x22:
                    break
        else:
            if byte == 0x2D or 0x30 <= byte <= 0x39:
                numeric += 1
                if numeric > numeric_limit:
                    raise Refusal("resource_budget_exceeded")
            else:
                nodes += 1
            while offset < n and data[offset] not in enders:
                offset += 1
            if nodes > 65_536:
                raise Refusal("resource_budget_exceeded")
            continue
        nodes += 1
        if nodes > 65_536:
            raise Refusal("resource_budget_exceeded")


# ----------------------------------------------------------------------------------------------- strict parsing

class _Missing:
    pass


MISSING = _Missing()


def _no_duplicates(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise ValueError("duplicate field")
        out[k] = v
    return out


def parse_json_line(data: bytes):
    try:
        text = data.decode("utf-8")
        return json.loads(text, object_pairs_hook=_no_duplicates, parse_constant=_reject_constant)
    except (ValueError, UnicodeError, RecursionError):
        raise Refusal("invalid_request") from None


def _reject_constant(name):
    raise ValueError(name)   # NaN / Infinity are not JSON


def _uint(v, limit):
    if isinstance(v, bool) or not isinstance(v, int) or v < 0 or v > limit:
        raise Refusal("invalid_request")
    return v


def _boolean(v):
    if not isinstance(v, bool):
        raise Refusal("invalid_request")
    return v


def _string(v):
    if not isinstance(v, str):
        raise Refusal("invalid_request")
    return v


def _number(v):
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise Refusal("invalid_request")
    return float(v)


def _f32(v):
    x = _number(v)
    y = struct.unpack("<f", struct.pack("<f", max(min(x, 3.4028234663852886e38), -3.4028234663852886e38)))[0]
    return y if math.isfinite(x) else x


def _ids(v, limit=U32_MAX):
    if not isinstance(v, list):
        raise Refusal("invalid_request")
    return [_uint(x, limit) for x in v]


def _strings(v):
    if not isinstance(v, list):
        raise Refusal("invalid_request")
    return [_string(x) for x in v]


class Fields:
    """One tagged request object with serde's ``deny_unknown_fields``: every key must be taken."""

    def __init__(self, obj: dict, tag: str):
        if not isinstance(obj, dict):
            raise Refusal("invalid_request")
        self.obj = dict(obj)
        self.obj.pop(tag, None)

    def required(self, name, convert):
        if name not in self.obj:
            raise Refusal("invalid_request")
        return convert(self.obj.pop(name))

    def defaulted(self, name, convert, default):
        """``#[serde(default)]`` on a plain field: absent means the default, null is a type error."""
        if name not in self.obj:
            return default
        return convert(self.obj.pop(name))

    def optional(self, name, convert):
        """``#[serde(default)] Option<T>``: absent or null mean None."""
        v = self.obj.pop(name, None)
        return None if v is None else convert(v)

    def present(self, name, convert):
        """``deserialize_with = present_value``: absent means None, an explicit null is invalid."""
        if name not in self.obj:
            return None
        return convert(self.obj.pop(name))

    def done(self):
        if self.obj:
            raise Refusal("invalid_request")


def parse_sampling(v) -> dict:
    if not isinstance(v, dict) or not isinstance(v.get("mode"), str):
        raise Refusal("invalid_request")
    f = Fields(v, "mode")
    if v["mode"] == "greedy":
        f.done()
        return {"mode": "greedy"}
    if v["mode"] == "stochastic":
        out = {"mode": "stochastic", "temperature": f.required("temperature", _f32),
               "top_k": f.optional("top_k", lambda x: _uint(x, U32_MAX)), "top_p": f.optional("top_p", _f32),
               "min_p": f.optional("min_p", _f32)}
        f.done()
        return out
    raise Refusal("invalid_request")


def validate_sampling(s: dict, vocab: int) -> None:
    """generation.rs:67-111."""
    if s["mode"] != "stochastic":
        return
    t, k, p, m = s["temperature"], s["top_k"], s["top_p"], s["min_p"]
    bad = (not math.isfinite(t) or t <= 0.0 or not math.isfinite(1.0 / t) or t > 100.0
           or (k is not None and (k == 0 or k > vocab))
           or (p is not None and (not math.isfinite(p) or p <= 0.0 or p > 1.0))
           or (m is not None and (not math.isfinite(m) or not 0.0 <= m <= 1.0)))
    if bad:
        raise Refusal("invalid_sampling_request")


# ----------------------------------------------------------------------------------------------- process plumbing

def protocol_output():
    """Replies go to a duplicate of stdout; the process' own stdout and stderr are pointed at /dev/null so that no
    diagnostic of a native library can enter the protocol stream."""
    import fcntl
    null = os.open("/dev/null", os.O_WRONLY)
    fd = fcntl.fcntl(1, fcntl.F_DUPFD_CLOEXEC, 3)
    os.dup2(null, 1)
    os.dup2(null, 2)
    return os.fdopen(fd, "wb", buffering=0)


def write_reply(out, value) -> None:
    try:
        out.write(json.dumps(value, separators=(",", ":"), allow_nan=False).encode("utf-8") + b"\n")
        out.flush()
    except (OSError, ValueError):
        raise Refusal("protocol_write_failed") from None


class CancelSignal:
    """Request-scoped cancellation over an inherited FIFO: 8-byte little-endian request ids (cancel.rs)."""

    def __init__(self, fd: int):
        self.fd, self.pending = fd, b""

    @classmethod
    def from_environment(cls):
        value = os.environ.pop("STARK_CANCEL_FD", None)
        if value is None:
            return None
        import fcntl
        try:
            fd = int(value)
            if fd < 3 or not stat.S_ISFIFO(os.fstat(fd).st_mode):
                raise ValueError
            fcntl.fcntl(fd, fcntl.F_SETFL, fcntl.fcntl(fd, fcntl.F_GETFL) | os.O_NONBLOCK)
            fcntl.fcntl(fd, fcntl.F_SETFD, fcntl.FD_CLOEXEC)
        except (ValueError, OSError):
            raise Refusal("invalid_cancel_channel") from None
        return cls(fd)

    def check(self, request_id: int) -> bool:
        cancelled = False
        while True:
            try:
                chunk = os.read(self.fd, 256)
            except BlockingIOError:
                return cancelled
            except InterruptedError:
                continue
            except OSError:
                raise Refusal("cancel_channel_failed") from None
            if not chunk:
                return True   # the owning client vanished
            self.pending += chunk
            while len(self.pending) >= 8:
                cancelled |= struct.unpack("<Q", self.pending[:8])[0] == request_id
                self.pending = self.pending[8:]


def read_frame(stream, wire_bytes: int):
    """One line of at most wire_bytes bytes; returns (bytes, oversize).  An oversize frame is drained to its
    newline so that the next request stays independent (generation.rs:1627-1646)."""
    data = stream.readline(wire_bytes + 1)
    if not data:
        return None, False
    if len(data) > wire_bytes:
        while not data.endswith(b"\n"):
            data = stream.readline(1 << 20)
            if not data:
                break
        return b"", True
    return data, False


# ----------------------------------------------------------------------------------------------- backend

class B200Backend:
    """The engine behind both workers: a converted-model directory (``config.json`` + ``model.safetensors`` in the
    reference's layout, optional ``tokenizer.json``) on one B200."""

    def __init__(self, path: Path, context_tokens: int | None = None):
        config = path / "config.json"
        if not config.is_file():
            raise Refusal("model_config_unavailable")
        try:
            root = json.loads(config.read_text())
        except (OSError, ValueError):
            raise Refusal("invalid_model_config") from None
        from .artifact import ArtifactError, read_artifact
        from .engine import DenseModel
        try:
            cfg, weights = read_artifact(path)
        except (ArtifactError, KeyError, TypeError, OSError, ValueError):
            raise Refusal("invalid_model_config") from None
        try:
            layer0 = root["decoder_config"]["transformer_config"]["layer_configs"][0]
            model_max = int(layer0["rope_config"].get("max_sequence_length") or 32768)
        except (KeyError, IndexError, TypeError, ValueError):
            model_max = 32768
        want = context_tokens or int(os.environ.get("STARK_B200_WORKER_CONTEXT", "8192"))
        self.capacity = max(2, min(model_max, want))
        generation = root.get("generation_config") or {}
        self.eos = [int(t) for t in generation.get("stop_token_ids", []) if 0 <= int(t) < cfg["vocab"]]
        self.cfg = cfg
        self.tokenizer = None
        if (path / "tokenizer.json").is_file():
            try:
                from tokenizers import Tokenizer
                self.tokenizer = Tokenizer.from_file(str(path / "tokenizer.json"))
            except Exception:  # noqa: BLE001 - a tokenizer that does not load is a model that does not load
                raise Refusal("tokenizer_unavailable") from None
        try:
            self.model = DenseModel.load(cfg, weights, context_tokens=self.capacity)
        except Exception:  # noqa: BLE001
            raise Refusal("model_load_failed") from None
        self.has_head = bool(cfg.get("mtp"))
        self.rounds = None   # speculative state of the request in flight
        self._newline = None
        self.key = hashlib.sha256((path / "model.safetensors").stat().st_size.to_bytes(8, "little")
                                  + config.read_bytes()).hexdigest()
        self.position_tokens: list[int] = []   # tokens whose rows the cache currently holds

    # -- identity
    def vocab_size(self) -> int:
        return self.cfg["vocab"]

    def max_context_length(self) -> int:
        return self.capacity

    def eos_token_ids(self) -> list[int]:
        return self.eos

    # -- speculative decoding (GenerationBackend::mtp_capabilities and friends, generation.rs:585-615)
    def mtp_capabilities(self):
        if not self.has_head:
            return None
        return {"max_drafts": 4, "recommended_drafts": 2, "sampling": "exact-rejection-v1",
                "verification": "dense-target-verify-rows-v1"}

    def supports_mtp_scheduling(self) -> bool:
        return self.has_head

    def plan_context_length(self, input_tokens: int, maximum: int, drafts: int):
        """The largest context up to `maximum` this engine can serve now.  The paged cache is allocated when the model
        loads (`capacity` rows: 147 KB each for the 8B shape), so a context costs nothing further; what a request may
        still allocate are the working buffers of a prompt pass (4 096 rows of every intermediate) and, with
        proposals, the rows of the verify pass.  They have to fit the device memory that is free, with a reserve."""
        import ctypes as C
        from . import _lib
        c = self.cfg
        rows = 4096
        qkv = (c["q_heads"] + 2 * c["kv_heads"]) * c["head_dim"]
        scratch = rows * 2 * (2 * c["hidden"] + qkv + c["q_heads"] * c["head_dim"] + c["inter"])
        if drafts:
            scratch += 16 * 2 * (c["vocab"] + 4 * c["hidden"])
        free, total = C.c_uint64(0), C.c_uint64(0)
        try:
            _lib.check(_lib.load().stark_b200_device_memory(C.byref(free), C.byref(total)), "device_memory")
        except Exception:  # noqa: BLE001
            return None
        reserve = 512 << 20
        if getattr(self, "_scratch_ready", False):
            scratch = 0
        if free.value < scratch + reserve:
            return None
        return min(maximum, self.capacity)

    def prefix_cache_supported(self) -> bool:
        return not self.has_head    # the head's cache cannot be cut inside a prompt

    def effective_mtp_drafts(self, drafts: int, sampling: dict) -> int:
        """Greedy requests are accepted on the device (arg-max compare); stochastic ones go through the exact
        rejection sampler on the host, with the head's greedy proposals as point masses."""
        return drafts

    def newline_tokens(self):
        from .mtp_schedule import NewlineTokens
        if self._newline is None:
            tk = self.tokenizer
            self._newline = NewlineTokens(self.cfg["vocab"] if tk is not None else 0,
                                          (lambda i: "\n" in tk.decode([i], skip_special_tokens=False)) if tk is not None
                                          else (lambda i: False))
        return self._newline

    # -- text
    def tokenize(self, text: str, add_special_tokens: bool) -> list[int]:
        if self.tokenizer is None:
            raise Refusal("tokenizer_unavailable")
        try:
            return [int(t) for t in self.tokenizer.encode(text, add_special_tokens=add_special_tokens).ids]
        except Exception:  # noqa: BLE001
            raise Refusal("tokenization_failed") from None

    def decode(self, ids: list[int], skip_special_tokens: bool) -> str:
        if self.tokenizer is None:
            return ""   # token-id service: the reply's text stays empty
        try:
            return self.tokenizer.decode(ids, skip_special_tokens=skip_special_tokens)
        except Exception:  # noqa: BLE001
            raise Refusal("decoding_failed") from None

    # -- generation
    def begin(self, input_ids: list[int], reuse_rows: int, sampling: dict, seed: int, mtp: dict | None = None,
              budget_tokens: int = 0) -> None:
        """Brings the cache to the end of the prompt (reusing `reuse_rows` rows it already holds) with the
        prompt's last row read out; `next_token` then samples.  mtp = {"drafts", "adaptive", "lookup"}: tokens
        come from speculative rounds planned by a RoundScheduler (greedy acceptance)."""
        from ._lib import StarkB200Error
        import numpy as np
        self.rounds = None
        try:
            if reuse_rows and self.position_tokens[:reuse_rows] == input_ids[:reuse_rows]:
                self.model.rewind(reuse_rows)
            else:
                reuse_rows = 0
                self.model.reset()
            self.position_tokens = list(input_ids[:reuse_rows])
            self.model.prefill(np.asarray(input_ids[reuse_rows:], np.uint32))
            self._scratch_ready = True    # the prompt pass has its working buffers now
            self.position_tokens = list(input_ids)
        except StarkB200Error:
            self.position_tokens = []
            raise Refusal("native_generation_failed") from None
        self.sampling, self.seed, self.sampled = sampling, seed, 0
        if mtp and mtp["drafts"] > 0:
            from .mtp_schedule import B200_QWEN3_8B_V1, PromptLookup, RoundScheduler
            lookup = PromptLookup(input_ids, self.newline_tokens()) if mtp["lookup"] else None
            sampler = None
            try:
                if sampling["mode"] == "greedy":
                    first = self.model.mtp_initial()
                else:
                    # hybrid/mtp.rs: the request's seed drives the target stream, proposals have their own
                    from .mtp_sampler import ExactMtpSampler, SamplerError
                    sampler = ExactMtpSampler(sampling, seed, dense_filters=True)
                    try:
                        first = sampler.sample_initial(self.model.logits())
                    except SamplerError:
                        raise Refusal("native_generation_failed") from None
            except StarkB200Error:
                self.position_tokens = []
                raise Refusal("native_generation_failed") from None
            self.rounds = dict(scheduler=RoundScheduler(mtp["adaptive"], B200_QWEN3_8B_V1.greedy, mtp["drafts"], lookup,
                                                        B200_QWEN3_8B_V1.id),
                               queue=[first], pending=first, sampler=sampler, budget=budget_tokens, handed=0, count=0, proposed=0,
                               accepted=0, by_accepted=[0] * (mtp["drafts"] + 1), verified_rows=0, seconds=0.0)

    def _round(self) -> None:
        """One speculative round: the pending token and the accepted proposals enter the cache, the accepted
        proposals and the next pending token join the queue."""
        import time as _time
        r = self.rounds
        cap = max(0, min(r["scheduler"].planner.limit, r["budget"] - r["handed"] - 1))
        plan = r["scheduler"].plan(cap)
        t0 = _time.perf_counter()
        held = r["sampler"] is not None
        if plan[0] == "lookup":
            out = self.model.mtp_round_lookup(r["pending"], plan[1], held=held)
        else:
            out = self.model.mtp_round(r["pending"], plan[1], held=held)
        if held:
            out = self._decide(out)
        seconds = _time.perf_counter() - t0
        r["scheduler"].observe(plan, out["accepted"], out["tokens"], seconds)
        if plan[0] == "lookup" or plan[1] == 0:
            r["scheduler"].record_head_advance(0.0)
        r["count"] += 1
        r["proposed"] += out["proposed"]
        r["accepted"] += out["accepted"]
        r["by_accepted"][out["accepted"]] += 1
        r["verified_rows"] += out["proposed"] + 1
        r["seconds"] += seconds
        self.position_tokens.extend(out["tokens"])
        r["queue"] = out["tokens"][1:] + [out["next_pending"]]
        r["pending"] = out["next_pending"]

    def _decide(self, out: dict) -> dict:
        """Acceptance by the exact rejection sampler over the rows of a held round: the proposals (the head's
        arg-max picks, or tokens copied from the context) are point masses, so a proposal is kept with probability
        p(token) and a rejection draws from p without it (hybrid/mtp.rs:193-262)."""
        from .mtp_sampler import SamplerError
        sampler = self.rounds["sampler"]
        proposals = out["tokens"][1:]
        try:
            sampler.begin_round()
            for token in proposals:
                sampler.draft_point_mass(token)
            accepted, drawn = 0, None
            for row in range(len(proposals) + 1):
                proposal = proposals[row] if row < len(proposals) else None
                drawn = sampler.target(self.model.mtp_row_logits(row), proposal)
                if proposal is None or drawn != proposal or sampler.phase == sampler.FINISHED:
                    break
                accepted += 1
        except SamplerError:
            self.position_tokens = []
            raise Refusal("native_generation_failed") from None
        return self.model.mtp_commit(accepted, drawn)

    def mtp_metadata(self):
        r = self.rounds
        if r is None:
            return None
        return {"rounds": r["count"], "proposed": r["proposed"], "accepted": r["accepted"],
                "rounds_by_accepted_drafts": r["by_accepted"], "verified_rows": r["verified_rows"],
                "round_seconds": r["seconds"], "schedule": r["scheduler"].stats.as_json()}

    def next_token(self) -> int:
        """Samples from the logits of the last row and feeds the sample back (one decode step)."""
        from ._lib import StarkB200Error
        from .engine import position_seed
        if self.rounds is not None:
            try:
                if not self.rounds["queue"]:
                    self._round()
                self.rounds["handed"] += 1
                return self.rounds["queue"].pop(0)
            except StarkB200Error:
                self.position_tokens = []
                raise Refusal("native_generation_failed") from None
        try:
            if self.sampling["mode"] == "greedy":
                token = self.model.argmax()
            else:
                s = self.sampling
                token = self.model.sample(seed=position_seed(self.seed, len(self.position_tokens)),
                                          temperature=s["temperature"], top_k=s["top_k"], top_p=s["top_p"],
                                          min_p=s["min_p"])
            self._pending = token
            return token
        except StarkB200Error:
            self.position_tokens = []
            raise Refusal("native_generation_failed") from None

    def advance(self, token: int) -> None:
        """Feeds an accepted sample so that the next `next_token` sees its row (skipped after the last sample)."""
        from ._lib import StarkB200Error
        if self.rounds is not None:
            return   # a round feeds its own tokens
        try:
            self.model.step_async(int(token))
            self.position_tokens.append(int(token))
        except StarkB200Error:
            self.position_tokens = []
            raise Refusal("native_generation_failed") from None

    def fenced(self) -> bool:
        try:
            return bool(self.model.info().fenced)
        except Exception:  # noqa: BLE001
            return True

    def forget(self) -> None:
        self.position_tokens = []

    # -- scoring
    def score(self, input_ids: list[int]):
        """Full-vocabulary f32 logits of the next token after `input_ids`, on a fresh state."""
        from ._lib import StarkB200Error
        import numpy as np
        try:
            t0 = time.perf_counter()
            self.model.reset()
            t1 = time.perf_counter()
            self.model.prefill(np.asarray(input_ids, np.uint32))
            self.model.drain()
            t2 = time.perf_counter()
            logits = self.model.logits()
            t3 = time.perf_counter()
        except StarkB200Error:
            raise Refusal("native_scoring_failed") from None
        return logits, (t1 - t0, t2 - t1, t3 - t2)


# ----------------------------------------------------------------------------------------------- generation worker

def reusable_prefill_rows(prompt_tokens: int, chunk: int = PREFIX_CHUNK) -> int:
    return max(prompt_tokens - 1, 0) // chunk * chunk


def parse_scope(scope: str):
    """32 lowercase hex digits (prefix_cache.rs: parse_scope)."""
    if len(scope) != 32 or any(c not in "0123456789abcdef" for c in scope):
        return None
    return bytes.fromhex(scope)


class GenerationWorker:
    def __init__(self, backend, budget: Budget, prefix_cache: bool, cancel=None, clock=time.monotonic):
        self.backend, self.budget, self.prefix_cache, self.cancel, self.clock = backend, budget, prefix_cache, cancel, clock
        self.retained = None      # (scope, context_tokens, prefix tokens) of the last published request
        self.pending_entry = None
        self.retained_at = 0.0

    # -- readiness
    def readiness(self) -> dict:
        b = self.backend
        max_context = b.max_context_length()
        ready = {"ready": True, "engine": "stark", "version": VERSION, "mode": "text-generation-v1",
                 "operations": ["tokenize", "decode", "generate"], "state_policy": "fresh-per-request",
                 "vocab_size": b.vocab_size(), "max_context_tokens": max_context,
                 "max_new_tokens": min(max(max_context - 1, 0), min(self.budget.input_bytes // 4, U32_MAX)),
                 "max_request_bytes": self.budget.wire_bytes, "request_budget_bytes": self.budget.input_bytes,
                 "eos_token_ids": b.eos_token_ids(), "sampling_modes": ["greedy", "stochastic"],
                 "streaming": "text-delta-v1", "generation_progress": "token-counts-v1", "stop_sequences": True,
                 "cancellation": "pipe-v1"}
        ready["prefix_cache"] = {"supported": True, "enabled": self.prefix_cache, "chunk_tokens": PREFIX_CHUNK,
                                 "idle_seconds": PREFIX_IDLE_SECONDS, "key": getattr(b, "key", "")}
        if self.prefix_cache:
            ready["state_policy"] = PREFIX_POLICY
            ready["operations"] = ["tokenize", "decode", "generate", "reset_cache"]
        caps = self.mtp_capabilities()
        if caps is None:
            ready["mtp"] = {"supported": False, "max_drafts": 0, "recommended_drafts": 0, "default_drafts": 0,
                            "operations": []}
        else:   # generation.rs:1562-1575
            ready["mtp"] = {"supported": True, "max_drafts": caps["max_drafts"],
                            "recommended_drafts": caps["recommended_drafts"], "default_drafts": 0,
                            "sampling": caps["sampling"], "verification": caps["verification"], "operations": ["generate"]}
            if self.backend.supports_mtp_scheduling():
                ready["mtp"].update(policies=["fixed", "adaptive"], default_policy="fixed", default_lookup=False, lookup=True)
        return ready

    def mtp_capabilities(self):
        fn = getattr(self.backend, "mtp_capabilities", None)
        return fn() if fn is not None else None

    def resolve_mtp(self, enabled, drafts) -> int:
        """generation.rs:788-821: `mtp` and `mtp_drafts` exclude each other; `mtp: true` takes the recommended count."""
        if enabled is not None and drafts is not None:
            raise Refusal("invalid_generation_request")
        caps = self.mtp_capabilities()
        if enabled is True:
            if caps is None:
                raise Refusal("mtp_not_supported")
            drafts = caps["recommended_drafts"]
        elif enabled is False or drafts is None:
            drafts = 0
        if drafts > 0:
            if caps is None:
                raise Refusal("mtp_not_supported")
            if drafts > caps["max_drafts"]:
                raise Refusal("invalid_generation_request")
        return drafts

    def resolve_mtp_scheduling(self, policy, lookup, explicit_drafts: bool, drafts: int):
        """generation.rs:823-860.  Returns (adaptive, lookup, drafts)."""
        if policy is not None and policy not in ("fixed", "adaptive"):
            raise Refusal("invalid_generation_request")
        adaptive = policy == "adaptive"
        lookup = bool(lookup) if lookup is not None else False
        if not adaptive and not lookup:
            return False, False, drafts
        if drafts == 0:
            raise Refusal("invalid_generation_request")
        supports = getattr(self.backend, "supports_mtp_scheduling", None)
        if supports is None or not supports():
            raise Refusal("mtp_not_supported")
        if adaptive and not explicit_drafts:
            drafts = self.mtp_capabilities()["max_drafts"]
        return adaptive, lookup, drafts

    # -- prefix policy
    def clear_prefix(self) -> None:
        self.retained, self.pending_entry = None, None
        self.backend.forget()

    def plan_reuse(self, input_ids, context_tokens, scope) -> int:
        if not self.prefix_cache or self.retained is None or scope is None:
            return 0
        if self.clock() - self.retained_at > PREFIX_IDLE_SECONDS:
            self.clear_prefix()
            return 0
        r_scope, r_context, prefix = self.retained
        if scope != r_scope or context_tokens != r_context:
            return 0
        common = 0
        for a, b in zip(prefix, input_ids):
            if a != b:
                break
            common += 1
        return min(common, reusable_prefill_rows(len(input_ids))) // PREFIX_CHUNK * PREFIX_CHUNK

    # -- requests
    def handle(self, obj, out):
        if not isinstance(obj, dict) or not isinstance(obj.get("operation"), str):
            raise Refusal("invalid_request")
        op = obj["operation"]
        f = Fields(obj, "operation")
        b = self.backend
        if op == "tokenize":
            text = f.required("text", _string)
            special = f.defaulted("add_special_tokens", _boolean, False)
            f.done()
            if len(text.encode("utf-8")) > self.budget.input_bytes:
                raise Refusal("resource_budget_exceeded")
            ids = b.tokenize(text, special)
            if any(t >= b.vocab_size() for t in ids):
                raise Refusal("invalid_tokenization_output")
            return {"token_ids": ids, "token_count": len(ids)}
        if op == "decode":
            ids = f.required("token_ids", _ids)
            skip = f.defaulted("skip_special_tokens", _boolean, False)
            f.done()
            if len(ids) > self.budget.input_bytes // 4:
                raise Refusal("resource_budget_exceeded")
            if any(t >= b.vocab_size() for t in ids):
                raise Refusal("invalid_decoding_request")
            text = b.decode(ids, skip)
            if len(text.encode("utf-8")) > self.budget.input_bytes:
                raise Refusal("resource_budget_exceeded")
            return {"text": text, "token_count": len(ids)}
        if op == "reset_cache":
            f.done()
            if not self.prefix_cache:
                raise Refusal("invalid_request")
            self.clear_prefix()
            return {"cache_reset": True}
        if op == "generate":
            return self.generate(f, out)
        if op == "plan_generation":
            plan = {name: f.required(name, lambda x: _uint(x, U32_MAX)) for name in ("input_tokens", "context_tokens")}
            plan["input_token_ids"] = f.present("input_token_ids", _ids)
            plan["cache_scope"] = f.present("cache_scope", _string)
            plan["mtp"] = f.present("mtp", _boolean)
            plan["mtp_drafts"] = f.present("mtp_drafts", lambda x: _uint(x, U32_MAX))
            sampling = f.defaulted("sampling", parse_sampling, {"mode": "greedy"})
            f.done()
            return self.plan_generation(plan, sampling)
        if op in ("prepare_image", "generate_image", "discard_image"):
            raise Refusal("images_not_supported" if op != "discard_image" else "invalid_request")
        raise Refusal("invalid_request")

    def plan_generation(self, obj: dict, sampling: dict):
        """generation.rs:1114-1182: the largest context the loaded model can serve for this input within the
        memory that is left.  The fields were type-checked by the caller."""
        b = self.backend
        planner = getattr(b, "plan_context_length", None)
        if planner is None:
            raise Refusal("context_planning_unavailable")
        input_tokens, context_tokens = obj["input_tokens"], obj["context_tokens"]
        token_limit = min(self.budget.input_bytes // 4, U32_MAX)
        maximum = min(input_tokens + token_limit, context_tokens, b.max_context_length())
        if input_tokens == 0 or input_tokens > token_limit or maximum <= input_tokens:
            raise Refusal("invalid_generation_request")
        ids = obj.get("input_token_ids")
        if ids is not None and (len(ids) != input_tokens or any(t >= b.vocab_size() for t in ids)):
            raise Refusal("invalid_generation_request")
        drafts = self.resolve_mtp(obj.get("mtp"), obj.get("mtp_drafts"))
        scope_text = obj.get("cache_scope")
        if scope_text is not None and (not self.prefix_cache or parse_scope(scope_text) is None):
            raise Refusal("invalid_generation_request")
        validate_sampling(sampling, b.vocab_size())
        if drafts:
            effective = b.effective_mtp_drafts(drafts, sampling)
            if effective > drafts or (effective != 0 and effective != drafts):
                raise Refusal("invalid_generation_output")
            drafts = effective
        capacity = planner(input_tokens, maximum, drafts)
        if capacity is None or capacity <= input_tokens or capacity > maximum:
            raise Refusal("resource_budget_exceeded")
        return {"context_tokens": capacity, "max_new_tokens": capacity - input_tokens,
                "context_capacity_known": True, "budget_kind": "memory"}

    def generate(self, f: Fields, out):
        b = self.backend
        rendered = f.optional("rendered_prompt", _string)
        input_ids = f.optional("input_token_ids", _ids)
        context_tokens = f.required("context_tokens", lambda x: _uint(x, U32_MAX))
        max_new = f.required("max_new_tokens", lambda x: _uint(x, U32_MAX))
        seed = f.defaulted("seed", lambda x: _uint(x, U64_MAX), 0)
        sampling = f.defaulted("sampling", parse_sampling, {"mode": "greedy"})
        mtp = f.present("mtp", _boolean)
        mtp_drafts = f.present("mtp_drafts", lambda x: _uint(x, U32_MAX))
        mtp_policy = f.present("mtp_policy", _string)
        mtp_lookup = f.present("mtp_lookup", _boolean)
        stop_ids = f.defaulted("stop_token_ids", _ids, [])
        stream = f.defaulted("stream", _boolean, False)
        stop = f.defaulted("stop", _strings, [])
        request_id = f.defaulted("request_id", lambda x: _uint(x, U64_MAX), 0)
        scope_text = f.present("cache_scope", _string)
        f.done()
        # generation.rs:1199-1243: cache scope, MTP selectors, options, then the input
        scope = None
        if scope_text is not None:
            scope = parse_scope(scope_text) if self.prefix_cache else None
            if scope is None:
                raise Refusal("invalid_generation_request")
        drafts = self.resolve_mtp(mtp, mtp_drafts)
        adaptive, lookup, drafts = self.resolve_mtp_scheduling(mtp_policy, mtp_lookup, mtp_drafts is not None, drafts)
        vocab = b.vocab_size()
        if (context_tokens == 0 or max_new == 0 or len(stop_ids) > MAX_EXTRA_STOPS or len(stop) > 4
                or any(not s or len(s) > 1024 for s in stop) or any(t >= vocab for t in stop_ids)
                or len(set(stop_ids)) != len(stop_ids)):
            raise Refusal("invalid_generation_request")
        if max_new > self.budget.input_bytes // 4:
            raise Refusal("resource_budget_exceeded")
        if context_tokens > b.max_context_length():
            raise Refusal("context_overflow")
        validate_sampling(sampling, vocab)
        if rendered is not None and input_ids is None:
            if len(rendered.encode("utf-8")) > self.budget.input_bytes:
                raise Refusal("resource_budget_exceeded")
            ids = b.tokenize(rendered, False)
        elif rendered is None and input_ids is not None:
            if len(input_ids) > self.budget.input_bytes // 4:
                raise Refusal("resource_budget_exceeded")
            ids = input_ids
        else:
            raise Refusal("invalid_generation_request")
        if not ids or any(t >= vocab for t in ids):
            raise Refusal("invalid_generation_request")
        if len(ids) >= context_tokens or len(ids) + max_new > context_tokens:
            raise Refusal("context_overflow")
        return self.complete(ids, dict(context_tokens=context_tokens, max_new_tokens=max_new, seed=seed,
                                       sampling=sampling, stop_ids=stop_ids, stop=stop, request_id=request_id,
                                       scope=scope, mtp_drafts=drafts, mtp_adaptive=adaptive, mtp_lookup=lookup),
                             stream, out)

    def cancelled(self, request_id: int) -> bool:
        return self.cancel.check(request_id) if self.cancel is not None else False

    def complete(self, ids, o, stream, out):
        """generate_completion + collect_tokens (generation.rs:889-1060, 452-526)."""
        b = self.backend
        started = time.perf_counter()
        input_tokens = len(ids)
        budget_tokens = min(o["context_tokens"] - input_tokens, o["max_new_tokens"])
        reused = self.plan_reuse(ids, o["context_tokens"], o["scope"])
        if reused >= input_tokens or reused % PREFIX_CHUNK:
            raise Refusal("invalid_generation_output")

        def progress(sampled, elapsed, prefill):
            frame = {"event": "progress", "input_tokens": input_tokens, "sampled_tokens": sampled,
                     "output_token_budget": budget_tokens, "elapsed_seconds": elapsed, "prefill_seconds": prefill}
            if self.prefix_cache:
                frame["reused_input_tokens"] = reused
            return frame
        if stream:
            write_reply(out, progress(0, 0.0, None))
        if self.cancelled(o["request_id"]):
            raise Refusal("generation_cancelled")
        self.pending_entry = None
        requested_drafts = o.get("mtp_drafts", 0)
        effective_drafts = requested_drafts
        if requested_drafts:
            effective_drafts = b.effective_mtp_drafts(requested_drafts, o["sampling"])
            if effective_drafts > requested_drafts or (effective_drafts != 0 and effective_drafts != requested_drafts):
                raise Refusal("invalid_generation_output")
        if effective_drafts:
            b.begin(ids, reused, o["sampling"], o["seed"],
                    mtp={"drafts": effective_drafts, "adaptive": o["mtp_adaptive"], "lookup": o["mtp_lookup"]},
                    budget_tokens=budget_tokens)
        else:
            b.begin(ids, reused, o["sampling"], o["seed"])
        generated, sampled, emitted = [], 0, ""
        finish = "context" if o["context_tokens"] - input_tokens < o["max_new_tokens"] else "length"
        stop_token, first_sample, last_sample, text_so_far = None, None, None, ""
        holdback = max((len(s) for s in o["stop"]), default=1) - 1
        eos = set(b.eos_token_ids())
        for i in range(budget_tokens):
            if self.cancelled(o["request_id"]):
                raise Refusal("generation_cancelled")
            if i:
                b.advance(generated[-1])
            token = b.next_token()
            if self.cancelled(o["request_id"]):
                raise Refusal("generation_cancelled")
            now = time.perf_counter() - started
            if not isinstance(token, int) or token < 0 or token >= b.vocab_size():
                raise Refusal("invalid_generation_output")
            first_sample = now if first_sample is None else first_sample
            last_sample = now
            sampled += 1
            if stream:
                write_reply(out, progress(sampled, now, first_sample))
            if token in eos:
                finish, stop_token = "eos", token
                break
            if token in o["stop_ids"]:
                finish, stop_token = "stop_token", token
                break
            generated.append(token)
            if o["stop"] or stream:
                text_so_far = b.decode(generated, False)
                cut = min((text_so_far.find(s) for s in o["stop"] if s in text_so_far), default=-1)
                if cut >= 0:
                    text_so_far = text_so_far[:cut]
                    finish = "stop_sequence"
                visible = text_so_far if cut >= 0 else text_so_far[:max(len(text_so_far) - holdback, len(emitted))]
                if stream and visible.startswith(emitted) and len(visible) > len(emitted):
                    write_reply(out, {"event": "delta", "text": visible[len(emitted):]})
                    emitted = visible
                if cut >= 0:
                    break
        if b.fenced():
            raise Refusal("native_generation_failed")
        text = text_so_far if finish == "stop_sequence" else b.decode(generated, False)
        if len(text.encode("utf-8")) + 4 * len(generated) > self.budget.input_bytes:
            raise Refusal("resource_budget_exceeded")
        if stream:
            if not text.startswith(emitted):
                raise Refusal("decoding_failed")
            if len(text) > len(emitted):
                write_reply(out, {"event": "delta", "text": text[len(emitted):]})
        if sampled > o["max_new_tokens"] or input_tokens + sampled > o["context_tokens"] \
                or sampled != len(generated) + (stop_token is not None):
            raise Refusal("invalid_generation_output")
        prefill_seconds = first_sample
        decode_seconds = (last_sample - first_sample) if sampled > 1 else None

        def rate(tokens, seconds):
            if seconds is None or not seconds > 0.0 or not math.isfinite(seconds) or tokens <= 0:
                return None
            return tokens / seconds
        reply = {"generated_token_ids": generated, "text": text, "input_tokens": input_tokens,
                 "output_tokens": len(generated), "sampled_tokens": sampled, "finish_reason": finish,
                 "stop_token_id": stop_token, "generation_seconds": time.perf_counter() - started,
                 "prefill_seconds": prefill_seconds, "decode_seconds": decode_seconds,
                 "input_tokens_per_second": rate(input_tokens - reused, prefill_seconds),
                 "output_tokens_per_second": rate(max(sampled - 1, 0), decode_seconds),
                 "timing_method": "first-token-wall-clock-v1"}
        caps = self.mtp_capabilities()
        if caps is not None:   # generation.rs:1029-1063
            meta_fn = getattr(b, "mtp_metadata", None)
            metadata = (meta_fn() if meta_fn is not None else None) or {}
            metadata.update(enabled=effective_drafts > 0, drafts=effective_drafts, sampling=caps["sampling"],
                            verification=caps["verification"])
            if o.get("mtp_adaptive") or o.get("mtp_lookup"):
                metadata.update(policy="adaptive" if o["mtp_adaptive"] else "fixed", lookup=bool(o["mtp_lookup"]))
            if effective_drafts != requested_drafts:
                metadata.update(requested_drafts=requested_drafts, fallback_reason="unsupported_sampling")
            reply["mtp"] = metadata
        if self.prefix_cache:
            reply["reused_input_tokens"] = reused
            if o["scope"] is not None:
                self.pending_entry = (o["scope"], o["context_tokens"], list(ids[:reusable_prefill_rows(len(ids))]))
        return reply

    def process_line(self, data: bytes, out) -> None:
        generate = False
        try:
            check_json_structure(data, self.budget)
            obj = parse_json_line(data)
            op = obj.get("operation") if isinstance(obj, dict) else None
            if op not in ("tokenize", "decode", "generate", "plan_generation"):
                self.clear_prefix()
            generate = op == "generate"
            value = self.handle(obj, out)
        except Refusal as e:
            self.clear_prefix()
            if e.code == "protocol_write_failed":
                raise
            write_reply(out, {"error": e.code})
            if e.code in FENCING_GENERATION:
                raise Refusal("native_operation_failed") from None
            return
        try:
            write_reply(out, value)
        except Refusal:
            self.clear_prefix()
            raise
        if generate and self.pending_entry is not None:
            # publish only state whose terminal reply reached the host
            self.retained, self.retained_at, self.pending_entry = self.pending_entry, self.clock(), None
        elif generate:
            self.retained = None


# ----------------------------------------------------------------------------------------------- scoring worker

def token_hash(ids) -> str:
    h = hashlib.sha256()
    for t in ids:
        h.update(struct.pack("<I", t))
    return h.hexdigest()


def candidate_readout(vocabulary_logits, candidates, temperature):
    """scoring.rs:299-336: log-probabilities against the whole vocabulary in f64; candidate probabilities from the
    raw candidate logits at the given temperature."""
    import numpy as np
    logits32 = np.asarray(vocabulary_logits, np.float32)
    if logits32.size == 0 or not np.isfinite(logits32).all() or any(c >= logits32.size for c in candidates):
        raise Refusal("invalid_score_values")
    maximum = float(logits32.max())
    log_partition = maximum + math.log(float(np.exp(logits32.astype(np.float64) - maximum).sum()))
    logits = [float(logits32[c]) for c in candidates]
    log_probabilities = [v - log_partition for v in logits]
    if not math.isfinite(temperature) or temperature <= 0.0:
        raise Refusal("invalid_score_values")
    top = max(logits)
    exps = [math.exp((v - top) / temperature) for v in logits]
    total = sum(exps)
    return logits, log_probabilities, [e / total for e in exps]


class ScoreWorker:
    def __init__(self, backend, budget: Budget, cache_enabled: bool):
        self.backend, self.budget, self.cache_enabled = backend, budget, cache_enabled
        self.entry, self.hits, self.native_score_calls = None, 0, 0

    def telemetry(self, pending_hit: bool) -> dict:
        return {"enabled": self.cache_enabled, "hits": self.hits + int(pending_hit),
                "native_score_calls": self.native_score_calls}

    def readiness(self, load_seconds: float) -> dict:
        b = self.backend
        return {"ready": True, "engine": "stark", "version": VERSION, "mode": "exact-token-scoring-cache-v1",
                "cache_policy": "consecutive-full-vocabulary-logits-v1" if self.cache_enabled else "fresh-state",
                "cache_enabled": self.cache_enabled, "cache_key": "exact-token-ids+context-tokens+model-instance",
                "cache": self.telemetry(False), "load_seconds": load_seconds, "vocab_size": b.vocab_size(),
                "max_context_tokens": b.max_context_length(), "max_request_bytes": self.budget.wire_bytes,
                "request_budget_bytes": self.budget.input_bytes, "peak_memory_bytes": None}

    def handle(self, obj):
        """Returns (reply, next cache entry or None, hit)."""
        if not isinstance(obj, dict) or not isinstance(obj.get("operation"), str):
            raise Refusal("invalid_request")
        op = obj["operation"]
        f = Fields(obj, "operation")
        b = self.backend
        if op == "reset_cache":
            f.done()
            self.entry = None
            return {"cache_reset": True, "cache": self.telemetry(False)}, MISSING, False
        if op == "tokenize":
            text = f.required("text", _string)
            special = f.defaulted("add_special_tokens", _boolean, False)
            f.done()
            if not text:
                raise Refusal("invalid_tokenization_request")
            if len(text.encode("utf-8")) > self.budget.input_bytes:
                raise Refusal("resource_budget_exceeded")
            started = time.perf_counter()
            ids = b.tokenize(text, special)
            if len(ids) > self.budget.input_bytes // 4:
                raise Refusal("resource_budget_exceeded")
            return {"token_ids": ids, "token_count": len(ids), "token_ids_sha256": token_hash(ids),
                    "vocab_size": b.vocab_size(), "tokenization_seconds": time.perf_counter() - started,
                    "cache": self.telemetry(False)}, MISSING, False
        if op != "score":
            raise Refusal("invalid_request")
        input_ids = f.required("input_token_ids", _ids)
        candidates = f.required("candidate_token_ids", _ids)
        context = f.required("context_tokens", lambda x: _uint(x, U32_MAX))
        temperature = f.required("temperature", _number)
        f.done()
        vocab = b.vocab_size()
        if vocab > self.budget.input_bytes // 4 or len(input_ids) > self.budget.input_bytes // 4 \
                or len(candidates) > self.budget.input_bytes // 4:
            raise Refusal("resource_budget_exceeded")
        started = time.perf_counter()
        # taking before validation leaves no committed entry on failure; a mismatch discards it (A/B/A cannot hit)
        previous, self.entry = self.entry, None
        if not (self.cache_enabled and previous is not None and previous[0] == input_ids and previous[1] == context):
            previous = None
        if (not input_ids or not 2 <= len(candidates) <= 16 or context == 0 or not math.isfinite(temperature)
                or temperature <= 0.0 or any(t >= vocab for t in input_ids + candidates)
                or len(set(candidates)) != len(candidates)):
            raise Refusal("invalid_scoring_request")
        if len(input_ids) > context or context > b.max_context_length():
            raise Refusal("context_overflow")
        scoring_started = time.perf_counter()
        hit = previous is not None
        if hit:
            logits, timings = previous[2], (0.0, 0.0, 0.0)
        else:
            self.native_score_calls += 1
            logits, timings = b.score(input_ids)
        import numpy as np
        if len(logits) != vocab or not np.isfinite(np.asarray(logits)).all():
            raise Refusal("invalid_score_values")
        readout_started = time.perf_counter()
        cand_logits, log_probs, cand_probs = candidate_readout(logits, candidates, temperature)
        now = time.perf_counter()
        reply = {"input_tokens": len(input_ids), "prompt_tokens_sha256": token_hash(input_ids),
                 "candidate_token_ids": candidates, "logits": cand_logits, "log_probabilities": log_probs,
                 "candidate_probabilities": cand_probs, "temperature": temperature, "cache_hit": hit,
                 "truncated": False,
                 "metrics": {"state_creation_seconds": timings[0], "prefill_seconds": timings[1],
                             "readout_seconds": timings[2] + (now - readout_started),
                             "score_seconds": now - scoring_started, "total_seconds": now - started},
                 "peak_memory_bytes": None, "cache": self.telemetry(hit)}
        entry = (input_ids, context, logits) if self.cache_enabled else None
        return reply, entry, hit

    def process_line(self, data: bytes, out) -> None:
        try:
            check_json_structure(data, self.budget)
            reply, entry, hit = self.handle(parse_json_line(data))
        except Refusal as e:
            self.entry = None
            write_reply(out, {"error": e.code, "cache": self.telemetry(False)})
            if e.code in FENCING_SCORING:
                raise Refusal("native_operation_failed") from None
            return
        try:
            write_reply(out, reply)
        except Refusal:
            self.entry = None
            raise
        if entry is not MISSING:
            self.entry = entry   # the only publication site follows the write
        self.hits += int(hit)


# ----------------------------------------------------------------------------------------------- entry points

def generation_arguments(args):
    """protocol.rs:18-53."""
    if len(args) < 2 or args[0] != "--model-path" or not args[1]:
        raise Refusal("invalid_arguments")
    prefix_cache, staging, rest = False, None, list(args[2:])
    while rest:
        flag = rest.pop(0)
        if flag == "--vision-staging-root" and staging is None:
            if not rest or not rest[0]:
                raise Refusal("invalid_arguments")
            staging = rest.pop(0)
        elif flag == "--prefix-cache" and not prefix_cache:
            prefix_cache = True
        else:
            raise Refusal("invalid_arguments")
    return Path(args[1]), prefix_cache


def scoring_arguments(args):
    """crates/stark-score/src/protocol.rs:10-26."""
    if len(args) < 2 or args[0] != "--score-model-path":
        raise Refusal("invalid_arguments")
    if len(args) == 2:
        return Path(args[1]), False
    if len(args) == 3 and args[2] == "--consecutive-cache":
        return Path(args[1]), True
    raise Refusal("invalid_arguments")


def serve_generation(worker: GenerationWorker, stdin, out) -> int:
    write_reply(out, worker.readiness())
    while True:
        data, oversize = read_frame(stdin, worker.budget.wire_bytes)
        if data is None:
            return 0
        if oversize:
            worker.clear_prefix()
            write_reply(out, {"error": "request_too_large"})
            continue
        worker.process_line(data, out)


def serve_scoring(worker: ScoreWorker, load_seconds: float, stdin, out) -> int:
    write_reply(out, worker.readiness(load_seconds))
    while True:
        data, oversize = read_frame(stdin, worker.budget.wire_bytes)
        if data is None:
            worker.entry = None
            return 0
        if oversize:
            worker.entry = None
            write_reply(out, {"error": "request_too_large", "cache": worker.telemetry(False)})
            return 0   # the scorer ends after an oversize frame (scoring.rs:858-863)
        worker.process_line(data, out)


def main(argv=None, backend_factory=None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    try:
        out = protocol_output()
    except OSError:
        return 1
    for name in list(os.environ):
        if name.startswith("STARK_CAPTURE_") or name.startswith("UZU_CAPTURE_"):
            del os.environ[name]
    factory = backend_factory or B200Backend
    try:
        scoring = bool(args) and args[0] == "--score-model-path"
        path, flag = scoring_arguments(args) if scoring else generation_arguments(args)
        budget = Budget.from_environment()
        cancel = None if scoring else CancelSignal.from_environment()
        started = time.perf_counter()
        backend = factory(path)
        if scoring:
            return serve_scoring(ScoreWorker(backend, budget, flag), time.perf_counter() - started, sys.stdin.buffer, out)
        supported = getattr(backend, "prefix_cache_supported", None)
        if flag and supported is not None and not supported():
            flag = False   # a model with a draft head: its cache cannot be cut inside a prompt
        return serve_generation(GenerationWorker(backend, budget, flag, cancel), sys.stdin.buffer, out)
    except Refusal as e:
        try:
            write_reply(out, {"ready": False, "error": e.code})
        except Refusal:
            pass
        return 1


if __name__ == "__main__":
    raise SystemExit(main())
