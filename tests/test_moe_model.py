"""The routed-expert decoder (f32 host-path conventions, GGUF Q8_0 attention + Q4_K expert banks): the
oracle's token step against an independent float64 restatement on CPU, and (GPU) the device decoder
against the oracle through the C ABI."""
import numpy as np
import pytest

from oracle import oracle as O
from stark_b200 import synthetic as S


def _dense(kind, blocks, rows, columns):
    """GGUF rows decoded through the pinned block decoder, as float64."""
    blocks = np.ascontiguousarray(blocks, np.uint8).reshape(rows, -1)
    return np.stack([O.gguf_decode_row(kind, blocks[r], columns) for r in range(rows)]).astype(np.float64)


class _Float64Decoder:
    """The same token step in float64 numpy with dense weights: no shared code with the C restatement beyond
    the block decoder.  Sums are numpy's, not sequential, so agreement is to rounding, not to the bit."""

    def __init__(self, cfg, w):
        self.c = cfg
        H, D, E, I = cfg["hidden"], cfg["head_dim"], cfg["experts"], cfg["inter"]
        qd, kd = cfg["q_heads"] * D, cfg["kv_heads"] * D
        self.table = _dense(8, w["token_table"], cfg["vocab"], H)
        self.output = _dense(8, w["output"], cfg["vocab"], H)
        self.final = w["final_norm"].astype(np.float64)
        self.layers = []
        for l in w["layers"]:
            self.layers.append(dict(
                qkv=_dense(8, l["qkv"], qd + 2 * kd, H), o=_dense(8, l["o"], H, qd), router=l["router"].astype(np.float64),
                gate=_dense(12, l["gate"], E * I, H).reshape(E, I, H), up=_dense(12, l["up"], E * I, H).reshape(E, I, H),
                down=_dense(12, l["down"], E * H, I).reshape(E, H, I),
                **{k: l[k].astype(np.float64) for k in ("attn_norm", "ffn_norm", "q_norm", "k_norm")}))
        self.keys = [[] for _ in w["layers"]]
        self.values = [[] for _ in w["layers"]]
        self.experts = []

    def _norm(self, x, w):
        return x / np.sqrt(np.mean(x * x) + self.c["eps"]) * w

    def _rope(self, head, position):
        d = head.size
        i = np.arange(d // 2)
        angle = position * self.c["rope_theta"] ** (-(2.0 * i) / d)
        a, b = head[:d // 2].copy(), head[d // 2:].copy()
        return np.concatenate([a * np.cos(angle) - b * np.sin(angle), a * np.sin(angle) + b * np.cos(angle)])

    def step(self, token):
        c = self.c
        D, QH, KV = c["head_dim"], c["q_heads"], c["kv_heads"]
        position = len(self.keys[0])
        x = self.table[token].copy()
        self.experts = []
        for li, l in enumerate(self.layers):
            n = self._norm(x, l["attn_norm"])
            qkv = l["qkv"] @ n
            q, k, v = qkv[:QH * D].reshape(QH, D), qkv[QH * D:(QH + KV) * D].reshape(KV, D), qkv[(QH + KV) * D:].reshape(KV, D)
            q = np.stack([self._rope(self._norm(h, l["q_norm"]), position) for h in q])
            k = np.stack([self._rope(self._norm(h, l["k_norm"]), position) for h in k])
            self.keys[li].append(k)
            self.values[li].append(v)
            K, V = np.stack(self.keys[li]), np.stack(self.values[li])  # [t, kv, d]
            att = np.empty((QH, D))
            for h in range(QH):
                g = h // (QH // KV)
                s = K[:, g] @ q[h] / np.sqrt(D)
                p = np.exp(s - s.max())
                att[h] = (p / p.sum()) @ V[:, g]
            x = x + l["o"] @ att.reshape(-1)
            n = self._norm(x, l["ffn_norm"])
            scores = l["router"] @ n
            ids = sorted(range(c["experts"]), key=lambda e: (-scores[e], e))[:c["active"]]
            p = np.exp(scores[ids] - scores[ids].max())
            p /= p.sum()
            mix = np.zeros_like(x)
            for e, pe in zip(ids, p):
                g = l["gate"][e] @ n
                mix += pe * (l["down"][e] @ (g / (1.0 + np.exp(-g)) * (l["up"][e] @ n)))
            x = x + mix
            self.experts.append(ids)
        return self.output @ self._norm(x, self.final)


def test_oracle_step_matches_float64_restatement():
    cfg = S.MOE_CONFIGS["moe-tiny"]
    w = S.moe_weights(cfg, seed=3)
    oracle, exact = O.MoEDecoder(cfg, w, 16, threads=2), _Float64Decoder(cfg, w)
    for token in (5, 400, 5, 77, 123):
        got, want = oracle.step(token), exact.step(token)
        assert oracle.last_experts.tolist() == exact.experts
        assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    assert oracle.position == 5
    with pytest.raises(ValueError):
        oracle.step(cfg["vocab"])


def test_rope_matches_the_closed_form():
    """ripple.rs:653-666: pairs (i, i + d/2) rotate by position * theta^(-2i/d)."""
    head = np.arange(1, 9, dtype=np.float32)
    out = head.copy()
    f = O.lib().so_rope_f32
    import ctypes as C
    f.restype, f.argtypes = None, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_float]
    f(out.ctypes.data, 8, 3, 10000.0)
    for i in range(4):
        ang = 3.0 * 10000.0 ** (-(2.0 * i) / 8.0)
        assert abs(out[i] - (head[i] * np.cos(ang) - head[i + 4] * np.sin(ang))) < 1e-5
        assert abs(out[i + 4] - (head[i] * np.sin(ang) + head[i + 4] * np.cos(ang))) < 1e-5
    same = head.copy()
    f(same.ctypes.data, 8, 0, 10000.0)
    assert same.tolist() == head.tolist()                                    # position 0 is the identity


def _close(got, want, bound=2e-4):
    return np.abs(got - want).max() <= bound * max(1.0, np.abs(want).max())


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["moe-tiny", "moe-small", "moe-a3b-layers"])
def test_device_decoder_matches_oracle(name):
    from stark_b200.engine import MoEModel
    cfg = S.MOE_CONFIGS[name]
    w = S.moe_weights(cfg, seed=1)
    context = 192
    model, oracle = MoEModel.load(cfg, w, context), O.MoEDecoder(cfg, w, context)
    prompt = S.prompt(cfg, 40, seed=2)
    # token by token: logits, routing and the greedy pick
    agree = 0
    for t in prompt[:12]:
        got, want = model.step(int(t)), oracle.step(int(t))
        assert np.isfinite(got).all() and _close(got, want)
        assert model.last_experts().tolist() == oracle.last_experts.tolist()
        agree += int(got.argmax() == want.argmax())
    assert agree >= 11
    # cache-only prompt rows, then a step: same as stepping through them
    model.ingest(prompt[12:])
    oracle.ingest(prompt[12:])
    assert model.position == oracle.position == 40
    got, want = model.step(9), oracle.step(9)
    assert _close(got, want)
    # greedy decode chained on the device follows the oracle's own greedy decode while no near-tie parts them
    first = int(want.argmax())
    picks = model.generate_greedy(first, 16)
    token, same = first, 0
    for i in range(16):
        lg = oracle.step(token)
        token = int(lg.argmax())
        same += int(picks[i] == token)
        if picks[i] != token:
            break
    assert same >= 8, (same, picks)
    assert model.position == 57
    # teacher-forced: both decoders are fed the oracle's greedy tokens, top-1 must agree on >= 99 % of 100 steps
    model.reset()
    oracle.reset()
    model.ingest(prompt[:-1])
    oracle.ingest(prompt[:-1])
    token, agree, steps = int(prompt[-1]), 0, 100
    for i in range(steps):
        got, want = model.step(token), oracle.step(token)
        assert _close(got, want, 1e-3)   # absolute tolerance on the f32 logits: 1e-3 of the largest magnitude
        agree += int(got.argmax() == want.argmax())
        token = int(want.argmax())
    assert agree >= 99, agree
    assert model.position == 39 + steps
    # reset: the first step reproduces itself bit for bit
    model.reset()
    a = model.step(int(prompt[0]))
    model.reset()
    b = model.step(int(prompt[0]))
    assert model.position == 1 and a.tobytes() == b.tobytes()
    assert model.launches_per_token >= 4 + 8 * cfg["layers"]
    model.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["moe-small", "moe-a3b-layers"])
def test_fused_hand_offs_change_no_bit(name, monkeypatch):
    """The residual add + norm inside the router kernel and the per-head norm + rope inside the attention kernel
    form their sums in the order of the separate kernels: logits, experts and tokens are the same bits."""
    from stark_b200.engine import MoEModel
    cfg = S.MOE_CONFIGS[name]
    w = S.moe_weights(cfg, seed=4)
    prompt = S.prompt(cfg, 70, seed=6)
    seen = []
    for fuse in ("1", "0"):
        monkeypatch.setenv("STARK_B200_MOE_FUSE", fuse)
        model = MoEModel.load(cfg, w, 128)
        assert model.launches_per_token == 4 + (8 if fuse == "1" else 10) * cfg["layers"]
        model.ingest(prompt[:-1])
        logits = model.step(int(prompt[-1]))
        experts = model.last_experts().tolist()
        picks = model.generate_greedy(int(logits.argmax()), 12)
        seen.append((logits.tobytes(), experts, picks.tolist(), model.step(3).tobytes()))
        model.close()
    assert seen[0] == seen[1]


@pytest.mark.gpu
def test_device_decoder_refuses_bad_calls():
    from stark_b200._lib import StarkB200Error
    from stark_b200.engine import MoEModel
    cfg = S.MOE_CONFIGS["moe-tiny"]
    w = S.moe_weights(cfg, seed=4)
    model = MoEModel(cfg, 4)
    with pytest.raises(StarkB200Error):                                      # nothing loaded yet
        model.step(1)
    model.set_globals(w["token_table"], w["output"], w["final_norm"])
    for i, l in enumerate(w["layers"]):
        model.set_layer(i, l)
    with pytest.raises(StarkB200Error):
        model.step(cfg["vocab"])
    with pytest.raises(StarkB200Error):
        model.ingest([1, 2, 3, 4, 5])                                        # more rows than the cache holds
    model.ingest([1, 2, 3])
    model.step(4)
    with pytest.raises(StarkB200Error):
        model.step(5)                                                        # the cache is full
    assert model.position == 4
    bad = dict(w["layers"][0])
    bad["attn_norm"] = np.full(cfg["hidden"], np.nan, np.float32)
    with pytest.raises(StarkB200Error):
        model.set_layer(0, bad)
    with pytest.raises(StarkB200Error):
        MoEModel(dict(cfg, head_dim=64), 4)
    model.close()
