"""Seeded synthetic weights and prompts in the reference's on-disk tensor layouts.

No checkpoint or dataset is available offline, so every configuration is random-init by
definition: codes uniform, bf16 scales uniform in a stated range, bias = -8 * scale (4 bit).  The
arrays use the MLX layout the reference reads (``uint32[rows, columns/8]`` codes with 8 nibbles per
word along K, planes ``[rows, columns/group]``;
crates/stark-engine/src/engine/hybrid/weights.rs:1157-1228).
"""
from __future__ import annotations

import numpy as np

# Shapes of the named configurations (Qwen3-shaped dense decoders).
CONFIGS = {
    "qwen3-0.6b": dict(layers=28, hidden=1024, q_heads=16, kv_heads=8, head_dim=128, inter=3072, vocab=151936,
                       tied=True, eps=1e-6, rope_theta=1e6),
    "qwen3-8b": dict(layers=36, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, inter=12288, vocab=151936,
                     tied=False, eps=1e-6, rope_theta=1e6),
    # two layers with the layer and vocabulary dimensions of the named shapes: every matrix width, head count
    # and the full-vocabulary read-out of those shapes at a cost the CPU oracle pays in seconds
    "qwen3-0.6b-layers": dict(layers=2, hidden=1024, q_heads=16, kv_heads=8, head_dim=128, inter=3072, vocab=151936,
                              tied=True, eps=1e-6, rope_theta=1e6),
    "qwen3-8b-layers": dict(layers=2, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, inter=12288, vocab=151936,
                            tied=False, eps=1e-6, rope_theta=1e6),
    # small shapes for parity tests (same graph, minutes -> milliseconds on the CPU oracle)
    "tiny": dict(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=128, inter=512, vocab=1024, tied=True,
                 eps=1e-6, rope_theta=1e6),
    "small": dict(layers=4, hidden=1024, q_heads=16, kv_heads=8, head_dim=128, inter=3072, vocab=8192, tied=False,
                  eps=1e-6, rope_theta=1e6),
}


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


def affine4_matrix(rng: np.random.Generator, rows: int, columns: int, scale_lo: float = 0.005,
                   scale_hi: float = 0.02, group: int = 64, zero_point: float = 8.0) -> dict:
    """One 4-bit MLX-affine matrix: nibbles uniform 0..15, scale U[lo, hi] (bf16), bias = -zero_point*scale.
    The default zero point of 8 is the benchmarked distribution; its weights have mean -scale/2, so every
    output carries a common-mode term.  7.5 gives zero-mean weights (input-dependent arg-max)."""
    words = rows * columns // 8
    codes = rng.integers(0, 1 << 32, size=words, dtype=np.uint32).reshape(rows, columns // 8)
    scales_f = rng.uniform(scale_lo, scale_hi, size=(rows, columns // group)).astype(np.float32)
    scales = f32_to_bf16(scales_f)
    biases = f32_to_bf16(-zero_point * bf16_to_f32(scales))
    return dict(codes=codes, scales=scales, biases=biases, n=rows, k=columns, bits=4, group=group)


def bf16_normal(rng: np.random.Generator, count: int, sigma: float = 1.0) -> np.ndarray:
    return f32_to_bf16((rng.standard_normal(count) * sigma).astype(np.float32))


def matvec_case(seed: int = 0, rows: int = 4096, columns: int = 4096) -> dict:
    """The single-matvec configuration: W 4096x4096, scales U[0.005, 0.02], x ~ N(0,1) in bf16."""
    rng = np.random.default_rng(seed)
    w = affine4_matrix(rng, rows, columns)
    w["x"] = bf16_normal(rng, columns)
    return w


def dense_weights(cfg: dict, seed: int = 0, zero_point: float = 8.0) -> dict:
    """Random-init weights for a Qwen3-shaped dense decoder.

    Scale ranges are the single-matvec range times 17.3/sqrt(K), which keeps every linear layer's
    output at the magnitude of its input (unit-variance rows) so that 28-36 layers stay in range.
    """
    rng = np.random.default_rng(seed)
    D, hd, I, V = cfg["hidden"], cfg["head_dim"], cfg["inter"], cfg["vocab"]
    qkv_n = (cfg["q_heads"] + 2 * cfg["kv_heads"]) * hd

    def mat(n, k, gain=1.0):
        c = gain * 17.3 / np.sqrt(k)
        return affine4_matrix(rng, n, k, 0.005 * c, 0.02 * c, zero_point=zero_point)

    def norm(n):
        return (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)

    layers = []
    for _ in range(cfg["layers"]):
        layers.append(dict(attn_norm=norm(D), mlp_norm=norm(D), q_norm=norm(hd), k_norm=norm(hd),
                           qkv=mat(qkv_n, D), o=mat(D, cfg["q_heads"] * hd, 0.5), upgate=mat(2 * I, D),
                           down=mat(D, I, 0.5)))
    embed = mat(V, D)
    lm_head = embed if cfg["tied"] else mat(V, D)
    return dict(layers=layers, embed=embed, lm_head=lm_head, final_norm=norm(D))


def mtp_weights(cfg: dict, seed: int = 0, zero_point: float = 8.0) -> dict:
    """Random-init draft head of the dense multi-token-prediction path: fusion [D, 2D], one decoder layer of the
    target's dimensions, and the three norms (embedding, incoming hidden, output)."""
    rng = np.random.default_rng(seed + 7919)
    D, hd, I = cfg["hidden"], cfg["head_dim"], cfg["inter"]
    qkv_n = (cfg["q_heads"] + 2 * cfg["kv_heads"]) * hd

    def mat(n, k, gain=1.0):
        c = gain * 17.3 / np.sqrt(k)
        return affine4_matrix(rng, n, k, 0.005 * c, 0.02 * c, zero_point=zero_point)

    def norm(n):
        return (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)

    layer = dict(attn_norm=norm(D), mlp_norm=norm(D), q_norm=norm(hd), k_norm=norm(hd), qkv=mat(qkv_n, D),
                 o=mat(D, cfg["q_heads"] * hd, 0.5), upgate=mat(2 * I, D), down=mat(D, I, 0.5))
    return dict(fusion=mat(D, 2 * D), layer=layer, embed_norm=norm(D), hidden_norm=norm(D), out_norm=norm(D))


def prompt(cfg: dict, length: int, seed: int = 1) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=length, dtype=np.uint32)


# ----------------------------------------------------------------------------- GGUF blocks

def _random_bytes(rng: np.random.Generator, count: int, pool: int = 1 << 23) -> np.ndarray:
    """`count` uniform random bytes.  Beyond `pool` bytes the sequence is one drawn pool repeated, each repeat
    XORed with its own drawn byte: hundreds of MB of expert banks then cost a copy instead of a draw."""
    if count <= pool:
        return rng.integers(0, 256, size=count, dtype=np.uint8)
    base = rng.integers(0, 256, size=pool, dtype=np.uint8)
    reps = -(-count // pool)
    masks = rng.integers(0, 256, size=reps, dtype=np.uint8)
    return (base[None, :] ^ masks[:, None]).reshape(-1)[:count].copy()


def q8_0_rows(rng: np.random.Generator, rows: int, columns: int, scale: float = 0.01) -> np.ndarray:
    """Random Q8_0 rows: per 32 values an f16 scale d ~ U[0.5, 1.5] * scale and 32 int8 codes."""
    blocks = rows * columns // 32
    out = np.empty((blocks, 34), np.uint8)
    d = (rng.uniform(0.5, 1.5, blocks) * scale).astype(np.float16)
    out[:, 0:2] = d.view(np.uint8).reshape(blocks, 2)
    out[:, 2:] = _random_bytes(rng, blocks * 32).reshape(blocks, 32)
    return out.reshape(rows, -1)


def q4_k_rows(rng: np.random.Generator, rows: int, columns: int, scale: float = 0.01) -> np.ndarray:
    """Random Q4_K rows: per 256 values f16 d and dmin, 12 bytes of packed 6-bit (scale, min) pairs, 128
    bytes of nibbles.  d is sized so that d * sc * q stays O(scale)."""
    blocks = rows * columns // 256
    out = _random_bytes(rng, blocks * 144).reshape(blocks, 144)
    d = (rng.uniform(0.5, 1.5, blocks) * scale / 32.0).astype(np.float16)
    dmin = (rng.uniform(0.5, 1.5, blocks) * scale / 8.0).astype(np.float16)
    out[:, 0:2] = d.view(np.uint8).reshape(blocks, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(blocks, 2)
    return out.reshape(rows, -1)


def affine8_matrix(rng: np.random.Generator, rows: int, columns: int, scale_lo: float = 0.0005,
                   scale_hi: float = 0.002, group: int = 64) -> dict:
    """One 8-bit MLX-affine matrix: codes uniform 0..255, bias = -128 * scale."""
    codes = rng.integers(0, 256, size=(rows, columns), dtype=np.uint8)
    scales = f32_to_bf16(rng.uniform(scale_lo, scale_hi, size=(rows, columns // group)).astype(np.float32))
    biases = f32_to_bf16(-128.0 * bf16_to_f32(scales))
    return dict(codes=codes, scales=scales, biases=biases, n=rows, k=columns, bits=8, group=group)


# ----------------------------------------------------------------------------- routed-expert decoder

MOE_CONFIGS = {
    # the Qwen3-30B-A3B shape: 128 experts, 8 active, expert intermediate 768
    "qwen3-30b-a3b": dict(layers=48, hidden=2048, q_heads=32, kv_heads=4, head_dim=128, experts=128, active=8,
                          inter=768, vocab=151936, eps=1e-6, rope_theta=1e6),
    # two layers of that shape over a small vocabulary: full-size layer dimensions at test cost
    "moe-a3b-layers": dict(layers=2, hidden=2048, q_heads=32, kv_heads=4, head_dim=128, experts=128, active=8,
                           inter=768, vocab=4096, eps=1e-6, rope_theta=1e6),
    "moe-tiny": dict(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=128, experts=8, active=2, inter=256,
                     vocab=512, eps=1e-6, rope_theta=1e6),
    "moe-small": dict(layers=3, hidden=512, q_heads=8, kv_heads=2, head_dim=128, experts=16, active=4, inter=256,
                      vocab=2048, eps=1e-6, rope_theta=1e6),
}


def moe_layer_weights(cfg: dict, rng: np.random.Generator) -> dict:
    """One layer: Q8_0 [q; k; v] and o, f32 router ~ N(0, 1/hidden) (unit-variance router logits on a
    normalised input), Q4_K gate / up / down banks, f32 norm weights near 1."""
    H, D, E, I = cfg["hidden"], cfg["head_dim"], cfg["experts"], cfg["inter"]
    qd, kd = cfg["q_heads"] * D, cfg["kv_heads"] * D
    near_one = lambda n: (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    return dict(
        qkv=q8_0_rows(rng, qd + 2 * kd, H, scale=3e-4), o=q8_0_rows(rng, H, qd, scale=3e-4),
        router=(rng.standard_normal((E, H)) / np.sqrt(H)).astype(np.float32),
        gate=q4_k_rows(rng, E * I, H, scale=4e-3), up=q4_k_rows(rng, E * I, H, scale=4e-3),
        down=q4_k_rows(rng, E * H, I, scale=4e-3),
        attn_norm=near_one(H), ffn_norm=near_one(H), q_norm=near_one(D), k_norm=near_one(D))


def moe_weights(cfg: dict, seed: int = 0) -> dict:
    """Random-init weights of a routed-expert decoder in GGUF blocks (Q8_0 attention / token table / output,
    Q4_K experts)."""
    rng = np.random.default_rng(seed)
    return dict(token_table=q8_0_rows(rng, cfg["vocab"], cfg["hidden"], scale=3e-4),
                output=q8_0_rows(rng, cfg["vocab"], cfg["hidden"], scale=3e-4),
                final_norm=(1.0 + 0.1 * rng.standard_normal(cfg["hidden"])).astype(np.float32),
                layers=[moe_layer_weights(cfg, rng) for _ in range(cfg["layers"])])
