"""The arithmetic of the tensor-memory prompt-attention kernel, restated in numpy and checked on the CPU: two passes
over the keys (row maximum first, then exp2(s - max) with no rescaling), probabilities carried into the second
product as bf16 hi + lo (two round-to-nearest conversions), values in bf16, accumulation in f32, one bf16 rounding
of the output.  What the split drops is at most 2^-16 of a probability, so the result sits within a rounding of the
f64 answer of attention_single_pass.rs:11-133."""
import numpy as np

from oracle import oracle as O
from stark_b200 import synthetic as S


def _to_bf16(x: np.ndarray) -> np.ndarray:
    return O.bf16_to_f32(S.f32_to_bf16(np.ascontiguousarray(x, np.float32))).astype(np.float32)


def _kernel_arithmetic(q, k, v, first_pos):
    """q [m, 128], k / v [rows, 128] as f32 values of bf16 numbers; returns the bf16 output as f32."""
    m, d = q.shape
    scale_log2 = np.float32(np.log2(np.e) / np.sqrt(d))
    s = (q.astype(np.float32) @ k.astype(np.float32).T).astype(np.float32)          # f32 accumulation of exact products
    visible = np.arange(k.shape[0])[None, :] <= (first_pos + np.arange(m))[:, None]
    mx = np.where(visible, s * scale_log2, -np.inf).max(axis=1, keepdims=True).astype(np.float32)   # pass 1
    p = np.where(visible, np.exp2((s * scale_log2 - mx).astype(np.float32)), 0.0).astype(np.float32)   # pass 2
    hi = _to_bf16(p)
    lo = _to_bf16(p - hi)
    assert np.all(np.abs(p - hi - lo) <= 2.0 ** -16 * p + 1e-45)   # what the split drops
    out = (hi.astype(np.float64) @ v + lo.astype(np.float64) @ v) / p.sum(axis=1, keepdims=True, dtype=np.float32)
    return O.bf16_to_f32(S.f32_to_bf16(out.astype(np.float32)))


def test_two_pass_split_probabilities_are_within_a_rounding_of_f64():
    rng = np.random.default_rng(3)
    for m, first_pos, spread in ((70, 0, 1.0), (130, 517, 1.0), (64, 2000, 4.0)):
        rows = first_pos + m
        bf = lambda a: O.bf16_to_f32(S.f32_to_bf16(a.astype(np.float32))).astype(np.float32)
        q, k, v = bf(spread * rng.standard_normal((m, 128))), bf(rng.standard_normal((rows, 128))), bf(rng.standard_normal((rows, 128)))
        got = _kernel_arithmetic(q, k, v, first_pos).astype(np.float64)
        s = q.astype(np.float64) @ k.astype(np.float64).T / np.sqrt(128.0)
        s = np.where(np.arange(rows)[None, :] <= (first_pos + np.arange(m))[:, None], s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        weights = p / p.sum(axis=1, keepdims=True)
        want = weights @ v.astype(np.float64)
        half_step = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(want), 2.0 ** -30))) - 8)   # the output's own bf16 rounding
        # plus what the split drops, against the magnitude of the terms (an output near zero is a cancellation of
        # terms that are not): 2^-16 of every term at most
        dropped = 2.0 ** -16 * (weights @ np.abs(v.astype(np.float64)))
        assert (np.abs(got - want) <= half_step * 1.01 + dropped + 2e-6).all()
