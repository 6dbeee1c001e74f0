"""Causal attention of a prompt pass over the paged cache, operator by operator: the mma.sync kernel and the tcgen05
kernel against an f64 restatement of attention_single_pass.rs:11-133 (scores q.k / sqrt(d) over the keys a row may
see, softmax, probability-weighted values) and against each other."""
import numpy as np
import pytest

from oracle import oracle as O
from stark_b200 import synthetic as S

PAGE, DIM = 64, 128


def _case(seed, m, first_pos, q_heads, kv_heads):
    rng = np.random.default_rng(seed)
    rows = first_pos + m
    pages = -(-rows // PAGE) + 1                      # one page more than needed: never read
    table = rng.permutation(pages).astype(np.int32)   # pages out of order, as a paged cache has them
    heads = q_heads + 2 * kv_heads
    qkv = S.f32_to_bf16(rng.standard_normal((m, heads, DIM)).astype(np.float32))
    k = S.f32_to_bf16(rng.standard_normal((rows, kv_heads, DIM)).astype(np.float32))
    v = S.f32_to_bf16(rng.standard_normal((rows, kv_heads, DIM)).astype(np.float32))
    keys = np.zeros((pages, kv_heads, PAGE, DIM), np.uint16)
    values = np.zeros_like(keys)
    for pos in range(rows):
        keys[table[pos // PAGE], :, pos % PAGE] = k[pos]
        values[table[pos // PAGE], :, pos % PAGE] = v[pos]
    return qkv, keys, values, table, k, v


def _reference(qkv, k, v, m, first_pos, q_heads, kv_heads):
    q = O.bf16_to_f32(qkv[:, :q_heads]).astype(np.float64)
    kf, vf = O.bf16_to_f32(k).astype(np.float64), O.bf16_to_f32(v).astype(np.float64)
    out = np.zeros((m, q_heads, DIM))
    group = q_heads // kv_heads
    for h in range(q_heads):
        s = q[:, h] @ kf[:, h // group].T / np.sqrt(DIM)                    # [m, rows]
        mask = np.arange(kf.shape[0])[None, :] <= (first_pos + np.arange(m))[:, None]
        s = np.where(mask, s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h] = (p / p.sum(axis=1, keepdims=True)) @ vf[:, h // group]
    return out


def _run(qkv, keys, values, table, m, first_pos, q_heads, kv_heads, variant):
    from stark_b200.ops import prompt_attention, take_device_error
    out = prompt_attention(qkv, keys, values, table, first_pos, q_heads, kv_heads, tensor_memory=bool(variant))
    assert out.shape == (m, q_heads, DIM) and take_device_error() == 0
    return O.bf16_to_f32(out).astype(np.float64)


CASES = [(128, 0, 4, 1), (200, 77, 8, 2), (40, 300, 4, 4), (384, 128, 4, 2), (129, 1023, 8, 1)]


@pytest.mark.gpu
@pytest.mark.parametrize("m,first_pos,q_heads,kv_heads", CASES)
@pytest.mark.parametrize("variant", [0, 1])
def test_prompt_attention_matches_f64(variant, m, first_pos, q_heads, kv_heads):
    qkv, keys, values, table, k, v = _case(m + first_pos, m, first_pos, q_heads, kv_heads)
    want = _reference(qkv, k, v, m, first_pos, q_heads, kv_heads)
    got = _run(qkv, keys, values, table, m, first_pos, q_heads, kv_heads, variant)
    # the output is one bf16 rounding of an f32 result whose probabilities carry about 16 bits
    err = np.abs(got - want)
    assert err.max() <= 2.0 ** -8 * max(1.0, np.abs(want).max()), (variant, err.max(), np.unravel_index(err.argmax(), err.shape))


@pytest.mark.gpu
def test_both_kernels_agree_to_a_rounding():
    m, first_pos, q_heads, kv_heads = 300, 500, 8, 2
    qkv, keys, values, table, k, v = _case(5, m, first_pos, q_heads, kv_heads)
    a = _run(qkv, keys, values, table, m, first_pos, q_heads, kv_heads, 0)
    b = _run(qkv, keys, values, table, m, first_pos, q_heads, kv_heads, 1)
    # the same f32 arithmetic up to summation order and the exponential's last bits: the bf16 outputs differ by at
    # most one unit in the last place (plus the f32 noise itself where an output is nearly zero), and rarely
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(a), 2.0 ** -20))) - 7)
    assert (np.abs(a - b) <= ulp + 2e-5).all()
    assert (a != b).mean() < 0.05
