"""The allocation-free attention entry point against the ordinary one, through the C ABI.

A worker that fixed its device-memory budget up front, or a decode loop that cannot take the
device-wide stall of an allocation, calls ``stark_b200_op_attention_decode_static``: it brings every
buffer itself (device pointers, the library's KV page layout) and the kernel's own working memory
is a fixed array inside the library.  The test feeds both entry points the same seeded inputs and
requires the same output, on two calls in a row (the second call sees what the first one left in
the shared array, and also reads the row the first one appended).

This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O
from stark_b200 import synthetic as S

pytestmark = pytest.mark.gpu
REL_TOL = 1e-2  # the per-operator bar of the other GPU tests; the two entry points should agree exactly
PAGE = 64


def to_pages(rows: np.ndarray, blocks: int) -> np.ndarray:
    """[n, kv_heads, 128] row-major cache -> the library's [page, kv_head, 64, 128] layout."""
    n, kvh, hd = rows.shape
    pages = np.zeros((blocks, kvh, PAGE, hd), np.uint16)
    for r in range(n):
        pages[r // PAGE, :, r % PAGE, :] = rows[r]
    return pages


def rope_tables(positions: int, theta: float):
    cos = np.zeros((positions, 128), np.float32)
    sin = np.zeros((positions, 128), np.float32)
    for p in range(positions):
        cos[p], sin[p] = O.rope_coeffs(p, 128, theta)
    return cos, sin


@pytest.mark.parametrize("q_heads,kv_heads,position,splits", [(32, 8, 300, 8), (16, 8, 63, 4)])
def test_static_entry_point_matches_the_allocating_one_twice_in_a_row(q_heads, kv_heads, position, splits):
    from stark_b200 import _lib, ops
    from stark_b200._lib import check
    lib = _lib.load()
    rng = np.random.default_rng(100 + position)
    hd, eps, theta = 128, 1e-6, 1e6
    capacity = position + 2
    keys = np.zeros((capacity, kv_heads, hd), np.uint16)
    values = np.zeros((capacity, kv_heads, hd), np.uint16)
    keys[:position] = S.bf16_normal(rng, position * kv_heads * hd).reshape(position, kv_heads, hd)
    values[:position] = S.bf16_normal(rng, position * kv_heads * hd).reshape(position, kv_heads, hd)
    qn = (1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kn = (1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    rows = [S.bf16_normal(rng, (q_heads + 2 * kv_heads) * hd, 2.0) for _ in range(2)]

    # the existing entry point (host buffers; it stages and allocates internally), two steps
    want = []
    for step, qkv in enumerate(rows):
        want.append(ops.attention_decode(qkv, keys, values, q_heads, kv_heads, position + step, eps, theta, qn, kn,
                                         splits=splits))

    # the static entry point: the caller owns every buffer (allocated here, once, before the calls)
    blocks = (position + 2 + PAGE - 1) // PAGE
    start = keys.copy()
    start[position:] = 0
    vstart = values.copy()
    vstart[position:] = 0
    cos, sin = rope_tables(position + 2, theta)
    bufs = dict(
        k=ops.DeviceBuffer(blocks * kv_heads * PAGE * hd * 2).upload(to_pages(start[:position], blocks)),
        v=ops.DeviceBuffer(blocks * kv_heads * PAGE * hd * 2).upload(to_pages(vstart[:position], blocks)),
        table=ops.DeviceBuffer(blocks * 4).upload(np.arange(blocks, dtype=np.int32)),
        qn=ops.DeviceBuffer(hd * 4).upload(qn), kn=ops.DeviceBuffer(hd * 4).upload(kn),
        cos=ops.DeviceBuffer(cos.nbytes).upload(cos), sin=ops.DeviceBuffer(sin.nbytes).upload(sin),
        qkv=ops.DeviceBuffer(rows[0].nbytes), out=ops.DeviceBuffer(q_heads * hd * 2),
    )
    for step, qkv in enumerate(rows):
        bufs["qkv"].upload(qkv)
        d = _lib.AttentionDesc(C.sizeof(_lib.AttentionDesc), _lib.ABI_VERSION, q_heads, kv_heads, hd,
                               position + step, 0, splits, eps, 0.0)
        check(lib.stark_b200_op_attention_decode_static(
            bufs["qkv"].ptr, bufs["k"].ptr, bufs["v"].ptr, bufs["table"].ptr, bufs["out"].ptr, bufs["qn"].ptr,
            bufs["kn"].ptr, bufs["cos"].ptr, bufs["sin"].ptr, C.byref(d), None), "op_attention_decode_static")
        got = bufs["out"].download(np.uint16, q_heads * hd)
        g = O.bf16_to_f32(got).astype(np.float64)
        w = O.bf16_to_f32(want[step]).astype(np.float64)
        assert np.all(np.abs(g - w) <= REL_TOL * np.maximum(np.abs(w), np.abs(w).mean())), f"call {step}"
        assert np.array_equal(got, want[step]), f"call {step}: same kernel, same split count, same bits"
        # and against the CPU oracle directly: the rows of earlier positions plus the row this call appended
        # (which the allocating entry point wrote back into the host cache, head norm and RoPE applied)
        seq = position + step + 1
        cosr, sinr = O.rope_coeffs(position + step, hd, theta)
        q = O.head_norm_bf16(qkv, qn, 0, q_heads, hd, eps)
        q = np.concatenate([O.rope_head_bf16(q[h * hd:(h + 1) * hd], cosr, sinr) for h in range(q_heads)])
        ref = O.attention_decode_bf16(q, keys[:seq].reshape(seq, -1), values[:seq].reshape(seq, -1), q_heads,
                                      kv_heads, hd, seq, 1.0 / np.sqrt(hd))
        r = O.bf16_to_f32(ref).astype(np.float64)
        assert np.all(np.abs(g - r) <= REL_TOL * np.maximum(np.abs(r), np.abs(r).mean())), f"call {step} vs oracle"
    # the rows both calls appended are the ones the allocating entry point wrote back to the host cache
    got_k = bufs["k"].download(np.uint16, blocks * kv_heads * PAGE * hd).reshape(blocks, kv_heads, PAGE, hd)
    for r in (position, position + 1):
        assert np.array_equal(got_k[r // PAGE, :, r % PAGE, :], keys[r])


def test_static_entry_point_rejects_what_does_not_fit():
    from stark_b200 import _lib
    lib = _lib.load()
    # 64 query heads x 32 splits x 520 bytes > 1 MiB - 1 KiB: refused before anything is launched
    d = _lib.AttentionDesc(C.sizeof(_lib.AttentionDesc), _lib.ABI_VERSION, 64, 8, 128, 10, 0, 32, 1e-6, 0.0)
    dummy = 0x1000  # never dereferenced: the size check comes first
    status = lib.stark_b200_op_attention_decode_static(dummy, dummy, dummy, dummy, dummy, None, None, None, None,
                                                       C.byref(d), None)
    assert status == _lib.STATUS_NAMES.index("context_limit")
    # more KV heads than the counter block holds, in a shape whose partials would fit (65 x 1 x 520 bytes): only
    # the head bound can refuse it
    d.splits = 1
    d.kv_heads = 65
    d.q_heads = 65
    assert lib.stark_b200_op_attention_decode_static(dummy, dummy, dummy, dummy, dummy, None, None, None, None,
                                                     C.byref(d), None) == _lib.STATUS_NAMES.index("context_limit")


def test_static_entry_point_accepts_the_largest_head_count():
    """64 KV heads is the last count the arrival-counter block holds; the call must run and agree with the
    allocating entry point."""
    from stark_b200 import _lib, ops
    from stark_b200._lib import check
    lib = _lib.load()
    rng = np.random.default_rng(7)
    heads, hd, position, eps, theta = 64, 128, 5, 1e-6, 1e6
    keys = np.zeros((position + 1, heads, hd), np.uint16)
    values = np.zeros((position + 1, heads, hd), np.uint16)
    keys[:position] = S.bf16_normal(rng, position * heads * hd).reshape(position, heads, hd)
    values[:position] = S.bf16_normal(rng, position * heads * hd).reshape(position, heads, hd)
    qkv = S.bf16_normal(rng, 3 * heads * hd, 2.0)
    want = ops.attention_decode(qkv, keys.copy(), values.copy(), heads, heads, position, eps, theta, None, None,
                                splits=2)
    cos, sin = rope_tables(position + 1, theta)
    k = ops.DeviceBuffer(heads * PAGE * hd * 2).upload(to_pages(keys[:position], 1))
    v = ops.DeviceBuffer(heads * PAGE * hd * 2).upload(to_pages(values[:position], 1))
    table = ops.DeviceBuffer(4).upload(np.zeros(1, np.int32))
    dc, ds = ops.DeviceBuffer(cos.nbytes).upload(cos), ops.DeviceBuffer(sin.nbytes).upload(sin)
    dq, out = ops.DeviceBuffer(qkv.nbytes).upload(qkv), ops.DeviceBuffer(heads * hd * 2)
    d = _lib.AttentionDesc(C.sizeof(_lib.AttentionDesc), _lib.ABI_VERSION, heads, heads, hd, position, 0, 2, eps, 0.0)
    check(lib.stark_b200_op_attention_decode_static(dq.ptr, k.ptr, v.ptr, table.ptr, out.ptr, None, None, dc.ptr,
                                                    ds.ptr, C.byref(d), None), "op_attention_decode_static")
    assert np.array_equal(out.download(np.uint16, heads * hd), want)
