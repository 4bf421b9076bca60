"""Decode attention without allocations: tl_attn_decode_f16_noalloc.

Who needs it: a caller that is not allowed to allocate device memory at the point of the call —
inside a stream capture, under a fixed memory budget handed down by the application embedding the
library, or in a serving loop that bans allocator calls after start-up. Such a caller cannot
provide the scratch buffer and the counters tl_attn_decode_f16 asks for; this entry point keeps
them in a fixed array inside the library.

The test drives both entry points through the C ABI on the same inputs, twice in a row with
different sequence lengths and split counts (the second call sees whatever the first left in the
shared array), and requires identical fp16 outputs: both run the same kernel with the same
split, so there is nothing to tolerate. It also checks that oversized requests are refused.
This file sorts last on purpose, so a run that stops at the first failure has already run
everything else.
"""
import numpy as np
import pytest

from tensorlib_b200 import synth

pytestmark = pytest.mark.gpu


def _attn_pair(tl, seed, n_heads, head_dim, seq_len, splits, max_seq):
    lib = tl.load()
    width = n_heads * head_dim
    q = synth.normal_f16(seed, 1, width, 1.0)
    k = synth.normal_f16(seed, 2, max_seq * width, 1.0)
    v = synth.normal_f16(seed, 3, max_seq * width, 1.0)
    dq, dk, dv = (tl.DeviceBuffer.from_numpy(a) for a in (q, k, v))
    out_ref, out_new = tl.DeviceBuffer(width * 2), tl.DeviceBuffer(width * 2)
    scratch = tl.DeviceBuffer(n_heads * splits * (head_dim + 2) * 4)
    counters = tl.DeviceBuffer.from_numpy(np.zeros(n_heads, dtype=np.uint32))
    tl.check(lib.tl_attn_decode_f16(dq.ptr, dk.ptr, dv.ptr, out_ref.ptr, scratch.ptr, counters.ptr,
                                    n_heads, head_dim, seq_len, splits, None), "tl_attn_decode_f16")
    tl.check(lib.tl_attn_decode_f16_noalloc(dq.ptr, dk.ptr, dv.ptr, out_new.ptr, n_heads, head_dim,
                                            seq_len, splits, None), "tl_attn_decode_f16_noalloc")
    a = out_ref.to_numpy(np.float16, (n_heads, head_dim))
    b = out_new.to_numpy(np.float16, (n_heads, head_dim))
    # sanity of the shared kernel itself against float64 attention
    qf = q.reshape(n_heads, head_dim).astype(np.float64)
    kf = k.reshape(max_seq, n_heads, head_dim)[:seq_len].astype(np.float64)
    vf = v.reshape(max_seq, n_heads, head_dim)[:seq_len].astype(np.float64)
    s = np.einsum("hd,shd->hs", qf, kf) / np.sqrt(head_dim)
    p = np.exp(s - s.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    want = np.einsum("hs,shd->hd", p, vf)
    assert np.abs(a.astype(np.float64) - want).max() <= 5e-3
    return a, b


def test_noalloc_attention_matches_the_allocating_entry_point_twice_in_a_row(tl):
    a1, b1 = _attn_pair(tl, seed=41, n_heads=32, head_dim=128, seq_len=333, splits=8, max_seq=512)
    assert np.array_equal(a1.view(np.uint16), b1.view(np.uint16))
    # second call: other shape, other split count, stale contents of the shared array in place
    a2, b2 = _attn_pair(tl, seed=42, n_heads=6, head_dim=48, seq_len=77, splits=3, max_seq=128)
    assert np.array_equal(a2.view(np.uint16), b2.view(np.uint16))
    assert tl.device_status() == 0


def test_noalloc_attention_rejects_requests_beyond_its_fixed_scratch(tl):
    lib = tl.load()
    d = tl.DeviceBuffer(1 << 16)
    # 129 heads: over the head limit; 64 heads x 16 splits x 258: over the partial-result limit;
    # a head size and a split count whose product with the rest would wrap a 64-bit size
    for (h, hd, splits) in ((129, 16, 1), (64, 256, 16), (2, 2 ** 31 - 2, 1), (128, 128, 2 ** 31 - 1)):
        rc = lib.tl_attn_decode_f16_noalloc(d.ptr, d.ptr, d.ptr, d.ptr, h, hd, 4, splits, None)
        assert rc == 1, "expected TL_ERR_INVALID_ARGUMENT"
        assert b"exceeds the built-in scratch" in lib.tl_last_error()
