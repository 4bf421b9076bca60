"""GPU parity, single operators, all through the C ABI.

Reference-order numerics must be BIT-IDENTICAL to the oracle (and to the golden fixtures the
reference itself produced). Fast numerics must stay within the stated tolerance:
matmul max relative error <= 1e-2 against the oracle (fp16 inputs, fp32 accumulate), where the
relative error of an element is |got - want| / max(|want|, row_scale) with row_scale the RMS of
the oracle's output row (a pure per-element ratio is meaningless next to cancellation zeros).
"""
import os
import sys

import numpy as np
import pytest

from conftest import assert_bit_equal

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import SEED, SWEEP, op_inputs  # noqa: E402

from tensorlib_b200 import synth  # noqa: E402

pytestmark = pytest.mark.gpu

MATMUL_RTOL = 1e-2


def max_rel_err(got: np.ndarray, want: np.ndarray) -> float:
    g, w = got.astype(np.float64), want.astype(np.float64)
    scale = np.sqrt((w * w).mean(axis=-1, keepdims=True)) + 1e-30
    return float((np.abs(g - w) / np.maximum(np.abs(w), scale)).max())


# ---- reference-order numerics: bit-exact -----------------------------------------------------------
def test_refmode_ops_bit_exact_vs_golden(tl, golden_ops):
    for name, args in op_inputs().items():
        if name.startswith("mm_"):
            assert_bit_equal(tl.matmul2d(*args, numerics=tl.REFERENCE_ORDER), golden_ops[name], name)
        elif name.startswith("norm"):
            assert_bit_equal(tl.rms_norm(*args, numerics=tl.REFERENCE_ORDER), golden_ops[name], name)
        elif name.startswith("rope"):
            assert_bit_equal(tl.apply_rotary_emb(*args), golden_ops[name], name)
        elif name == "softmax":
            assert_bit_equal(tl.softmax(*args, numerics=tl.REFERENCE_ORDER), golden_ops[name], name)
        elif name == "silu":
            assert_bit_equal(tl.silu(args[0], True), golden_ops["silu_float"], "silu_float")
            assert_bit_equal(tl.silu(args[0], False), golden_ops["silu_half"], "silu_half")
        elif name == "argmax":
            assert np.array_equal(tl.argmax(*args), golden_ops[name])


def test_refmode_elementwise_all_fp16_values(tl, oracle):
    allh = np.arange(65536, dtype=np.uint16).view(np.float16)
    fin = np.ascontiguousarray(allh[np.isfinite(allh)])
    rolled = np.ascontiguousarray(np.roll(fin, 12345))
    assert_bit_equal(tl.add(fin, rolled), oracle.ewise(fin, rolled, "add"), "add")
    assert_bit_equal(tl.mul(fin, rolled), oracle.ewise(fin, rolled, "mul"), "mul")
    assert_bit_equal(tl.silu(fin, True), oracle.silu(fin, True), "silu float")
    assert_bit_equal(tl.silu(fin, False), oracle.silu(fin, False), "silu half")
    for hd in (48, 128):
        s = float(np.sqrt(float(hd)))
        assert_bit_equal(tl.div_scalar(fin, s), oracle.ewise(fin, None, "sdiv", s), "scalar div")


@pytest.mark.parametrize("M,N,K", [(1, 288, 288), (1, 768, 288), (1, 288, 768), (7, 33, 129), (16, 300, 48),
                                   (1, 64, 11008), (3, 1000, 4096), (1, 1, 8), (2, 5, 1)])
def test_refmode_matmul_bit_exact_vs_oracle(tl, oracle, M, N, K):
    A = synth.normal_f16(21, 1, M * K, 1.0).reshape(M, K)
    W = synth.normal_f16(21, 2, N * K, 0.02).reshape(N, K)
    assert_bit_equal(tl.matmul2d(A, W, numerics=tl.REFERENCE_ORDER), oracle.matmul2d(A, W), f"matmul {M}x{N}x{K}")


def test_refmode_batched_matmul_broadcast(tl, oracle):
    a = synth.normal_f16(22, 1, 6 * 5 * 48, 1.0).reshape(6, 5, 48)
    b = synth.normal_f16(22, 2, 6 * 9 * 48, 1.0).reshape(6, 9, 48)
    assert_bit_equal(tl.matmul_batched(a, b, numerics=tl.REFERENCE_ORDER), oracle.bmm_nt(a, b), "bmm")
    b1 = np.ascontiguousarray(b[:1])
    want = oracle.bmm_nt(a, np.ascontiguousarray(np.broadcast_to(b1, b.shape)))
    assert_bit_equal(tl.matmul_batched(a, b1, numerics=tl.REFERENCE_ORDER), want, "bmm, broadcast rhs")


def test_refmode_softmax_and_norm_ragged(tl, oracle):
    for rows, cols in ((1, 1), (3, 17), (64, 144), (2, 2048)):
        x = synth.normal_f16(23, rows * 7 + cols, rows * cols, 3.0).reshape(rows, cols)
        assert_bit_equal(tl.softmax(x, numerics=tl.REFERENCE_ORDER), oracle.softmax(x), f"softmax {rows}x{cols}")
    for T, D in ((1, 288), (5, 768), (2, 4096), (1, 11008)):
        x = synth.normal_f16(24, T * 3 + D, T * D, 1.7).reshape(T, D)
        w = synth.normal_f16(24, 99, D, 1.0)
        assert_bit_equal(tl.rms_norm(x, w, numerics=tl.REFERENCE_ORDER), oracle.rmsnorm(x, w), f"rmsnorm {T}x{D}")


def test_rope_positions_to_the_end_of_the_context(tl, oracle):
    for (T, Hh, hd, pos) in ((1, 6, 48, 255), (4, 32, 128, 2044), (16, 6, 48, 0)):
        x = synth.normal_f16(25, pos + hd, T * Hh * hd, 1.0).reshape(T, Hh, hd)
        assert_bit_equal(tl.apply_rotary_emb(x, pos), oracle.rope(x, pos), f"rope hd={hd} pos={pos}")


def test_argmax_ties_and_embedding(tl, oracle):
    x = np.zeros((3, 32000), dtype=np.float16)          # all equal: index 0 wins
    x[1, 31999] = 1.0
    x[2, 7] = x[2, 9000] = 2.0
    assert tl.argmax(x).tolist() == [0, 31999, 7] == oracle.argmax(x).tolist()
    table = synth.normal_f16(26, 1, 100 * 288, 0.02).reshape(100, 288)
    tok = np.array([0, 99, 5, 5], dtype=np.int32)
    assert_bit_equal(tl.embedding(table, tok), table[tok], "embedding gather")


def test_empty_and_invalid_arguments(tl):
    e = np.zeros((0, 64), dtype=np.float16)
    w = np.zeros((16, 64), dtype=np.float16)
    assert tl.matmul2d(e, w).shape == (0, 16)
    with pytest.raises(tl.TLError) as err:
        tl.matmul2d(w, w, numerics=7)
    assert err.value.status == 1
    with pytest.raises(tl.TLError) as err:
        tl.div_scalar(w, 0.0)                             # reference: throws "Division by zero."
    assert err.value.status == 1 and "zero" in str(err.value)


# ---- fast numerics: tolerance ------------------------------------------------------------------------
@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 7, 8, 9, 16, 17, 25, 32])
def test_fast_gemv_small_m(tl, oracle, M):
    for (N, K) in ((288, 288), (768, 288), (288, 768), (1000, 4096), (513, 1032), (64, 11008)):
        A = synth.normal_f16(31, M, M * K, 1.0).reshape(M, K)
        W = synth.normal_f16(31, 2, N * K, 0.02).reshape(N, K)
        got, want = tl.matmul2d(A, W, numerics=tl.FAST), oracle.matmul2d(A, W)
        assert max_rel_err(got, want) <= MATMUL_RTOL, (M, N, K)


@pytest.mark.parametrize("M,N,K", [(16, 256, 1024), (130, 136, 264), (128, 512, 4096), (33, 77, 300), (300, 1000, 520)])
def test_fast_matmul_larger_m(tl, oracle, M, N, K):
    A = synth.normal_f16(32, 1, M * K, 1.0).reshape(M, K)
    W = synth.normal_f16(32, 2, N * K, 0.02).reshape(N, K)
    got, want = tl.matmul2d(A, W, numerics=tl.FAST), oracle.matmul2d(A, W)
    assert max_rel_err(got, want) <= MATMUL_RTOL, (M, N, K)


def test_fast_matmul_host_entry_point(tl, oracle):
    A = synth.normal_f16(33, 1, 4 * 4096, 1.0).reshape(4, 4096)
    W = synth.normal_f16(33, 2, 640 * 4096, 0.02).reshape(640, 4096)
    assert max_rel_err(tl.matmul2d_host(A, W, numerics=tl.FAST), oracle.matmul2d(A, W)) <= MATMUL_RTOL


def test_fast_sweep_shapes_vs_golden_heads(tl, golden_sweep):
    """Full-size sweep shapes at M = 1 and 8: first 64 outputs against the reference's own."""
    for (K, N) in SWEEP:
        W = synth.normal_f16(SEED, synth.TID_SWEEP_W, N * K, 0.02).reshape(N, K)
        for M in (1, 8):
            x = synth.normal_f16(SEED, synth.TID_SWEEP_X, M * K, 1.0).reshape(M, K)
            got = tl.matmul2d(x, W, numerics=tl.FAST).reshape(-1)[:64].astype(np.float64)
            want = golden_sweep[f"head_K{K}_N{N}_M{M}"].astype(np.float64)
            scale = np.sqrt((want * want).mean())
            assert (np.abs(got - want) / np.maximum(np.abs(want), scale)).max() <= MATMUL_RTOL, (K, N, M)


def test_fast_matmul_linearity_at_full_size(tl):
    """Size-independent property at a sweep shape too large for the CPU oracle in a test:
    W.(2x) == 2.(W.x) exactly (scaling by two is exact in fp16 and in the fp32 accumulator) for
    every output outside the fp16 subnormal range, where the final rounding step is absolute."""
    K, N, M = 4096, 11008, 128
    W = synth.normal_f16(34, 1, N * K, 0.02).reshape(N, K)
    x = synth.normal_f16(34, 2, M * K, 0.5).reshape(M, K)
    y1 = tl.matmul2d(x, W, numerics=tl.FAST).astype(np.float32)
    y2 = tl.matmul2d((x * np.float16(2)).astype(np.float16), W, numerics=tl.FAST).astype(np.float32)
    normal = np.abs(y1) >= 2.0 ** -13
    assert normal.mean() > 0.99
    assert np.array_equal(y2[normal], 2 * y1[normal])
    assert np.abs(y2 - 2 * y1).max() <= 2.0 ** -23
    rows = [0, 63, 127]                                   # spot rows against float64
    want = x[rows].astype(np.float64) @ W.astype(np.float64).T
    assert max_rel_err(y1[rows], want) <= MATMUL_RTOL


def test_fast_softmax_and_norm_close(tl, oracle):
    x = synth.normal_f16(35, 1, 40 * 300, 3.0).reshape(40, 300)
    got = tl.softmax(x, numerics=tl.FAST).astype(np.float64)
    xf = x.astype(np.float64)
    e = np.exp(xf - xf.max(axis=1, keepdims=True))
    exact = e / e.sum(axis=1, keepdims=True)
    assert np.abs(got - exact).max() <= 6e-4                 # half an fp16 ulp at 1.0
    # the reference sums the row in fp16, so it is only loosely comparable
    want = oracle.softmax(x).astype(np.float64)
    assert (np.abs(got - want) <= 3e-2 * want + 1e-4).all()
    xn = synth.normal_f16(35, 2, 4 * 4096, 1.0).reshape(4, 4096)
    w = synth.normal_f16(35, 3, 4096, 1.0)
    got = tl.rms_norm(xn, w, numerics=tl.FAST).astype(np.float64)
    xf = xn.astype(np.float64)
    want = xf / np.sqrt((xf * xf).mean(axis=1, keepdims=True) + 1e-5) * w.astype(np.float64)
    assert np.abs(got - want).max() <= 1e-2


# ---- fused prefill attention (tcgen05 / TMEM), head_dim 128 ---------------------------------------------
def _attention_f64(q, k, v, start_pos, n_heads):
    """softmax(q k^T / sqrt(hd) + causal mask) v in float64 on the fp16 inputs."""
    T, width = q.shape
    hd, S = width // n_heads, start_pos + q.shape[0]
    out = np.empty((T, width))
    for h in range(n_heads):
        qh, kh, vh = (a[:, h * hd:(h + 1) * hd].astype(np.float64) for a in (q, k[:S], v[:S]))
        s = qh @ kh.T / np.sqrt(hd)
        s[np.arange(S)[None, :] > (start_pos + np.arange(T))[:, None]] = -np.inf
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h * hd:(h + 1) * hd] = (p / p.sum(axis=1, keepdims=True)) @ vh
    return out


@pytest.mark.parametrize("T,start_pos,n_heads", [(128, 0, 2), (200, 0, 3), (64, 0, 1), (1, 0, 2), (130, 77, 2),
                                                  (333, 190, 2), (512, 0, 4)])
def test_fused_prefill_attention(tl, T, start_pos, n_heads):
    hd, S = 128, start_pos + T
    max_seq = S + 5
    q = synth.normal_f16(51, 1, T * n_heads * hd, 1.0).reshape(T, n_heads * hd)
    k = synth.normal_f16(51, 2, max_seq * n_heads * hd, 1.0).reshape(max_seq, n_heads * hd)
    v = synth.normal_f16(51, 3, max_seq * n_heads * hd, 1.0).reshape(max_seq, n_heads * hd)
    got = tl.attn_prefill(q, k, v, start_pos, n_heads).astype(np.float64)
    want = _attention_f64(q, k, v, start_pos, n_heads)
    assert tl.device_status() == 0
    # fp16 probabilities and an fp16 result: absolute error against unit-variance values
    assert np.abs(got - want).max() <= 8e-3, (T, start_pos, np.abs(got - want).max())


def test_fused_prefill_attention_peaked_scores_rescale(tl):
    """Scores that keep growing along the sequence force the running-max rescale of the accumulator."""
    T, n_heads, hd = 256, 1, 128
    q = np.full((T, hd), 0.25, np.float16)
    k = (np.linspace(0.0, 3.0, T, dtype=np.float64)[:, None] * np.ones((1, hd))).astype(np.float16)
    v = synth.normal_f16(52, 3, T * hd, 1.0).reshape(T, hd)
    got = tl.attn_prefill(q, k, v, 0, n_heads).astype(np.float64)
    want = _attention_f64(q, k, v, 0, n_heads)
    assert tl.device_status() == 0
    assert np.abs(got - want).max() <= 8e-3


def test_fused_prefill_attention_rejects_other_head_sizes(tl):
    d = tl.DeviceBuffer(1 << 16)
    rc = tl.load().tl_attn_prefill_f16(d.ptr, d.ptr, d.ptr, d.ptr, 4, 0, 2, 48, None)
    assert rc == 4  # TL_ERR_UNSUPPORTED


# ---- CTA-pair HGEMM (cta_group::2): forced onto small shapes in a child process -------------------------
_PAIR_CHILD = r"""
import sys, numpy as np
sys.path.insert(0, sys.argv[1])
import tensorlib_b200 as tl
from tensorlib_b200 import synth
tl.init(0)
worst = 0.0
for (M, N, K) in ((512, 1024, 512), (384, 768, 200), (2048, 512, 4096), (300, 256, 1032), (129, 512, 64), (1100, 2304, 2048)):
    A = synth.normal_f16(71, 1, M * K, 1.0).reshape(M, K)
    W = synth.normal_f16(71, 2, N * K, 0.02).reshape(N, K)
    want = A.astype(np.float64) @ W.astype(np.float64).T
    scale = np.sqrt((want * want).mean(axis=-1, keepdims=True)) + 1e-30
    for rep in range(2):      # twice: the stream-K arrival counters must be back at zero after a launch
        got = tl.matmul2d(A, W, numerics=tl.FAST).astype(np.float64)
        worst = max(worst, float((np.abs(got - want) / np.maximum(np.abs(want), scale)).max()))
assert tl.device_status() == 0
print("WORST", worst)
"""


@pytest.mark.parametrize("mode", ["always", "always512", "streamk", "streamk512", "never"])
def test_hgemm_pair_and_single_kernels_agree_with_float64(tl, mode, tmp_path):
    import subprocess
    script = tmp_path / "child.py"
    script.write_text(_PAIR_CHILD)
    root = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
    env = dict(os.environ, TL_HGEMM_PAIR=mode)
    r = subprocess.run([sys.executable, str(script), root], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    worst = float(r.stdout.strip().split("WORST")[-1])
    assert worst <= 2e-3, worst      # fp16 rounding of the result only: both kernels accumulate in fp32


@pytest.mark.parametrize("M,N,K", [(5, 4096, 1024), (32, 4224, 1032), (100, 4096, 2048), (128, 8192, 512), (2, 5000, 4096)])
def test_skinny_matmul_cluster_reduction_shapes(tl, oracle, M, N, K):
    """Shapes whose weight tiles split evenly over the SMs: the sharers of a tile reduce through
    distributed shared memory (ragged K, a last tile beyond N, M not a multiple of the split)."""
    A = synth.normal_f16(81, 1, M * K, 1.0).reshape(M, K)
    W = synth.normal_f16(81, 2, N * K, 0.02).reshape(N, K)
    got, want = tl.matmul2d(A, W, numerics=tl.FAST), oracle.matmul2d(A, W)
    assert tl.device_status() == 0
    assert max_rel_err(got, want) <= MATMUL_RTOL, (M, N, K)


def test_bounded_wait_runs_out_and_the_library_stays_usable(tl, oracle):
    """A consumer GEMV whose tensor-parallel input is never posted: the wait is limited to 1024
    polls, the kernel returns by itself, the status word reads TL_ERR_TIMEOUT exactly once, and the
    next ordinary call works. No trap, no fault, no unbounded spin."""
    assert tl.device_status() == 0
    tl.check(tl.load().tl_selftest_unposted_exchange(1024, None), "tl_selftest_unposted_exchange")
    assert tl.device_status() == 6                        # TL_ERR_TIMEOUT
    assert tl.device_status() == 0                        # reading it cleared it
    A = synth.normal_f16(91, 1, 4096, 1.0).reshape(1, 4096)
    W = synth.normal_f16(91, 2, 512 * 4096, 0.02).reshape(512, 4096)
    assert max_rel_err(tl.matmul2d(A, W, numerics=tl.FAST), oracle.matmul2d(A, W)) <= MATMUL_RTOL
    assert tl.device_status() == 0
    assert tl.load().tl_selftest_unposted_exchange(0, None) == 1      # out-of-range limit is refused


@pytest.mark.parametrize("world,owner,M,dim,K", [(2, 1, 512, 4096, 256), (4, 2, 512, 4096, 192), (8, 5, 1024, 4096, 128),
                                                 (8, 0, 2048, 512, 64), (4, 3, 1024, 5120, 64)])
def test_tp_prefill_exchange_with_the_ranks_emulated_on_one_gpu(tl, world, owner, M, dim, K):
    """The K-split matmul in signalling mode followed by the owner-side reduce + RMSNorm + gather kernel, for
    2, 4 and 8 ranks, on one GPU: every rank's partial is the same matrix P, so the owner's rows must come out
    as residual + half(world x P), normalised, in every destination copy, and nobody else's rows are touched."""
    A = synth.normal_f16(77, 1, M * K, 1.0).reshape(M, K)
    B = synth.normal_f16(77, 2, dim * K, 0.05).reshape(dim, K)
    rpo = M // world
    resid = synth.normal_f16(77, 3, rpo * dim, 1.0).reshape(rpo, dim)
    w = (1.0 + synth.normal_f16(77, 4, dim, 0.1).astype(np.float32)).astype(np.float16)
    h, xn = tl.selftest_tp_prefill_exchange(A, B, resid, w, world, owner)
    assert tl.device_status() == 0
    rows = slice(owner * rpo, (owner + 1) * rpo)
    P = (A[rows].astype(np.float32) @ B.astype(np.float32).T).astype(np.float16)          # the matmul's fp16 result
    # the kernel adds the `world` fp16 partials in fp32, rounds once, then adds the residual in fp16
    s16 = (P.astype(np.float32) * world).astype(np.float16)
    want_h = (resid.astype(np.float32) + s16.astype(np.float32)).astype(np.float16)
    # P itself carries the matmul's rounding: allow one fp16 ulp of P (times world) in h
    tol = np.maximum(np.abs(want_h.astype(np.float32)), 1.0) * 2e-3 * world
    assert np.all(np.abs(h.astype(np.float32) - want_h.astype(np.float32)) <= tol)
    hf = h.astype(np.float32)
    want_xn = hf * (1.0 / np.sqrt((hf * hf).mean(axis=1, keepdims=True) + 1e-5)) * w.astype(np.float32)
    for d in range(world):
        got = xn[d].astype(np.float32)
        assert np.max(np.abs(got[rows] - want_xn)) <= 4e-3 * max(1.0, float(np.abs(want_xn).max())), d
        mask = np.ones(M, bool); mask[rows] = False
        assert not got[mask].any(), d                               # other owners' rows untouched
        assert np.array_equal(xn[d][rows], xn[0][rows])             # every destination holds the same bits


def test_batched_matmul_with_a_batch_stride_that_is_not_a_multiple_of_8(tl, oracle):
    """Aligned pitches but an odd batch stride: the tensor-core kernels cannot take it, the call
    must fall through to the any-shape kernel instead of failing."""
    b, M, N, K = 3, 16, 24, 64
    pad = 4                                               # batch stride M*K + 4 elements
    A = synth.normal_f16(92, 1, b * (M * K + pad), 1.0)
    Bt = synth.normal_f16(92, 2, b * N * K, 0.05).reshape(b, N, K)
    dA, dB, dC = tl.DeviceBuffer.from_numpy(A), tl.DeviceBuffer.from_numpy(Bt), tl.DeviceBuffer(b * M * N * 2)
    tl.check(tl.load().tl_matmul_batched_f16(dA.ptr, dB.ptr, dC.ptr, b, M, N, K, K, K, N, M * K + pad, N * K, M * N,
                                             tl.FAST, None), "tl_matmul_batched_f16")
    got = dC.to_numpy(np.float16, (b, M, N))
    a3 = np.stack([A[i * (M * K + pad): i * (M * K + pad) + M * K].reshape(M, K) for i in range(b)])
    assert max_rel_err(got, oracle.bmm_nt(np.ascontiguousarray(a3), Bt)) <= MATMUL_RTOL


@pytest.mark.parametrize("T", [1, 3, 8, 20])
def test_linear_entry_point_matches_the_oracle(tl, oracle, T):
    """tl_linear_f16 (nn::Linear::forward with a constant weight): same results as the matmul entry point."""
    for (N, K) in ((768, 288), (1000, 4096), (4096, 11008)):
        x = synth.normal_f16(93, T, T * K, 1.0).reshape(T, K)
        W = synth.normal_f16(93, 2, N * K, 0.02).reshape(N, K)
        got = tl.linear(x, W)
        assert max_rel_err(got, oracle.matmul2d(x, W)) <= MATMUL_RTOL, (T, N, K)
        assert_bit_equal(got, tl.matmul2d(x, W, numerics=tl.FAST), "linear vs matmul2d")
    assert tl.device_status() == 0
