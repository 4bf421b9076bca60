"""GPU parity at the Llama2-7B layer shape (dim 4096, hidden 11008, 32 heads of 128) and over the
whole 24-point matmul sweep, all through the C ABI.

The model here is ONE 7B-shaped layer with a 2000-row vocabulary, so that the CPU oracle finishes
in seconds; the kernels, their tilings (K = 4096 / 11008, 148-CTA row splits, the last ring chunk
partly filled) and the fused epilogues are the ones every benchmark number comes from.

Two oracles are used on purpose. Reference-order numerics is compared BIT FOR BIT with the CPU
path as the reference ships it. Fast numerics is compared, within the stated tolerance, with the
oracle whose RMSNorm follows the reference's CUDA kernel (fp32 sum of squares): the CPU RMSNorm
sums in fp16 and loses 3-5 % of the scale at dim 4096 (pinned in tests/test_oracle.py), which is
a property of that CPU code, not a target for a fast kernel. The distance between the fast path
and the as-shipped CPU path is reported and bounded by that known scale loss.
"""
import os
import sys

import numpy as np
import pytest

from conftest import assert_bit_equal

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import SEED, SWEEP, SWEEP_LARGE_M, sweep_sample  # noqa: E402

from tensorlib_b200 import synth  # noqa: E402

pytestmark = pytest.mark.gpu

MATMUL_RTOL = 1e-2
# Logits of a whole layer pass: |got - want| <= 2e-2 * max(|want|, rms of the row), i.e. the matmul
# metric with twice its tolerance. (At this width the oracle itself sits 1.5e-2 away from float64
# arithmetic in absolute terms, with logits of rms 1.3 and magnitude up to 6; the float64 check below
# holds the fast path to the same distance from exact arithmetic as the reference's own.)
LOGIT_RTOL = 2e-2
LAYER = synth.LlamaConfig(dim=4096, hidden_dim=11008, n_layers=1, n_heads=32, vocab_size=2000, seq_len=256)


def max_rel_err(got, want) -> float:
    g, w = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    scale = np.sqrt((w * w).mean(axis=-1, keepdims=True)) + 1e-30
    return float((np.abs(g - w) / np.maximum(np.abs(w), scale)).max())


def rng_f16(seed: int, n: int, std: float) -> np.ndarray:
    """Seeded normals from numpy's generator: ten times faster than the counter-based fixture
    stream, and both sides of every comparison below get the same array."""
    return (np.random.default_rng(seed).standard_normal(n, dtype=np.float32) * std).astype(np.float16)


def layer_payload() -> np.ndarray:
    c = LAYER
    p = rng_f16(4096, c.payload_elems(), 0.02)
    V, d, L, h = c.vocab_size, c.dim, c.n_layers, c.hidden_dim
    # norm weights around 1 so that the norm-weight multiply is exercised too
    off = V * d
    p[off:off + L * d] = (1.0 + rng_f16(1, L * d, 0.1).astype(np.float32)).astype(np.float16)
    off += L * d + 4 * L * d * d
    p[off:off + L * d] = (1.0 + rng_f16(2, L * d, 0.1).astype(np.float32)).astype(np.float16)
    p[-d:] = (1.0 + rng_f16(3, d, 0.1).astype(np.float32)).astype(np.float16)
    return p


@pytest.fixture(scope="module")
def layer():
    return layer_payload()


def layer_tensors(payload):
    c = LAYER
    V, d, h = c.vocab_size, c.dim, c.hidden_dim
    off = V * d
    out = {}
    for name, n, shape in (("attention_norm", d, (d,)), ("wq", d * d, (d, d)), ("wk", d * d, (d, d)), ("wv", d * d, (d, d)),
                           ("wo", d * d, (d, d)), ("ffn_norm", d, (d,)), ("w1", h * d, (h, d)), ("w2", h * d, (d, h)),
                           ("w3", h * d, (h, d))):
        out[name] = payload[off:off + n].reshape(shape)
        off += n
    return out


def check_logits(got, want, what):
    got, want = got.astype(np.float32), want.astype(np.float32)
    err, rel = float(np.abs(got - want).max()), max_rel_err(got, want)
    print(f"{what}: max abs logit error {err:.4f}, relative (row-rms floor) {rel:.4f}, over {got.shape[0]} positions")
    assert rel <= LOGIT_RTOL, f"{what}: max relative logit error {rel} (abs {err})"
    s = np.sort(want, axis=1)
    clear = (s[:, -1] - s[:, -2]) > 2 * err
    assert np.array_equal(got.argmax(1)[clear], want.argmax(1)[clear]), what
    return err


def layer_forward_f64(payload, tokens):
    """The same layer in float64 on the fp16 weights: exact arithmetic up to 1e-15."""
    w, c = layer_tensors(payload), LAYER
    f = lambda a: a.astype(np.float64)
    emb = f(payload[:c.vocab_size * c.dim].reshape(c.vocab_size, c.dim))
    T, H, hd = len(tokens), c.n_heads, c.head_dim

    def norm(v, g):
        return v / np.sqrt((v * v).mean(-1, keepdims=True) + 1e-5) * f(g)

    def rope(v):
        v = v.reshape(T, H, hd // 2, 2)
        th = np.arange(T)[:, None] / (10000.0 ** (np.arange(0, hd, 2) / hd))[None, :]
        cs, sn = np.cos(th)[:, None, :], np.sin(th)[:, None, :]
        out = np.empty_like(v)
        out[..., 0] = v[..., 0] * cs - v[..., 1] * sn
        out[..., 1] = v[..., 0] * sn + v[..., 1] * cs
        return out.reshape(T, H * hd)

    x = emb[tokens]
    xn = norm(x, w["attention_norm"])
    q, k, v = rope(xn @ f(w["wq"]).T), rope(xn @ f(w["wk"]).T), xn @ f(w["wv"]).T
    att = np.empty_like(q)
    for h in range(H):
        sl = slice(h * hd, (h + 1) * hd)
        s = q[:, sl] @ k[:, sl].T / np.sqrt(float(hd))
        s[np.triu_indices(T, 1)] = -np.inf
        pr = np.exp(s - s.max(1, keepdims=True))
        att[:, sl] = (pr / pr.sum(1, keepdims=True)) @ v[:, sl]
    hres = x + att @ f(w["wo"]).T
    xn = norm(hres, w["ffn_norm"])
    g, u = xn @ f(w["w1"]).T, xn @ f(w["w3"]).T
    x2 = hres + ((g / (1 + np.exp(-g))) * u) @ f(w["w2"]).T
    return norm(x2, payload[-c.dim:]) @ emb.T


def test_fast_numerics_7b_layer_prefill_continuation_and_decode(tl, oracle, layer):
    tokens = synth.token_ids(4096, 5, 240, LAYER.vocab_size)
    m = tl.Llama2(LAYER, numerics=tl.FAST)
    m.load_payload(layer, shared_classifier=True)
    mo = oracle.llama2(LAYER, layer)
    CUDA_NORM = 3                                    # SiLU through float + RMSNorm with an fp32 sum
    # fused prefill (tcgen05 HGEMMs with the RoPE / residual / SiLU*up epilogues, flash attention)
    got200, want200 = m.forward(tokens[:200], 0, all_logits=True), mo.forward(tokens[:200], 0, CUDA_NORM)
    check_logits(got200, want200, "prefill T=200")
    exact = layer_forward_f64(layer, tokens[:200])
    e_fast, e_oracle = np.abs(got200.astype(np.float64) - exact).max(), np.abs(want200.astype(np.float64) - exact).max()
    print(f"against float64: fast path {e_fast:.4f}, oracle {e_oracle:.4f}")
    assert e_fast <= 1.25 * e_oracle + 2e-3, (e_fast, e_oracle)
    # chunked continuations over the same cache: 12 rows (skinny kernel), then 3 rows (GEMV ring, 3 columns)
    check_logits(m.forward(tokens[200:212], 200, all_logits=True), mo.forward(tokens[200:212], 200, CUDA_NORM), "chunk T=12")
    check_logits(m.forward(tokens[212:215], 212, all_logits=True), mo.forward(tokens[212:215], 212, CUDA_NORM), "chunk T=3")
    # single-token steps through forward(T=1): the five fused decode kernels per layer
    got, want = [], []
    for p in range(215, 223):
        got.append(m.forward(tokens[p:p + 1], p, all_logits=True))
        want.append(mo.forward(tokens[p:p + 1], p, CUDA_NORM))
    err = check_logits(np.concatenate(got), np.concatenate(want), "decode steps 215..222")
    # device-resident decode (CUDA-graph replay): free-running ids, judged by the oracle run along them
    first = int(got[-1][0].astype(np.float32).argmax())
    ids = m.decode_device(223, 8)
    assert tl.device_status() == 0
    tok, tol = first, 2 * max(err, 4e-3)
    for i, gid in enumerate(ids):
        lo = mo.forward(np.array([tok], dtype=np.int32), 223 + i, CUDA_NORM)[0].astype(np.float32)
        assert lo[gid] >= lo.max() - tol, f"graph decode step {i}: id {gid} is {lo.max() - lo[gid]:.4f} below the oracle's best"
        tok = int(gid)
    # the as-shipped CPU path for the record: its fp16 RMSNorm sum costs 3-5 % of scale at dim 4096
    shipped = mo.forward(tokens[:8], 0, 1).astype(np.float32)
    fast8 = m.forward(tokens[:8], 0, all_logits=True).astype(np.float32)
    rel = float(np.abs(fast8 - shipped).max() / np.abs(shipped).max())
    print(f"fast vs CPU path as shipped (fp16 RMSNorm sum): max |diff| / max |logit| = {rel:.3f}")
    assert rel <= 0.15
    m.close()


def test_reference_order_numerics_7b_layer_is_bit_identical_to_the_cpu_path(tl, oracle, layer):
    tokens = synth.token_ids(4096, 6, 20, LAYER.vocab_size)
    m = tl.Llama2(LAYER, numerics=tl.REFERENCE_ORDER)
    m.load_payload(layer, shared_classifier=True)
    mo = oracle.llama2(LAYER, layer)
    assert_bit_equal(m.forward(tokens[:16], 0, all_logits=True), mo.forward(tokens[:16], 0, 1), "prefill T=16")
    for p in range(16, 19):
        assert_bit_equal(m.forward(tokens[p:p + 1], p, all_logits=True), mo.forward(tokens[p:p + 1], p, 1), f"step {p}")
    m.close()


@pytest.mark.parametrize("n_heads_local", [32, 3])
def test_fused_entry_point_rmsnorm_qkv_rope(tl, oracle, layer, n_heads_local):
    """tl_rmsnorm_qkv_rope_f16 at (n_q 4096, dim 4096) and at a ragged width of 3 heads."""
    w = layer_tensors(layer)
    hd, dim, n_q, pos, max_seq = 128, 4096, n_heads_local * 128, 37, 64
    x = rng_f16(11, dim, 1.3)
    wq, wk, wv = (np.ascontiguousarray(w[k][:n_q]) for k in ("wq", "wk", "wv"))
    kc = rng_f16(12, max_seq * n_q, 1.0).reshape(max_seq, n_q)
    vc = rng_f16(13, max_seq * n_q, 1.0).reshape(max_seq, n_q)
    q, kc2, vc2 = tl.rmsnorm_qkv_rope(x, w["attention_norm"], wq, wk, wv, kc, vc, hd, pos)
    assert tl.device_status() == 0
    xn = oracle.rmsnorm_cuda_route(x.reshape(1, dim), w["attention_norm"])
    want_q = oracle.rope(oracle.matmul2d(xn, wq).reshape(1, n_heads_local, hd), pos).reshape(-1)
    want_k = oracle.rope(oracle.matmul2d(xn, wk).reshape(1, n_heads_local, hd), pos).reshape(-1)
    want_v = oracle.matmul2d(xn, wv).reshape(-1)
    assert max_rel_err(q, want_q) <= MATMUL_RTOL
    assert max_rel_err(kc2[pos], want_k) <= MATMUL_RTOL
    assert max_rel_err(vc2[pos], want_v) <= MATMUL_RTOL
    others = np.arange(max_seq) != pos                      # every other cache row is untouched
    assert_bit_equal(kc2[others], kc[others], "k cache rows")
    assert_bit_equal(vc2[others], vc[others], "v cache rows")


@pytest.mark.parametrize("N,K,which", [(4096, 11008, "w2"), (4096, 4096, "wo"), (1234, 4096, "wo"), (2, 11008, "w2")])
def test_fused_entry_point_gemv_residual(tl, oracle, layer, N, K, which):
    """tl_gemv_residual_f16 at the w2 / wo shapes and at ragged widths."""
    W = np.ascontiguousarray(layer_tensors(layer)[which][:N])
    x, res = rng_f16(21, K, 0.7), rng_f16(22, N, 1.0)
    got = tl.gemv_residual(x, W, res)
    assert tl.device_status() == 0
    lin = oracle.matmul2d(x.reshape(1, K), W)
    want = oracle.ewise(res, lin.reshape(-1), "add")
    # the sum before the residual add differs by fp32 summation order; the add itself is exact fp16
    assert np.abs(got.astype(np.float64) - want.astype(np.float64)).max() <= MATMUL_RTOL * max(1.0, float(np.abs(lin.astype(np.float64)).max()))
    assert max_rel_err(got, want) <= MATMUL_RTOL


@pytest.mark.parametrize("hidden", [11008, 1366])
def test_fused_entry_point_rmsnorm_gateup_swiglu(tl, oracle, layer, hidden):
    """tl_rmsnorm_gateup_swiglu_f16 (the kernel whose roofline the benchmark reports) at
    (hidden 11008, dim 4096) and at a ragged hidden width."""
    w = layer_tensors(layer)
    dim = 4096
    x = rng_f16(31, dim, 0.9)
    w1, w3 = np.ascontiguousarray(w["w1"][:hidden]), np.ascontiguousarray(w["w3"][:hidden])
    got = tl.rmsnorm_gateup_swiglu(x, w["ffn_norm"], w1, w3)
    assert tl.device_status() == 0
    xn = oracle.rmsnorm_cuda_route(x.reshape(1, dim), w["ffn_norm"])
    g = oracle.silu(oracle.matmul2d(xn, w1).reshape(-1), True)
    want = oracle.ewise(g, oracle.matmul2d(xn, w3).reshape(-1), "mul")
    # a product of two matmul results: twice the matmul tolerance
    assert max_rel_err(got, want) <= 2 * MATMUL_RTOL


def test_matmul_sweep_all_24_points(tl, oracle, golden_sweep):
    """Every (K, N) x M point of the benchmark's matmul sweep at full size. M = 1 and 8: every
    output against the oracle and the reference-made fixture heads. M = 32..2048: sixteen seeded
    rows x all N columns against the oracle (each output is an independent dot product) and the
    fixture samples the reference produced."""
    for (K, N) in SWEEP:
        W = synth.normal_f16(SEED, synth.TID_SWEEP_W, N * K, 0.02).reshape(N, K)
        x_all = synth.normal_f16(SEED, synth.TID_SWEEP_X, 2048 * K, 1.0).reshape(2048, K)
        for M in (1, 8):
            x = np.ascontiguousarray(x_all.reshape(-1)[:M * K].reshape(M, K))
            got = tl.matmul2d(x, W, numerics=tl.FAST)
            assert max_rel_err(got, oracle.matmul2d(x, W)) <= MATMUL_RTOL, (K, N, M)
            head, want = got.reshape(-1)[:64].astype(np.float64), golden_sweep[f"head_K{K}_N{N}_M{M}"].astype(np.float64)
            scale = np.sqrt((want * want).mean())
            assert (np.abs(head - want) / np.maximum(np.abs(want), scale)).max() <= MATMUL_RTOL, (K, N, M)
        for M in SWEEP_LARGE_M:
            x = np.ascontiguousarray(x_all.reshape(-1)[:M * K].reshape(M, K))
            got = tl.matmul2d(x, W, numerics=tl.FAST)
            rows = np.unique(np.concatenate([np.random.default_rng(M + K + N).choice(M, 13, replace=False), [0, M // 2 + 1, M - 1]]))
            want = oracle.matmul2d(np.ascontiguousarray(x[rows]), W)
            assert max_rel_err(got[rows], want) <= MATMUL_RTOL, (K, N, M)
            r3, cols = sweep_sample(M, N)
            fixture = golden_sweep[f"sample_K{K}_N{N}_M{M}"]
            assert max_rel_err(got[np.ix_(r3, cols)], fixture) <= MATMUL_RTOL, (K, N, M)
            assert np.isfinite(got.astype(np.float32)).all()
        assert tl.device_status() == 0
