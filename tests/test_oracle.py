"""CPU suite, part 1: the oracle is pinned.

* the plain-C restatement (oracle/tl_oracle.c) reproduces the golden fixtures that were generated
  by the reference's own CPU code (tests/golden/make_golden.py);
* where oracle/_ref is built, the restatement is compared live with the reference on further
  seeded inputs, including every finite fp16 value for the elementwise operators.
"""
import hashlib
import os
import sys

import numpy as np
import pytest

from conftest import assert_bit_equal

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import N_GEN, SEED, SWEEP, op_inputs  # noqa: E402

from tensorlib_b200 import synth  # noqa: E402


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).view(np.uint8).tobytes()).hexdigest()


def test_ops_match_golden(oracle, golden_ops):
    for name, args in op_inputs().items():
        if name.startswith("mm_"):
            assert_bit_equal(oracle.matmul2d(*args), golden_ops[name], name)
        elif name.startswith("norm"):
            assert_bit_equal(oracle.rmsnorm(*args), golden_ops[name], name)
        elif name.startswith("rope"):
            assert_bit_equal(oracle.rope(*args), golden_ops[name], name)
        elif name == "softmax":
            assert_bit_equal(oracle.softmax(*args), golden_ops[name], name)
        elif name == "silu":
            assert_bit_equal(oracle.silu(args[0], True), golden_ops["silu_float"], "silu_float")
            assert_bit_equal(oracle.silu(args[0], False), golden_ops["silu_half"], "silu_half")
        elif name == "argmax":
            assert np.array_equal(oracle.argmax(*args), golden_ops[name])
            assert golden_ops[name][1] == 500  # lowest index wins the tie planted at 500 / 20000


def test_sweep_small_m_matches_golden(oracle, golden_sweep):
    K, N = SWEEP[0]
    W = synth.normal_f16(SEED, synth.TID_SWEEP_W, N * K, 0.02).reshape(N, K)
    for M in (1, 8):
        x = synth.normal_f16(SEED, synth.TID_SWEEP_X, M * K, 1.0).reshape(M, K)
        y = oracle.matmul2d(x, W)
        assert sha(y) == str(golden_sweep[f"sha_K{K}_N{N}_M{M}"])
        assert_bit_equal(y.reshape(-1)[:64], golden_sweep[f"head_K{K}_N{N}_M{M}"], "sweep head")


@pytest.mark.parametrize("tag,mode", [("A", 0), ("B", 1)])
def test_tiny_llama2_matches_golden(oracle, golden_tiny, tiny_payload, tag, mode):
    model = oracle.llama2(synth.TINY, tiny_payload)
    prompt = golden_tiny["prompt"]
    assert np.array_equal(prompt, synth.prompt_tokens(synth.TINY, SEED, prompt.size))
    ids, logits = model.generate(prompt, N_GEN, silu_mode=mode, keep_logits=True)
    assert np.array_equal(ids, golden_tiny[f"ids_{tag}"])
    assert sha(logits) == str(golden_tiny[f"logits_sha_{tag}"])
    assert_bit_equal(logits[list(golden_tiny["keep_steps"])], golden_tiny[f"logits_{tag}"], "kept logits")


@pytest.mark.parametrize("tag,mode", [("A", 0), ("B", 1)])
def test_tiny_llama2_teacher_forced_matches_golden(oracle, golden_tiny, tiny_payload, tag, mode):
    model = oracle.llama2(synth.TINY, tiny_payload)
    forced = golden_tiny["forced_tokens"]
    lg = [model.forward(forced[:16], 0, mode)]
    for i in range(16, 24):
        lg.append(model.forward(forced[i:i + 1], i, mode))
    lg = np.concatenate(lg, axis=0)
    assert sha(lg) == str(golden_tiny[f"forced_sha_{tag}"])
    assert np.array_equal(oracle.argmax(np.ascontiguousarray(lg)), golden_tiny[f"forced_argmax_{tag}"])


def test_oracle_is_thread_count_independent(oracle):
    A = synth.normal_f16(3, 1, 4 * 512, 1.0).reshape(4, 512)
    W = synth.normal_f16(3, 2, 96 * 512, 0.02).reshape(96, 512)
    n = oracle.max_threads()
    oracle.set_threads(1)
    y1 = oracle.matmul2d(A, W)
    oracle.set_threads(n)
    assert_bit_equal(y1, oracle.matmul2d(A, W), "1 vs N threads")


# ---- live comparison with the compiled reference (skipped where it is not built) ----------------
def test_restatement_vs_reference_elementwise_all_values(oracle, ref):
    allh = np.arange(65536, dtype=np.uint16).view(np.float16)
    fin = np.ascontiguousarray(allh[np.isfinite(allh)])
    rolled = np.ascontiguousarray(np.roll(fin, 12345))
    assert_bit_equal(oracle.silu(fin, True), ref.silu(fin, True), "silu float")
    assert_bit_equal(oracle.silu(fin, False), ref.silu(fin, False), "silu half")
    assert_bit_equal(oracle.ewise(fin, rolled, "add"), ref.ewise(fin, rolled, "add"), "add")
    assert_bit_equal(oracle.ewise(fin, rolled, "mul"), ref.ewise(fin, rolled, "mul"), "mul")
    for hd in (48, 128):
        s = float(np.sqrt(float(hd)))
        assert_bit_equal(oracle.ewise(fin, None, "sdiv", s), ref.ewise(fin, None, "sdiv", s), "scalar div")


def test_restatement_vs_reference_ops(oracle, ref):
    x = synth.normal_f16(11, 1, 6 * 768, 1.5).reshape(6, 768)
    w = synth.normal_f16(11, 2, 768, 1.0)
    assert_bit_equal(oracle.rmsnorm(x, w), ref.rmsnorm(x, w), "rmsnorm")
    W = synth.normal_f16(11, 3, 100 * 768, 0.02).reshape(100, 768)
    assert_bit_equal(oracle.matmul2d(x, W), ref.matmul2d(x, W), "matmul2d")
    assert_bit_equal(oracle.linear(x, W), ref.linear(x, W), "linear via Tensor::matmul")
    a = synth.normal_f16(11, 4, 3 * 4 * 48, 1.0).reshape(3, 4, 48)
    b = synth.normal_f16(11, 5, 3 * 9 * 48, 1.0).reshape(3, 9, 48)
    assert_bit_equal(oracle.bmm_nt(a, b), ref.bmm_nt(a, b), "batched matmul")
    r = synth.normal_f16(11, 6, 5 * 6 * 48, 1.0).reshape(5, 6, 48)
    assert_bit_equal(oracle.rope(r, 250), ref.rope(r, 250), "rope")
    s = synth.normal_f16(11, 7, 20 * 257, 4.0).reshape(20, 257)
    assert_bit_equal(oracle.softmax(s), ref.softmax(s), "softmax")


def test_restatement_vs_reference_model(oracle, ref, tiny_payload):
    mo, mr = oracle.llama2(synth.TINY, tiny_payload), ref.llama2(synth.TINY, tiny_payload)
    tok = synth.token_ids(77, 1, 12, synth.TINY.vocab_size)
    for mode in (0, 1):
        lo, ho = mo.forward(tok, 0, mode, want_hidden=True)
        lr, hr = mr.forward(tok, 0, mode, want_hidden=True)
        assert_bit_equal(ho, hr, "hidden states")
        assert_bit_equal(lo, lr, "prefill logits")
        assert_bit_equal(mo.forward(tok[:1], 12, mode), mr.forward(tok[:1], 12, mode), "decode logits")


# ---- the RMSNorm of the reference at the 7B width --------------------------------------------------
def test_cpu_rmsnorm_fp16_sum_loses_scale_at_dim_4096_and_the_cuda_route_does_not(oracle, ref):
    """The reference's CPU RMSNorm adds the squares in fp16: once the running sum reaches 2048 an
    addend below 1 is rounded away, so at dim 4096 the mean comes out too small and the result
    3-5 % too large. The reference's CUDA kernel sums in fp32; the oracle restates both. This pins
    the size of the effect (and that the restatement of the CPU form still equals the reference at
    this width), which is why fast-numerics parity at dim 4096 is stated against the CUDA form."""
    D = 4096
    x = synth.normal_f16(41, 1, 3 * D, 1.0).reshape(3, D)
    w = synth.normal_f16(41, 2, D, 1.0)
    xf = x.astype(np.float64)
    exact = xf / np.sqrt((xf * xf).mean(axis=1, keepdims=True) + 1e-5) * w.astype(np.float64)
    cpu = oracle.rmsnorm(x, w)
    assert_bit_equal(cpu, ref.rmsnorm(x, w), "CPU form at dim 4096")
    big = np.abs(exact) > 0.5
    ratio = cpu.astype(np.float64)[big] / exact[big]
    assert 1.03 <= ratio.min() and ratio.max() <= 1.06, (ratio.min(), ratio.max())
    cuda_form = oracle.rmsnorm_cuda_route(x, w).astype(np.float64)
    # half(rms) carries 2^-11 relative error and the two fp16 roundings another 2^-11 each
    assert np.abs(cuda_form - exact).max() <= 3 * 2.0 ** -11 * np.abs(exact).max()
    # at the tiny model's width the two forms agree to fp16 rounding
    xs = synth.normal_f16(41, 3, 2 * 288, 1.0).reshape(2, 288)
    ws = np.ones(288, dtype=np.float16)
    a, b = oracle.rmsnorm(xs, ws).astype(np.float64), oracle.rmsnorm_cuda_route(xs, ws).astype(np.float64)
    assert np.abs(a - b).max() <= 4e-3 * np.abs(b).max()


# ---- the rest of the Device<half> surface: restatement against the reference's CPU<half> ------------
def test_restatement_vs_reference_unary_binary_reduce_cast(oracle, ref):
    import device_cases as dc
    fin, pos = dc.finite_halfs(), dc.positive_halfs()
    for op in dc.UNARY_ON_ALL:
        assert_bit_equal(oracle.unary(fin, op), ref.unary(fin, op), op)
    for op in dc.UNARY_ON_POSITIVE:
        assert_bit_equal(oracle.unary(pos, op), ref.unary(pos, op), op)
    rolled = np.ascontiguousarray(np.roll(fin, 777))
    for op in ("add", "sub", "mul"):
        assert_bit_equal(oracle.binary(fin, rolled, op), ref.binary(fin, rolled, op), op)
    nz = np.ascontiguousarray(np.roll(pos, 4321)[:fin.size - 30000])
    a = np.ascontiguousarray(fin[:nz.size])
    assert_bit_equal(oracle.binary(a, nz, "div"), ref.binary(a, nz, "div"), "div")
    for s in dc.SCALARS:
        for op in ("add", "sub", "mul", "div"):
            assert_bit_equal(oracle.binary(fin, s, op), ref.binary(fin, s, op), f"{op} {s}")
        assert_bit_equal(oracle.binary(pos, s, "pow"), ref.binary(pos, s, "pow"), f"pow {s}")
    x = synth.normal_f16(19, 1, 37 * 301, 2.0).reshape(37, 301)
    x[3, 5] = x[3, 200] = x[3].max()                       # ties: the first one wins
    x[4, :] = 0.0
    x[4, 17] = -0.0
    for op in ("max", "min", "sum", "mean"):
        assert_bit_equal(oracle.reduce(x, op), ref.reduce(x, op), op)
    assert np.array_equal(oracle.argreduce(x, False), ref.argreduce(x, False))
    assert np.array_equal(oracle.argreduce(x, True), ref.argreduce(x, True))
    wide = synth.normal_f16(19, 2, 3 * 5000, 1.0).reshape(3, 5000)   # long rows: the fp16 running sum drifts
    assert_bit_equal(oracle.reduce(wide, "sum"), ref.reduce(wide, "sum"), "sum of 5000")
    assert_bit_equal(oracle.reduce(wide, "mean"), ref.reduce(wide, "mean"), "mean of 5000")
    assert np.array_equal(oracle.cast(fin, np.float32), ref.cast(fin, np.float32))
    f32 = (np.random.default_rng(5).standard_normal(20000) * 300).astype(np.float32)
    assert_bit_equal(oracle.cast(f32, np.float16), ref.cast(f32, np.float16), "float -> half")
    small = np.ascontiguousarray(fin[np.abs(fin.astype(np.float32)) < 30000])
    assert np.array_equal(oracle.cast(small, np.int32), ref.cast(small, np.int32))
    i32 = np.random.default_rng(6).integers(-70000, 70000, 20000).astype(np.int32)
    assert_bit_equal(oracle.cast(i32, np.float16), ref.cast(i32, np.float16), "int -> half")


def test_restatement_vs_reference_strided_copies(oracle, ref):
    import device_cases as dc
    for view in dc.STRIDED_VIEWS:
        name, _, shape, stride, offset = view
        buf = dc.buffer_for(view)
        want = ref.contiguous(buf, shape, stride, offset)
        assert_bit_equal(oracle.contiguous(buf, shape, stride, offset), want, name)
        if 0 in stride:
            continue                                       # writing through a broadcast view is a race in the reference
        src = synth.normal_f16(18, 3, int(np.prod(shape)), 1.0)
        assert_bit_equal(oracle.set_item(buf, src, shape, stride, offset), ref.set_item(buf, src, shape, stride, offset), name)
        assert_bit_equal(oracle.set_item(buf, 2.5, shape, stride, offset), ref.set_item(buf, 2.5, shape, stride, offset), name)


def test_restatement_vs_reference_strided_batched_matmul(oracle, ref):
    import device_cases as dc
    for name, lhs, rhs, ls, rs, lo, ro, shape, K in dc.strided_matmul_cases():
        assert_bit_equal(oracle.matmul_strided(lhs, rhs, ls, rs, lo, ro, shape, K),
                         ref.matmul_strided(lhs, rhs, ls, rs, lo, ro, shape, K), name)
