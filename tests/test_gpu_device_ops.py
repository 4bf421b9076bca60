"""GPU parity of the remaining Device<half> operators (strided copies, unary family, binary and
scalar arithmetic, reductions, casts) through the C ABI: bit-exact against the oracle, which
tests/test_oracle.py pins against the reference's own CPU<half> on the same inputs."""
import numpy as np
import pytest

import device_cases as dc
from conftest import assert_bit_equal

from tensorlib_b200 import synth

pytestmark = pytest.mark.gpu


def test_unary_family_on_every_fp16_value(tl, oracle):
    fin, pos = dc.finite_halfs(), dc.positive_halfs()
    for op in dc.UNARY_ON_ALL:
        assert_bit_equal(tl.unary(fin, op), oracle.unary(fin, op), op)
    for op in dc.UNARY_ON_POSITIVE:
        assert_bit_equal(tl.unary(pos, op), oracle.unary(pos, op), op)
    # the shared-memory table path (>= 2^20 elements, 16-byte aligned) and a ragged tail on the gather path
    big = np.resize(fin, (1 << 20) + 8 * 1000)
    for op in ("exp", "tanh", "silu"):
        assert_bit_equal(tl.unary(big, op), oracle.unary(big, op), op + " (large)")
        assert_bit_equal(tl.unary(big[:-3], op), oracle.unary(np.ascontiguousarray(big[:-3]), op), op + " (ragged)")
    for op in ("neg", "abs"):
        assert_bit_equal(tl.unary(big[:1001], op), oracle.unary(np.ascontiguousarray(big[:1001]), op), op + " (ragged)")
    # where the reference's CPU code throws, the IEEE value comes back (as from its CUDA kernels)
    z = np.array([0.0, -4.0, 4.0], dtype=np.float16)
    got = tl.unary(z, "sqrt").astype(np.float32)
    assert got[0] == 0.0 and np.isnan(got[1]) and got[2] == 2.0
    assert np.isinf(tl.unary(z, "rsqrt").astype(np.float32)[0])
    assert tl.unary(np.zeros(0, np.float16), "sin").size == 0
    with pytest.raises(tl.TLError):
        tl._unary_like("tl_unary_f16", z, z.size, 99, None)


def test_binary_and_scalar_arithmetic_on_every_fp16_value(tl, oracle):
    fin, pos = dc.finite_halfs(), dc.positive_halfs()
    rolled = np.ascontiguousarray(np.roll(fin, 777))
    for op in ("add", "sub", "mul"):
        assert_bit_equal(tl.binary(fin, rolled, op), oracle.binary(fin, rolled, op), op)
    nz = np.ascontiguousarray(np.roll(pos, 4321)[:fin.size - 30000])
    a = np.ascontiguousarray(fin[:nz.size])
    assert_bit_equal(tl.binary(a, nz, "div"), oracle.binary(a, nz, "div"), "div")
    odd = np.ascontiguousarray(fin[:1003])                        # not a multiple of eight: scalar path
    assert_bit_equal(tl.binary(odd, np.ascontiguousarray(rolled[:1003]), "sub"), oracle.binary(odd, np.ascontiguousarray(rolled[:1003]), "sub"), "sub ragged")
    for s in dc.SCALARS:
        for op in ("add", "sub", "mul", "div"):
            assert_bit_equal(tl.binary(fin, s, op), oracle.binary(fin, s, op), f"{op} {s}")
        assert_bit_equal(tl.binary(pos, s, "pow"), oracle.binary(pos, s, "pow"), f"pow {s}")
    assert_bit_equal(tl.binary(pos, 2.0, "pow"), oracle.binary(pos, 2.0, "pow"), "pow 2 again (cached table)")
    with pytest.raises(tl.TLError, match="zero"):                 # the reference throws "Division by zero."
        tl.binary(fin, 0.0, "div")
    q = tl.binary(np.array([1.0, -1.0], np.float16), np.array([0.0, 0.0], np.float16), "div").astype(np.float32)
    assert np.isposinf(q[0]) and np.isneginf(q[1])                # tensor divisor: IEEE, like the reference's CUDA kernel


def test_reductions_both_numerics_and_arg_forms(tl, oracle):
    x = synth.normal_f16(19, 1, 37 * 301, 2.0).reshape(37, 301)
    x[3, 5] = x[3, 200] = x[3].max()
    x[4, :] = 0.0
    x[4, 17] = -0.0
    for op in ("max", "min", "sum", "mean"):
        assert_bit_equal(tl.reduce(x, op, numerics=tl.REFERENCE_ORDER), oracle.reduce(x, op), op)
    for op in ("max", "min"):                                     # exact in the parallel form too
        assert_bit_equal(tl.reduce(x, op, numerics=tl.FAST), oracle.reduce(x, op), op + " fast")
    assert np.array_equal(tl.argreduce(x, False), oracle.argreduce(x, False))
    assert np.array_equal(tl.argreduce(x, True), oracle.argreduce(x, True))
    assert np.array_equal(tl.argreduce(x, False), tl.argmax(x))
    wide = synth.normal_f16(19, 2, 3 * 5000, 1.0).reshape(3, 5000)
    for op in ("sum", "mean"):
        assert_bit_equal(tl.reduce(wide, op, numerics=tl.REFERENCE_ORDER), oracle.reduce(wide, op), op + " of 5000")
        exact = getattr(wide.astype(np.float64), op)(axis=1)
        fast = tl.reduce(wide, op, numerics=tl.FAST).astype(np.float64)
        assert np.abs(fast - exact).max() <= 2.0 ** -10 * max(1.0, np.abs(exact).max())     # one fp16 rounding of an fp32 sum
    one = synth.normal_f16(19, 3, 64, 1.0).reshape(64, 1)         # runs of one element
    assert_bit_equal(tl.reduce(one, "sum", numerics=tl.REFERENCE_ORDER), one.reshape(-1), "runs of 1")
    with pytest.raises(tl.TLError):
        tl.check(tl.load().tl_reduce_f16(None, None, 7, 20, 0, tl.FAST, None), "tl_reduce_f16")   # 20 is not a multiple of 7


def test_casts(tl, oracle):
    fin = dc.finite_halfs()
    assert np.array_equal(tl.cast(fin, np.float32), oracle.cast(fin, np.float32))
    f32 = (np.random.default_rng(5).standard_normal(20000) * 300).astype(np.float32)
    f32[:4] = [65519.9, 65520.0, 1e-8, -7e4]                        # the rounding boundary to inf, underflow, overflow
    assert_bit_equal(tl.cast(f32, np.float16), oracle.cast(f32, np.float16), "float -> half")
    small = np.ascontiguousarray(fin[np.abs(fin.astype(np.float32)) < 30000])
    assert np.array_equal(tl.cast(small, np.int32), oracle.cast(small, np.int32))
    i32 = np.random.default_rng(6).integers(-70000, 70000, 20000).astype(np.int32)
    assert_bit_equal(tl.cast(i32, np.float16), oracle.cast(i32, np.float16), "int -> half")


def test_strided_copies(tl, oracle):
    for view in dc.STRIDED_VIEWS:
        name, _, shape, stride, offset = view
        buf = dc.buffer_for(view)
        assert_bit_equal(tl.contiguous(buf, shape, stride, offset), oracle.contiguous(buf, shape, stride, offset), name)
        if 0 in stride:
            continue
        src = synth.normal_f16(18, 3, int(np.prod(shape)), 1.0)
        assert_bit_equal(tl.set_item(buf, src, shape, stride, offset), oracle.set_item(buf, src, shape, stride, offset), name)
        assert_bit_equal(tl.set_item(buf, 2.5, shape, stride, offset), oracle.set_item(buf, 2.5, shape, stride, offset), name)
    # the Llama2 forward's own re-layout at the 7B width: (S, H, hd) cache rows read as (H, S, hd)
    S, H, hd = 200, 32, 128
    cache = synth.normal_f16(18, 9, S * H * hd, 1.0)
    got = tl.contiguous(cache, (H, S, hd), (hd, H * hd, 1), 0)
    assert_bit_equal(got, cache.reshape(S, H, hd).transpose(1, 0, 2), "cache re-layout")
    with pytest.raises(tl.TLError):                                # num_elements must be the product of the shape
        sh = np.array([4, 4], np.int32)
        d = tl.DeviceBuffer(64)
        tl.check(tl.load().tl_contiguous_f16(d.ptr, d.ptr, sh.ctypes.data, sh.ctypes.data, 2, 0, 15, None), "tl_contiguous_f16")


def test_strided_batched_device_matmul(tl, oracle):
    """Device::matmul with per-dimension strides: bit-exact in reference order, within the matmul
    tolerance in fast numerics (tensor-core kernels where the reduction dimension is contiguous)."""
    for name, lhs, rhs, ls, rs, lo, ro, shape, K in dc.strided_matmul_cases():
        want = oracle.matmul_strided(lhs, rhs, ls, rs, lo, ro, shape, K)
        assert_bit_equal(tl.matmul_strided(lhs, rhs, ls, rs, lo, ro, shape, K, numerics=tl.REFERENCE_ORDER), want, name)
        got = tl.matmul_strided(lhs, rhs, ls, rs, lo, ro, shape, K, numerics=tl.FAST).astype(np.float64)
        w = want.astype(np.float64)
        scale = np.sqrt((w * w).mean(axis=-1, keepdims=True)) + 1e-30
        assert (np.abs(got - w) / np.maximum(np.abs(w), scale)).max() <= 1e-2, name
    assert tl.device_status() == 0
