"""Seeded inputs shared by the CPU pin (oracle against the compiled reference) and the GPU parity
test (product against the oracle) of the remaining Device<half> operators."""
import numpy as np

from tensorlib_b200 import synth


def finite_halfs() -> np.ndarray:
    allh = np.arange(65536, dtype=np.uint16).view(np.float16)
    return np.ascontiguousarray(allh[np.isfinite(allh)])


def positive_halfs() -> np.ndarray:
    f = finite_halfs()
    return np.ascontiguousarray(f[f > 0])


UNARY_ON_ALL = ("neg", "sin", "cos", "exp", "abs", "tanh", "silu", "silu_cpu_half")
UNARY_ON_POSITIVE = ("log", "sqrt", "rsqrt")        # the reference throws (sqrt, rsqrt) or returns nan / -inf (log) elsewhere
SCALARS = (2.0, 0.5, -1.5, 3.0, 1e-3, 11.3125)

# (name, elements of the underlying buffer, shape, stride, offset): views a Tensor program produces
STRIDED_VIEWS = (
    ("row slice", 64 * 48, (16, 48), (48, 1), 48 * 5),
    ("transpose", 37 * 53, (53, 37), (1, 53), 0),
    ("heads of a (T,H,hd) cache as (H,T,hd)", 9 * 6 * 48, (6, 9, 48), (48, 6 * 48, 1), 0),
    ("column block, 16-byte aligned", 32 * 256, (32, 64), (256, 1), 128),
    ("column block, odd offset", 32 * 256, (32, 64), (256, 1), 3),
    ("broadcast row", 300, (7, 300), (0, 1), 0),
    ("every other element", 1000, (500,), (2,), 1),
    ("five dimensions", 2 * 3 * 4 * 5 * 16, (3, 2, 5, 4, 16), (4 * 5 * 16, 3 * 4 * 5 * 16, 16, 5 * 16, 1), 0),
    ("single element", 10, (1, 1), (5, 1), 7),
    ("contiguous", 4096, (4, 1024), (1024, 1), 0),
    ("ragged inner", 23 * 19, (23, 19), (19, 1), 0),
)


def buffer_for(view) -> np.ndarray:
    return synth.normal_f16(17, len(view[0]), view[1], 1.0)


def strided_matmul_cases():
    """(name, lhs buffer, rhs buffer, lhs_stride, rhs_stride, lhs_offset, rhs_offset, result_shape, K):
    the operand layouts the reference's Tensor::matmul hands to Device::matmul."""
    cases = []
    T, K, N = 5, 64, 24                                   # Linear: x (1,T,K) . W[N,K] viewed as (1,K,N)
    cases.append(("linear", synth.normal_f16(23, 1, T * K, 1.0), synth.normal_f16(23, 2, N * K, 0.1),
                  (T * K, K, 1), (0, 1, K), 0, 0, (1, T, N), K))
    H, T, S, hd = 3, 4, 9, 16                             # scores: q (T,H,hd) as (1,H,T,hd), keys (S,H,hd) as (1,H,hd,S)
    q, kc = synth.normal_f16(23, 3, T * H * hd, 1.0), synth.normal_f16(23, 4, S * H * hd, 1.0)
    cases.append(("q.k^T over in-place heads", q, kc, (T * H * hd, hd, H * hd, 1), (S * H * hd, hd, 1, H * hd), 0, 0,
                  (1, H, T, S), hd))
    p, vc = synth.normal_f16(23, 5, H * T * S, 0.3), synth.normal_f16(23, 6, S * H * hd, 1.0)
    cases.append(("p.v, reduction dimension strided in the cache", p, vc, (H * T * S, T * S, S, 1), (S * H * hd, hd, H * hd, 1),
                  0, 0, (1, H, T, hd), S))
    a, b = synth.normal_f16(23, 7, 2 * 3 * 4 * 5 * 6, 1.0), synth.normal_f16(23, 8, 4 * 6 * 7, 1.0)
    cases.append(("three batch dimensions, rhs broadcast over two", a, b, (3 * 4 * 5 * 6, 4 * 5 * 6, 5 * 6, 6, 1),
                  (0, 0, 6 * 7, 7, 1), 0, 0, (2, 3, 4, 5, 7), 6))
    a2, b2 = synth.normal_f16(23, 9, 1000, 1.0), synth.normal_f16(23, 10, 1000, 1.0)
    cases.append(("odd offsets and pitches", a2, b2, (37, 1), (1, 29), 3, 5, (7, 11), 13))
    big_a, big_w = synth.normal_f16(23, 11, 40 * 256, 1.0), synth.normal_f16(23, 12, 96 * 256, 0.05)
    cases.append(("aligned, tensor-core sized", big_a, big_w, (40 * 256, 256, 1), (0, 1, 256), 0, 0, (1, 40, 96), 256))
    return cases
