"""tensorlib_b200 — B200 (sm_100a) matmul backend for tensorLib's Tensor::matmul -> Llama2 path.

This module is a thin ctypes binding of the C ABI in include/tensorlib_b200.h (built in-tree as
tensorlib_b200/libtensorlib_b200.so by ``python -m tensorlib_b200.build``). There is no CPU or
PyTorch fallback: if the library is missing or no sm_100 GPU is present, loading / init raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libtensorlib_b200.so")

REFERENCE_ORDER = 0
FAST = 1

_vp = C.c_void_p
_sz = C.c_size_t
_int = C.c_int


class TLError(RuntimeError):
    def __init__(self, status: int, where: str, msg: str):
        super().__init__(f"{where}: status {status}: {msg}")
        self.status = status


class tl_llama2_config(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads",
                                       "vocab_size", "max_seq_len", "numerics", "silu_via_float",
                                       "tp_rank", "tp_world", "one_kernel_decode")]


# name -> argtypes; every function returns int status unless listed in _OTHER_RESTYPE
_SIGS = {
    "tl_init": [_int],
    "tl_device_count": [C.POINTER(_int)],
    "tl_device_status": [C.POINTER(_int)],
    "tl_host_lookup_tables": [_vp, _vp, _vp],
    "tl_host_rope_table": [_int, _int, _vp, _vp],
    "tl_malloc": [C.POINTER(_vp), _sz],
    "tl_free": [_vp],
    "tl_memcpy_h2d": [_vp, _vp, _sz, _vp],
    "tl_memcpy_d2h": [_vp, _vp, _sz, _vp],
    "tl_memcpy_d2d": [_vp, _vp, _sz, _vp],
    "tl_memset": [_vp, _int, _sz, _vp],
    "tl_stream_synchronize": [_vp],
    "tl_malloc_host": [C.POINTER(_vp), _sz],
    "tl_free_host": [_vp],
    "tl_matmul2d_f16": [_vp, _vp, _vp, _sz, _sz, _sz, _int, _vp],
    "tl_matmul_batched_f16": [_vp, _vp, _vp] + [_sz] * 10 + [_int, _vp],
    "tl_matmul2d_f16_host": [_vp, _vp, _vp, _sz, _sz, _sz, _int],
    "tl_linear_f16": [_vp, _vp, _vp, _sz, _sz, _sz, _vp],
    "tl_matmul_strided_f16": [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _vp, _int, _sz, _sz, _int, _vp],
    "tl_rms_norm_f16": [_vp, _vp, _vp, C.c_float, _int, _int, _int, _vp],
    "tl_apply_rotary_emb_f16": [_vp, _vp, _int, _int, _int, _int, _int, _vp],
    "tl_softmax_f16": [_vp, _vp, _sz, _sz, _int, _vp],
    "tl_silu_f16": [_vp, _vp, _sz, _int, _vp],
    "tl_add_f16": [_vp, _vp, _vp, _sz, _vp],
    "tl_mul_f16": [_vp, _vp, _vp, _sz, _vp],
    "tl_div_scalar_f16": [_vp, _vp, C.c_double, _sz, _vp],
    "tl_argmax_f16": [_vp, _vp, _sz, _sz, _vp],
    "tl_embedding_f16": [_vp, _vp, _vp, _int, _int, _int, _vp],
    "tl_llama2_create": [C.POINTER(tl_llama2_config), C.POINTER(_vp)],
    "tl_llama2_destroy": [_vp],
    "tl_llama2_load_payload_host": [_vp, _vp, _int],
    "tl_llama2_load_file": [_vp, C.c_char_p],
    "tl_llama2_init_random": [_vp, C.c_uint64, C.c_float],
    "tl_matmul_plan": [C.c_size_t, C.c_size_t, C.c_size_t, _int] + [C.POINTER(_int)] * 5,
    "tl_llama2_forward": [_vp, _vp, _int, _int, _vp, _vp],
    "tl_llama2_generate": [_vp, _vp, _int, _int, _int, _vp, C.POINTER(_int), C.POINTER(C.c_double),
                           C.POINTER(C.c_double)],
    "tl_llama2_generate_at": [_vp, _int, _vp, _int, _int, _int, _vp, C.POINTER(_int), C.POINTER(C.c_double),
                              C.POINTER(C.c_double)],
    "tl_llama2_decode_device": [_vp, _int, _int, _vp, _vp],
    "tl_llama2_set_next_token": [_vp, _int],
    "tl_llama2_kernel_launches": [_vp, C.POINTER(C.c_longlong)],
    "tl_llama2_weight_bytes": [_vp, C.POINTER(C.c_longlong)],
    "tl_llama2_tensor": [_vp, C.c_char_p, _int, C.POINTER(_vp), C.POINTER(_int), C.POINTER(_int)],
    "tl_llama2_decode_profile": [_vp, _int, _int, _vp, _int, C.POINTER(_int)],
    "tl_rmsnorm_qkv_rope_f16": [_vp, _vp, C.c_float] + [_vp] * 6 + [_int, _int, _int, _int, _vp],
    "tl_attn_decode_f16": [_vp] * 6 + [_int, _int, _int, _int, _vp],
    "tl_attn_decode_f16_noalloc": [_vp] * 4 + [_int, _int, _int, _int, _vp],
    "tl_attn_prefill_f16": [_vp] * 4 + [_int, _int, _int, _int, _vp],
    "tl_gemv_residual_f16": [_vp, _vp, _vp, _vp, _int, _int, _vp],
    "tl_rmsnorm_gateup_swiglu_f16": [_vp, _vp, C.c_float, _vp, _vp, _vp, _int, _int, _vp],
    "tl_tp_unique_id": [_vp, _int],
    "tl_tp_init": [_vp, _int, _int, _int],
    "tl_tp_attach": [_vp],
    "tl_tp_allreduce_f32": [_vp, _sz, _vp],
    "tl_tp_destroy": [],
    "tl_tp_exchange_export": [_vp, _vp, _int],
    "tl_tp_exchange_open": [_vp, _vp, _int],
    "tl_tp_exchange_close": [_vp],
    "tl_tp_shard": [_int] * 5 + [C.POINTER(_int)] * 4,
    "tl_selftest_unposted_exchange": [_int, _vp],
    "tl_selftest_tp_prefill_exchange": [_vp] * 6 + [_int] * 5 + [C.c_float, _vp],
    "tl_contiguous_f16": [_vp, _vp, _vp, _vp, _int, _sz, _sz, _vp],
    "tl_set_item_f16": [_vp, _vp, _vp, _vp, _int, _sz, _sz, _vp],
    "tl_set_item_scalar_f16": [_vp, C.c_uint16, _vp, _vp, _int, _sz, _sz, _vp],
    "tl_unary_f16": [_vp, _vp, _sz, _int, _vp],
    "tl_binary_f16": [_vp, _vp, _vp, _sz, _int, _vp],
    "tl_binary_scalar_f16": [_vp, _vp, C.c_uint16, _sz, _int, _vp],
    "tl_reduce_f16": [_vp, _vp, _sz, _sz, _int, _int, _vp],
    "tl_argreduce_f16": [_vp, _vp, _sz, _sz, _int, _vp],
    "tl_cast": [_vp, _vp, _sz, _int, _vp],
}
_OTHER_RESTYPE = {"tl_strerror": (C.c_char_p, [_int]), "tl_last_error": (C.c_char_p, []),
                  "tl_version": (_int, [])}
_OPTIONAL = {}

_lib = None


def load() -> C.CDLL:
    """dlopen the native library (no GPU needed for this step)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: run `python -m tensorlib_b200.build` "
                          "(this package has no fallback implementation)")
    lib = C.CDLL(LIB_PATH)
    for name, args in _SIGS.items():
        f = getattr(lib, name)
        f.argtypes = args
        f.restype = _int
    for name, (res, args) in _OTHER_RESTYPE.items():
        f = getattr(lib, name)
        f.argtypes = args
        f.restype = res
    for name, args in _OPTIONAL.items():
        if hasattr(lib, name):
            f = getattr(lib, name)
            f.argtypes = args
            f.restype = _int
    _lib = lib
    return lib


def exported_symbols() -> list[str]:
    return list(_SIGS) + list(_OTHER_RESTYPE)


def check(status: int, where: str) -> None:
    if status != 0:
        raise TLError(status, where, load().tl_last_error().decode(errors="replace"))


_initialized_device = None


def init(device: int = 0) -> None:
    global _initialized_device
    check(load().tl_init(device), "tl_init")
    _initialized_device = device


def device_count() -> int:
    n = _int(0)
    load().tl_device_count(C.byref(n))
    return n.value


def _np_ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_vp)


class DeviceBuffer:
    """Owned device allocation (what CUDA<dtype> holds in the reference, CUDA.cu:17-32)."""

    def __init__(self, nbytes: int):
        p = _vp()
        check(load().tl_malloc(C.byref(p), nbytes), "tl_malloc")
        self.ptr, self.nbytes = p.value, nbytes

    @classmethod
    def from_numpy(cls, a: np.ndarray) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        b = cls(a.nbytes)
        if a.nbytes:
            check(load().tl_memcpy_h2d(b.ptr, _np_ptr(a), a.nbytes, None), "tl_memcpy_h2d")
            check(load().tl_stream_synchronize(None), "sync")
        return b

    def to_numpy(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes <= self.nbytes
        if out.nbytes:
            check(load().tl_memcpy_d2h(_np_ptr(out), self.ptr, out.nbytes, None), "tl_memcpy_d2h")
        check(load().tl_stream_synchronize(None), "sync")
        return out

    def free(self):
        if self.ptr:
            load().tl_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def device_status() -> int:
    """0, or the status a kernel recorded when one of its bounded waits ran out (synchronises)."""
    v = _int(0)
    check(load().tl_device_status(C.byref(v)), "tl_device_status")
    return v.value


def synchronize(stream=None) -> None:
    check(load().tl_stream_synchronize(stream), "tl_stream_synchronize")


# -------------------------------------------------------------------------------------------------
# numpy-in / numpy-out helpers around the device entry points (tests, smoke)
# -------------------------------------------------------------------------------------------------
def matmul2d(A: np.ndarray, B: np.ndarray, numerics: int = FAST) -> np.ndarray:
    """C[M,N] = A[M,K] @ B[N,K]^T through tl_matmul2d_f16 on device buffers."""
    M, K = A.shape
    N, K2 = B.shape
    assert K == K2 and A.dtype == np.float16 and B.dtype == np.float16
    dA, dB, dC = DeviceBuffer.from_numpy(A), DeviceBuffer.from_numpy(B), DeviceBuffer(max(M * N * 2, 2))
    check(load().tl_matmul2d_f16(dA.ptr, dB.ptr, dC.ptr, M, N, K, numerics, None), "tl_matmul2d_f16")
    return dC.to_numpy(np.float16, (M, N))


def linear(x: np.ndarray, W: np.ndarray) -> np.ndarray:
    """nn::Linear::forward: x[T, in] @ W[out, in]^T through tl_linear_f16."""
    T, K = x.shape
    N, _ = W.shape
    dx, dW, dy = DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(W), DeviceBuffer(max(T * N * 2, 2))
    check(load().tl_linear_f16(dx.ptr, dW.ptr, dy.ptr, T, K, N, None), "tl_linear_f16")
    return dy.to_numpy(np.float16, (T, N))


def matmul2d_host(A: np.ndarray, B: np.ndarray, numerics: int = FAST) -> np.ndarray:
    M, K = A.shape
    N, _ = B.shape
    A, B = np.ascontiguousarray(A), np.ascontiguousarray(B)
    Cm = np.empty((M, N), dtype=np.float16)
    check(load().tl_matmul2d_f16_host(_np_ptr(A), _np_ptr(B), _np_ptr(Cm), M, N, K, numerics),
          "tl_matmul2d_f16_host")
    return Cm


def matmul_batched(A: np.ndarray, Bt: np.ndarray, numerics: int = FAST) -> np.ndarray:
    """A (batch,M,K), Bt (batch or 1,N,K) -> (batch,M,N); batch stride 0 broadcasts Bt."""
    b, M, K = A.shape
    bb, N, _ = Bt.shape
    dA, dB, dC = DeviceBuffer.from_numpy(A), DeviceBuffer.from_numpy(Bt), DeviceBuffer(max(b * M * N * 2, 2))
    check(load().tl_matmul_batched_f16(dA.ptr, dB.ptr, dC.ptr, b, M, N, K, K, K, N, M * K,
                                       0 if bb == 1 else N * K, M * N, numerics, None), "tl_matmul_batched_f16")
    return dC.to_numpy(np.float16, (b, M, N))


def matmul_strided(lhs: np.ndarray, rhs: np.ndarray, lhs_stride, rhs_stride, lhs_offset: int, rhs_offset: int,
                   result_shape, K: int, numerics: int = FAST) -> np.ndarray:
    """Device::matmul on flat fp16 buffers with per-dimension strides (tl_matmul_strided_f16)."""
    n = int(np.prod(result_shape))
    ls, lsp = _ints(lhs_stride)
    rs, rsp = _ints(rhs_stride)
    sh, shp = _ints(result_shape)
    dl, dr, dc = DeviceBuffer.from_numpy(lhs), DeviceBuffer.from_numpy(rhs), DeviceBuffer(max(n * 2, 2))
    check(load().tl_matmul_strided_f16(dl.ptr, dr.ptr, dc.ptr, lsp, rsp, lhs_offset, rhs_offset, shp, len(result_shape), n, K,
                                       numerics, None), "tl_matmul_strided_f16")
    return dc.to_numpy(np.float16, tuple(result_shape))


def _unary_like(fn_name, x: np.ndarray, *args):
    dx, dy = DeviceBuffer.from_numpy(x), DeviceBuffer(max(x.nbytes, 2))
    check(getattr(load(), fn_name)(dy.ptr, dx.ptr, *args), fn_name)
    return dy.to_numpy(np.float16, x.shape)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float = 1e-5, numerics: int = FAST) -> np.ndarray:
    T, D = x.shape
    dx, dw, dy = DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(w), DeviceBuffer(max(x.nbytes, 2))
    check(load().tl_rms_norm_f16(dy.ptr, dx.ptr, dw.ptr, eps, D, T, numerics, None), "tl_rms_norm_f16")
    return dy.to_numpy(np.float16, x.shape)


def apply_rotary_emb(x: np.ndarray, start_pos: int) -> np.ndarray:
    T, Hh, hd = x.shape
    dx, dy = DeviceBuffer.from_numpy(x), DeviceBuffer(max(x.nbytes, 2))
    check(load().tl_apply_rotary_emb_f16(dx.ptr, dy.ptr, start_pos, 1, T, Hh, hd, None), "tl_apply_rotary_emb_f16")
    return dy.to_numpy(np.float16, x.shape)


def softmax(x: np.ndarray, numerics: int = FAST) -> np.ndarray:
    R, Cc = x.shape
    return _unary_like("tl_softmax_f16", x, R, Cc, numerics, None)


def silu(x: np.ndarray, via_float: bool = True) -> np.ndarray:
    return _unary_like("tl_silu_f16", x, x.size, int(via_float), None)


def add(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    da, db, dy = DeviceBuffer.from_numpy(a), DeviceBuffer.from_numpy(b), DeviceBuffer(max(a.nbytes, 2))
    check(load().tl_add_f16(dy.ptr, da.ptr, db.ptr, a.size, None), "tl_add_f16")
    return dy.to_numpy(np.float16, a.shape)


def mul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    da, db, dy = DeviceBuffer.from_numpy(a), DeviceBuffer.from_numpy(b), DeviceBuffer(max(a.nbytes, 2))
    check(load().tl_mul_f16(dy.ptr, da.ptr, db.ptr, a.size, None), "tl_mul_f16")
    return dy.to_numpy(np.float16, a.shape)


def div_scalar(a: np.ndarray, scalar: float) -> np.ndarray:
    da, dy = DeviceBuffer.from_numpy(a), DeviceBuffer(max(a.nbytes, 2))
    check(load().tl_div_scalar_f16(dy.ptr, da.ptr, float(scalar), a.size, None), "tl_div_scalar_f16")
    return dy.to_numpy(np.float16, a.shape)


def argmax(x: np.ndarray) -> np.ndarray:
    R, Cc = x.shape
    dx, di = DeviceBuffer.from_numpy(x), DeviceBuffer(max(R * 4, 4))
    check(load().tl_argmax_f16(di.ptr, dx.ptr, R, Cc, None), "tl_argmax_f16")
    return di.to_numpy(np.int32, (R,))


def embedding(table: np.ndarray, tokens: np.ndarray) -> np.ndarray:
    V, D = table.shape
    tok = np.ascontiguousarray(tokens, dtype=np.int32)
    dt, dk, dy = DeviceBuffer.from_numpy(table), DeviceBuffer.from_numpy(tok), DeviceBuffer(max(tok.size * D * 2, 2))
    check(load().tl_embedding_f16(dy.ptr, dt.ptr, dk.ptr, tok.size, D, V, None), "tl_embedding_f16")
    return dy.to_numpy(np.float16, (tok.size, D))


def attn_prefill(q: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray, start_pos: int, n_heads: int) -> np.ndarray:
    """Causal attention of T query rows (T, n_heads*hd) at positions start_pos.. over the first
    start_pos+T rows of the caches (max_seq, n_heads*hd): tl_attn_prefill_f16."""
    T, width = q.shape
    hd = width // n_heads
    S = start_pos + T
    dq, dk, dv = (DeviceBuffer.from_numpy(np.ascontiguousarray(a, dtype=np.float16)) for a in (q, k_cache, v_cache))
    out = DeviceBuffer(T * width * 2)
    check(load().tl_attn_prefill_f16(dq.ptr, dk.ptr, dv.ptr, out.ptr, T, start_pos, n_heads, hd, None),
          "tl_attn_prefill_f16")
    synchronize()
    return out.to_numpy(np.float16, (T, width))


def rmsnorm_qkv_rope(x, norm_w, wq, wk, wv, k_cache, v_cache, head_dim: int, pos: int, eps: float = 1e-5):
    """tl_rmsnorm_qkv_rope_f16: x[dim] -> (q[n_q], k_cache', v_cache') with row `pos` of the caches
    (max_seq, n_q) written in place on device copies, which are returned."""
    n_q, dim = wq.shape
    bufs = [DeviceBuffer.from_numpy(np.ascontiguousarray(a, dtype=np.float16))
            for a in (x, norm_w, wq, wk, wv, k_cache, v_cache)]
    dq = DeviceBuffer(n_q * 2)
    check(load().tl_rmsnorm_qkv_rope_f16(bufs[0].ptr, bufs[1].ptr, eps, bufs[2].ptr, bufs[3].ptr, bufs[4].ptr, dq.ptr,
                                         bufs[5].ptr, bufs[6].ptr, dim, n_q, head_dim, pos, None), "tl_rmsnorm_qkv_rope_f16")
    return (dq.to_numpy(np.float16, (n_q,)), bufs[5].to_numpy(np.float16, k_cache.shape),
            bufs[6].to_numpy(np.float16, v_cache.shape))


def gemv_residual(x, W, residual):
    """tl_gemv_residual_f16: residual[N] + W[N,K] x[K]."""
    N, K = W.shape
    dx, dW, dr = (DeviceBuffer.from_numpy(np.ascontiguousarray(a, dtype=np.float16)) for a in (x, W, residual))
    dy = DeviceBuffer(N * 2)
    check(load().tl_gemv_residual_f16(dx.ptr, dW.ptr, dr.ptr, dy.ptr, N, K, None), "tl_gemv_residual_f16")
    return dy.to_numpy(np.float16, (N,))


def rmsnorm_gateup_swiglu(x, norm_w, w1, w3, eps: float = 1e-5):
    """tl_rmsnorm_gateup_swiglu_f16: silu(w1 n) * (w3 n) with n = rmsnorm(x) * norm_w."""
    hidden, dim = w1.shape
    dx, dn, d1, d3 = (DeviceBuffer.from_numpy(np.ascontiguousarray(a, dtype=np.float16)) for a in (x, norm_w, w1, w3))
    dy = DeviceBuffer(hidden * 2)
    check(load().tl_rmsnorm_gateup_swiglu_f16(dx.ptr, dn.ptr, eps, d1.ptr, d3.ptr, dy.ptr, hidden, dim, None),
          "tl_rmsnorm_gateup_swiglu_f16")
    return dy.to_numpy(np.float16, (hidden,))


UNARY_OPS = {"neg": 0, "sin": 1, "cos": 2, "exp": 3, "log": 4, "abs": 5, "tanh": 6, "silu": 7, "sqrt": 8, "rsqrt": 9,
             "silu_cpu_half": 10}
BINARY_OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3, "pow": 4}
REDUCE_OPS = {"max": 0, "min": 1, "sum": 2, "mean": 3}


def selftest_tp_prefill_exchange(A, B, residual, norm_w, world: int, owner: int, eps: float = 1e-5):
    """tl_selftest_tp_prefill_exchange: the tensor-parallel prefill exchange of rank `owner` of `world`, the ranks
    emulated on one GPU. Returns (residual_out [M / world, dim], xn [world, M, dim]; xn starts as zeros)."""
    M, K = A.shape
    dim = B.shape[0]
    dA, dB, dr, dw = (DeviceBuffer.from_numpy(np.ascontiguousarray(a, dtype=np.float16)) for a in (A, B, residual, norm_w))
    dout = DeviceBuffer(M // world * dim * 2)
    dxn = DeviceBuffer.from_numpy(np.zeros((world, M, dim), np.float16))
    check(load().tl_selftest_tp_prefill_exchange(dA.ptr, dB.ptr, dr.ptr, dw.ptr, dout.ptr, dxn.ptr, M, dim, K, world, owner,
                                                 eps, None), "tl_selftest_tp_prefill_exchange")
    return dout.to_numpy(np.float16, (M // world, dim)), dxn.to_numpy(np.float16, (world, M, dim))


def _ints(v):
    a = np.ascontiguousarray(v, dtype=np.int32)
    return a, a.ctypes.data_as(_vp)


def contiguous(data: np.ndarray, shape, stride, offset: int = 0) -> np.ndarray:
    """Device::contiguous of the view (shape, stride, offset) over the flat fp16 array `data`."""
    n = int(np.prod(shape)) if len(shape) else 1
    sh, shp = _ints(shape)
    sd, sdp = _ints(stride)
    dd, dr = DeviceBuffer.from_numpy(data), DeviceBuffer(max(n * 2, 2))
    check(load().tl_contiguous_f16(dr.ptr, dd.ptr, shp, sdp, len(shape), offset, n, None), "tl_contiguous_f16")
    return dr.to_numpy(np.float16, tuple(shape))


def set_item(data: np.ndarray, src, shape, stride, offset: int = 0) -> np.ndarray:
    """Device::setItemEwise (src an array of prod(shape) values) or setItemScalar (src a scalar)
    into the view (shape, stride, offset) of `data`; returns the updated flat array."""
    n = int(np.prod(shape)) if len(shape) else 1
    sh, shp = _ints(shape)
    sd, sdp = _ints(stride)
    dd = DeviceBuffer.from_numpy(data)
    if np.ndim(src) == 0:
        bits = int(np.float16(src).view(np.uint16))
        check(load().tl_set_item_scalar_f16(dd.ptr, bits, shp, sdp, len(shape), offset, n, None), "tl_set_item_scalar_f16")
    else:
        ds = DeviceBuffer.from_numpy(np.ascontiguousarray(src, dtype=np.float16))
        check(load().tl_set_item_f16(dd.ptr, ds.ptr, shp, sdp, len(shape), offset, n, None), "tl_set_item_f16")
    return dd.to_numpy(np.float16, data.shape)


def unary(x: np.ndarray, op: str) -> np.ndarray:
    return _unary_like("tl_unary_f16", x, x.size, UNARY_OPS[op], None)


def binary(a: np.ndarray, b, op: str) -> np.ndarray:
    """a (op) b with b an array of a's shape or a scalar."""
    da, dy = DeviceBuffer.from_numpy(a), DeviceBuffer(max(a.nbytes, 2))
    if np.ndim(b) == 0:
        bits = int(np.float16(b).view(np.uint16))
        check(load().tl_binary_scalar_f16(dy.ptr, da.ptr, bits, a.size, BINARY_OPS[op], None), "tl_binary_scalar_f16")
    else:
        db = DeviceBuffer.from_numpy(np.ascontiguousarray(b, dtype=np.float16))
        check(load().tl_binary_f16(dy.ptr, da.ptr, db.ptr, a.size, BINARY_OPS[op], None), "tl_binary_f16")
    return dy.to_numpy(np.float16, a.shape)


def reduce(x: np.ndarray, op: str, numerics: int = FAST) -> np.ndarray:
    """max / min / sum / mean over the last dimension of a 2-D array."""
    R, Cc = x.shape
    dx, dy = DeviceBuffer.from_numpy(x), DeviceBuffer(max(R * 2, 2))
    check(load().tl_reduce_f16(dy.ptr, dx.ptr, Cc, x.size, REDUCE_OPS[op], numerics, None), "tl_reduce_f16")
    return dy.to_numpy(np.float16, (R,))


def argreduce(x: np.ndarray, want_min: bool) -> np.ndarray:
    R, Cc = x.shape
    dx, di = DeviceBuffer.from_numpy(x), DeviceBuffer(max(R * 4, 4))
    check(load().tl_argreduce_f16(di.ptr, dx.ptr, Cc, x.size, int(want_min), None), "tl_argreduce_f16")
    return di.to_numpy(np.int32, (R,))


def cast(x: np.ndarray, to) -> np.ndarray:
    """half <-> float32 / int32 through tl_cast."""
    kinds = {(np.float16, np.float32): 0, (np.float32, np.float16): 1, (np.float16, np.int32): 2, (np.int32, np.float16): 3}
    kind = kinds[(x.dtype.type, np.dtype(to).type)]
    dx, dy = DeviceBuffer.from_numpy(x), DeviceBuffer(max(x.size * np.dtype(to).itemsize, 4))
    check(load().tl_cast(dy.ptr, dx.ptr, x.size, kind, None), "tl_cast")
    return dy.to_numpy(np.dtype(to), x.shape)


PLAN_NAMES = {0: "reference_order", 1: "gemv_ring", 2: "gemv_small", 3: "skinny_streamk", 4: "skinny_cluster",
              5: "hgemm", 6: "hgemm_pair", 7: "hgemm_pair512", 8: "hgemm_splitk"}


def matmul_plan(M: int, N: int, K: int, sm_count: int = 148) -> dict:
    """Host-only: the kernel and work split tl_matmul2d_f16 would use (tl_matmul_plan)."""
    out = [_int(0) for _ in range(5)]
    check(load().tl_matmul_plan(M, N, K, sm_count, *[C.byref(o) for o in out]), "tl_matmul_plan")
    k, grid, tile_n, per, cluster = (o.value for o in out)
    return {"kernel": PLAN_NAMES[k], "grid": grid, "tile_n": tile_n, "k_blocks_per_cta": per, "cluster": cluster}


def host_lookup_tables():
    e, sf, sh = (np.empty(65536, dtype=np.float16) for _ in range(3))
    check(load().tl_host_lookup_tables(_np_ptr(e), _np_ptr(sf), _np_ptr(sh)), "tl_host_lookup_tables")
    return e, sf, sh


def host_rope_table(head_dim: int, rows: int):
    c = np.empty((rows, head_dim // 2), dtype=np.float16)
    s = np.empty_like(c)
    check(load().tl_host_rope_table(head_dim, rows, _np_ptr(c), _np_ptr(s)), "tl_host_rope_table")
    return c, s


class Llama2:
    """Handle on the native Llama2 model (Transformer<half> + Llama2<half>::generate)."""

    def __init__(self, cfg, numerics: int = FAST, silu_via_float: bool = True, one_kernel_decode: bool = False, tp_rank: int = 0,
                 tp_world: int = 1):
        self.cfg = cfg
        self.c = tl_llama2_config(cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.n_heads, cfg.n_heads,
                                  cfg.vocab_size, cfg.seq_len, numerics, int(silu_via_float), tp_rank, tp_world,
                                  int(one_kernel_decode))
        h = _vp()
        check(load().tl_llama2_create(C.byref(self.c), C.byref(h)), "tl_llama2_create")
        self.h = h

    def load_payload(self, payload: np.ndarray, shared_classifier: bool) -> None:
        assert payload.dtype == np.float16
        payload = np.ascontiguousarray(payload)
        check(load().tl_llama2_load_payload_host(self.h, _np_ptr(payload), int(shared_classifier)),
              "tl_llama2_load_payload_host")

    def load_file(self, path: str) -> None:
        check(load().tl_llama2_load_file(self.h, path.encode()), "tl_llama2_load_file")

    def init_random(self, seed: int, std: float = 0.02) -> None:
        check(load().tl_llama2_init_random(self.h, seed, std), "tl_llama2_init_random")

    def forward(self, tokens, start_pos: int, all_logits: bool = True) -> np.ndarray:
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        V = self.cfg.vocab_size
        if all_logits:
            out = np.empty((tok.size, V), dtype=np.float16)
            check(load().tl_llama2_forward(self.h, _np_ptr(tok), tok.size, start_pos, _np_ptr(out), None),
                  "tl_llama2_forward")
        else:
            out = np.empty((1, V), dtype=np.float16)
            check(load().tl_llama2_forward(self.h, _np_ptr(tok), tok.size, start_pos, None, _np_ptr(out)),
                  "tl_llama2_forward")
        return out

    def generate(self, prompt, max_new: int, stop_on_eos: bool = False, start_pos: int = 0):
        """Prefill `prompt` at start_pos (0: a fresh conversation; > 0: continue over the KV cache of
        earlier turns), then greedy decode. Returns (ids, prefill seconds, decode seconds)."""
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.empty(max_new, dtype=np.int32)
        n = _int(0)
        tp, td = C.c_double(0), C.c_double(0)
        check(load().tl_llama2_generate_at(self.h, int(start_pos), _np_ptr(p), p.size, max_new, int(stop_on_eos),
                                           _np_ptr(out), C.byref(n), C.byref(tp), C.byref(td)), "tl_llama2_generate_at")
        return out[: n.value].copy(), tp.value, td.value

    def set_next_token(self, token: int) -> None:
        check(load().tl_llama2_set_next_token(self.h, int(token)), "tl_llama2_set_next_token")

    def decode_device(self, start_pos: int, steps: int, fetch: bool = True, stream=None):
        out = np.empty(steps, dtype=np.int32) if fetch else None
        check(load().tl_llama2_decode_device(self.h, start_pos, steps, _np_ptr(out) if fetch else None, stream),
              "tl_llama2_decode_device")
        return out

    def decode_profile(self, start_pos: int, cta: int = 0) -> np.ndarray:
        """One decode step with device timestamps (ns, %globaltimer): array [phases, 3] = (start,
        activation vector staged, done) per GEMV phase in launch order (tl_llama2_decode_profile).
        Under tensor parallelism every rank must call it together."""
        cap = 3 * (5 * self.cfg.n_layers + 2)
        buf = np.zeros(cap, dtype=np.uint64)
        n = _int(0)
        check(load().tl_llama2_decode_profile(self.h, start_pos, cta, buf.ctypes.data_as(_vp), cap, C.byref(n)),
              "tl_llama2_decode_profile")
        return buf[:3 * n.value].reshape(n.value, 3)

    def kernel_launches(self) -> int:
        v = C.c_longlong(0)
        check(load().tl_llama2_kernel_launches(self.h, C.byref(v)), "tl_llama2_kernel_launches")
        return v.value

    def weight_bytes(self) -> int:
        v = C.c_longlong(0)
        check(load().tl_llama2_weight_bytes(self.h, C.byref(v)), "tl_llama2_weight_bytes")
        return v.value

    def close(self) -> None:
        if getattr(self, "h", None):
            load().tl_llama2_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
