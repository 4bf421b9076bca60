"""TEST INFRASTRUCTURE — ctypes bindings of the two checkers. Not part of the product.

* ``RefLib``    : oracle/_ref/libtl_ref.so, the reference's own CPU code behind ref_harness.cpp.
* ``OracleLib`` : oracle/_build/libtl_oracle.so, the plain-C restatement (tl_oracle.c).

Both expose the same function set with the prefixes ``ref_`` / ``orc_`` so a test can run one
against the other. Arrays are numpy fp16 / int32, C-contiguous.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_SO = os.path.join(HERE, "_ref", "libtl_ref.so")
ORACLE_SO = os.path.join(HERE, "_build", "libtl_oracle.so")

_u16p = C.POINTER(C.c_uint16)
_i32p = C.POINTER(C.c_int)


def _p16(a: np.ndarray):
    assert a.dtype == np.float16 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_u16p)


def _pi(a: np.ndarray):
    assert a.dtype == np.int32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_i32p)


class _Lib:
    prefix = ""
    path = ""

    def __init__(self):
        if not os.path.exists(self.path):
            raise FileNotFoundError(self.path)
        self.lib = C.CDLL(self.path)
        p = self.prefix
        L = self.lib
        self._fn = {}
        sigs = {
            "matmul2d_f16": [_u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_int],
            "linear_f16": [_u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_int],
            "bmm_nt_f16": [_u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_int, C.c_int],
            "rmsnorm_f16": [_u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_float],
            "rope_f16": [_u16p, _u16p, C.c_int, C.c_int, C.c_int, C.c_int],
            "softmax_f16": [_u16p, _u16p, C.c_int, C.c_int],
            "silu_f16": [_u16p, _u16p, C.c_int, C.c_int],
            "ewise_f16": [_u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_double],
            "argmax_f16": [_u16p, _i32p, C.c_int, C.c_int],
            "llama2_load": [C.c_void_p, _u16p, C.c_int],
            "llama2_forward": [C.c_void_p, _i32p, C.c_int, C.c_int, C.c_int, _u16p, _u16p],
        }
        for name, args in sigs.items():
            f = getattr(L, p + name)
            f.argtypes = args
            f.restype = C.c_int
            self._fn[name] = f
        self._create = getattr(L, p + "llama2_create")
        self._create.argtypes = [C.c_int] * 6
        self._create.restype = C.c_void_p
        self._destroy = getattr(L, p + "llama2_destroy")
        self._destroy.argtypes = [C.c_void_p]
        self._destroy.restype = None
        self._err = getattr(L, p + "last_error")
        self._err.restype = C.c_char_p
        self._maxthr = getattr(L, p + "omp_max_threads")
        self._maxthr.restype = C.c_int
        self._setthr = getattr(L, p + "omp_set_threads")
        self._setthr.argtypes = [C.c_int]
        ip, vp, sz = _i32p, C.c_void_p, C.c_size_t
        for name, args in {
            "unary_f16": [_u16p, _u16p, C.c_int, C.c_int],
            "binary_f16": [_u16p, _u16p, _u16p, C.c_int, C.c_int],
            "binary_scalar_f16": [_u16p, C.c_uint16, _u16p, C.c_int, C.c_int],
            "reduce_f16": [_u16p, _u16p, sz, sz, C.c_int],
            "argreduce_f16": [_u16p, ip, sz, sz, C.c_int],
            "cast": [vp, vp, sz, C.c_int],
            "matmul_strided_f16": [_u16p, _u16p, _u16p, ip, ip, sz, sz, ip, C.c_int, sz, sz],
        }.items():
            self._bind(name, args)
        self._bind_extra()

    def _bind_extra(self):
        pass

    def _bind(self, name, args):
        f = getattr(self.lib, self.prefix + name)
        f.argtypes = args
        f.restype = C.c_int
        self._fn[name] = f

    def _call(self, name, *args):
        rc = self._fn[name](*args)
        if rc != 0:
            raise RuntimeError(f"{self.prefix}{name}: {self._err().decode()}")

    # -- threads -------------------------------------------------------------------------------
    def max_threads(self) -> int:
        return int(self._maxthr())

    def set_threads(self, n: int) -> None:
        self._setthr(int(n))

    # -- single operators -----------------------------------------------------------------------
    def matmul2d(self, A: np.ndarray, B: np.ndarray) -> np.ndarray:
        """A[M,K] x B[N,K]^T -> C[M,N] (the Device::matmul2d contract)."""
        M, K = A.shape
        N, K2 = B.shape
        assert K == K2
        Cm = np.empty((M, N), dtype=np.float16)
        self._call("matmul2d_f16", _p16(A), _p16(B), _p16(Cm), M, N, K)
        return Cm

    def linear(self, x: np.ndarray, W: np.ndarray) -> np.ndarray:
        T, K = x.shape
        N, K2 = W.shape
        assert K == K2
        y = np.empty((T, N), dtype=np.float16)
        self._call("linear_f16", _p16(x), _p16(W), _p16(y), T, K, N)
        return y

    def bmm_nt(self, a: np.ndarray, bt: np.ndarray) -> np.ndarray:
        B, M, K = a.shape
        B2, N, K2 = bt.shape
        assert B == B2 and K == K2
        c = np.empty((B, M, N), dtype=np.float16)
        self._call("bmm_nt_f16", _p16(a), _p16(bt), _p16(c), B, M, N, K)
        return c

    def rmsnorm(self, x: np.ndarray, w: np.ndarray, eps: float = 1e-5) -> np.ndarray:
        T, D = x.shape
        y = np.empty_like(x)
        self._call("rmsnorm_f16", _p16(x), _p16(w), _p16(y), T, D, eps)
        return y

    def rope(self, x: np.ndarray, start_pos: int) -> np.ndarray:
        T, H, hd = x.shape
        y = np.empty_like(x)
        self._call("rope_f16", _p16(x), _p16(y), start_pos, T, H, hd)
        return y

    def rope_table(self, max_pos: int, hd: int):
        """(cos, sin) fp16 tables [max_pos, hd/2] exactly as the rotation uses them: rotating
        the pair (1, 0) returns (cos, sin) with no further rounding."""
        x = np.zeros((max_pos, 1, hd), dtype=np.float16)
        x[:, :, 0::2] = 1.0
        y = self.rope(x, 0)
        return np.ascontiguousarray(y[:, 0, 0::2]), np.ascontiguousarray(y[:, 0, 1::2])

    def softmax(self, x: np.ndarray) -> np.ndarray:
        R, Cc = x.shape
        y = np.empty_like(x)
        self._call("softmax_f16", _p16(x), _p16(y), R, Cc)
        return y

    def silu(self, x: np.ndarray, via_float: bool) -> np.ndarray:
        y = np.empty_like(x)
        self._call("silu_f16", _p16(x), _p16(y), x.size, int(via_float))
        return y

    def ewise(self, a: np.ndarray, b, op: str, scalar: float = 0.0) -> np.ndarray:
        y = np.empty_like(a)
        code = {"add": 0, "mul": 1, "sdiv": 2}[op]
        bb = a if b is None else b
        self._call("ewise_f16", _p16(a), _p16(bb), _p16(y), a.size, code, scalar)
        return y

    def argmax(self, x: np.ndarray) -> np.ndarray:
        R, Cc = x.shape
        idx = np.empty(R, dtype=np.int32)
        self._call("argmax_f16", _p16(x), _pi(idx), R, Cc)
        return idx

    # -- the rest of the Device<half> surface (op names as in tensorlib_b200: UNARY_OPS, ...) -------
    UNARY = {"neg": 0, "sin": 1, "cos": 2, "exp": 3, "log": 4, "abs": 5, "tanh": 6, "silu": 7, "sqrt": 8, "rsqrt": 9,
             "silu_cpu_half": 10}
    BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "pow": 4}
    REDUCE = {"max": 0, "min": 1, "sum": 2, "mean": 3}

    def unary(self, x: np.ndarray, op: str) -> np.ndarray:
        y = np.empty_like(x)
        self._call("unary_f16", _p16(x), _p16(y), x.size, self.UNARY[op])
        return y

    def binary(self, a: np.ndarray, b, op: str) -> np.ndarray:
        y = np.empty_like(a)
        if np.ndim(b) == 0:
            self._call("binary_scalar_f16", _p16(a), int(np.float16(b).view(np.uint16)), _p16(y), a.size, self.BINARY[op])
        else:
            self._call("binary_f16", _p16(a), _p16(np.ascontiguousarray(b)), _p16(y), a.size, self.BINARY[op])
        return y

    def reduce(self, x: np.ndarray, op: str) -> np.ndarray:
        R, Cc = x.shape
        y = np.empty(R, dtype=np.float16)
        self._call("reduce_f16", _p16(x), _p16(y), Cc, x.size, self.REDUCE[op])
        return y

    def argreduce(self, x: np.ndarray, want_min: bool) -> np.ndarray:
        R, Cc = x.shape
        idx = np.empty(R, dtype=np.int32)
        self._call("argreduce_f16", _p16(x), _pi(idx), Cc, x.size, int(want_min))
        return idx

    def cast(self, x: np.ndarray, to) -> np.ndarray:
        kinds = {(np.float16, np.float32): 0, (np.float32, np.float16): 1, (np.float16, np.int32): 2, (np.int32, np.float16): 3}
        x = np.ascontiguousarray(x)
        y = np.empty(x.shape, dtype=to)
        self._call("cast", x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), x.size, kinds[(x.dtype.type, np.dtype(to).type)])
        return y

    def matmul_strided(self, lhs, rhs, lhs_stride, rhs_stride, lhs_offset, rhs_offset, result_shape, K) -> np.ndarray:
        """Device::matmul with per-dimension strides over flat fp16 buffers."""
        ls, rs, sh = (np.ascontiguousarray(v, dtype=np.int32) for v in (lhs_stride, rhs_stride, result_shape))
        out = np.empty(tuple(result_shape), dtype=np.float16)
        self._call("matmul_strided_f16", _p16(lhs), _p16(rhs), _p16(out), _pi(ls), _pi(rs), lhs_offset, rhs_offset, _pi(sh),
                   sh.size, out.size, K)
        return out

    def contiguous(self, data: np.ndarray, shape, stride, offset: int = 0) -> np.ndarray:
        raise NotImplementedError

    def set_item(self, data: np.ndarray, src, shape, stride, offset: int = 0) -> np.ndarray:
        raise NotImplementedError

    # -- model ---------------------------------------------------------------------------------
    def llama2(self, cfg, payload: np.ndarray) -> "_Model":
        return _Model(self, cfg, payload)


class _Model:
    def __init__(self, lib: _Lib, cfg, payload: np.ndarray):
        self.lib, self.cfg = lib, cfg
        self.h = lib._create(cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.n_heads, cfg.vocab_size,
                             cfg.seq_len)
        if not self.h:
            raise RuntimeError("llama2_create: " + lib._err().decode())
        assert payload.dtype == np.float16 and payload.size == cfg.payload_elems()
        lib._call("llama2_load", self.h, _p16(payload), int(cfg.shared_classifier))

    def forward(self, tokens, start_pos: int, silu_mode: int = 1, want_hidden: bool = False):
        """silu_mode 0 / 1: the SiLU route (CPU fp16 as shipped / through float). OracleLib only:
        +2 computes RMSNorm as the reference's CUDA backend does (fp32 sum) instead of the CPU's
        fp16 running sum, which loses 3-5 % at dim 4096."""
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        T = tok.size
        logits = np.empty((T, self.cfg.vocab_size), dtype=np.float16)
        hidden = np.empty((self.cfg.n_layers, T, self.cfg.dim), dtype=np.float16) if want_hidden else None
        hp = _p16(hidden) if want_hidden else C.cast(None, _u16p)
        self.lib._call("llama2_forward", self.h, _pi(tok), T, start_pos, silu_mode, _p16(logits), hp)
        return (logits, hidden) if want_hidden else logits

    def generate(self, prompt, n_gen: int, silu_mode: int = 1, keep_logits: bool = False):
        """Greedy decode like Llama2::generate (model/llama2_7b/src/llama2.cpp:15-101) without
        the stop-on-id-1/2 rule: prefill the prompt, then n_gen-1 single-token steps. Returns the
        n_gen sampled ids (and the last-position logits of every forward)."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        out, all_logits = [], []
        logits = self.forward(prompt, 0, silu_mode)
        last = logits[-1:]
        pos = prompt.size
        for _ in range(n_gen):
            nxt = int(self.lib.argmax(np.ascontiguousarray(last))[0])
            out.append(nxt)
            if keep_logits:
                all_logits.append(last[0].copy())
            if len(out) == n_gen:
                break
            last = self.forward(np.array([nxt], dtype=np.int32), pos, silu_mode)
            pos += 1
        ids = np.array(out, dtype=np.int32)
        return (ids, np.stack(all_logits)) if keep_logits else ids

    def close(self):
        if self.h:
            self.lib._destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class RefLib(_Lib):
    prefix = "ref_"
    path = REF_SO

    def _bind_extra(self):
        self._bind("cuda_rms_norm_f16", [_u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_float])
        self._bind("cuda_matmul2d_f16", [_u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                         C.POINTER(C.c_double)])
        self._cuda_count = self.lib.ref_cuda_device_count
        self._cuda_count.restype = C.c_int
        self._bind("contiguous_f16", [_u16p, _u16p, C.c_size_t, _i32p, _i32p, C.c_int, C.c_size_t, C.c_size_t])
        self._bind("set_item_f16", [_u16p, C.c_size_t, _u16p, C.c_int, _i32p, _i32p, C.c_int, C.c_size_t, C.c_size_t])

    def contiguous(self, data, shape, stride, offset=0):
        sh, sd = np.ascontiguousarray(shape, dtype=np.int32), np.ascontiguousarray(stride, dtype=np.int32)
        n = int(np.prod(sh)) if sh.size else 1
        out = np.empty(n, dtype=np.float16)
        self._call("contiguous_f16", _p16(out), _p16(data), data.size, _pi(sh), _pi(sd), sh.size, offset, n)
        return out.reshape(tuple(shape))

    def set_item(self, data, src, shape, stride, offset=0):
        sh, sd = np.ascontiguousarray(shape, dtype=np.int32), np.ascontiguousarray(stride, dtype=np.int32)
        n = int(np.prod(sh)) if sh.size else 1
        out = data.copy()
        scalar = np.ndim(src) == 0
        v = np.array([src], dtype=np.float16) if scalar else np.ascontiguousarray(src, dtype=np.float16).reshape(-1)
        self._call("set_item_f16", _p16(out), out.size, _p16(v), int(scalar), _pi(sh), _pi(sd), sh.size, offset, n)
        return out

    # -- the reference's CUDA backend (needs a GPU): a baseline and a cross-check, never an oracle ----
    def cuda_device_count(self) -> int:
        return int(self._cuda_count())

    def cuda_rms_norm(self, x: np.ndarray, w: np.ndarray, eps: float = 1e-5) -> np.ndarray:
        """nn::RMSNorm<half>::forward on "cuda" tensors (rms_norm_kernel_v1)."""
        T, D = x.shape
        y = np.empty_like(x)
        self._call("cuda_rms_norm_f16", _p16(x), _p16(w), _p16(y), T, D, eps)
        return y

    def cuda_matmul2d(self, A: np.ndarray, B: np.ndarray, reps: int = 0, b_copies: int = 1):
        """CUDA<half>::matmul2d (gemv_v6 / gemv_v4 / hgemm_cublas) on device copies; returns
        (C, mean microseconds per call or None)."""
        M, K = A.shape
        N, _ = B.shape
        Cm = np.empty((M, N), dtype=np.float16)
        us = C.c_double(0.0)
        self._call("cuda_matmul2d_f16", _p16(A), _p16(B), _p16(Cm), M, N, K, reps, b_copies, C.byref(us))
        return Cm, (us.value if reps > 0 else None)


class OracleLib(_Lib):
    prefix = "orc_"
    path = ORACLE_SO

    def _bind_extra(self):
        self._bind("rmsnorm_cuda_route_f16", [_u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_float])
        self._bind("contiguous_f16", [_u16p, _u16p, _i32p, _i32p, C.c_int, C.c_size_t, C.c_size_t])
        self._bind("set_item_f16", [_u16p, _u16p, _i32p, _i32p, C.c_int, C.c_size_t, C.c_size_t])
        self._bind("set_item_scalar_f16", [_u16p, C.c_uint16, _i32p, _i32p, C.c_int, C.c_size_t, C.c_size_t])

    def contiguous(self, data, shape, stride, offset=0):
        sh, sd = np.ascontiguousarray(shape, dtype=np.int32), np.ascontiguousarray(stride, dtype=np.int32)
        n = int(np.prod(sh)) if sh.size else 1
        out = np.empty(n, dtype=np.float16)
        self._call("contiguous_f16", _p16(out), _p16(data), _pi(sh), _pi(sd), sh.size, offset, n)
        return out.reshape(tuple(shape))

    def set_item(self, data, src, shape, stride, offset=0):
        sh, sd = np.ascontiguousarray(shape, dtype=np.int32), np.ascontiguousarray(stride, dtype=np.int32)
        n = int(np.prod(sh)) if sh.size else 1
        out = data.copy()
        if np.ndim(src) == 0:
            self._call("set_item_scalar_f16", _p16(out), int(np.float16(src).view(np.uint16)), _pi(sh), _pi(sd), sh.size, offset, n)
        else:
            self._call("set_item_f16", _p16(out), _p16(np.ascontiguousarray(src, dtype=np.float16).reshape(-1)), _pi(sh), _pi(sd),
                       sh.size, offset, n)
        return out

    def rmsnorm_cuda_route(self, x: np.ndarray, w: np.ndarray, eps: float = 1e-5) -> np.ndarray:
        """RMSNorm as the reference's CUDA backend computes it (fp32 sum of squares)."""
        T, D = x.shape
        y = np.empty_like(x)
        self._call("rmsnorm_cuda_route_f16", _p16(x), _p16(w), _p16(y), T, D, eps)
        return y


def have_ref() -> bool:
    return os.path.exists(REF_SO)


def have_oracle() -> bool:
    return os.path.exists(ORACLE_SO)
