"""ctypes loader for oracle/liboracle.so, the CPU restatement used as the checker in tests."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_lib = C.CDLL(os.path.join(ROOT, "oracle", "liboracle.so"))
u32, u64, vp = C.c_uint32, C.c_uint64, C.c_void_p
_lib.oracle_gen_x_i8.argtypes = [vp, u64, u32]
_lib.oracle_gen_fixed.argtypes = [u32, u32, u32, vp]
_lib.oracle_gen_iid.argtypes = [u32, u32, C.c_double, u64, vp]
_lib.oracle_build_lists.argtypes = [vp, u32, u32, u32, C.c_uint16, vp, vp, vp, vp]
_lib.oracle_build_lists.restype = C.c_int64
_lib.oracle_encode_div.argtypes = [vp, u32, u32, u32, vp]
_lib.oracle_delta_lists.argtypes = [vp, u32, u32, vp]
_lib.oracle_delta_lists.restype = u64
_lib.oracle_encode_delta_div256.argtypes = [vp, u32, u32, vp]
_lib.oracle_gemv_i8_div.argtypes = [vp, vp, vp, vp, u32, u32, u32, u32, u32]
_lib.oracle_gemv_i8_delta256.argtypes = [vp, vp, vp, vp, u32, u32, u32, u32]
_lib.oracle_gemv_i8_dense.argtypes = [vp, vp, vp, u32, u32, u32]
_lib.oracle_gemv_i8_lists.argtypes = [vp, vp, vp, vp, vp, u32, vp, u32, u32, u32]
_lib.oracle_gemv_f32_lists.argtypes = [vp, vp, vp, vp, vp, u32, vp, vp, vp, u32, u32, u32]
_lib.oracle_i2s_pack16.argtypes = [vp]
_lib.oracle_i2s_pack16.restype = u32
_lib.oracle_i2s_unpack16.argtypes = [u32, vp]
_lib.oracle_gemv_i8_div_mt.argtypes = [vp, vp, vp, vp, u32, u32, u32, u32, u32, u32]
_lib.oracle_gemv_i8_div_mt.restype = C.c_int


def _p(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def gen_x_i8(count: int, seed: int) -> np.ndarray:
    x = np.empty(count, dtype=np.int8)
    _lib.oracle_gen_x_i8(_p(x), count, seed)
    return x


def gen_fixed(K: int, N: int, S: int) -> np.ndarray:
    W = np.empty((N, K), dtype=np.int8)
    assert _lib.oracle_gen_fixed(K, N, S, _p(W)) == 0
    return W


def gen_iid(K: int, N: int, p_zero: float, seed: int) -> np.ndarray:
    W = np.empty((N, K), dtype=np.int8)
    assert _lib.oracle_gen_iid(K, N, p_zero, seed, _p(W)) == 0
    return W


def build_lists(W: np.ndarray, cap: int, sentinel: int):
    N, K = W.shape
    pos = np.empty((N, cap), dtype=np.uint16)
    neg = np.empty((N, cap), dtype=np.uint16)
    npos = np.empty(N, dtype=np.uint32)
    nneg = np.empty(N, dtype=np.uint32)
    mx = _lib.oracle_build_lists(_p(W), K, N, cap, sentinel, _p(pos), _p(neg), _p(npos), _p(nneg))
    assert mx >= 0, "a column overflows cap"
    return pos, neg, npos, nneg


def encode_div(lst: np.ndarray, split: int) -> np.ndarray:
    N, half = lst.shape
    out = np.zeros(half * N, dtype=np.uint16)
    _lib.oracle_encode_div(_p(lst), half, N, split, _p(out))
    return out


def delta_lists(lst: np.ndarray):
    N, half = lst.shape
    gaps = np.empty((N, half), dtype=np.uint8)
    lossy = _lib.oracle_delta_lists(_p(lst), half, N, _p(gaps))
    return gaps, int(lossy)


def encode_delta_div256(gaps: np.ndarray) -> np.ndarray:
    N, half = gaps.shape
    out = np.zeros(256 * N * ((half + 255) // 256), dtype=np.uint8)
    _lib.oracle_encode_delta_div256(_p(gaps), half, N, _p(out))
    return out


def gemv_i8_div(X, wpos, wneg, M, K, N, S, split) -> np.ndarray:
    Cm = np.empty((M, N), dtype=np.int32)
    _lib.oracle_gemv_i8_div(_p(X), _p(wpos), _p(wneg), _p(Cm), M, K, N, S, split)
    return Cm


def gemv_i8_div_mt(X, wpos, wneg, M, K, N, S, split, threads) -> np.ndarray:
    Cm = np.empty((M, N), dtype=np.int32)
    assert _lib.oracle_gemv_i8_div_mt(_p(X), _p(wpos), _p(wneg), _p(Cm), M, K, N, S, split, threads) == 0
    return Cm


def gemv_i8_delta256(X, dpos, dneg, M, K, N, S) -> np.ndarray:
    Cm = np.empty((M, N), dtype=np.int32)
    _lib.oracle_gemv_i8_delta256(_p(X), _p(dpos), _p(dneg), _p(Cm), M, K, N, S)
    return Cm


def gemv_i8_dense(X, W) -> np.ndarray:
    N, K = W.shape
    M = X.size // K
    Cm = np.empty((M, N), dtype=np.int32)
    _lib.oracle_gemv_i8_dense(_p(X), _p(W), _p(Cm), M, K, N)
    return Cm


def gemv_i8_lists(X, pos, neg, npos, nneg, K) -> np.ndarray:
    N, cap = pos.shape
    M = X.size // K
    Cm = np.empty((M, N), dtype=np.int32)
    _lib.oracle_gemv_i8_lists(_p(X), _p(pos), _p(neg), _p(npos), _p(nneg), cap, _p(Cm), M, K, N)
    return Cm


def gemv_f32_lists(X32, pos, neg, npos, nneg, K):
    """Returns (fp32 in the reference's order, double sum, sum of |x|)."""
    N, cap = pos.shape
    M = X32.size // K
    ref = np.empty((M, N), dtype=np.float32)
    dbl = np.empty((M, N), dtype=np.float64)
    ab = np.empty((M, N), dtype=np.float64)
    _lib.oracle_gemv_f32_lists(_p(X32), _p(pos), _p(neg), _p(npos), _p(nneg), cap, _p(ref), _p(dbl), _p(ab), M, K, N)
    return ref, dbl, ab


def i2s_pack16(w16: np.ndarray) -> int:
    w16 = np.ascontiguousarray(w16, dtype=np.int8)
    return int(_lib.oracle_i2s_pack16(_p(w16)))


def i2s_unpack16(word: int) -> np.ndarray:
    out = np.empty(16, dtype=np.int8)
    _lib.oracle_i2s_unpack16(word, _p(out))
    return out


_lib.oracle_quant_absmax_i8.argtypes = [vp, u32, vp, u32, u32, u32, vp, vp]
_lib.oracle_fnv1a64.argtypes = [vp, u64]
_lib.oracle_fnv1a64.restype = u64


_lib.oracle_ternarise_absmean.argtypes = [vp, u32, u32, vp, vp]


def ternarise_absmean(W: np.ndarray):
    """fp32 weights of shape (N, K) -> (int8 ternary, scale): the oracle's absmean rule."""
    W = np.ascontiguousarray(W, dtype=np.float32)
    N, K = W.shape
    out = np.empty((N, K), dtype=np.int8)
    scale = np.zeros(1, dtype=np.float32)
    _lib.oracle_ternarise_absmean(_p(W), K, N, _p(out), _p(scale))
    return out, float(scale[0])


def fnv1a64(a) -> str:
    a = np.ascontiguousarray(a)
    return "%016x" % _lib.oracle_fnv1a64(_p(a), a.nbytes)


def quant_absmax_i8(A: np.ndarray, B=None):
    """A (and optional B): int32 (M, K) possibly strided views; returns (int8 (M,K), float32 scale (M,))."""
    M, K = A.shape
    lda = A.strides[0] // 4
    ldb = B.strides[0] // 4 if B is not None else 0
    out = np.empty((M, K), dtype=np.int8)
    scale = np.empty(M, dtype=np.float32)
    _lib.oracle_quant_absmax_i8(A.ctypes.data, lda, B.ctypes.data if B is not None else None, ldb, M, K, _p(out), _p(scale))
    return out, scale
