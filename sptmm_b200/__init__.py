"""sptmm_b200 -- thin Python binding over libsptmm.so (the C ABI in include/sptmm.h).

The library is the product; this module only marshals arguments with ctypes.  There is no
Python or CPU fallback: importing without a built library raises, and every compute call goes
through the C ABI into the CUDA kernels.

Names follow the reference program's operator surface (Ogiwara-CostlierRain464/SpTMM main.cu):
``row_split3_small`` / ``row_split_delta2`` are its two SpTMM modes (flags at main.cu:39-40),
``i2s`` its 2-bit comparator (main.cu:41).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
# SPTMM_B200_TUNING=1 loads the tuning build (build.py --tuning: kernel timelines, overridable launch
# constants) instead of the product library; only measurement scripts set it.
TUNING = os.environ.get("SPTMM_B200_TUNING", "") not in ("", "0")
LIB_PATH = os.path.join(_PKG, "libsptmm_tuning.so" if TUNING else "libsptmm.so")

FMT_U16_DIV, FMT_DELTA_DIV256, FMT_U16_V256, FMT_DELTA_LANE, FMT_I2S = 1, 2, 3, 4, 5
I8, F16, F32 = 0, 1, 2
X_COLMAJOR, C_COLMAJOR, LAUNCH_PDL = 1, 2, 4

_NP_DTYPE = {I8: np.int8, F16: np.float16, F32: np.float32}
_OUT_DTYPE = {I8: np.int32, F16: np.float32, F32: np.float32}


class SptmmError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__("sptmm error %d: %s" % (code, message))
        self.code = code
        self.message = message


class WeightsInfo(C.Structure):
    _fields_ = [("K", C.c_uint32), ("N", C.c_uint32), ("format", C.c_uint32), ("split", C.c_uint32),
                ("S", C.c_uint32), ("max_count", C.c_uint32), ("nnz", C.c_uint64),
                ("stream_bytes", C.c_uint64), ("lossy_entries", C.c_uint64), ("n_arrays", C.c_uint32),
                ("device", C.c_int32), ("k_tile", C.c_uint32), ("n_tiles", C.c_uint32)]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError("%s is not built: run `python sptmm_b200/build.py%s` (needs nvcc)"
                          % (os.path.basename(LIB_PATH), " --tuning" if TUNING else ""))
    lib = C.CDLL(LIB_PATH)
    u32, u64, vp, i32 = C.c_uint32, C.c_uint64, C.c_void_p, C.c_int
    sigs = {
        "sptmm_last_error": (C.c_char_p, []),
        "sptmm_version": (i32, []),
        "sptmm_gen_ternary_fixed": (i32, [u32, u32, u32, vp]),
        "sptmm_gen_ternary_iid": (i32, [u32, u32, C.c_double, u64, vp]),
        "sptmm_ternarise_absmean": (i32, [vp, u32, u32, u32, vp, C.POINTER(C.c_float)]),
        "sptmm_encode": (i32, [vp, u32, u32, u32, u32, u32, C.POINTER(vp)]),
        "sptmm_encode_ktiled": (i32, [vp, u32, u32, u32, C.POINTER(vp)]),
        "sptmm_weights_tile": (i32, [vp, u32, C.POINTER(vp)]),
        "sptmm_weights_info_get": (i32, [vp, C.POINTER(WeightsInfo)]),
        "sptmm_weights_array": (i32, [vp, u32, C.POINTER(vp), C.POINTER(vp), C.POINTER(u64), C.POINTER(C.c_char_p)]),
        "sptmm_weights_upload": (i32, [vp]),
        "sptmm_weights_upload_replicas": (i32, [vp, u32]),
        "sptmm_weights_free": (i32, [vp]),
        "sptmm_gemv": (i32, [vp, vp, u32, u32, vp, u32, u32, vp]),
        "sptmm_weights_save": (i32, [vp, C.c_char_p]),
        "sptmm_weights_load": (i32, [C.c_char_p, C.POINTER(C.c_void_p)]),
        "sptmm_gemv_status": (i32, [vp, C.POINTER(u32)]),
        "sptmm_quantize_absmax": (i32, [vp, u32, u32, u32, u32, u32, vp, vp, u32, vp]),
        "sptmm_gemv_scaled": (i32, [vp, vp, u32, vp, vp, C.c_float, u32, u32, vp]),
        "sptmm_gemv_reduce": (i32, [vp, vp, u32, u32, vp, u32, u32, u32, vp]),
        "sptmm_gemv_host": (i32, [vp, vp, u32, u32, vp, u32, u32]),
        "sptmm_gemv_host_async": (i32, [vp, vp, u32, u32, vp, u32, u32, u32]),
        "sptmm_gemv_host_wait": (i32, [vp, u32]),
        "sptmm_gemv_host_batch": (i32, [vp, u32, vp, vp, vp, u32, u32, u32, u32, u32]),
        "sptmm_row_split3_small": (i32, [vp, vp, vp, vp, u32, u32, u32, u32, u32, vp]),
        "sptmm_row_split_delta2": (i32, [vp, vp, vp, vp, u32, u32, u32, u32, u32, vp]),
        "sptmm_dense_cublas_gemm": (i32, [vp, vp, vp, u32, u32, u32, vp]),
        "sptmm_dense_cublas_gemm_f16": (i32, [vp, vp, vp, u32, u32, u32, vp]),
        "sptmm_seq_create": (i32, [vp, u32, u32, C.POINTER(vp)]),
        "sptmm_seq_create_shared": (i32, [vp, u32, u32, vp, vp, u32, u32, C.POINTER(vp)]),
        "sptmm_seq_shared_bytes": (u64, [u32]),
        "sptmm_seq_shared_bytes_for": (u64, [vp, u32, u32]),
        "sptmm_seq_run": (i32, [vp, vp]),
        "sptmm_seq_run_static": (i32, [vp, u32, u32, vp, C.POINTER(u32)]),
        "sptmm_seq_status": (i32, [vp, C.POINTER(u32), C.POINTER(u64)]),
        "sptmm_seq_set_wait_limit": (i32, [vp, u32]),
        "sptmm_seq_free": (i32, [vp]),
        "sptmm_stack_weights_create": (i32, [vp, C.POINTER(vp)]),
        "sptmm_stack_weights_info": (i32, [vp, C.POINTER(u64), C.POINTER(u64)]),
        "sptmm_stack_weights_matrix": (i32, [vp, u32, C.POINTER(vp)]),
        "sptmm_stack_weights_free": (i32, [vp]),
        "sptmm_stack_arena_bytes": (u64, [vp, u32, u32]),
        "sptmm_stack_create": (i32, [vp, u32, u32, vp, C.POINTER(vp)]),
        "sptmm_stack_set_input": (i32, [vp, vp]),
        "sptmm_stack_forward": (i32, [vp, vp]),
        "sptmm_stack_buffer": (i32, [vp, C.c_char_p, vp, C.POINTER(u32)]),
        "sptmm_stack_status": (i32, [vp, C.POINTER(u32)]),
        "sptmm_stack_exchange": (i32, [vp, C.POINTER(u32)]),
        "sptmm_stack_sequence": (i32, [vp, C.POINTER(vp)]),
        "sptmm_stack_wait_limit": (i32, [vp, u32]),
        "sptmm_stack_free": (i32, [vp]),
        "sptmm_splitk_k_range": (i32, [u32, u32, u32, C.POINTER(u32), C.POINTER(u32)]),
        "sptmm_splitk_col_range": (i32, [u32, u32, u32, C.POINTER(u32), C.POINTER(u32)]),
        "sptmm_splitk_arena_bytes": (u64, [u32, u32, u32]),
        "sptmm_splitk_create": (i32, [vp, u32, u32, u32, u32, C.POINTER(vp), C.POINTER(vp)]),
        "sptmm_splitk_forward": (i32, [vp, vp, u32, vp]),
        "sptmm_splitk_clear": (i32, [vp, vp]),
        "sptmm_splitk_barrier": (i32, [vp, vp]),
        "sptmm_splitk_accumulate": (i32, [vp, vp, u32, vp]),
        "sptmm_splitk_output": (i32, [vp, C.POINTER(vp), C.POINTER(u32)]),
        "sptmm_splitk_status": (i32, [vp, C.POINTER(u32)]),
        "sptmm_splitk_set_wait_limit": (i32, [vp, u64]),
        "sptmm_splitk_free": (i32, [vp]),
        "sptmm_device_count": (i32, [C.POINTER(C.c_int)]),
        "sptmm_set_device": (i32, [C.c_int]),
        "sptmm_dev_alloc": (i32, [C.POINTER(vp), u64]),
        "sptmm_dev_free": (i32, [vp]),
        "sptmm_memcpy_h2d": (i32, [vp, vp, u64]),
        "sptmm_memcpy_d2h": (i32, [vp, vp, u64]),
        "sptmm_device_sync": (i32, []),
        "sptmm_stream_wait": (i32, [vp]),
    }
    if TUNING:                           # csrc/tuning.h
        sigs["sptmm_seq_set_trace"] = (i32, [vp, vp])
        sigs["sptmm_set_trace_buffer"] = (i32, [vp])
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)          # AttributeError if the header and the library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()
EXPORTS = ["sptmm_last_error", "sptmm_version", "sptmm_gen_ternary_fixed", "sptmm_gen_ternary_iid", "sptmm_ternarise_absmean",
           "sptmm_encode", "sptmm_encode_ktiled", "sptmm_weights_tile", "sptmm_weights_info_get", "sptmm_weights_array", "sptmm_weights_upload",
           "sptmm_weights_upload_replicas", "sptmm_weights_free", "sptmm_weights_save", "sptmm_weights_load", "sptmm_gemv", "sptmm_gemv_status", "sptmm_quantize_absmax", "sptmm_gemv_scaled", "sptmm_gemv_reduce", "sptmm_gemv_host", "sptmm_gemv_host_async", "sptmm_gemv_host_wait", "sptmm_gemv_host_batch",
           "sptmm_row_split3_small", "sptmm_row_split_delta2", "sptmm_dense_cublas_gemm", "sptmm_dense_cublas_gemm_f16",
           "sptmm_seq_create", "sptmm_seq_create_shared", "sptmm_seq_shared_bytes", "sptmm_seq_shared_bytes_for", "sptmm_seq_run", "sptmm_seq_run_static", "sptmm_seq_status", "sptmm_seq_set_wait_limit", "sptmm_seq_free",
           "sptmm_stack_weights_create", "sptmm_stack_weights_info", "sptmm_stack_weights_matrix", "sptmm_stack_weights_free",
           "sptmm_stack_arena_bytes", "sptmm_stack_create", "sptmm_stack_set_input", "sptmm_stack_forward", "sptmm_stack_buffer",
           "sptmm_stack_status", "sptmm_stack_exchange", "sptmm_stack_sequence", "sptmm_stack_wait_limit", "sptmm_stack_free",
           "sptmm_splitk_k_range", "sptmm_splitk_col_range", "sptmm_splitk_arena_bytes", "sptmm_splitk_create", "sptmm_splitk_forward",
           "sptmm_splitk_clear", "sptmm_splitk_barrier", "sptmm_splitk_accumulate", "sptmm_splitk_output", "sptmm_splitk_status",
           "sptmm_splitk_set_wait_limit", "sptmm_splitk_free",
           "sptmm_device_count", "sptmm_set_device", "sptmm_dev_alloc", "sptmm_dev_free",
           "sptmm_memcpy_h2d", "sptmm_memcpy_d2h", "sptmm_device_sync", "sptmm_stream_wait"]


def check(rc: int) -> None:
    if rc != 0:
        raise SptmmError(rc, lib.sptmm_last_error().decode("utf-8", "replace"))


def _ptr(x) -> int:
    """Address of a numpy array (host), a torch tensor (host or device) or a raw integer."""
    if isinstance(x, (int, np.integer)):
        return int(x)
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    raise TypeError("expected numpy array, torch tensor or address, got %r" % type(x))


def device_count() -> int:
    n = C.c_int(0)
    rc = lib.sptmm_device_count(C.byref(n))
    return n.value if rc == 0 else 0


def gen_ternary_fixed(K: int, N: int, S: int) -> np.ndarray:
    """Reference generator (main.cu:248-265): returns W as int8 array of shape (N, K), i.e.
    column-major K x N -- W[c] is column c."""
    W = np.empty((N, K), dtype=np.int8)
    check(lib.sptmm_gen_ternary_fixed(K, N, S, W.ctypes.data))
    return W


def gen_ternary_iid(K: int, N: int, p_zero: float, seed: int) -> np.ndarray:
    W = np.empty((N, K), dtype=np.int8)
    check(lib.sptmm_gen_ternary_iid(K, N, float(p_zero), int(seed), W.ctypes.data))
    return W


def ternarise_absmean(W: np.ndarray) -> tuple[np.ndarray, float]:
    """fp16 / fp32 weights of shape (N, K) (column c of the K x N matrix is row c) -> (int8 ternary
    matrix of the same shape, scale): the absmean rule of BitNet b1.58 (sptmm_ternarise_absmean)."""
    if W.dtype not in (np.float16, np.float32) or W.ndim != 2:
        raise ValueError("W must be a 2-D float16 or float32 array")
    W = np.ascontiguousarray(W)
    N, K = W.shape
    out = np.empty((N, K), dtype=np.int8)
    scale = C.c_float(0)
    check(lib.sptmm_ternarise_absmean(W.ctypes.data, F16 if W.dtype == np.float16 else F32, K, N, out.ctypes.data, C.byref(scale)))
    return out, scale.value


class Weights:
    """An encoded ternary matrix (host-owned handle; optionally uploaded to the current device)."""

    def __init__(self, W_colmajor: np.ndarray, fmt: int = FMT_U16_V256, split: int = 32, S: int = 0, k_tile: int = 0):
        """k_tile > 0: the matrix is cut into K-tiles of that many rows (native u16 format only)."""
        W = np.ascontiguousarray(W_colmajor, dtype=np.int8)
        if W.ndim != 2:
            raise ValueError("W must be 2-D with shape (N, K): one row per column of the K x N matrix")
        N, K = W.shape
        h = C.c_void_p()
        if k_tile:
            if fmt != FMT_U16_V256:
                raise ValueError("K-tiles come in the native u16 format only")
            check(lib.sptmm_encode_ktiled(W.ctypes.data, K, N, k_tile, C.byref(h)))
        else:
            check(lib.sptmm_encode(W.ctypes.data, K, N, fmt, split, S, C.byref(h)))
        self._h = h
        self.info = self._info()

    @classmethod
    def borrow(cls, handle) -> "Weights":
        """A view of a handle somebody else owns (it is not freed with this object)."""
        self = cls.__new__(cls)
        self._h = handle
        self._borrowed = True
        self.info = self._info()
        return self

    @classmethod
    def load(cls, path: str) -> "Weights":
        """An encoded matrix written by save(); ready for upload()."""
        h = C.c_void_p()
        check(lib.sptmm_weights_load(os.fsencode(path), C.byref(h)))
        self = cls.__new__(cls)
        self._h = h
        self.info = self._info()
        return self

    def tile(self, t: int) -> "Weights":
        """K-tile `t` of a K-tiled matrix as a handle of its own (owned by this object)."""
        h = C.c_void_p()
        check(lib.sptmm_weights_tile(self._h, t, C.byref(h)))
        return Weights.borrow(h)

    def save(self, path: str) -> None:
        check(lib.sptmm_weights_save(self._h, os.fsencode(path)))

    def _info(self) -> WeightsInfo:
        info = WeightsInfo()
        check(lib.sptmm_weights_info_get(self._h, C.byref(info)))
        return info

    @property
    def K(self) -> int: return self.info.K
    @property
    def N(self) -> int: return self.info.N
    @property
    def stream_bytes(self) -> int: return self.info.stream_bytes

    def array(self, i: int) -> tuple[str, np.ndarray, Optional[int]]:
        """(name, host bytes as uint8 array copy, device address of replica 0 or None)."""
        hp, dp, nb, name = C.c_void_p(), C.c_void_p(), C.c_uint64(), C.c_char_p()
        check(lib.sptmm_weights_array(self._h, i, C.byref(hp), C.byref(dp), C.byref(nb), C.byref(name)))
        buf = (C.c_uint8 * nb.value).from_address(hp.value) if nb.value else (C.c_uint8 * 0)()
        return name.value.decode(), np.frombuffer(buf, dtype=np.uint8).copy(), dp.value

    def upload(self, replicas: int = 1) -> "Weights":
        check(lib.sptmm_weights_upload_replicas(self._h, replicas))
        self.info = self._info()
        return self

    def gemv(self, X, M: int, out, dtype: int = I8, flags: int = 0, replica: int = 0, stream: int = 0) -> None:
        """C = X*W on the device; X and out are device tensors (or addresses)."""
        check(lib.sptmm_gemv(self._h, _ptr(X), dtype, M, _ptr(out), flags, replica, stream))

    def gemv_scaled(self, X, M: int, out, row_scale=None, w_scale: float = 1.0, flags: int = 0, replica: int = 0, stream: int = 0) -> None:
        """C (float) = float(X*W) * (row_scale[m] * w_scale) for int8 X: the de-quantising epilogue."""
        check(lib.sptmm_gemv_scaled(self._h, _ptr(X), M, _ptr(out), _ptr(row_scale) if row_scale is not None else None,
                                    float(w_scale), flags, replica, stream))

    def status(self) -> int:
        """Waits for the device; 0 unless a bounded wait inside a kernel ran out since upload."""
        st = C.c_uint32(0)
        check(lib.sptmm_gemv_status(self._h, C.byref(st)))
        return st.value

    def gemv_reduce(self, X, M: int, C_peers, dtype: int = I8, flags: int = 0, replica: int = 0, stream: int = 0) -> None:
        """Split-K step: adds this rank's partial sums X*W into every column's owner buffer
        (C_peers[r]: rank r's M x shard-width buffer, device tensors or addresses)."""
        arr = (C.c_void_p * len(C_peers))(*[_ptr(c) for c in C_peers])
        check(lib.sptmm_gemv_reduce(self._h, _ptr(X), dtype, M, arr, len(C_peers), flags, replica, stream))

    def gemv_host(self, X: np.ndarray, dtype: int = I8, flags: int = 0, replica: int = 0, out: Optional[np.ndarray] = None) -> np.ndarray:
        """Host-buffer call: copies X to the device, runs, copies C back."""
        X = np.ascontiguousarray(X, dtype=_NP_DTYPE[dtype])
        M = X.shape[0] if X.ndim == 2 else 1
        if flags & X_COLMAJOR:
            M = X.shape[1]
        if out is None:
            out = np.empty((self.N, M) if flags & C_COLMAJOR else (M, self.N), dtype=_OUT_DTYPE[dtype])
        check(lib.sptmm_gemv_host(self._h, X.ctypes.data, dtype, M, out.ctypes.data, flags, replica))
        return out

    def gemv_host_async(self, X: np.ndarray, out: np.ndarray, slot: int, dtype: int = I8, flags: int = 0, replica: int = 0) -> None:
        """First half of a host-buffer call on `slot` (0..15): returns once the work is enqueued.  X
        and out must be C-contiguous arrays of the right dtype; `out` is filled by gemv_host_wait."""
        M = X.shape[0] if X.ndim == 2 else 1
        if flags & X_COLMAJOR:
            M = X.shape[1]
        check(lib.sptmm_gemv_host_async(self._h, X.ctypes.data, dtype, M, out.ctypes.data, flags, replica, slot))

    def gemv_host_wait(self, slot: int) -> None:
        check(lib.sptmm_gemv_host_wait(self._h, slot))

    def gemv_host_batch(self, Xs, outs, replicas=None, dtype: int = I8, flags: int = 0, slot0: int = 0, nslots: int = 4,
                        M: Optional[int] = None) -> None:
        """A list of independent host-buffer calls (Xs[i] -> outs[i], weight copy replicas[i]) kept
        `nslots` at a time in flight on slots slot0..; returns when all have delivered.  Entries are
        C-contiguous numpy arrays, or host addresses (then M must be given)."""
        n = len(Xs)
        if len(outs) != n or (replicas is not None and len(replicas) != n):
            raise ValueError("gemv_host_batch: list lengths differ")
        if n == 0:
            return
        if M is None:
            M = Xs[0].shape[0] if Xs[0].ndim == 2 else 1
            if flags & X_COLMAJOR:
                M = Xs[0].shape[1]
        xp = (C.c_void_p * n)(*[_ptr(x) for x in Xs])
        cp = (C.c_void_p * n)(*[_ptr(o) for o in outs])
        rp = (C.c_uint32 * n)(*replicas) if replicas is not None else None
        check(lib.sptmm_gemv_host_batch(self._h, n, xp, cp, rp, dtype, M, flags, slot0, nslots))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            if not getattr(self, "_borrowed", False):
                lib.sptmm_weights_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class SeqStep(C.Structure):
    _fields_ = [("w", C.c_void_p), ("replica", C.c_uint32), ("x_kind", C.c_uint32), ("X", C.c_void_p),
                ("X2", C.c_void_p), ("C", C.c_void_p), ("scale_out", C.c_void_p),
                ("ldx", C.c_uint32), ("ldx2", C.c_uint32), ("ldc", C.c_uint32), ("dep", C.c_int32), ("c_kind", C.c_uint32)]


def _seq_steps(steps):
    arr = (SeqStep * len(steps))()
    for a, s in zip(arr, steps):
        a.w = s["w"]._h
        a.replica = s.get("replica", 0)
        a.x_kind = s.get("x_kind", 0)
        a.X = _ptr(s["X"])
        a.X2 = _ptr(s["X2"]) if s.get("X2") is not None else None
        a.C = _ptr(s["C"]) if s.get("C") is not None else None
        a.scale_out = _ptr(s["scale_out"]) if s.get("scale_out") is not None else None
        a.ldx, a.ldx2, a.ldc = s.get("ldx", 0), s.get("ldx2", 0), s.get("ldc", 0)
        a.dep = s.get("dep", -1); a.c_kind = s.get("c_kind", 0)
    return arr


def seq_shared_bytes(steps, M: int) -> int:
    """Bytes of one rank's synchronisation area for this step list (sptmm_seq_shared_bytes_for);
    only the kinds, dependencies and weights of the steps matter, not their buffer addresses."""
    arr = _seq_steps(steps)
    n = int(lib.sptmm_seq_shared_bytes_for(C.cast(arr, C.c_void_p), len(steps), M))
    if n == 0:
        raise ValueError("seq_shared_bytes: bad step list or M")
    return n


class Sequence:
    """A fixed list of matmul steps run by one persistent kernel (sptmm_seq_* in the C ABI).

    steps: dicts with keys w (Weights), X, C and optionally replica, x_kind, X2, scale_out, ldx,
    ldx2, ldc, dep (index of the step whose output this one reads; default -1 = none)."""

    def __init__(self, steps, M: int = 1, counter_peers=None, rank: int = 0):
        """counter_peers: for a multi-GPU sequence, the peer-mapped addresses of every rank's
        counter array (len = ranks); each step then carries "C_peers", one address per rank."""
        arr = _seq_steps(steps)
        self._keep = list(steps)                     # keep tensors and handles alive
        h = C.c_void_p()
        if counter_peers is None:
            check(lib.sptmm_seq_create(C.cast(arr, C.c_void_p), len(steps), M, C.byref(h)))
        else:
            n = len(counter_peers)
            cp = (C.c_void_p * (len(steps) * n))(*[int(a) for s in steps for a in s["C_peers"]])
            kp = (C.c_void_p * n)(*[int(a) for a in counter_peers])
            check(lib.sptmm_seq_create_shared(C.cast(arr, C.c_void_p), len(steps), M, C.cast(cp, C.c_void_p),
                                              C.cast(kp, C.c_void_p), n, rank, C.byref(h)))
        self._h = h

    @classmethod
    def borrow(cls, handle) -> "Sequence":
        """A view of a sequence somebody else owns (it is not freed with this object)."""
        self = cls.__new__(cls)
        self._h, self._keep, self._borrowed = handle, [], True
        return self

    def run(self, stream: int = 0) -> None:
        check(lib.sptmm_seq_run(self._h, stream))

    def status(self) -> int:
        st = C.c_uint32(0)
        check(lib.sptmm_seq_status(self._h, C.byref(st), None))
        return st.value

    @property
    def stream_bytes(self) -> int:
        nb = C.c_uint64(0)
        check(lib.sptmm_seq_status(self._h, None, C.byref(nb)))
        return nb.value

    def set_wait_limit(self, polls: int) -> None:
        """Reloads before a device-side wait gives up and raises the status word (0 = default)."""
        check(lib.sptmm_seq_set_wait_limit(self._h, polls))

    def set_trace(self, dev_tensor) -> None:
        """Tuning build only (SPTMM_B200_TUNING=1)."""
        check(lib.sptmm_seq_set_trace(self._h, _ptr(dev_tensor) if dev_tensor is not None else None))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            if not getattr(self, "_borrowed", False):
                lib.sptmm_seq_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def quantize_absmax(X, M: int, K: int, out, scale=None, ldx: int = 0, shard: int = 0, pair: bool = False, flags: int = 0,
                    stream: int = 0) -> None:
    """int32 rows -> int8 with a per-row absmax scale (sptmm_quantize_absmax); device buffers."""
    check(lib.sptmm_quantize_absmax(_ptr(X), M, K, ldx, shard, 1 if pair else 0, _ptr(out),
                                    _ptr(scale) if scale is not None else None, flags, stream))


def row_split3_small(X, W_pos_div, W_neg_div, out, M: int, K: int, N: int, S: int, split: int, stream: int = 0) -> None:
    """Raw-pointer form of the reference's -row_split3_small launch (main.cu:556-594)."""
    check(lib.sptmm_row_split3_small(_ptr(X), _ptr(W_pos_div), _ptr(W_neg_div), _ptr(out), M, K, N, S, split, stream))


def row_split_delta2(X, W_pos_delta, W_neg_delta, out, M: int, K: int, N: int, S: int, split: int = 32, stream: int = 0) -> None:
    """Raw-pointer form of the reference's -row_split_delta2 launch (main.cu:599-764)."""
    check(lib.sptmm_row_split_delta2(_ptr(X), _ptr(W_pos_delta), _ptr(W_neg_delta), _ptr(out), M, K, N, S, split, stream))


def run_sequence_static(steps, M: int = 1, stream: int = 0, wait: bool = True) -> int:
    """sptmm_seq_run_static: run up to 16 steps (dicts as for Sequence) without allocating device
    memory -- for callers that may not call cudaMalloc at that point; the kernel's scratch is a
    fixed array inside the library.  With wait=True the call waits and returns the status word."""
    arr = _seq_steps(steps)
    st = C.c_uint32(0)
    check(lib.sptmm_seq_run_static(C.cast(arr, C.c_void_p), len(steps), M, stream, C.byref(st) if wait else None))
    return st.value


def dense_cublas_gemm(X_colmajor, W_dense, out_colmajor, M: int, K: int, N: int, stream: int = 0) -> None:
    check(lib.sptmm_dense_cublas_gemm(_ptr(X_colmajor), _ptr(W_dense), _ptr(out_colmajor), M, K, N, stream))


def dense_cublas_gemm_f16(X_colmajor, W_dense, out_colmajor, M: int, K: int, N: int, stream: int = 0) -> None:
    """fp16 x fp16 -> fp32 dense comparator (column-major operands, W holds -1/0/+1 as fp16)."""
    check(lib.sptmm_dense_cublas_gemm_f16(_ptr(X_colmajor), _ptr(W_dense), _ptr(out_colmajor), M, K, N, stream))
