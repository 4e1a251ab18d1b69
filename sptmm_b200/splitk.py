"""A ternary matmul split along K over the GPUs of one node, with the reduce-scatter fused in.

A thin wrapper over the C ABI's sptmm_splitk_* (shard arithmetic, arena layout, the phases of a
pass and the barrier kernel between them live in csrc/splitk.cu): every rank holds rows k0..k1 of W
and the same slice of X, and its kernel adds each column's partial sum straight into the buffer of
the rank that owns the column (a plain reduction over NVLink).  What is left here is the allocation
of the per-rank arenas in memory every rank can address.  The reference is single-GPU and has no
counterpart; the shapes this is meant for are the large K x N sweeps (K up to 28672) where one
GPU's HBM time dominates.

`forward_nccl` is the unfused comparator: a full-width partial product per rank, then NCCL's
reduce-scatter.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

import sptmm_b200 as sp


def k_range(K: int, rank: int, world: int) -> tuple[int, int]:
    """Rows of W (and elements of an X row) that `rank` owns (sptmm_splitk_k_range: contiguous,
    boundaries on multiples of 16 so that 16-byte row loads of int8 activations stay aligned)."""
    k0, k1 = C.c_uint32(0), C.c_uint32(0)
    sp.check(sp.lib.sptmm_splitk_k_range(K, rank, world, C.byref(k0), C.byref(k1)))
    return k0.value, k1.value


def col_range(N: int, rank: int, world: int) -> tuple[int, int]:
    """Columns of the result that `rank` owns after the reduce-scatter (sptmm_splitk_col_range)."""
    c0, c1 = C.c_uint32(0), C.c_uint32(0)
    sp.check(sp.lib.sptmm_splitk_col_range(N, rank, world, C.byref(c0), C.byref(c1)))
    return c0.value, c1.value


class SplitKMatmul:
    """sptmm_splitk_* with torch doing what a C++ host would do with CUDA IPC or the virtual memory
    API: one zeroed arena per rank, mapped into every rank (symmetric memory)."""

    def __init__(self, W: np.ndarray, M: int, dtype: int = sp.I8, rank: int = 0, world: int = 1, group=None, weights=None,
                 arena_peers=None):
        """W: the full (N, K) int8 ternary matrix, identical on every rank; only this rank's K range
        is encoded and uploaded -- or `weights`, an uploaded encoding of that range made earlier (for
        example this rank's tile of a K-tiled encoding), is used as it is.  `arena_peers`: addresses
        of every rank's zeroed arena for a caller that has mapped them itself (one device playing
        several ranks in turn, say); by default they come from torch's symmetric memory."""
        import torch
        self.torch, self.M, self.dtype, self.rank, self.world = torch, M, dtype, rank, world
        self.N, self.K = W.shape
        self.k0, self.k1 = k_range(self.K, rank, world)
        self.w = weights if weights is not None else sp.Weights(np.ascontiguousarray(W[:, self.k0:self.k1]), sp.FMT_U16_V256).upload()
        self.out_dtype = torch.int32 if dtype == sp.I8 else torch.float32
        nbytes = int(sp.lib.sptmm_splitk_arena_bytes(M, self.N, world))
        if nbytes == 0:
            raise sp.SptmmError(-1, "split-K: bad M, N or rank count")
        self.dist = None
        if arena_peers is not None:
            self.arena = None
            peers = [int(p) for p in arena_peers]
        elif world > 1:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm
            self.dist = dist
            self.arena = symm.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
            self.arena.zero_()
            self.handle = symm.rendezvous(self.arena, group=group if group is not None else dist.group.WORLD)
            peers = [int(p) for p in self.handle.buffer_ptrs]
        else:
            self.arena = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
            peers = [self.arena.data_ptr()]
        arr = (C.c_void_p * world)(*peers)
        h = C.c_void_p()
        sp.check(sp.lib.sptmm_splitk_create(self.w._h, dtype, M, rank, world, arr, C.byref(h)))
        self._h = h
        ptr, width = C.c_void_p(), C.c_uint32(0)
        sp.check(sp.lib.sptmm_splitk_output(self._h, C.byref(ptr), C.byref(width)))
        self.width = width.value
        if self.arena is not None:
            self.out = self.arena[: M * self.width * 4].view(self.out_dtype).view(M, self.width)
        else:
            self.out = None
        self.out_ptr = ptr.value
        self.partial = None
        if self.dist is not None:
            torch.cuda.synchronize()
            self.dist.barrier()              # every rank's arena is zeroed and its object exists before any pass starts

    def _stream(self):
        return self.torch.cuda.current_stream().cuda_stream

    def forward(self, x_slice) -> "torch.Tensor":
        """x_slice: device tensor M x (k1-k0) -- this rank's part of every row of X.  Queues a whole
        pass (clear | barrier | add partial sums to their owners | barrier) on the current stream and
        returns this rank's columns of X*W, valid once the stream has run."""
        sp.check(sp.lib.sptmm_splitk_forward(self._h, sp._ptr(x_slice), 0, self._stream()))
        return self.out

    # the phases one by one, for a caller with its own barrier or one device playing the ranks in turn
    def clear(self):
        sp.check(sp.lib.sptmm_splitk_clear(self._h, self._stream()))

    def accumulate(self, x_slice):
        sp.check(sp.lib.sptmm_splitk_accumulate(self._h, sp._ptr(x_slice), 0, self._stream()))

    def barrier(self):
        sp.check(sp.lib.sptmm_splitk_barrier(self._h, self._stream()))

    def status(self) -> int:
        st = C.c_uint32(0)
        sp.check(sp.lib.sptmm_splitk_status(self._h, C.byref(st)))
        return st.value

    def set_wait_limit(self, polls: int):
        sp.check(sp.lib.sptmm_splitk_set_wait_limit(self._h, polls))

    def close(self):
        if getattr(self, "_h", None):
            sp.lib.sptmm_splitk_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def forward_nccl(self, x_slice) -> "torch.Tensor":
        """Comparator: the full-width partial product, then NCCL reduce-scatter (N % world == 0)."""
        torch = self.torch
        if self.partial is None:
            self.partial = torch.zeros(self.M, self.N, dtype=self.out_dtype, device="cuda")
            self.rs_in = torch.zeros(self.world, self.M, self.N // self.world, dtype=self.out_dtype, device="cuda")
            self.rs_out = torch.zeros(self.M, self.N // self.world, dtype=self.out_dtype, device="cuda")
        self.w.gemv(x_slice, self.M, self.partial, self.dtype, stream=self._stream())
        if self.world == 1:
            return self.partial
        self.rs_in.copy_(self.partial.view(self.M, self.world, self.N // self.world).transpose(0, 1))
        self.dist.reduce_scatter_tensor(self.rs_out, self.rs_in)
        return self.rs_out

    @property
    def stream_bytes(self) -> int:
        return self.w.stream_bytes
