"""A ternary matmul split along K over the GPUs of one node, with the reduce-scatter fused in.

Plumbing only (buffers, shard arithmetic, stream-ordered barriers); the compute is the C ABI's
sptmm_gemv_reduce: every rank holds rows k0..k1 of W and the same slice of X, and its kernel adds
each column's partial sum straight into the buffer of the rank that owns the column (a plain
reduction over NVLink).  The reference is single-GPU and has no counterpart; the shapes this is
meant for are the large K x N sweeps (K up to 28672) where one GPU's HBM time dominates.

`forward_nccl` is the unfused comparator: a full-width partial product per rank, then NCCL's
reduce-scatter.
"""
from __future__ import annotations

import numpy as np

import sptmm_b200 as sp


def k_range(K: int, rank: int, world: int, align: int = 16) -> tuple[int, int]:
    """Rows of W (and elements of an X row) that `rank` owns: contiguous, boundaries on multiples of
    `align` so that 16-byte row loads of int8 activations stay aligned."""
    units = -(-K // align)
    return min(K, units * rank // world * align), min(K, units * (rank + 1) // world * align)


def col_range(N: int, rank: int, world: int) -> tuple[int, int]:
    """Columns of the result that `rank` owns after the reduce-scatter (the kernel's own rule)."""
    return N * rank // world, N * (rank + 1) // world


class SplitKMatmul:
    def __init__(self, W: np.ndarray, M: int, dtype: int = sp.I8, rank: int = 0, world: int = 1, group=None, weights=None):
        """W: the full (N, K) int8 ternary matrix, identical on every rank; only this rank's K range
        is encoded and uploaded -- or `weights`, an uploaded encoding of that range made earlier (for
        example this rank's tile of a K-tiled encoding), is used as it is."""
        import torch
        self.torch, self.M, self.dtype, self.rank, self.world = torch, M, dtype, rank, world
        self.N, self.K = W.shape
        self.k0, self.k1 = k_range(self.K, rank, world)
        self.w = weights if weights is not None else sp.Weights(np.ascontiguousarray(W[:, self.k0:self.k1]), sp.FMT_U16_V256).upload()
        self.out_dtype = torch.int32 if dtype == sp.I8 else torch.float32
        widths = [col_range(self.N, r, world)[1] - col_range(self.N, r, world)[0] for r in range(world)]
        self.width = widths[rank]
        nbytes = (M * max(widths) * 4 + 255) & ~255
        if world > 1:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm
            self.dist = dist
            self.arena = symm.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
            self.handle = symm.rendezvous(self.arena, group=group if group is not None else dist.group.WORLD)
            self.peers = [int(p) for p in self.handle.buffer_ptrs]
            self.token = torch.zeros(1, dtype=torch.int32, device="cuda")
        else:
            self.dist = None
            self.arena = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
            self.peers = [self.arena.data_ptr()]
        self.out = self.arena[: M * self.width * 4].view(self.out_dtype).view(M, self.width)
        self.partial = None

    def _barrier(self):
        """All ranks' streams reach this point before any goes on (a one-word all-reduce: ordered on
        the stream, the host does not wait)."""
        if self.world > 1:
            self.dist.all_reduce(self.token)

    def forward(self, x_slice) -> "torch.Tensor":
        """x_slice: device tensor M x (k1-k0) -- this rank's part of every row of X.  Returns this
        rank's columns of X*W (valid once the current stream has run)."""
        self.out.zero_()
        self._barrier()                      # nobody adds into a buffer that is not yet cleared
        self.w.gemv_reduce(x_slice, self.M, self.peers, self.dtype, stream=self.torch.cuda.current_stream().cuda_stream)
        self._barrier()                      # every rank's additions have landed
        return self.out

    def forward_nccl(self, x_slice) -> "torch.Tensor":
        """Comparator: the full-width partial product, then NCCL reduce-scatter (N % world == 0)."""
        torch = self.torch
        if self.partial is None:
            self.partial = torch.zeros(self.M, self.N, dtype=self.out_dtype, device="cuda")
            self.rs_in = torch.zeros(self.world, self.M, self.N // self.world, dtype=self.out_dtype, device="cuda")
            self.rs_out = torch.zeros(self.M, self.N // self.world, dtype=self.out_dtype, device="cuda")
        self.w.gemv(x_slice, self.M, self.partial, self.dtype, stream=torch.cuda.current_stream().cuda_stream)
        if self.world == 1:
            return self.partial
        self.rs_in.copy_(self.partial.view(self.M, self.world, self.N // self.world).transpose(0, 1))
        self.dist.reduce_scatter_tensor(self.rs_out, self.rs_in)
        return self.rs_out

    @property
    def stream_bytes(self) -> int:
        return self.w.stream_bytes
