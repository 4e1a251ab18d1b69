"""A BitNet-b1.58-shaped stack of ternary layers run as one persistent sequence per forward pass.

Plumbing only: the stack itself -- weight generation, this rank's column shard of every matrix,
the buffer layout, the step list -- is the C ABI's sptmm_stack_* (host C++, csrc/stack.cpp) over
its sequence kernel; this module allocates the peer-visible arena and marshals arguments.  The reference has no layer stack, no quantiser and no
multi-GPU path; the shapes are the ones its dispatch ladders hard-code (main.cu:1107-1190: fused
qkv N=3840 and gate|up N=13824 at K=2560, down 6912x2560).

Per layer, four dependent steps (int8 activations, int32 results, per-row absmax re-quantisation
fused into the next step's input stage):
    qkv  = Wqkv(x)          hidden -> hidden + 2*kv       x: previous layer's `down` output
    o    = Wo(qkv[:, :hidden])                            (stand-in for attention: the q part)
    gu   = Wgu(o)           hidden -> ffn                 (gate | up fused along N with their columns
                                                           interleaved; the step stores gate_j + up_j)
    down = Wdown(gu)                                      ffn -> hidden

Multi-GPU: every matrix is sharded by contiguous column ranges over the ranks of one node; each
rank's kernel stores its output columns into every rank's buffers over NVLink and the step
counters live in the same peer-mapped arena (torch symmetric memory), so a forward pass is still
one kernel launch per rank with no collective call inside.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

import sptmm_b200 as sp


def shard_range(n_cols: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous column range of `rank`; sizes differ by at most one."""
    return n_cols * rank // world, n_cols * (rank + 1) // world


def layer_shapes(hidden: int, ffn: int, kv: int):
    """(name, K, N) of the four fused matrices of one layer, in execution order."""
    return [("qkv", hidden, hidden + 2 * kv), ("o", hidden, hidden), ("gu", hidden, 2 * ffn), ("down", ffn, hidden)]


def matrix_seed(seed: int, layer: int, which: int) -> int:
    return (seed * 1000003 + layer * 16 + which) & 0xFFFFFFFFFFFFFFFF


def stack_weights(layers: int, hidden: int, ffn: int, kv: int, p_zero: float, seed: int):
    """Yields (layer, name, W) with W the full (N, K) int8 matrix -- identical on every rank."""
    for l in range(layers):
        for i, (name, K, N) in enumerate(layer_shapes(hidden, ffn, kv)):
            yield l, name, sp.gen_ternary_iid(K, N, p_zero, matrix_seed(seed, l, i))


class StackConfig(C.Structure):
    _fields_ = [("layers", C.c_uint32), ("hidden", C.c_uint32), ("ffn", C.c_uint32), ("kv", C.c_uint32),
                ("p_zero", C.c_double), ("seed", C.c_uint64), ("rank", C.c_uint32), ("world", C.c_uint32)]


AUTO, COUNTERS, TAGGED, ROW_MAXIMA, PRODUCER_QUANT, SETTLED, SETTLED_HALVES = 0, 1, 2, 3, 4, 5, 6      # sptmm.h: SPTMM_STACK_*


class StackWeights:
    """This rank's column shard of every matrix of the stack, generated, encoded and uploaded by
    sptmm_stack_weights_create; independent of M, so stacks for several batch sizes share one set."""

    def __init__(self, layers=30, hidden=2560, ffn=6912, kv=640, p_zero=1 / 3, seed=0, rank=0, world=1, keep_dense=False):
        self.shape = (layers, hidden, ffn, kv)
        self.rank, self.world = rank, world
        cfg = StackConfig(layers, hidden, ffn, kv, float(p_zero), int(seed) & 0xFFFFFFFFFFFFFFFF, rank, world)
        h = C.c_void_p()
        sp.check(sp.lib.sptmm_stack_weights_create(C.byref(cfg), C.byref(h)))
        self._h = h
        nb, npar = C.c_uint64(), C.c_uint64()
        sp.check(sp.lib.sptmm_stack_weights_info(h, C.byref(nb), C.byref(npar)))
        self.stream_bytes, self.params = nb.value, npar.value
        self.weights = []
        for i in range(4 * layers):
            wh = C.c_void_p()
            sp.check(sp.lib.sptmm_stack_weights_matrix(h, i, C.byref(wh)))
            self.weights.append(sp.Weights.borrow(wh))
        # the dense matrices, for tests that compare with the oracle chain (the same seeds)
        self.dense = [W for _, _, W in stack_weights(layers, hidden, ffn, kv, p_zero, seed)] if keep_dense else None

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            sp.lib.sptmm_stack_weights_free(self._h)
            self._h = C.c_void_p()
            self.weights = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class TernaryStack:
    """sptmm_stack_* behind a Python face: this class allocates the arena (torch symmetric memory
    across GPUs, so that every rank can address every rank's copy) and marshals arguments; weight
    generation, sharding, the buffer layout and the step list are the library's."""

    def __init__(self, layers=30, hidden=2560, ffn=6912, kv=640, M=1, p_zero=1 / 3, seed=0,
                 rank=0, world=1, group=None, keep_dense=False, tagged=None, row_maxima=False, producer_quant=None,
                 settled=None, weights=None, exchange=None, arena_peers=None):
        """weights: a StackWeights built for the same shapes, rank and world (else one is built here).
        exchange: one of AUTO, COUNTERS, TAGGED, ROW_MAXIMA, PRODUCER_QUANT, SETTLED, SETTLED_HALVES;
        the boolean arguments are the older way of naming the same choice.  arena_peers: addresses of
        every rank's zeroed arena (arena_bytes() each) for a caller that has mapped them itself; by
        default they come from torch's symmetric memory."""
        import torch
        self.torch = torch
        self.layers, self.hidden, self.ffn, self.kv, self.M = layers, hidden, ffn, kv, M
        self.rank, self.world = rank, world
        if exchange is None:
            if settled:
                exchange = SETTLED
            elif producer_quant:
                exchange = PRODUCER_QUANT
            elif row_maxima:
                exchange = ROW_MAXIMA
            elif tagged:
                exchange = TAGGED
            elif tagged is False or producer_quant is False or settled is False:
                exchange = COUNTERS              # the newer exchanges were declined by name
            else:
                exchange = AUTO
        if weights is None:
            weights = StackWeights(layers, hidden, ffn, kv, p_zero, seed, rank, world, keep_dense)
        assert weights.shape == (layers, hidden, ffn, kv) and (weights.rank, weights.world) == (rank, world)
        self.shared_weights = weights
        self.weights, self.stream_bytes, self.params, self.dense = weights.weights, weights.stream_bytes, weights.params, weights.dense
        nbytes = int(sp.lib.sptmm_stack_arena_bytes(weights._h, M, exchange))
        if nbytes == 0:
            raise sp.SptmmError(-1, "sptmm_stack_arena_bytes: " + sp.lib.sptmm_last_error().decode("utf-8", "replace"))
        h = C.c_void_p()
        self.arena_bytes = nbytes
        if arena_peers is not None:
            self.arena = None
            bases = (C.c_void_p * world)(*[int(p) for p in arena_peers])
            sp.check(sp.lib.sptmm_stack_create(weights._h, M, exchange, bases, C.byref(h)))
        elif world > 1:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm
            self.arena = symm.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
            self.arena.zero_()
            self.handle = symm.rendezvous(self.arena, group=group if group is not None else dist.group.WORLD)
            bases = (C.c_void_p * world)(*[int(p) for p in self.handle.buffer_ptrs])
            torch.cuda.synchronize()
            dist.barrier()
            sp.check(sp.lib.sptmm_stack_create(weights._h, M, exchange, bases, C.byref(h)))
        else:
            self.arena = None
            sp.check(sp.lib.sptmm_stack_create(weights._h, M, exchange, None, C.byref(h)))
        self._h = h
        ex = C.c_uint32()
        sp.check(sp.lib.sptmm_stack_exchange(h, C.byref(ex)))
        self.exchange = ex.value
        self.tagged, self.settled, self.producer_quant = ex.value in (TAGGED, SETTLED, SETTLED_HALVES), ex.value in (SETTLED, SETTLED_HALVES), ex.value == PRODUCER_QUANT
        self.n_steps = 4 * layers * (2 if ex.value == SETTLED_HALVES else 1)
        sh = C.c_void_p()
        sp.check(sp.lib.sptmm_stack_sequence(h, C.byref(sh)))
        self.seq = sp.Sequence.borrow(sh)

    def set_input(self, x_i8: np.ndarray) -> None:
        x = np.ascontiguousarray(x_i8, dtype=np.int8).reshape(self.M, self.hidden)
        sp.check(sp.lib.sptmm_stack_set_input(self._h, x.ctypes.data))

    def forward(self, stream: int = 0) -> None:
        sp.check(sp.lib.sptmm_stack_forward(self._h, stream))

    def buffer(self, name: str) -> np.ndarray:
        """This rank's copy of an activation buffer (int32, M x width), after a synchronise: the
        last values written to "qkv", "o", "gu" and, as "down", the stack's final result."""
        width = C.c_uint32()
        sp.check(sp.lib.sptmm_stack_buffer(self._h, name.encode(), None, C.byref(width)))
        out = np.empty((self.M, width.value), dtype=np.int32)
        sp.check(sp.lib.sptmm_stack_buffer(self._h, name.encode(), out.ctypes.data, None))
        return out

    def status(self) -> int:
        st = C.c_uint32()
        sp.check(sp.lib.sptmm_stack_status(self._h, C.byref(st)))
        return st.value

    def set_wait_limit(self, polls: int) -> None:
        sp.check(sp.lib.sptmm_stack_wait_limit(self._h, polls))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            sp.lib.sptmm_stack_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def reference_forward(dense, layers, hidden, ffn, kv, x_i8, gemv_dense, quant):
    """The same chain on the host, given the oracle's dense matmul and quantiser; returns the
    int32 outputs of the last layer's four steps (for parity tests on small stacks)."""
    M = x_i8.shape[0]
    x = np.ascontiguousarray(x_i8, dtype=np.int8)
    out = {}
    for l in range(layers):
        Wqkv, Wo, Wgu, Wd = dense[4 * l: 4 * l + 4]
        if l > 0:
            x, _ = quant(out["down"])
        out["qkv"] = gemv_dense(x.reshape(-1), Wqkv).reshape(M, -1)
        xq, _ = quant(np.ascontiguousarray(out["qkv"][:, :hidden]))
        out["o"] = gemv_dense(xq.reshape(-1), Wo).reshape(M, -1)
        xo, _ = quant(out["o"])
        gu = gemv_dense(xo.reshape(-1), Wgu).reshape(M, -1)
        out["gu"] = gu[:, :ffn] + gu[:, ffn:]                  # the stack stores gate_j + up_j
        xg, _ = quant(np.ascontiguousarray(out["gu"]))
        out["down"] = gemv_dense(xg.reshape(-1), Wd).reshape(M, -1)
    return out


class NcclStack:
    """The same column-sharded stack with NCCL between the steps instead of the fused exchange: per
    step one per-call matmul on this rank's columns (sptmm_gemv), an all-gather of the int32
    results (ncclAllGather through torch.distributed) and the quantiser kernel
    (sptmm_quantize_absmax) on what arrived; a whole pass is captured in one CUDA graph.  It is the
    comparator the fused exchange is measured against, and a second implementation of the same
    numbers (bit-exact with TernaryStack).  NCCL's buffers stay NCCL's: nothing of this library
    touches peer memory here."""

    def __init__(self, weights: StackWeights, M=1, group=None):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.group = torch, dist, group
        self.layers, self.hidden, self.ffn, self.kv = weights.shape
        self.M, self.rank, self.world, self.w = M, weights.rank, weights.world, weights.weights
        self.stream_bytes = weights.stream_bytes
        hidden, ffn, kv = self.hidden, self.ffn, self.kv
        # (output columns of the step, columns the next step reads, pair sums?)
        self.plan = [(hidden + 2 * kv, hidden, False), (hidden, hidden, False), (2 * ffn, ffn, True), (hidden, hidden, False)]
        self.x_in = torch.zeros(M, hidden, dtype=torch.int8, device="cuda")
        self.xq = [torch.zeros(M, max(hidden, ffn), dtype=torch.int8, device="cuda") for _ in range(2)]
        self.part = {n: torch.zeros(M, (n * (self.rank + 1)) // self.world - (n * self.rank) // self.world, dtype=torch.int32, device="cuda")
                     for n in {p[0] for p in self.plan}}
        self.full = {n: torch.zeros(self.world, M, n // self.world, dtype=torch.int32, device="cuda") for n in {p[0] for p in self.plan}}
        for n in self.full:
            assert n % self.world == 0, "the NCCL variant needs equal shards"
        self.scales = torch.zeros(4 * self.layers, M, dtype=torch.float32, device="cuda")
        self.graph = None

    def set_input(self, x_i8: np.ndarray) -> None:
        self.x_in.copy_(self.torch.from_numpy(np.ascontiguousarray(x_i8, dtype=np.int8).reshape(self.M, self.hidden)))

    def _pass(self, stream: int) -> None:
        x = self.x_in
        for s in range(4 * self.layers):
            n_out, k_next, pair = self.plan[s % 4]
            part, full = self.part[n_out], self.full[n_out]
            self.w[s].gemv(x, self.M, part, sp.I8, stream=stream)
            if self.world > 1:
                self.dist.all_gather_into_tensor(full, part, group=self.group)
            else:
                full.copy_(part.view(1, self.M, n_out))
            if s + 1 < 4 * self.layers:
                x = self.xq[s & 1]
                sp.quantize_absmax(full, self.M, k_next, x, self.scales[s + 1], shard=n_out // self.world, pair=pair, stream=stream)
        self.last = full

    def forward(self) -> None:
        """One pass on the current stream: the first call runs eagerly (NCCL sets itself up), the
        second captures the pass in a CUDA graph, later calls replay it."""
        torch = self.torch
        st = torch.cuda.current_stream()
        if self.graph is not None:
            self.graph.replay()
        elif getattr(self, "_warm", False):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st if st != torch.cuda.default_stream() else None):
                self._pass(torch.cuda.current_stream().cuda_stream)
            self.graph = g
            g.replay()
        else:
            self._pass(st.cuda_stream)
            self._warm = True

    def result(self) -> np.ndarray:
        """The last step's int32 output (M x hidden), after a synchronise."""
        return self.last.cpu().numpy().transpose(1, 0, 2).reshape(self.M, -1)
