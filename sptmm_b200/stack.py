"""A BitNet-b1.58-shaped stack of ternary layers run as one persistent sequence per forward pass.

Plumbing only: this module generates seeded weights, encodes and uploads this rank's column
shard of every matrix, lays out the activation buffers and builds the step list; all compute is
the C ABI's sequence kernel (sptmm_seq_*).  The reference has no layer stack, no quantiser and no
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


class StackWeights:
    """This rank's column shard of every matrix of the stack, encoded and uploaded; independent of M,
    so stacks for several batch sizes can share one set."""

    def __init__(self, layers=30, hidden=2560, ffn=6912, kv=640, p_zero=1 / 3, seed=0, rank=0, world=1, keep_dense=False):
        self.shape = (layers, hidden, ffn, kv)
        self.rank, self.world = rank, world
        self.dense = [] if keep_dense else None
        self.weights, self.stream_bytes, self.params = [], 0, 0
        for l, name, W in stack_weights(layers, hidden, ffn, kv, p_zero, seed):
            if keep_dense:
                self.dense.append(W)
            if name == "gu":                    # columns g0,u0,g1,u1,...: a pair-summing step adds gate_j and up_j
                W = np.ascontiguousarray(W.reshape(2, ffn, W.shape[1]).transpose(1, 0, 2).reshape(2 * ffn, W.shape[1]))
            c0, c1 = shard_range(W.shape[0], rank, world)
            assert name != "gu" or (c0 % 2 == 0 and c1 % 2 == 0), "pair sums need even shard boundaries"
            w = sp.Weights(W[c0:c1], sp.FMT_U16_V256).upload()
            self.weights.append(w)
            self.stream_bytes += w.stream_bytes
            self.params += W.shape[0] * W.shape[1]

    def close(self):
        for w in self.weights:
            w.close()
        self.weights = []


class TernaryStack:
    def __init__(self, layers=30, hidden=2560, ffn=6912, kv=640, M=1, p_zero=1 / 3, seed=0,
                 rank=0, world=1, group=None, keep_dense=False, tagged=None, row_maxima=False, producer_quant=None,
                 settled=None, weights=None):
        """weights: a StackWeights built for the same shapes, rank and world (else one is built here)."""
        import torch
        self.torch = torch
        self.layers, self.hidden, self.ffn, self.kv, self.M = layers, hidden, ffn, kv, M
        self.rank, self.world = rank, world
        # How a step's int32 output becomes the next step's int8 input:
        #  - producer_quant (x_kind 4): the producing step quantises its own columns after a small
        #    exchange of row maxima and stores int8; readers fetch M*K bytes.  For M >= 4 (None picks
        #    it there), where every CTA quantising all M rows for itself is what a step costs.
        #  - tagged (x_kind 2): readers quantise; outputs travel as tagged words, no counters, no
        #    fences.  Measured on B200: across GPUs that beats the step counters for M <= 4 (2 GPUs,
        #    M=1: 1.20 ms per pass against 1.51 ms), on one GPU it does not; None picks accordingly.
        #  - settled (x_kind 5): tagged words as above, but every word is watched by one CTA per GPU,
        #    the CTAs of a GPU meet at local counters, and for M > 1 each CTA quantises only its own
        #    columns into a local int8 tile that all fetch with one bulk copy.
        #    Measured on B200 (30 layers, us per pass; counters / settled): one GPU M=1 1 240 / 1 380,
        #    M=4 1 890 / 1 900, M=16 4 280 / 3 350; two GPUs M=1 950 (polled tags) / 930, M=4 1 510 / 1 420,
        #    M=16 3 540 / 2 420.  None picks it across GPUs and, on one GPU, from eight rows upward.
        explicit = tagged is not None or producer_quant is not None or row_maxima
        if settled is None:
            settled = not explicit and (world > 1 or M >= 8)
        if producer_quant is None:
            producer_quant = False
        if settled:
            tagged, producer_quant = True, False         # the producers store tagged words
        elif tagged is None:
            tagged = world > 1 and M <= 4 and not producer_quant
        self.tagged, self.producer_quant, self.settled = tagged, producer_quant, settled
        shapes = layer_shapes(hidden, ffn, kv)
        widths = {name: N for name, _, N in shapes}

        # ---- weights: this rank's columns of every matrix
        if weights is None:
            weights = StackWeights(layers, hidden, ffn, kv, p_zero, seed, rank, world, keep_dense)
        assert weights.shape == (layers, hidden, ffn, kv) and (weights.rank, weights.world) == (rank, world)
        self.shared_weights = weights
        self.weights, self.stream_bytes, self.params, self.dense = weights.weights, weights.stream_bytes, weights.params, weights.dense

        # ---- activation buffers (full width on every rank) and step counters in one arena
        n_steps = 4 * layers
        off, cur = {}, 0
        # step counters + row maxima (+ the producers' packed int8 outputs): the size depends on the
        # step kinds and shapes only, so a list without buffer addresses gives it
        xk = 5 if settled else (4 if producer_quant else (2 if tagged else 1))
        sizing = [{"w": self.weights[s], "X": 1, "C": 1, "dep": s - 1, "x_kind": (0 if s == 0 else xk)} for s in range(n_steps)]
        off["counters"] = cur; cur += int(sp.seq_shared_bytes(sizing, M))
        widths["gu"] = ffn                       # stored as pair sums
        widths["out"] = widths["down"]           # the last step's result: never tagged, no reader inside the kernel
        for name in ("qkv", "o", "gu", "down", "out"):
            cur = (cur + 255) & ~255
            off[name] = cur; cur += M * widths[name] * 4
        cur = (cur + 255) & ~255
        if world > 1:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm
            self.arena = symm.empty(cur, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
            self.arena.zero_()
            self.handle = symm.rendezvous(self.arena, group=group if group is not None else dist.group.WORLD)
            bases = [int(p) for p in self.handle.buffer_ptrs]
            dist.barrier()
        else:
            self.arena = torch.zeros(cur, dtype=torch.uint8, device="cuda")
            bases = [self.arena.data_ptr()]
        self.bases, self.off = bases, off
        mine = bases[rank]
        self.x_in = torch.zeros(M, hidden, dtype=torch.int8, device="cuda")
        self.scales = torch.zeros(n_steps, M, dtype=torch.float32, device="cuda")

        # ---- the step list
        steps = []
        xk = 5 if settled else (4 if producer_quant else (2 if tagged else 1))       # a reader of part of a row finds the row's absmax itself
        xw = 5 if settled else (4 if producer_quant else (2 if tagged else (3 if row_maxima else 1)))    # row_maxima: a reader of a whole row gets its absmax from the producer
        for l in range(layers):
            for i, (name, K, N) in enumerate(shapes):
                s = 4 * l + i
                c0, _ = shard_range(N, rank, world)
                st = {"w": self.weights[s], "dep": s - 1, "ldc": widths[name], "scale_out": self.scales[s]}
                if name == "qkv":
                    if l == 0:
                        st.update(X=self.x_in, x_kind=0)
                    else:
                        st.update(X=mine + off["down"], x_kind=xw, ldx=hidden)
                elif name == "o":
                    st.update(X=mine + off["qkv"], x_kind=xk, ldx=widths["qkv"])
                elif name == "gu":
                    st.update(X=mine + off["o"], x_kind=xw, ldx=hidden, c_kind=1)
                else:
                    st.update(X=mine + off["gu"], x_kind=xw, ldx=ffn)
                dst = "out" if s == n_steps - 1 else name
                o0 = c0 // 2 if name == "gu" else c0      # where this rank's first output column lands
                if world > 1:
                    st["C_peers"] = [b + off[dst] + o0 * 4 for b in bases]
                else:
                    st["C"] = mine + off[dst] + o0 * 4
                steps.append(st)
        counter_peers = [b + off["counters"] for b in bases] if world > 1 else None
        self.seq = sp.Sequence(steps, M=M, counter_peers=counter_peers, rank=rank)
        self.n_steps = n_steps

    def set_input(self, x_i8: np.ndarray) -> None:
        self.x_in.copy_(self.torch.from_numpy(np.ascontiguousarray(x_i8, dtype=np.int8).reshape(self.M, self.hidden)))

    def forward(self, stream: int = 0) -> None:
        self.seq.run(stream)

    def buffer(self, name: str) -> np.ndarray:
        """This rank's copy of an activation buffer (int32, M x width), after a synchronise: the
        last values written to "qkv", "o", "gu" and, as "down", the stack's final result."""
        width = self.ffn if name == "gu" else dict((n, N) for n, _, N in layer_shapes(self.hidden, self.ffn, self.kv))[name]
        src = "out" if name == "down" else name
        t = self.arena[self.off[src]: self.off[src] + self.M * width * 4].view(self.torch.int32)
        v = t.cpu().numpy().reshape(self.M, width)
        if self.tagged and src != "out":
            v = (v << 8) >> 8                    # drop the tag byte, sign-extend the 24-bit value
        return v

    def status(self) -> int:
        return self.seq.status()


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
