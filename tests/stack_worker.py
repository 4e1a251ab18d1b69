"""Child process of tests/test_stack.py, started by torch.distributed.run (one process per rank).

  cpu-shards   gloo, no GPU: every rank encodes its column shard of a small stack; the shards'
               non-zero counts must add up to the full matrices'.
  gpu-parity   nccl (bootstrap and symmetric-memory rendezvous only), one GPU per rank: a small
               stack through the fused peer-store exchange; every rank's buffers must equal the
               oracle chain.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import torch
import torch.distributed as dist

import sptmm_b200 as sp
from sptmm_b200 import stack as S


def cpu_shards():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    layers, hidden, ffn, kv = 2, 64, 160, 16
    mine, total = 0, 0
    for l, name, W in S.stack_weights(layers, hidden, ffn, kv, 0.5, 11):
        c0, c1 = S.shard_range(W.shape[0], rank, world)
        w = sp.Weights(W[c0:c1], sp.FMT_U16_V256)            # host-side encode only
        assert w.info.N == c1 - c0 and w.info.K == W.shape[1]
        mine += w.info.nnz
        total += int((W != 0).sum())
    t = torch.tensor([mine], dtype=torch.int64)
    dist.all_reduce(t)
    assert int(t.item()) == total, (int(t.item()), total)
    if rank == 0:
        print("shards ok", total)
    dist.destroy_process_group()


def gpu_parity():
    import oracle_lib as O
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    layers, hidden, ffn, kv = 3, 256, 512, 64
    for M, tagged, row_maxima, pq in ((1, False, False, False), (4, False, True, False), (1, True, False, False), (4, True, False, False),
                                      (1, False, False, True), (4, False, False, True), (16, False, False, True),
                                      (1, None, False, None), (3, None, False, None), (4, None, False, None), (16, None, False, None),
                                      (4, "settled", False, None), (16, "settled", False, None), (6, None, False, None)):
        # None everywhere = the library's own choice (two half-batches from four even rows upward)
        kw = dict(exchange=S.SETTLED) if tagged == "settled" else dict(tagged=tagged, row_maxima=row_maxima, producer_quant=pq)
        st = S.TernaryStack(layers, hidden, ffn, kv, M=M, p_zero=1 / 3, seed=3, rank=rank, world=world, keep_dense=True, **kw)
        x = O.gen_x_i8(M * hidden, 9).reshape(M, hidden)
        st.set_input(x)
        want = S.reference_forward(st.dense, layers, hidden, ffn, kv, x, O.gemv_i8_dense, O.quant_absmax_i8)
        for _ in range(3):
            dist.barrier()                    # ranks leave and enter a pass together (host side)
            st.forward()
            torch.cuda.synchronize()
            assert st.status() == 0, "a bounded wait ran out on rank %d" % rank
            dist.barrier()
            for name in ("qkv", "o", "gu", "down"):
                assert (st.buffer(name) == want[name]).all(), (rank, M, tagged, row_maxima, pq, name)
        del st
    dist.barrier()
    if rank == 0:
        print("multi-gpu parity ok on %d GPUs" % world)
    dist.destroy_process_group()


if __name__ == "__main__":
    {"cpu-shards": cpu_shards, "gpu-parity": gpu_parity}[sys.argv[1]]()
