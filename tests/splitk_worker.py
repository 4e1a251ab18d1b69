"""Child process of tests/test_splitk.py, started by torch.distributed.run (one process per rank).

  cpu   gloo, no GPU: every rank takes its K range of a small matrix, forms its partial product
        with the oracle, the partials are summed with an all-reduce and each rank checks its
        column range of the sum against the full product (the shard arithmetic of the split-K
        path, without a device).
  gpu   nccl, one GPU per rank: the fused matmul + reduce-scatter (sptmm_gemv_reduce over peer
        buffers) against the oracle and against the unfused NCCL reduce-scatter.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import torch
import torch.distributed as dist

import oracle_lib as O
import sptmm_b200 as sp
from sptmm_b200 import splitk as SK


def cpu():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    K, N, M = 400, 96, 3
    W = sp.gen_ternary_iid(K, N, 0.5, 21)
    X = O.gen_x_i8(M * K, 22).reshape(M, K)
    k0, k1 = SK.k_range(K, rank, world)
    w = sp.Weights(np.ascontiguousarray(W[:, k0:k1]), sp.FMT_U16_V256)          # host-side encode only
    assert w.info.K == k1 - k0 and w.info.N == N
    part = O.gemv_i8_dense(np.ascontiguousarray(X[:, k0:k1]).reshape(-1), np.ascontiguousarray(W[:, k0:k1])).reshape(M, N)
    t = torch.from_numpy(part.astype(np.int64))
    dist.all_reduce(t)
    full = O.gemv_i8_dense(X.reshape(-1), W).reshape(M, N)
    c0, c1 = SK.col_range(N, rank, world)
    assert (t.numpy()[:, c0:c1] == full[:, c0:c1]).all()
    if rank == 0:
        print("split-k shards ok")
    dist.destroy_process_group()


def gpu():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    K, N = 1024, 256 * world
    W = sp.gen_ternary_iid(K, N, 0.5, 31)
    for M, dtype in ((1, sp.I8), (5, sp.I8), (4, sp.F16)):
        if dtype == sp.I8:
            X = O.gen_x_i8(M * K, 32).reshape(M, K)
            want = O.gemv_i8_dense(X.reshape(-1), W).reshape(M, N)
        else:
            X = np.random.default_rng(33).standard_normal((M, K)).astype(np.float16)
            want = X.astype(np.float64) @ W.T.astype(np.float64)
        mm = SK.SplitKMatmul(W, M, dtype, rank, world)
        xs = torch.from_numpy(np.ascontiguousarray(X[:, mm.k0:mm.k1])).cuda()
        c0, c1 = SK.col_range(N, rank, world)
        for _ in range(3):
            got = mm.forward(xs)
            torch.cuda.synchronize()
            ref = mm.forward_nccl(xs)
            torch.cuda.synchronize()
            if dtype == sp.I8:
                assert (got.cpu().numpy() == want[:, c0:c1]).all(), (rank, M)
                assert (ref.cpu().numpy() == want[:, c0:c1]).all(), (rank, M)
            else:
                scale = np.abs(X.astype(np.float64)) @ np.abs(W.T.astype(np.float64))
                err = np.abs(got.cpu().numpy() - want[:, c0:c1]) / scale[:, c0:c1]
                assert err.max() <= 1e-3, (rank, err.max())          # fp16 activations: 1e-3 relative to sum |x|
        del mm
    dist.barrier()
    if rank == 0:
        print("split-k multi-gpu parity ok on %d GPUs" % world)
    dist.destroy_process_group()


if __name__ == "__main__":
    {"cpu": cpu, "gpu": gpu}[sys.argv[1]]()
