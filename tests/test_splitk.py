"""Split-K over GPUs (sptmm_gemv_reduce): shard arithmetic on CPU (incl. a 2-rank gloo run), the
fused add-to-owner epilogue on one GPU with emulated ranks, and the real multi-GPU path."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

import oracle_lib as O
import sptmm_b200 as sp
from sptmm_b200 import splitk as SK

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "splitk_worker.py")


def test_k_ranges_partition_the_rows_on_aligned_boundaries():
    for K in (16, 400, 2560, 6912, 28672, 100):
        for world in (1, 2, 3, 4, 8):
            cuts = [SK.k_range(K, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == K
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            assert all(a % 16 == 0 for a, _ in cuts)


def test_col_ranges_follow_the_kernel_rule():
    for N in (256, 2560, 28672, 17):
        for world in (1, 2, 4, 8):
            cuts = [SK.col_range(N, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == N and all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))


def test_split_k_partials_add_up_gloo():
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29541", WORKER, "cpu"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "split-k shards ok" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("M,dtype,ranks", [(1, sp.I8, 2), (5, sp.I8, 3), (16, sp.I8, 2), (4, sp.F16, 2), (2, sp.F32, 4)])
def test_fused_reduce_scatter_with_emulated_ranks(M, dtype, ranks):
    """One GPU plays every rank in turn: each has its K range of W and adds its partial sums into
    per-rank output buffers; afterwards buffer r holds rank r's columns of the full product."""
    import torch
    torch.cuda.set_device(0)
    K, N = 1040, 200                                         # N not divisible by 3: ragged column ranges
    W = sp.gen_ternary_iid(K, N, 0.5, 41)
    rng = np.random.default_rng(42)
    if dtype == sp.I8:
        X = O.gen_x_i8(M * K, 43).reshape(M, K)
        want = O.gemv_i8_dense(X.reshape(-1), W).reshape(M, N)
        out_t = torch.int32
    else:
        X = rng.standard_normal((M, K)).astype(np.float16 if dtype == sp.F16 else np.float32)
        want = X.astype(np.float64) @ W.T.astype(np.float64)
        out_t = torch.float32
    cols = [SK.col_range(N, r, ranks) for r in range(ranks)]
    bufs = [torch.zeros(M, c1 - c0, dtype=out_t, device="cuda") for c0, c1 in cols]
    for r in range(ranks):
        k0, k1 = SK.k_range(K, r, ranks)
        w = sp.Weights(np.ascontiguousarray(W[:, k0:k1]), sp.FMT_U16_V256).upload()
        xs = torch.from_numpy(np.ascontiguousarray(X[:, k0:k1])).cuda()
        w.gemv_reduce(xs, M, bufs, dtype)
        torch.cuda.synchronize()
    got = np.concatenate([b.cpu().numpy() for b in bufs], axis=1)
    if dtype == sp.I8:
        assert (got == want).all()
    else:
        scale = np.abs(X.astype(np.float64)) @ np.abs(W.T.astype(np.float64))
        tol = 1e-3 if dtype == sp.F16 else 1e-5
        assert (np.abs(got - want) / scale).max() <= tol


@pytest.mark.gpu
@pytest.mark.parametrize("M,ranks", [(1, 2), (7, 4)])
def test_fused_reduce_scatter_from_one_k_tiled_encoding(M, ranks):
    """The same with ONE encoding of the matrix cut into K-tiles: every emulated rank takes its tile
    out of it (sptmm_weights_tile), uploads only that, and adds its partial sums to the owners."""
    import torch
    torch.cuda.set_device(0)
    K, N = 1024, 200
    kt = K // ranks
    W = sp.gen_ternary_iid(K, N, 0.5, 41)
    X = O.gen_x_i8(M * K, 43).reshape(M, K)
    want = O.gemv_i8_dense(X.reshape(-1), W).reshape(M, N)
    whole = sp.Weights(W, sp.FMT_U16_V256, k_tile=kt)
    cols = [SK.col_range(N, r, ranks) for r in range(ranks)]
    bufs = [torch.zeros(M, c1 - c0, dtype=torch.int32, device="cuda") for c0, c1 in cols]
    for r in range(ranks):
        tile = whole.tile(r)
        tile.upload()
        xs = torch.from_numpy(np.ascontiguousarray(X[:, r * kt:(r + 1) * kt])).cuda()
        tile.gemv_reduce(xs, M, bufs, sp.I8)
        torch.cuda.synchronize()
    assert (np.concatenate([b.cpu().numpy() for b in bufs], axis=1) == want).all()
    with pytest.raises(sp.SptmmError):
        whole.gemv_reduce(xs, M, bufs, sp.I8)                  # the parent is not one matrix


@pytest.mark.gpu
@pytest.mark.parametrize("M,dtype,ranks", [(1, sp.I8, 2), (6, sp.I8, 3), (4, sp.F16, 4)])
def test_splitk_object_phases_with_emulated_ranks(M, dtype, ranks):
    """The C object (sptmm_splitk_*) with one GPU playing the ranks in turn: arenas of the size the
    library asks for, every rank clears its block, then every rank adds its partial sums; no barrier
    kernel runs (its ranks would wait for kernels queued behind them on the same device)."""
    import torch
    torch.cuda.set_device(0)
    K, N = 1040, 200
    W = sp.gen_ternary_iid(K, N, 0.5, 51)
    if dtype == sp.I8:
        X = O.gen_x_i8(M * K, 52).reshape(M, K)
        want = O.gemv_i8_dense(X.reshape(-1), W).reshape(M, N)
    else:
        X = np.random.default_rng(53).standard_normal((M, K)).astype(np.float16)
        want = X.astype(np.float64) @ W.T.astype(np.float64)
    nbytes = int(sp.lib.sptmm_splitk_arena_bytes(M, N, ranks))
    assert nbytes >= M * (-(-N // ranks)) * 4 + 8 * ranks and nbytes % 256 == 0
    arenas = [torch.full((nbytes,), 0, dtype=torch.uint8, device="cuda") for _ in range(ranks)]
    objs = [SK.SplitKMatmul(W, M, dtype, r, ranks, arena_peers=[a.data_ptr() for a in arenas]) for r in range(ranks)]
    xs = [torch.from_numpy(np.ascontiguousarray(X[:, o.k0:o.k1])).cuda() for o in objs]
    for rep in range(2):                                     # the second pass starts from dirty blocks
        for o in objs:
            o.clear()
        for o, x in zip(objs, xs):
            o.accumulate(x)
        torch.cuda.synchronize()
        parts = []
        for r, o in enumerate(objs):
            assert o.out_ptr == arenas[r].data_ptr() and o.width == SK.col_range(N, r, ranks)[1] - SK.col_range(N, r, ranks)[0]
            raw = arenas[r][: M * o.width * 4].view(torch.int32 if dtype == sp.I8 else torch.float32).view(M, o.width)
            parts.append(raw.cpu().numpy())
        got = np.concatenate(parts, axis=1)
        if dtype == sp.I8:
            assert (got == want).all()
        else:
            scale = np.abs(X.astype(np.float64)) @ np.abs(W.T.astype(np.float64))
            assert (np.abs(got - want) / scale).max() <= 1e-3          # fp16 activations: 1e-3 of sum |x|
    assert all(o.status() == 0 for o in objs)
    for o in objs:
        o.close()


@pytest.mark.gpu
def test_splitk_single_rank_forward_and_validation():
    import torch
    torch.cuda.set_device(0)
    K, N, M = 512, 96, 3
    W = sp.gen_ternary_iid(K, N, 0.4, 61)
    X = O.gen_x_i8(M * K, 62).reshape(M, K)
    mm = SK.SplitKMatmul(W, M, sp.I8)                          # one rank: the library's barrier is a no-op
    x = torch.from_numpy(X).cuda()
    for _ in range(2):
        out = mm.forward(x)
        torch.cuda.synchronize()
        assert (out.cpu().numpy() == O.gemv_i8_dense(X.reshape(-1), W).reshape(M, N)).all()
    assert mm.status() == 0
    w = mm.w
    with pytest.raises(sp.SptmmError):
        SK.SplitKMatmul(W, M, sp.I8, rank=2, world=2, weights=w, arena_peers=[1 << 20, 2 << 20])      # rank outside the world
    with pytest.raises(sp.SptmmError):
        SK.SplitKMatmul(W, M, sp.I8, rank=0, world=2, weights=w, arena_peers=[mm.out_ptr, mm.out_ptr + 8])   # misaligned arena
    wd = sp.Weights(sp.gen_ternary_fixed(256, 64, 128), sp.FMT_U16_DIV, split=32).upload()
    with pytest.raises(sp.SptmmError):
        SK.SplitKMatmul(sp.gen_ternary_fixed(256, 64, 128), 1, sp.I8, weights=wd)                      # native format only
    mm.close()


@pytest.mark.gpu
def test_splitk_barrier_gives_up_on_a_rank_that_never_arrives():
    """Rank 0 of two whose second rank never runs (its arena is plain local memory nobody writes):
    the barrier's bounded poll runs out, the pass finishes with status bit 0 set, nothing hangs and
    the device stays usable."""
    import torch
    torch.cuda.set_device(0)
    K, N, M = 512, 128, 2
    W = sp.gen_ternary_iid(K, N, 0.4, 71)
    nbytes = int(sp.lib.sptmm_splitk_arena_bytes(M, N, 2))
    arenas = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    mm = SK.SplitKMatmul(W, M, sp.I8, 0, 2, arena_peers=[a.data_ptr() for a in arenas])
    mm.set_wait_limit(1 << 10)
    x = torch.from_numpy(np.ascontiguousarray(O.gen_x_i8(M * K, 72).reshape(M, K)[:, mm.k0:mm.k1])).cuda()
    mm.forward(x)
    torch.cuda.synchronize()
    assert mm.status() & 1
    mm.close()
    ok = SK.SplitKMatmul(W, M, sp.I8)
    xf = torch.from_numpy(O.gen_x_i8(M * K, 72).reshape(M, K)).cuda()
    out = ok.forward(xf)
    torch.cuda.synchronize()
    assert ok.status() == 0 and (out.cpu().numpy() == O.gemv_i8_dense(O.gen_x_i8(M * K, 72), W).reshape(M, N)).all()
    ok.close()


def test_splitk_shard_arithmetic_is_validated():
    k0, k1 = C.c_uint32(0), C.c_uint32(0)
    assert sp.lib.sptmm_splitk_k_range(256, 2, 2, C.byref(k0), C.byref(k1)) != 0
    assert sp.lib.sptmm_splitk_col_range(256, 0, 0, C.byref(k0), C.byref(k1)) != 0
    assert sp.lib.sptmm_splitk_arena_bytes(0, 256, 2) == 0 and sp.lib.sptmm_splitk_arena_bytes(4, 256, 9) == 0
    assert sp.lib.sptmm_splitk_arena_bytes(4, 250, 4) == ((4 * 63 * 4 + 255) & ~255) + 256


@pytest.mark.gpu
def test_gemv_reduce_is_validated():
    import torch
    torch.cuda.set_device(0)
    W = sp.gen_ternary_iid(256, 64, 0.5, 0)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    wd = sp.Weights(sp.gen_ternary_fixed(256, 64, 128), sp.FMT_U16_DIV, split=32).upload()
    x = torch.from_numpy(O.gen_x_i8(256, 1)).cuda()
    c = torch.zeros(64, dtype=torch.int32, device="cuda")
    with pytest.raises(sp.SptmmError):
        wd.gemv_reduce(x, 1, [c])                              # native format only
    with pytest.raises(sp.SptmmError):
        w.gemv_reduce(x, 1, [c] * 9)                           # at most 8 ranks
    with pytest.raises(sp.SptmmError):
        w.gemv_reduce(x, 1, [c], flags=sp.C_COLMAJOR)
    w.gemv_reduce(x, 1, [c])                                   # one rank: plain accumulate
    torch.cuda.synchronize()
    assert (c.cpu().numpy() == O.gemv_i8_dense(O.gen_x_i8(256, 1), W).reshape(-1)).all()


@pytest.mark.gpu
def test_split_k_multi_gpu():
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2 if n < 4 else 4
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % world,
                        "--master-addr", "127.0.0.1", "--master-port", "29542", WORKER, "gpu"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "split-k multi-gpu parity ok" in r.stdout
