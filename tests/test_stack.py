"""Layer stack: sharding logic on CPU (incl. a 2-rank gloo run), parity of a small stack on one
GPU against the oracle chain, and the multi-GPU fused-exchange path (2+ GPUs) as child processes."""
import os
import subprocess
import sys

import numpy as np
import pytest

import oracle_lib as O
import sptmm_b200 as sp
from sptmm_b200 import stack as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "stack_worker.py")


def test_shard_ranges_partition_the_columns():
    for n in (640, 2560, 3840, 13824, 17, 7):
        for world in (1, 2, 3, 4, 8):
            cuts = [S.shard_range(n, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            sizes = [b - a for a, b in cuts]
            assert max(sizes) - min(sizes) <= 1


def test_layer_shapes_are_the_bitnet_2b_ones():
    shapes = S.layer_shapes(2560, 6912, 640)
    assert shapes == [("qkv", 2560, 3840), ("o", 2560, 2560), ("gu", 2560, 13824), ("down", 6912, 2560)]
    assert sum(K * N for _, K, N in shapes) == 69468160          # parameters per layer


def test_stack_weights_are_seeded_and_distinct():
    a = list(S.stack_weights(2, 64, 128, 16, 1 / 3, 5))
    b = list(S.stack_weights(2, 64, 128, 16, 1 / 3, 5))
    assert len(a) == 8 and all((x[2] == y[2]).all() for x, y in zip(a, b))
    assert not (a[0][2] == a[4][2]).all()                         # layers differ
    assert not (a[0][2] == list(S.stack_weights(1, 64, 128, 16, 1 / 3, 6))[0][2]).all()


def test_sharded_encoding_covers_every_nonzero_gloo():
    """Two CPU ranks (gloo) each encode their column shard; together they hold every non-zero."""
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", WORKER, "cpu-shards"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "shards ok" in r.stdout


def _oracle_chain(dense, layers, hidden, ffn, kv, x):
    return S.reference_forward(dense, layers, hidden, ffn, kv, x, O.gemv_i8_dense, O.quant_absmax_i8)


@pytest.mark.gpu
@pytest.mark.parametrize("tagged,row_maxima,producer_quant", [(False, False, False), (True, False, False), (False, True, False),
                                                              (False, False, True), (None, False, None)])
@pytest.mark.parametrize("M", [1, 2, 4, 11, 16])
def test_small_stack_single_gpu(M, tagged, row_maxima, producer_quant):
    import torch
    torch.cuda.set_device(0)
    layers, hidden, ffn, kv = 3, 256, 512, 64
    st = S.TernaryStack(layers, hidden, ffn, kv, M=M, p_zero=1 / 3, seed=3, keep_dense=True, tagged=tagged, row_maxima=row_maxima,
                        producer_quant=producer_quant)
    x = O.gen_x_i8(M * hidden, 9).reshape(M, hidden)
    st.set_input(x)
    for _ in range(2):
        st.forward()
        assert st.status() == 0
        want = _oracle_chain(st.dense, layers, hidden, ffn, kv, x)
        for name in ("qkv", "o", "gu", "down"):
            assert (st.buffer(name) == want[name]).all(), name


@pytest.mark.gpu
@pytest.mark.parametrize("M", [2, 4, 10, 16])
def test_small_stack_two_half_batches(M):
    """SETTLED_HALVES: the rows run as two half-batches whose steps alternate in the one kernel
    (two, eight-row and sixteen-row tiles); same numbers as the oracle chain, row for row."""
    import torch
    torch.cuda.set_device(0)
    layers, hidden, ffn, kv = 3, 256, 512, 64
    st = S.TernaryStack(layers, hidden, ffn, kv, M=M, p_zero=1 / 3, seed=3, keep_dense=True, exchange=S.SETTLED_HALVES)
    assert st.n_steps == 2 * 4 * layers
    x = O.gen_x_i8(M * hidden, 9).reshape(M, hidden)
    st.set_input(x)
    want = _oracle_chain(st.dense, layers, hidden, ffn, kv, x)
    for _ in range(3):
        st.forward()
        assert st.status() == 0
        for name in ("qkv", "o", "gu", "down"):
            assert (st.buffer(name) == want[name]).all(), name
    with pytest.raises(sp.SptmmError):
        S.TernaryStack(layers, hidden, ffn, kv, M=3, weights=st.shared_weights, exchange=S.SETTLED_HALVES)


@pytest.mark.gpu
def test_stack_multi_gpu_fused_exchange():
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2 if n < 4 else 4
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % world,
                        "--master-addr", "127.0.0.1", "--master-port", "29534", WORKER, "gpu-parity"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "multi-gpu parity ok" in r.stdout
