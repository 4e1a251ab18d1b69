"""What a sequence does when a peer never delivers: every device-side wait is bounded, so the run
ends by itself, the status word says which kind of wait ran out, and the device stays usable.

The missing peer is made on the host, without a second GPU and without any fault: the sequence is
created as rank 0 of TWO ranks (sptmm_seq_create_shared), the second rank's output and counter
areas are ordinary local buffers, and no second rank ever runs.  Its arrivals (half of every step
counter's target) and its columns of every output therefore never come; with the wait limit set
to a few thousand reloads the run returns within milliseconds."""
import numpy as np
import pytest

import oracle_lib as O
import sptmm_b200 as sp

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _device():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    yield
    torch.cuda.synchronize()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("x_kind,M", [(1, 1), (1, 4), (5, 1), (5, 4)])
def test_missing_peer_ends_the_run_with_a_status(x_kind, M):
    K, N = 256, 128                                     # the full layer; this "rank" owns columns 0..63
    W1 = sp.gen_ternary_iid(K, N, 0.4, 1)
    W2 = sp.gen_ternary_iid(N, N, 0.5, 2)
    w1 = sp.Weights(W1[: N // 2], sp.FMT_U16_V256).upload()
    w2 = sp.Weights(W2[: N // 2], sp.FMT_U16_V256).upload()
    X = O.gen_x_i8(M * K, 3)
    steps = [{"w": w1, "X": dev(X), "dep": -1, "ldc": N}, {"w": w2, "X": 0, "x_kind": x_kind, "dep": 0, "ldx": N, "ldc": N},
             {"w": w2, "X": 0, "x_kind": x_kind, "dep": 1, "ldx": N, "ldc": N}]
    # rank 0's buffers and the never-running rank 1's: plain local memory, zeroed
    bufs = [[torch.zeros((M, N), dtype=torch.int32, device="cuda") for _ in range(2)] for _ in range(3)]
    steps[1]["X"], steps[2]["X"] = bufs[0][0], bufs[1][0]
    for s, st in enumerate(steps):
        st["C_peers"] = [b.data_ptr() for b in bufs[s]]          # this rank's shard starts at column 0 of both
    nbytes = sp.seq_shared_bytes([dict(st, C=1) for st in steps], M)
    areas = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    seq = sp.Sequence(steps, M=M, counter_peers=[a.data_ptr() for a in areas], rank=0)
    seq.set_wait_limit(1 << 12)
    seq.run()
    status = seq.status()                               # waits for the device: the run came back by itself
    assert status & 2, "the wait for the producer's output must have run out (status %d)" % status
    assert status & ~(2 | 16) == 0, status
    # the first step has no dependency and is complete: this rank's columns, in both copies
    want = O.gemv_i8_dense(X, W1[: N // 2]).reshape(M, N // 2)
    for b in bufs[0]:
        got = b.cpu().numpy()[:, : N // 2]
        got = (got << 8) >> 8 if x_kind == 5 else got   # the settled exchange stores tagged words
        assert (got == want).all()
    seq.close()

    # the device is as usable as before: a complete sequence on the same weights is exact
    c1 = torch.zeros((M, N // 2), dtype=torch.int32, device="cuda")
    ok = sp.Sequence([{"w": w1, "X": dev(X), "C": c1}], M=M)
    ok.run()
    assert ok.status() == 0
    assert (c1.cpu().numpy() == want).all()


def test_missing_peer_with_the_settle_warps_running_ahead():
    """Two interleaved chains make the sequence use the pipelined kernel (settle warps one step ahead,
    two tile buffers): there, too, a peer that never delivers ends the run with a status instead of
    hanging the settle warps or the consumers that wait for their tile."""
    M, K, N = 4, 256, 128
    W1 = sp.gen_ternary_iid(K, N, 0.4, 1)
    W2 = sp.gen_ternary_iid(N, N, 0.5, 2)
    w1 = sp.Weights(W1[: N // 2], sp.FMT_U16_V256).upload()
    w2 = sp.Weights(W2[: N // 2], sp.FMT_U16_V256).upload()
    xa, xb = dev(O.gen_x_i8(M * K, 3)), dev(O.gen_x_i8(M * K, 4))
    bufs = [[torch.zeros((M, N), dtype=torch.int32, device="cuda") for _ in range(2)] for _ in range(6)]
    steps = [{"w": w1, "X": xa, "ldc": N}, {"w": w1, "X": xb, "ldc": N},
             {"w": w2, "X": bufs[0][0], "x_kind": 5, "dep": 0, "ldx": N, "ldc": N}, {"w": w2, "X": bufs[1][0], "x_kind": 5, "dep": 1, "ldx": N, "ldc": N},
             {"w": w2, "X": bufs[2][0], "x_kind": 5, "dep": 2, "ldx": N, "ldc": N}, {"w": w2, "X": bufs[3][0], "x_kind": 5, "dep": 3, "ldx": N, "ldc": N}]
    for s, st in enumerate(steps):
        st["C_peers"] = [b.data_ptr() for b in bufs[s]]
    nbytes = sp.seq_shared_bytes([dict(st, C=1) for st in steps], M)
    areas = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    seq = sp.Sequence(steps, M=M, counter_peers=[a.data_ptr() for a in areas], rank=0)
    seq.set_wait_limit(1 << 12)
    seq.run()
    status = seq.status()
    assert status & 2 and status & ~(1 | 2 | 4 | 16) == 0, status
    want = O.gemv_i8_dense(O.gen_x_i8(M * K, 3), W1[: N // 2]).reshape(M, N // 2)
    assert ((((bufs[0][0].cpu().numpy()) << 8) >> 8)[:, : N // 2] == want).all()      # the first steps are complete
    seq.close()
    c1 = torch.zeros((M, N // 2), dtype=torch.int32, device="cuda")
    ok = sp.Sequence([{"w": w1, "X": xa, "C": c1}], M=M)
    ok.run()
    assert ok.status() == 0 and (c1.cpu().numpy() == want).all()


@pytest.mark.parametrize("M,rank", [(1, 0), (4, 3), (16, 7), (16, 0)])
def test_one_rank_of_eight_stores_to_every_rank_and_gives_up_on_the_missing_seven(M, rank):
    """The layer stack as ONE rank of eight whose other ranks never run (their arenas are plain local
    buffers): the plan, the arena layout and the peer tables of an eight-rank run are exercised on one
    GPU.  The rank's outputs must land at the same place in every rank's arena; its waits for the
    others' words run out (status, no hang); the device stays usable.  M=16 takes the pipelined
    exchange (two half-batches), M=1 and M=4 the settled one."""
    from sptmm_b200 import stack as SM
    world = 8
    wts = SM.StackWeights(2, 256, 512, 64, p_zero=1 / 3, seed=3, rank=rank, world=world)
    nbytes = int(sp.lib.sptmm_stack_arena_bytes(wts._h, M, SM.AUTO))
    arenas = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    stk = SM.TernaryStack(2, 256, 512, 64, M=M, rank=rank, world=world, weights=wts, arena_peers=[a.data_ptr() for a in arenas])
    assert stk.exchange == (SM.SETTLED_HALVES if M == 16 else SM.SETTLED)
    stk.set_wait_limit(1 << 10)
    stk.set_input(O.gen_x_i8(M * 256, 5).reshape(M, 256))
    stk.forward()
    torch.cuda.synchronize()
    status = stk.status()
    assert status & 2 and status & ~(1 | 2 | 4 | 16) == 0, status
    own = arenas[rank].cpu().numpy()
    others = [arenas[r].cpu().numpy() for r in range(world) if r != rank]
    for other in others:
        nz = other != 0
        assert nz.sum() >= M * 48 and (own[nz] == other[nz]).all()         # at least the first step's 48 qkv columns
        assert (other == others[0]).all()                                  # every missing rank received the same bytes
    stk.close()
    one = SM.TernaryStack(2, 256, 512, 64, M=M, p_zero=1 / 3, seed=3, keep_dense=True)
    x = O.gen_x_i8(M * 256, 5).reshape(M, 256)
    one.set_input(x)
    one.forward()
    torch.cuda.synchronize()
    want = SM.reference_forward(one.dense, 2, 256, 512, 64, x, O.gemv_i8_dense, lambda a: O.quant_absmax_i8(a))
    assert one.status() == 0 and (one.buffer("down") == want["down"]).all()
    one.close()


def test_wait_limit_rejects_a_null_handle_and_restores_the_default():
    W = sp.gen_ternary_iid(64, 32, 0.5, 1)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    c = torch.zeros(32, dtype=torch.int32, device="cuda")
    seq = sp.Sequence([{"w": w, "X": dev(O.gen_x_i8(64, 1)), "C": c}])
    seq.set_wait_limit(0)                                # back to the default
    seq.run()
    assert seq.status() == 0
    assert sp.lib.sptmm_seq_set_wait_limit(None, 5) != 0
