"""GPU parity tests of the persistent sequence kernel (sptmm_seq_*): independent steps against
the per-call results and the oracle, dependent chains with the fused int32 -> int8 quantiser
against an oracle chain, repeated runs, and the fused-shape layer of a BitNet-like stack."""
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


@pytest.mark.parametrize("M", [1, 3, 4, 16])
def test_independent_steps_match_oracle(M):
    shapes = [(512, 384, 1 / 3), (384, 700, 0.5), (1037, 333, 0.75), (64, 1, 0.2), (700, 40, 1.0)]
    Ws = [sp.gen_ternary_iid(K, N, p0, 10 + i) for i, (K, N, p0) in enumerate(shapes)]
    ws = [sp.Weights(W, sp.FMT_U16_V256).upload() for W in Ws]
    Xs = [O.gen_x_i8(M * K, 20 + i) for i, (K, N, _) in enumerate(shapes)]
    xd = [dev(x) for x in Xs]
    outs = [torch.full((M * N,), -5, dtype=torch.int32, device="cuda") for (K, N, _) in shapes]
    seq = sp.Sequence([{"w": w, "X": x, "C": o} for w, x, o in zip(ws, xd, outs)], M=M)
    for _ in range(3):                                  # repeated runs reuse the counters
        for o in outs:
            o.fill_(-5)
        seq.run()
        assert seq.status() == 0
        for W, X, o in zip(Ws, Xs, outs):
            assert (o.cpu().numpy().reshape(M, -1) == O.gemv_i8_dense(X, W)).all()


def test_full_size_rotating_replicas():
    K, N, S, M = 6912, 2560, 4096, 1
    W = sp.gen_ternary_fixed(K, N, S)
    w = sp.Weights(W, sp.FMT_U16_V256).upload(replicas=4)
    X = O.gen_x_i8(K, 1)
    xd = dev(X)
    outs = [torch.zeros(N, dtype=torch.int32, device="cuda") for _ in range(12)]
    steps = [{"w": w, "replica": i % 4, "X": xd, "C": o, "dep": i - 1} for i, o in enumerate(outs)]
    seq = sp.Sequence(steps, M=M)
    seq.run()
    assert seq.status() == 0
    want = O.gemv_i8_dense(X, W).reshape(-1)
    for o in outs:
        assert (o.cpu().numpy() == want).all()
    assert seq.stream_bytes == 12 * w.stream_bytes


@pytest.mark.parametrize("M", [1, 4, 9])
def test_dependent_chain_with_fused_quantiser(M):
    """x -> W1 -> quant -> W2 (fused two-halves output) -> quant(sum of halves) -> W3."""
    K1, N1, H, N3 = 512, 384, 320, 200
    W1 = sp.gen_ternary_iid(K1, N1, 0.4, 1)
    W2 = sp.gen_ternary_iid(N1, 2 * H, 0.5, 2)          # "gate|up" fused along N
    W3 = sp.gen_ternary_iid(H, N3, 1 / 3, 3)
    w1, w2, w3 = (sp.Weights(W, sp.FMT_U16_V256).upload() for W in (W1, W2, W3))
    X = O.gen_x_i8(M * K1, 4)
    c1 = torch.zeros((M, N1), dtype=torch.int32, device="cuda")
    c2 = torch.zeros((M, 2 * H), dtype=torch.int32, device="cuda")
    c3 = torch.zeros((M, N3), dtype=torch.int32, device="cuda")
    s2 = torch.zeros(M, dtype=torch.float32, device="cuda")
    s3 = torch.zeros(M, dtype=torch.float32, device="cuda")
    seq = sp.Sequence([
        {"w": w1, "X": dev(X), "C": c1},
        {"w": w2, "X": c1, "C": c2, "x_kind": 1, "dep": 0, "scale_out": s2},
        {"w": w3, "X": c2, "X2": c2[:, H:], "ldx": 2 * H, "ldx2": 2 * H, "C": c3, "x_kind": 1, "dep": 1, "scale_out": s3},
    ], M=M)
    for _ in range(2):
        seq.run()
        assert seq.status() == 0
        r1 = O.gemv_i8_dense(X, W1)
        q1, sc1 = O.quant_absmax_i8(r1)
        r2 = O.gemv_i8_dense(q1.reshape(-1), W2)
        q2, sc2 = O.quant_absmax_i8(r2[:, :H], r2[:, H:])
        r3 = O.gemv_i8_dense(q2.reshape(-1), W3)
        assert (c1.cpu().numpy() == r1).all()
        assert (c2.cpu().numpy() == r2).all()
        assert (c3.cpu().numpy() == r3).all()
        assert (s2.cpu().numpy() == sc1).all() and (s3.cpu().numpy() == sc2).all()


@pytest.mark.parametrize("M", [1, 3, 16])
def test_dependent_chain_with_tagged_exchange(M):
    """The same chain with x_kind 2: producers store (tag << 24 | value) and readers wait for the
    words themselves instead of a step counter.  Several runs in a row (the tag changes every
    run), a buffer written by two steps of one run, results bit-exact as before."""
    K1, N1, H, N3 = 512, 384, 320, 200
    W1 = sp.gen_ternary_iid(K1, N1, 0.4, 1)
    W2 = sp.gen_ternary_iid(N1, 2 * H, 0.5, 2)
    W3 = sp.gen_ternary_iid(H, N1, 1 / 3, 3)            # back to width N1: its output reuses W1's buffer
    W4 = sp.gen_ternary_iid(N1, N3, 0.6, 4)
    w1, w2, w3, w4 = (sp.Weights(W, sp.FMT_U16_V256).upload() for W in (W1, W2, W3, W4))
    X = O.gen_x_i8(M * K1, 4)
    c1 = torch.zeros((M, N1), dtype=torch.int32, device="cuda")      # written by steps 0 and 2
    c2 = torch.zeros((M, 2 * H), dtype=torch.int32, device="cuda")
    c4 = torch.zeros((M, N3), dtype=torch.int32, device="cuda")
    seq = sp.Sequence([
        {"w": w1, "X": dev(X), "C": c1},
        {"w": w2, "X": c1, "C": c2, "x_kind": 2, "dep": 0},
        {"w": w3, "X": c2, "X2": c2[:, H:], "ldx": 2 * H, "ldx2": 2 * H, "C": c1, "x_kind": 2, "dep": 1},
        {"w": w4, "X": c1, "C": c4, "x_kind": 2, "dep": 2},
    ], M=M)
    r1 = O.gemv_i8_dense(X, W1)
    q1, _ = O.quant_absmax_i8(r1)
    r2 = O.gemv_i8_dense(q1.reshape(-1), W2)
    q2, _ = O.quant_absmax_i8(r2[:, :H], r2[:, H:])
    r3 = O.gemv_i8_dense(q2.reshape(-1), W3)
    q3, _ = O.quant_absmax_i8(r3)
    r4 = O.gemv_i8_dense(q3.reshape(-1), W4)
    for run in range(4):
        seq.run()
        assert seq.status() == 0
        assert (c4.cpu().numpy() == r4).all(), "run %d" % run
        assert (((c1.cpu().numpy() << 8) >> 8) == r3).all()         # intermediate buffers hold tagged words
        assert (((c2.cpu().numpy() << 8) >> 8) == r2).all()
        tags = np.unique(c2.cpu().numpy().view(np.uint32) >> 24)
        assert len(tags) == 1 and tags[0] != 0


@pytest.mark.parametrize("M", [1, 4, 13])
def test_pair_sums_and_producer_side_row_maxima(M):
    """c_kind 1: a step stores result[2j] + result[2j+1]; x_kind 3: its reader quantises with the
    row maxima the producer recorded, in one pass.  Same numbers as the two-source, two-pass chain
    of test_dependent_chain_with_fused_quantiser; several runs (the maxima are kept per run)."""
    K1, N1, H, N3 = 512, 384, 320, 200
    W1 = sp.gen_ternary_iid(K1, N1, 0.4, 1)
    W2 = sp.gen_ternary_iid(N1, 2 * H, 0.5, 2)                                  # gate | up
    W2i = np.ascontiguousarray(W2.reshape(2, H, N1).transpose(1, 0, 2).reshape(2 * H, N1))    # g0 u0 g1 u1 ...
    W3 = sp.gen_ternary_iid(H, N3, 1 / 3, 3)
    w1, w2, w3 = (sp.Weights(W, sp.FMT_U16_V256).upload() for W in (W1, W2i, W3))
    X = O.gen_x_i8(M * K1, 4)
    c1 = torch.zeros((M, N1), dtype=torch.int32, device="cuda")
    c2 = torch.zeros((M, H), dtype=torch.int32, device="cuda")
    c3 = torch.zeros((M, N3), dtype=torch.int32, device="cuda")
    s2 = torch.zeros(M, dtype=torch.float32, device="cuda")
    s3 = torch.zeros(M, dtype=torch.float32, device="cuda")
    seq = sp.Sequence([
        {"w": w1, "X": dev(X), "C": c1},
        {"w": w2, "X": c1, "C": c2, "x_kind": 3, "dep": 0, "scale_out": s2, "c_kind": 1},
        {"w": w3, "X": c2, "C": c3, "x_kind": 3, "dep": 1, "scale_out": s3},
    ], M=M)
    r1 = O.gemv_i8_dense(X, W1)
    q1, sc1 = O.quant_absmax_i8(r1)
    r2 = O.gemv_i8_dense(q1.reshape(-1), W2)
    q2, sc2 = O.quant_absmax_i8(r2[:, :H], r2[:, H:])
    r3 = O.gemv_i8_dense(q2.reshape(-1), W3)
    for run in range(4):
        seq.run()
        assert seq.status() == 0
        assert (c1.cpu().numpy() == r1).all()
        assert (c2.cpu().numpy() == r2[:, :H] + r2[:, H:]).all()
        assert (c3.cpu().numpy() == r3).all(), "run %d" % run
        assert (s2.cpu().numpy() == sc1).all() and (s3.cpu().numpy() == sc2).all()
    with pytest.raises(sp.SptmmError):          # pair sums need an even number of columns
        sp.Sequence([{"w": sp.Weights(sp.gen_ternary_iid(64, 33, 0.5, 1), sp.FMT_U16_V256).upload(), "X": dev(O.gen_x_i8(64, 1)),
                      "C": c1, "c_kind": 1}])
    with pytest.raises(sp.SptmmError):          # x_kind 3 takes one source and needs its producer
        sp.Sequence([{"w": w1, "X": dev(X), "C": c1}, {"w": w2, "X": c1, "X2": c1, "C": c2, "x_kind": 3, "dep": 0}], M=M)


@pytest.mark.parametrize("M", [1, 2, 3, 4, 7, 13, 16])
def test_producer_side_quantiser(M):
    """x_kind 4: the producing step quantises the columns its reader names (a part of its row, or
    the pair sums of a fused gate|up step) and hands them on as packed int8; the reader fetches
    bytes.  Same numbers as the reader-side quantiser and the oracle chain; several runs (the
    packed words carry a tag that changes every run); the int32 outputs stay plain."""
    K1, N1, off, K2, H, N3 = 512, 448, 64, 320, 288, 200
    W1 = sp.gen_ternary_iid(K1, N1, 0.4, 1)
    W2 = sp.gen_ternary_iid(K2, 2 * H, 0.5, 2)                                  # gate | up, reads columns off..off+K2 of step 0
    W2i = np.ascontiguousarray(W2.reshape(2, H, K2).transpose(1, 0, 2).reshape(2 * H, K2))    # g0 u0 g1 u1 ...
    W3 = sp.gen_ternary_iid(H, N3, 1 / 3, 3)
    w1, w2, w3 = (sp.Weights(W, sp.FMT_U16_V256).upload() for W in (W1, W2i, W3))
    X = O.gen_x_i8(M * K1, 4)
    c1 = torch.zeros((M, N1), dtype=torch.int32, device="cuda")
    c2 = torch.zeros((M, H), dtype=torch.int32, device="cuda")
    c3 = torch.zeros((M, N3), dtype=torch.int32, device="cuda")
    s2 = torch.zeros(M, dtype=torch.float32, device="cuda")
    s3 = torch.zeros(M, dtype=torch.float32, device="cuda")
    seq = sp.Sequence([
        {"w": w1, "X": dev(X), "C": c1},
        {"w": w2, "X": c1[:, off:], "C": c2, "x_kind": 4, "dep": 0, "scale_out": s2, "c_kind": 1},
        {"w": w3, "X": c2, "C": c3, "x_kind": 4, "dep": 1, "scale_out": s3},
    ], M=M)
    r1 = O.gemv_i8_dense(X, W1)
    q1, sc1 = O.quant_absmax_i8(np.ascontiguousarray(r1[:, off:off + K2]))
    r2 = O.gemv_i8_dense(q1.reshape(-1), W2)
    q2, sc2 = O.quant_absmax_i8(r2[:, :H], r2[:, H:])
    r3 = O.gemv_i8_dense(q2.reshape(-1), W3)
    for run in range(4):
        seq.run()
        assert seq.status() == 0
        assert (c1.cpu().numpy() == r1).all()
        assert (c2.cpu().numpy() == r2[:, :H] + r2[:, H:]).all()
        assert (c3.cpu().numpy() == r3).all(), "run %d" % run
        assert (s2.cpu().numpy() == sc1).all() and (s3.cpu().numpy() == sc2).all()
    with pytest.raises(sp.SptmmError):          # the producer must be named
        sp.Sequence([{"w": w1, "X": dev(X), "C": c1}, {"w": w2, "X": c1, "C": c2, "x_kind": 4, "c_kind": 1}], M=M)
    with pytest.raises(sp.SptmmError):          # two readers of one producer must read the same columns
        sp.Sequence([{"w": w1, "X": dev(X), "C": c1}, {"w": w2, "X": c1[:, off:], "C": c2, "x_kind": 4, "dep": 0, "c_kind": 1},
                     {"w": w2, "X": c1, "C": c2, "x_kind": 4, "dep": 0, "c_kind": 1}], M=M)


def test_producer_side_quantiser_full_width_rows():
    """The layer shapes of the 2B stack at M=16 (K up to 6912: more columns than one pass of the
    CTA's threads covers), one layer, against the oracle chain."""
    M, hidden, ffn = 16, 2560, 6912
    Wgu = sp.gen_ternary_iid(hidden, 2 * ffn, 1 / 3, 11)
    Wgui = np.ascontiguousarray(Wgu.reshape(2, ffn, hidden).transpose(1, 0, 2).reshape(2 * ffn, hidden))
    Wd = sp.gen_ternary_iid(ffn, hidden, 1 / 3, 12)
    Wq = sp.gen_ternary_iid(hidden, 512, 1 / 3, 13)
    wgu, wd, wq = (sp.Weights(W, sp.FMT_U16_V256).upload() for W in (Wgui, Wd, Wq))
    X = O.gen_x_i8(M * hidden, 5)
    cg = torch.zeros((M, ffn), dtype=torch.int32, device="cuda")
    cd = torch.zeros((M, hidden), dtype=torch.int32, device="cuda")
    cq = torch.zeros((M, 512), dtype=torch.int32, device="cuda")
    seq = sp.Sequence([
        {"w": wgu, "X": dev(X), "C": cg, "c_kind": 1},
        {"w": wd, "X": cg, "C": cd, "x_kind": 4, "dep": 0},
        {"w": wq, "X": cd, "C": cq, "x_kind": 4, "dep": 1},
    ], M=M)
    r1 = O.gemv_i8_dense(X, Wgu)
    q1, _ = O.quant_absmax_i8(r1[:, :ffn], r1[:, ffn:])
    r2 = O.gemv_i8_dense(q1.reshape(-1), Wd)
    q2, _ = O.quant_absmax_i8(r2)
    r3 = O.gemv_i8_dense(q2.reshape(-1), Wq)
    for _ in range(2):
        seq.run()
        assert seq.status() == 0
        assert (cd.cpu().numpy() == r2).all()
        assert (cq.cpu().numpy() == r3).all()


@pytest.mark.parametrize("M", [1, 2, 4, 5, 16])
def test_settled_exchange(M):
    """x_kind 5: tagged words watched by one CTA each, local counters, and (M > 1) a local int8 tile
    fetched by bulk copy.  Parts of rows, pair sums, a buffer written twice in a run, several runs;
    bit-exact against the oracle chain.  Row lengths that are no multiple of 4 are refused."""
    K1, N1, off, K2, H, N3 = 512, 448, 64, 320, 288, 200
    W1 = sp.gen_ternary_iid(K1, N1, 0.4, 1)
    W2 = sp.gen_ternary_iid(K2, 2 * H, 0.5, 2)
    W2i = np.ascontiguousarray(W2.reshape(2, H, K2).transpose(1, 0, 2).reshape(2 * H, K2))
    W3 = sp.gen_ternary_iid(H, N1, 1 / 3, 3)            # back to width N1: its output reuses W1's buffer
    W4 = sp.gen_ternary_iid(N1 - 4, N3, 0.6, 4)         # part of a row again (444 columns)
    w1, w2, w3, w4 = (sp.Weights(W, sp.FMT_U16_V256).upload() for W in (W1, W2i, W3, W4))
    X = O.gen_x_i8(M * K1, 4)
    c1 = torch.zeros((M, N1), dtype=torch.int32, device="cuda")      # written by steps 0 and 2
    c2 = torch.zeros((M, H), dtype=torch.int32, device="cuda")
    c4 = torch.zeros((M, N3), dtype=torch.int32, device="cuda")
    s2 = torch.zeros(M, dtype=torch.float32, device="cuda")
    s3 = torch.zeros(M, dtype=torch.float32, device="cuda")
    seq = sp.Sequence([
        {"w": w1, "X": dev(X), "C": c1},
        {"w": w2, "X": c1[:, off:], "ldx": N1, "C": c2, "x_kind": 5, "dep": 0, "c_kind": 1, "scale_out": s2},
        {"w": w3, "X": c2, "C": c1, "x_kind": 5, "dep": 1, "scale_out": s3},
        {"w": w4, "X": c1, "ldx": N1, "C": c4, "x_kind": 5, "dep": 2},
    ], M=M)
    r1 = O.gemv_i8_dense(X, W1)
    q1, sc1 = O.quant_absmax_i8(np.ascontiguousarray(r1[:, off:off + K2]))
    r2 = O.gemv_i8_dense(q1.reshape(-1), W2)
    q2, sc2 = O.quant_absmax_i8(r2[:, :H], r2[:, H:])
    r3 = O.gemv_i8_dense(q2.reshape(-1), W3)
    q3, _ = O.quant_absmax_i8(np.ascontiguousarray(r3[:, :N1 - 4]))
    r4 = O.gemv_i8_dense(q3.reshape(-1), W4)
    for run in range(5):
        seq.run()
        assert seq.status() == 0
        assert (c4.cpu().numpy() == r4).all(), "run %d" % run
        assert (((c1.cpu().numpy() << 8) >> 8) == r3).all()
        assert (((c2.cpu().numpy() << 8) >> 8) == r2[:, :H] + r2[:, H:]).all()
        assert (s2.cpu().numpy() == sc1).all() and (s3.cpu().numpy() == sc2).all()
    wodd = sp.Weights(sp.gen_ternary_iid(N1 - 3, N3, 0.6, 4), sp.FMT_U16_V256).upload()
    with pytest.raises(sp.SptmmError):
        sp.Sequence([{"w": w1, "X": dev(X), "C": c1}, {"w": wodd, "X": c1, "ldx": N1, "C": c4, "x_kind": 5, "dep": 0}], M=M)
    with pytest.raises(sp.SptmmError):          # the settled exchange does not mix with the polling ones
        sp.Sequence([{"w": w1, "X": dev(X), "C": c1}, {"w": w3, "X": c2, "C": c1, "x_kind": 5, "dep": 0},
                     {"w": w4, "X": c1, "ldx": N1, "C": c4, "x_kind": 1, "dep": 1}], M=M)


@pytest.mark.parametrize("x_kind", [1, 2, 3, 5])
@pytest.mark.parametrize("M", [1, 4, 11])
def test_dequantising_epilogue_of_the_last_step(M, x_kind):
    """c_kind 2: the last step of a chain stores float(sum) * (absmax/127 of its quantised input row),
    bit-exact against the same fp32 product in numpy, whichever way its input arrived; an int8 input
    (x_kind 0) has scale 1.  A step may not read such an output."""
    K1, N1, N2 = 512, 384, 200
    W1 = sp.gen_ternary_iid(K1, N1, 0.4, 1)
    W2 = sp.gen_ternary_iid(N1, N2, 0.5, 2)
    w1, w2 = (sp.Weights(W, sp.FMT_U16_V256).upload() for W in (W1, W2))
    X = O.gen_x_i8(M * K1, 4)
    c1 = torch.zeros((M, N1), dtype=torch.int32, device="cuda")
    c1f = torch.zeros((M, N1), dtype=torch.float32, device="cuda")
    c2 = torch.zeros((M, N2), dtype=torch.float32, device="cuda")
    s2 = torch.zeros(M, dtype=torch.float32, device="cuda")
    seq = sp.Sequence([{"w": w1, "X": dev(X), "C": c1},
                       {"w": w2, "X": c1, "C": c2, "x_kind": x_kind, "dep": 0, "scale_out": s2, "c_kind": 2}], M=M)
    r1 = O.gemv_i8_dense(X, W1)
    q1, sc1 = O.quant_absmax_i8(r1)
    r2 = O.gemv_i8_dense(q1.reshape(-1), W2).reshape(M, N2)
    want = r2.astype(np.float32) * sc1.astype(np.float32)[:, None]
    for _ in range(3):
        seq.run()
        assert seq.status() == 0
        assert (c2.cpu().numpy() == want).all()
        assert (s2.cpu().numpy() == sc1).all()
    first = sp.Sequence([{"w": w1, "X": dev(X), "C": c1f, "c_kind": 2}], M=M)      # int8 input: the sums as floats
    first.run()
    assert first.status() == 0
    assert (c1f.cpu().numpy() == r1.astype(np.float32)).all()
    with pytest.raises(sp.SptmmError):
        sp.Sequence([{"w": w1, "X": dev(X), "C": c1f, "c_kind": 2},
                     {"w": w2, "X": c1f, "C": c2, "x_kind": 1, "dep": 0}], M=M)


def test_tagged_exchange_is_validated():
    W = sp.gen_ternary_iid(256, 256, 0.5, 0)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    x = dev(O.gen_x_i8(256, 1))
    a = torch.zeros(256, dtype=torch.int32, device="cuda")
    b = torch.zeros(256, dtype=torch.int32, device="cuda")
    with pytest.raises(sp.SptmmError):          # a tagged reader must name its producer
        sp.Sequence([{"w": w, "X": x, "C": a}, {"w": w, "X": a, "C": b, "x_kind": 2}])
    with pytest.raises(sp.SptmmError):          # a counter-waiting reader of a tagged output
        sp.Sequence([{"w": w, "X": x, "C": a}, {"w": w, "X": a, "C": b, "x_kind": 2, "dep": 0},
                     {"w": w, "X": a, "C": b, "x_kind": 1, "dep": 0}])
    with pytest.raises(sp.SptmmError):          # tagged and plain writers of one buffer
        sp.Sequence([{"w": w, "X": x, "C": a}, {"w": w, "X": a, "C": b, "x_kind": 2, "dep": 0},
                     {"w": w, "X": x, "C": a}])
    with pytest.raises(sp.SptmmError):          # X outside the producer's output
        sp.Sequence([{"w": w, "X": x, "C": a}, {"w": w, "X": b, "C": b, "x_kind": 2, "dep": 0}])


def test_sequence_errors():
    W = sp.gen_ternary_iid(256, 64, 0.5, 0)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    wd = sp.Weights(sp.gen_ternary_fixed(256, 64, 128), sp.FMT_U16_DIV, split=32).upload()
    x = dev(O.gen_x_i8(256, 1))
    c = torch.zeros(64, dtype=torch.int32, device="cuda")
    with pytest.raises(sp.SptmmError):
        sp.Sequence([{"w": wd, "X": x, "C": c}])                     # not the native format
    with pytest.raises(sp.SptmmError):
        sp.Sequence([{"w": w, "X": x, "C": c, "dep": 0}])            # depends on itself
    with pytest.raises(sp.SptmmError):
        sp.Sequence([{"w": w, "X": x, "C": c}], M=17)
    with pytest.raises(sp.SptmmError):
        sp.Sequence([{"w": sp.Weights(W, sp.FMT_U16_V256), "X": x, "C": c}])   # not uploaded
