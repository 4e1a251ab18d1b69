"""GPU parity tests: every kernel, called through the C ABI, against the CPU oracle on the same
seeded inputs.  int8 -> int32 must be bit-exact; fp16 within 1e-3 and fp32 within 1e-5, relative
to the sum of |x| over the gathered entries (summation order differs from the reference's)."""
import json
import os

import numpy as np
import pytest

import oracle_lib as O
import sptmm_b200 as sp

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FP16_RTOL, FP32_RTOL = 1e-3, 1e-5


@pytest.fixture(scope="module", autouse=True)
def _device():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    yield
    torch.cuda.synchronize()


def dev(a: np.ndarray):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_i8(w: sp.Weights, X: np.ndarray, M: int, flags: int = 0, **kw) -> np.ndarray:
    xd = dev(X)
    out = torch.full((M * w.N,), -7, dtype=torch.int32, device="cuda")
    w.gemv(xd, M, out, sp.I8, flags, **kw)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def lists_of(W):
    N, K = W.shape
    cap = max(1, int(max((W == 1).sum(1).max(), (W == -1).sum(1).max())))
    return O.build_lists(W, cap, K)


# ---------------------------------------------------------------- native u16 format

@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8, 16, 17])
def test_native_u16_small_fixed(M):
    K, N, S = 256, 32, 128
    W = sp.gen_ternary_fixed(K, N, S)
    X = O.gen_x_i8(M * K, 100 + M)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    assert (run_i8(w, X, M).reshape(M, N) == O.gemv_i8_dense(X, W)).all()


@pytest.mark.parametrize("p0", [1 / 3, 0.5, 0.75, 0.97, 1.0])
@pytest.mark.parametrize("K,N", [(700, 40), (1037, 333), (64, 1)])
def test_native_u16_ragged_iid(p0, K, N):
    W = sp.gen_ternary_iid(K, N, p0, 5)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    for M in (1, 4):
        X = O.gen_x_i8(M * K, 17)
        pos, neg, npos, nneg = lists_of(W)
        want = O.gemv_i8_lists(X, pos, neg, npos, nneg, K)
        assert (want == O.gemv_i8_dense(X, W)).all()
        assert (run_i8(w, X, M).reshape(M, N) == want).all()


def test_native_u16_extreme_columns():
    # a dense +1 column, a dense -1 column, an empty column and one-entry columns side by side
    K, N = 1500, 24
    W = np.zeros((N, K), dtype=np.int8)
    W[0, :] = 1
    W[1, :] = -1
    W[3, K - 1] = 1
    W[4, 0] = -1
    W[5:, ::3] = 1
    W[5:, 1::3] = -1
    X = np.full(2 * K, 127, dtype=np.int8)
    X[K:] = -127
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    got = run_i8(w, X, 2).reshape(2, N)
    assert (got == O.gemv_i8_dense(X, W)).all()
    assert got[0, 0] == 127 * K and got[1, 1] == 127 * K and (got[:, 2] == 0).all()


@pytest.mark.parametrize("M", [1, 4])
def test_native_u16_full_size_fixed_s4096(M):
    # the headline benchmark shape with the reference's own generator (-S=4096)
    K, N, S = 6912, 2560, 4096
    W = sp.gen_ternary_fixed(K, N, S)
    X = O.gen_x_i8(M * K, 1)
    pos, neg, _, _ = O.build_lists(W, S // 2, K)
    want = O.gemv_i8_div(X, O.encode_div(pos, 32), O.encode_div(neg, 32), M, K, N, S, 32)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    assert w.info.stream_bytes == 2 * S * N + (2 * N + 1) * 4
    assert (run_i8(w, X, M).reshape(M, N) == want).all()


def test_native_u16_full_size_iid_third():
    # headline configuration: i.i.d. P=1/3 each, seed 0, M=1, int8 uniform
    K, N = 6912, 2560
    W = sp.gen_ternary_iid(K, N, 1 / 3, 0)
    X = O.gen_x_i8(K, 1)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    assert (run_i8(w, X, 1).reshape(1, N) == O.gemv_i8_dense(X, W)).all()


def _float_case(K, N, M, p0, dtype):
    W = sp.gen_ternary_iid(K, N, p0, 21)
    rng = np.random.default_rng(2)
    Xh = rng.standard_normal((M, K)).astype(np.float16 if dtype == sp.F16 else np.float32)
    pos, neg, npos, nneg = lists_of(W)
    ref, dbl, ab = O.gemv_f32_lists(np.ascontiguousarray(Xh.astype(np.float32)), pos, neg, npos, nneg, K)
    return W, Xh, ref, dbl, ab


@pytest.mark.parametrize("dtype,rtol", [(sp.F16, FP16_RTOL), (sp.F32, FP32_RTOL)])
@pytest.mark.parametrize("K,N,M", [(700, 40, 1), (700, 40, 4), (6912, 2560, 4), (2560, 640, 16), (1024, 64, 9)])
def test_native_u16_float(dtype, rtol, K, N, M):
    # the M=4 configuration: M=4, K=6912, N=2560, fp16 N(0,1), fp32 accumulation
    W, Xh, ref, dbl, ab = _float_case(K, N, M, 1 / 3, dtype)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    out = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    w.gemv(dev(Xh), M, out, dtype)
    torch.cuda.synchronize()
    got = out.cpu().numpy().astype(np.float64)
    err = np.abs(got - dbl)
    assert (err <= rtol * ab + 1e-30).all(), "max err/scale = %g" % (err / np.maximum(ab, 1e-30)).max()
    # the reference-order fp32 sum sits inside the same band
    assert (np.abs(ref - dbl) <= rtol * ab + 1e-30).all()
    # repeated runs give identical bits (no atomics, fixed fold order)
    out2 = torch.zeros_like(out)
    w.gemv(dev(Xh), M, out2, dtype)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)


# ---------------------------------------------------------------- K-tiled matrices

@pytest.mark.parametrize("K,N,kt", [(400, 24, 128), (2560, 640, 1024), (6912, 320, 2304)])
@pytest.mark.parametrize("M", [1, 4, 16, 37])
def test_k_tiled_matrix_int8(K, N, kt, M):
    """A matrix cut into K-tiles (sptmm_encode_ktiled): tile after tile, the first storing and the
    others adding, gives the same int32 results as the whole matrix -- bit-exact against the dense
    oracle, also when the last tile is shorter, for both layouts of X and with several replicas."""
    W = sp.gen_ternary_iid(K, N, 0.5, 31)
    w = sp.Weights(W, sp.FMT_U16_V256, k_tile=kt).upload(2)
    X = O.gen_x_i8(M * K, 8)
    want = O.gemv_i8_dense(X, W).reshape(M, N)
    out = torch.full((M, N), -7, dtype=torch.int32, device="cuda")
    w.gemv(dev(X), M, out, sp.I8, replica=1)
    torch.cuda.synchronize()
    assert (out.cpu().numpy() == want).all()
    xc = np.ascontiguousarray(X.reshape(M, K).T)                  # X column-major: X(m,k) at k*M+m
    out.fill_(-7)
    w.gemv(dev(xc), M, out, sp.I8, sp.X_COLMAJOR | sp.LAUNCH_PDL)
    torch.cuda.synchronize()
    assert (out.cpu().numpy() == want).all()
    assert w.status() == 0
    got = w.gemv_host(X.reshape(M, K), sp.I8)                     # host buffers in and out
    assert (got == want).all()


@pytest.mark.parametrize("M", [4, 16, 64])
def test_k_tiled_matrix_fp16_long_rows(M):
    """K = 28672 fp16 rows do not fit shared memory sixteen at a time; K-tiles of 4096 do.  Within
    the fp16 tolerance of the double-precision sum, like the untiled path."""
    K, N = 28672, 96
    W, Xh, ref, dbl, ab = _float_case(K, N, M, 0.5, sp.F16)
    out = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    for kt in (4096, 8192):
        w = sp.Weights(W, sp.FMT_U16_V256, k_tile=kt).upload()
        out.zero_()
        w.gemv(dev(Xh), M, out, sp.F16)
        torch.cuda.synchronize()
        err = np.abs(out.cpu().numpy().astype(np.float64) - dbl)
        assert (err <= FP16_RTOL * ab + 1e-30).all(), "max err/scale = %g" % (err / np.maximum(ab, 1e-30)).max()
        w.close()


# ---------------------------------------------------------------- native lane-delta format

@pytest.mark.parametrize("p0", [1 / 3, 0.5, 0.75, 0.97, 1.0])
@pytest.mark.parametrize("K,N", [(700, 40), (6912, 97), (64, 1)])
def test_delta_lane_ragged_iid(p0, K, N):
    """Dense lists (all steps full), sparse ones (steps cut short by gaps of more than 255 rows),
    empty ones; bit-exact against the oracle and the u16 path."""
    W = sp.gen_ternary_iid(K, N, p0, 6)
    w = sp.Weights(W, sp.FMT_DELTA_LANE).upload()
    wu = sp.Weights(W, sp.FMT_U16_V256).upload()
    for M in (1, 3, 4, 16, 17):
        X = O.gen_x_i8(M * K, 18)
        want = O.gemv_i8_dense(X, W)
        assert (run_i8(w, X, M).reshape(M, N) == want).all()
        assert (run_i8(wu, X, M).reshape(M, N) == want).all()


@pytest.mark.parametrize("S", [4608, 4096, 3456, 1728])
def test_delta_lane_sparsity_sweep_full_size(S):
    # the delta-format configuration on the native narrow-integer format: bit-exact vs the undecoded u16 path
    K, N = 6912, 2560
    W = sp.gen_ternary_fixed(K, N, S)
    X = O.gen_x_i8(K, 1)
    wd = sp.Weights(W, sp.FMT_DELTA_LANE).upload()
    wu = sp.Weights(W, sp.FMT_U16_V256).upload()
    assert wd.info.stream_bytes < 0.75 * wu.info.stream_bytes
    got = run_i8(wd, X, 1)
    assert (got == run_i8(wu, X, 1)).all()
    assert (got.reshape(1, N) == O.gemv_i8_dense(X, W)).all()


@pytest.mark.parametrize("dtype,rtol", [(sp.F16, FP16_RTOL), (sp.F32, FP32_RTOL)])
def test_delta_lane_float(dtype, rtol):
    K, N, M = 2560, 640, 4
    W, Xh, ref, dbl, ab = _float_case(K, N, M, 1 / 3, dtype)
    w = sp.Weights(W, sp.FMT_DELTA_LANE).upload()
    out = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    w.gemv(dev(Xh), M, out, dtype)
    torch.cuda.synchronize()
    err = np.abs(out.cpu().numpy().astype(np.float64) - dbl)
    assert (err <= rtol * ab + 1e-30).all(), "max err/scale = %g" % (err / np.maximum(ab, 1e-30)).max()


def test_native_u16_layout_flags():
    K, N, M = 512, 48, 4
    W = sp.gen_ternary_iid(K, N, 0.4, 9)
    X = O.gen_x_i8(M * K, 5).reshape(M, K)
    want = O.gemv_i8_dense(X, W)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    got = run_i8(w, np.ascontiguousarray(X.T), M, sp.X_COLMAJOR | sp.C_COLMAJOR).reshape(N, M)
    assert (got.T == want).all()
    got = run_i8(w, X, M, sp.C_COLMAJOR).reshape(N, M)
    assert (got.T == want).all()


def test_pdl_chain_over_replicas():
    # back-to-back launches with programmatic dependent launch over distinct weight copies
    K, N, S, M = 2048, 512, 1024, 1
    W = sp.gen_ternary_fixed(K, N, S)
    w = sp.Weights(W, sp.FMT_U16_V256).upload(replicas=4)
    X = O.gen_x_i8(M * K, 3)
    want = O.gemv_i8_dense(X, W)
    xd = dev(X)
    outs = [torch.zeros(N, dtype=torch.int32, device="cuda") for _ in range(12)]
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for i, o in enumerate(outs):
            w.gemv(xd, M, o, sp.I8, sp.LAUNCH_PDL, replica=i % 4, stream=st.cuda_stream)
    st.synchronize()
    for o in outs:
        assert (o.cpu().numpy().reshape(1, N) == want).all()


def test_pdl_chain_respects_data_dependency():
    # layer 2 consumes what layer 1 wrote: the prefetch may overlap, the read of X may not
    K = N = 512
    W1 = sp.gen_ternary_iid(K, N, 0.9, 1)       # sparse, so int8 re-quantisation is not needed
    W2 = sp.gen_ternary_iid(K, N, 0.9, 2)
    w1 = sp.Weights(W1, sp.FMT_U16_V256).upload()
    w2 = sp.Weights(W2, sp.FMT_U16_V256).upload()
    X = np.random.default_rng(0).standard_normal(K).astype(np.float32)
    h = torch.zeros(N, dtype=torch.float32, device="cuda")
    y = torch.zeros(N, dtype=torch.float32, device="cuda")
    xd = dev(X)
    st = torch.cuda.Stream()
    for _ in range(3):
        h.zero_(); y.zero_()
        torch.cuda.synchronize()
        w1.gemv(xd, 1, h, sp.F32, sp.LAUNCH_PDL, stream=st.cuda_stream)
        w2.gemv(h, 1, y, sp.F32, sp.LAUNCH_PDL, stream=st.cuda_stream)
        st.synchronize()
        h_ref = X.astype(np.float64) @ W1.T.astype(np.float64)
        y_ref = h.cpu().numpy().astype(np.float64) @ W2.T.astype(np.float64)
        assert np.allclose(h.cpu().numpy(), h_ref, rtol=1e-4, atol=1e-4)
        assert np.allclose(y.cpu().numpy(), y_ref, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("M", [1, 4, 16])
@pytest.mark.parametrize("flags", [0, sp.LAUNCH_PDL])
def test_activation_request_order_both_ways(M, flags):
    # without the flag a call asks for X before its weights, with it X is read only after the
    # previous kernel has finished: both orders, every row-tile width, int8 and fp16
    K, N, S = 2304, 640, 1152
    W = sp.gen_ternary_fixed(K, N, S)
    w = sp.Weights(W, sp.FMT_U16_V256).upload(replicas=2)
    X = O.gen_x_i8(M * K, 5)
    want = O.gemv_i8_dense(X, W)
    xd = dev(X)
    Xf = np.random.default_rng(M).standard_normal((M, K)).astype(np.float16)
    xf = dev(Xf)
    want_f = Xf.astype(np.float64) @ W.T.astype(np.float64)
    scale = np.abs(Xf.astype(np.float64)) @ np.abs(W.T.astype(np.float64))
    st = torch.cuda.Stream()
    oi = [torch.zeros(M * N, dtype=torch.int32, device="cuda") for _ in range(4)]
    of = [torch.zeros(M * N, dtype=torch.float32, device="cuda") for _ in range(4)]
    with torch.cuda.stream(st):
        for i in range(4):
            w.gemv(xd, M, oi[i], sp.I8, flags, replica=i % 2, stream=st.cuda_stream)
            w.gemv(xf, M, of[i], sp.F16, flags, replica=i % 2, stream=st.cuda_stream)
    st.synchronize()
    for i in range(4):
        assert (oi[i].cpu().numpy().reshape(M, N) == want).all()
        assert (np.abs(of[i].cpu().numpy().reshape(M, N) - want_f) <= 1e-3 * scale + 1e-6).all()


def test_plain_stream_order_chain_reads_fresh_activations():
    # no programmatic overlap: layer 2 asks for its X first thing, which stream order makes final
    K = N = 1024
    W1 = sp.gen_ternary_iid(K, N, 0.9, 11)
    W2 = sp.gen_ternary_iid(K, N, 0.9, 12)
    w1 = sp.Weights(W1, sp.FMT_U16_V256).upload()
    w2 = sp.Weights(W2, sp.FMT_U16_V256).upload()
    st = torch.cuda.Stream()
    h = torch.zeros(N, dtype=torch.float32, device="cuda")
    y = torch.zeros(N, dtype=torch.float32, device="cuda")
    for seed in range(4):
        X = np.random.default_rng(seed).standard_normal(K).astype(np.float32)
        xd = dev(X)
        w1.gemv(xd, 1, h, sp.F32, 0, stream=st.cuda_stream)
        w2.gemv(h, 1, y, sp.F32, 0, stream=st.cuda_stream)
        st.synchronize()
        h_ref = X.astype(np.float64) @ W1.T.astype(np.float64)
        y_ref = h.cpu().numpy().astype(np.float64) @ W2.T.astype(np.float64)
        assert np.allclose(h.cpu().numpy(), h_ref, rtol=1e-4, atol=1e-4)
        assert np.allclose(y.cpu().numpy(), y_ref, rtol=1e-4, atol=1e-3)


def test_gemv_host_roundtrip():
    K, N, S = 6912, 2560, 4096
    W = sp.gen_ternary_fixed(K, N, S)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    for M in (1, 4):
        X = O.gen_x_i8(M * K, 8).reshape(M, K)
        assert (w.gemv_host(X, sp.I8) == O.gemv_i8_dense(X, W)).all()


def test_gemv_host_async_slots_overlap_independent_calls():
    """Sixteen slots in flight, every call its own activations; results land in the right buffers,
    a busy slot is waited for on reuse, and waiting on an idle slot is a no-op."""
    K, N = 1024, 320
    W = sp.gen_ternary_iid(K, N, 0.5, 7)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    calls = 40
    Xs = [O.gen_x_i8(K, 100 + i).reshape(1, K) for i in range(calls)]
    outs = [np.full((1, N), -7, dtype=np.int32) for _ in range(calls)]
    for i in range(calls):
        w.gemv_host_async(Xs[i], outs[i], slot=i % 16)         # reusing a slot first delivers its previous result
    for s in range(16):
        w.gemv_host_wait(s)
        w.gemv_host_wait(s)
    for i in range(calls):
        assert (outs[i] == O.gemv_i8_dense(Xs[i].reshape(-1), W)).all(), i
    with pytest.raises(sp.SptmmError):
        w.gemv_host_async(Xs[0], outs[0], slot=16)


def test_gemv_host_batch_delivers_every_call():
    K, N = 1536, 384
    W = sp.gen_ternary_iid(K, N, 0.4, 21)
    w = sp.Weights(W, sp.FMT_U16_V256).upload(replicas=3)
    n = 25
    for M in (1, 3):
        Xs = [O.gen_x_i8(M * K, 300 + i).reshape(M, K) for i in range(n)]
        outs = [np.full((M, N), -7, dtype=np.int32) for _ in range(n)]
        w.gemv_host_batch(Xs, outs, [i % 3 for i in range(n)], slot0=2, nslots=3)
        for i in range(n):
            assert (outs[i] == O.gemv_i8_dense(Xs[i].reshape(-1), W)).all(), (M, i)
    w.gemv_host_batch([], [])
    with pytest.raises(sp.SptmmError):
        w.gemv_host_batch(Xs, outs, None, slot0=14, nslots=4)       # slots 14..17 of 16
    with pytest.raises(sp.SptmmError):
        w.gemv_host_batch(Xs[:3], outs[:3], [0, 1, 9], nslots=2)    # no weight copy 9
    outs2 = [np.zeros((M, N), dtype=np.int32) for _ in range(2)]
    w.gemv_host_batch(Xs[:2], outs2, None, nslots=2)                # the handle is usable after an error
    assert (outs2[1] == O.gemv_i8_dense(Xs[1].reshape(-1), W)).all()


def test_gemv_host_slots_from_two_host_threads():
    """Two host threads, each with its own pair of slots, issue calls at the same time."""
    import threading
    K, N = 2048, 512
    W = sp.gen_ternary_iid(K, N, 0.5, 9)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    calls = 60
    Xs = [[O.gen_x_i8(K, 1000 * t + i).reshape(1, K) for i in range(calls)] for t in range(2)]
    outs = [[np.full((1, N), -7, dtype=np.int32) for _ in range(calls)] for t in range(2)]
    errors = []

    def work(t):
        try:
            torch.cuda.set_device(0)
            for i in range(calls):
                w.gemv_host_async(Xs[t][i], outs[t][i], slot=2 * t + i % 2)
            w.gemv_host_wait(2 * t)
            w.gemv_host_wait(2 * t + 1)
        except Exception as e:      # surfaced in the main thread below
            errors.append(e)

    th = [threading.Thread(target=work, args=(t,)) for t in range(2)]
    for x in th:
        x.start()
    for x in th:
        x.join()
    assert not errors, errors
    for t in range(2):
        for i in range(calls):
            assert (outs[t][i] == O.gemv_i8_dense(Xs[t][i].reshape(-1), W)).all(), (t, i)


# ---------------------------------------------------------------- reference layouts

@pytest.mark.parametrize("split", [8, 16, 32])
@pytest.mark.parametrize("M", [1, 4, 8, 11])
def test_row_split3_small_raw_pointers(split, M):
    # arrays built by the ORACLE's restatement of prepareW_map, consumed as-is
    K, N, S = 512, 48, 256
    W = O.gen_fixed(K, N, S)
    X = O.gen_x_i8(M * K, 4)
    pos, neg, _, _ = O.build_lists(W, S // 2, K)
    wp, wn = O.encode_div(pos, split), O.encode_div(neg, split)
    out = torch.full((M, N), -3, dtype=torch.int32, device="cuda")
    sp.row_split3_small(dev(X), dev(wp), dev(wn), out, M, K, N, S, split)
    torch.cuda.synchronize()
    assert (out.cpu().numpy() == O.gemv_i8_div(X, wp, wn, M, K, N, S, split)).all()


@pytest.mark.parametrize("split", [8, 16, 32])
@pytest.mark.parametrize("M", [1, 4])
def test_row_split3_small_full_size(split, M):
    K, N, S = 6912, 2560, 4096
    W = sp.gen_ternary_fixed(K, N, S)
    X = O.gen_x_i8(M * K, 1)
    w = sp.Weights(W, sp.FMT_U16_DIV, split=split, S=S).upload()
    pos, neg, _, _ = O.build_lists(W, S // 2, K)
    want = O.gemv_i8_div(X, O.encode_div(pos, split), O.encode_div(neg, split), M, K, N, S, split)
    assert (run_i8(w, X, M).reshape(M, N) == want).all()


def test_row_split3_small_ragged_padding():
    K, N = 700, 64
    W = sp.gen_ternary_iid(K, N, 0.5, 4)
    X = O.gen_x_i8(3 * K, 2)
    w = sp.Weights(W, sp.FMT_U16_DIV, split=16).upload()
    assert (run_i8(w, X, 3).reshape(3, N) == O.gemv_i8_dense(X, W)).all()


@pytest.mark.parametrize("S", [512, 384, 64])
@pytest.mark.parametrize("M", [1, 4, 9])
def test_row_split_delta2_raw_pointers(S, M):
    K, N = 1024, 32
    W = O.gen_fixed(K, N, S)
    X = O.gen_x_i8(M * K, 6)
    pos, neg, _, _ = O.build_lists(W, S // 2, K)
    gp, _ = O.delta_lists(pos)
    gn, _ = O.delta_lists(neg)
    dp, dn = O.encode_delta_div256(gp), O.encode_delta_div256(gn)
    out = torch.full((M, N), -3, dtype=torch.int32, device="cuda")
    sp.row_split_delta2(dev(X), dev(dp), dev(dn), out, M, K, N, S, 32)
    torch.cuda.synchronize()
    assert (out.cpu().numpy() == O.gemv_i8_delta256(X, dp, dn, M, K, N, S)).all()
    assert (out.cpu().numpy() == O.gemv_i8_dense(X, W)).all()


@pytest.mark.parametrize("S", [4608, 4096, 3456, 1728])
def test_row_split_delta2_sparsity_sweep(S):
    # the delta-format sweep: M=1, 6912x2560, P(0) in {.33,.5,.75} <-> S in {4608,3456,1728};
    # the delta result must equal the undecoded u16 path bit for bit
    K, N = 6912, 2560
    W = sp.gen_ternary_fixed(K, N, S)
    X = O.gen_x_i8(K, 1)
    wd = sp.Weights(W, sp.FMT_DELTA_DIV256, S=S).upload()
    wu = sp.Weights(W, sp.FMT_U16_V256).upload()
    assert wd.info.lossy_entries == 0
    got = run_i8(wd, X, 1)
    assert (got == run_i8(wu, X, 1)).all()
    assert (got.reshape(1, N) == O.gemv_i8_dense(X, W)).all()


def test_row_split_delta2_lossy_matches_reference_semantics():
    # a gap above 255 is stored truncated; the kernel rebuilds the same wrong index the
    # reference does (mod 65536) -- checked against the oracle's faithful restatement
    K, N = 1024, 16
    W = np.zeros((N, K), dtype=np.int8)
    W[:, 300] = 1; W[:, 310] = 1
    W[:, 5] = -1; W[:, 6] = -1
    X = O.gen_x_i8(K, 3)
    w = sp.Weights(W, sp.FMT_DELTA_DIV256).upload()
    assert w.info.lossy_entries == N
    pos, neg, _, _ = O.build_lists(W, 2, K)
    gp, _ = O.delta_lists(pos)
    gn, _ = O.delta_lists(neg)
    want = O.gemv_i8_delta256(X, O.encode_delta_div256(gp), O.encode_delta_div256(gn), 1, K, N, 4)
    assert (run_i8(w, X, 1).reshape(1, N) == want).all()


def test_row_split3_small_clamps_indices_beyond_k():
    """A caller-built reference layout may hold anything: an index past K reads the zero row instead
    of addressing shared memory beyond the activation tile."""
    K, N, S, split = 256, 32, 128, 32
    W = sp.gen_ternary_fixed(K, N, S)
    pos, neg, _, _ = O.build_lists(W, S // 2, K)
    wp, wn = O.encode_div(pos, split).copy(), O.encode_div(neg, split).copy()
    rng = np.random.default_rng(5)
    bad = rng.choice(wp.size, 40, replace=False)
    X = O.gen_x_i8(K, 1)
    good = O.gemv_i8_div(X, wp, wn, 1, K, N, S, split).reshape(-1).astype(np.int64)
    # what the clamped entries contributed before they were overwritten
    flat = wp.reshape(-1)
    cols = (bad % (split * N)) // split
    lost = np.zeros(N, dtype=np.int64)
    np.add.at(lost, cols, X[flat[bad]].astype(np.int64))
    flat[bad] = 65535
    out = torch.zeros(N, dtype=torch.int32, device="cuda")
    sp.row_split3_small(dev(X), dev(wp), dev(wn), out, 1, K, N, S, split)
    torch.cuda.synchronize()
    assert (out.cpu().numpy() == good - lost).all()


def test_launch_errors():
    K, N, S = 512, 48, 256
    W = O.gen_fixed(K, N, S)
    pos, neg, _, _ = O.build_lists(W, S // 2, K)
    wp, wn = dev(O.encode_div(pos, 32)), dev(O.encode_div(neg, 32))
    x = dev(O.gen_x_i8(K, 1))
    out = torch.zeros(N, dtype=torch.int32, device="cuda")
    with pytest.raises(sp.SptmmError) as e:
        sp.row_split3_small(x, wp, wn, out, 1, K, N, S, 64)
    assert "Wrong split size" in e.value.message
    with pytest.raises(sp.SptmmError) as e:
        sp.row_split_delta2(x, wp, wn, out, 1, K, N, S, 16)
    assert "Wrong split size" in e.value.message
    with pytest.raises(sp.SptmmError):
        sp.row_split3_small(x, wp, wn, out, 1, K, N, S + 2, 32)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    with pytest.raises(sp.SptmmError):
        w.gemv(x, 0, out)
    with pytest.raises(sp.SptmmError):
        w.gemv(x, 1, out, replica=3)
    # the context is still usable afterwards
    w.gemv(x, 1, out)
    torch.cuda.synchronize()


# ---------------------------------------------------------------- comparators

@pytest.mark.parametrize("K,N,M", [(64, 16, 1), (6912, 2560, 1), (6912, 2560, 4), (2560, 6912, 8), (1040, 50, 3),
                                   (2560, 3840, 1), (4096, 777, 1), (8192, 3000, 1), (1040, 50, 1), (10240, 96, 1), (6144, 5, 1)])
def test_i2s_comparator(K, N, M):
    """One row with K a multiple of 64 up to 8192 takes the register form of the kernel (one to four
    16-byte vectors of codes per lane and column); everything else the shared-memory form."""
    W = sp.gen_ternary_iid(K, N, 1 / 3, 0)
    X = O.gen_x_i8(M * K, 1)
    w = sp.Weights(W, sp.FMT_I2S).upload()
    assert (run_i8(w, X, M).reshape(M, N) == O.gemv_i8_dense(X, W)).all()


def test_i2s_comparator_with_activations_off_a_16_byte_boundary():
    K, N = 2560, 300
    W = sp.gen_ternary_iid(K, N, 0.5, 5)
    X = O.gen_x_i8(K, 6)
    w = sp.Weights(W, sp.FMT_I2S).upload()
    buf = torch.zeros(K + 16, dtype=torch.int8, device="cuda")
    buf[4:4 + K] = torch.from_numpy(X).cuda()
    out = torch.zeros(N, dtype=torch.int32, device="cuda")
    w.gemv(buf[4:4 + K], 1, out)                      # 4 bytes off: the register form needs 16-byte loads of X
    torch.cuda.synchronize()
    assert (out.cpu().numpy() == O.gemv_i8_dense(X, W).reshape(-1)).all()


def test_cublas_comparator():
    M, K, N = 4, 6912, 2560
    W = sp.gen_ternary_iid(K, N, 1 / 3, 0)
    X = O.gen_x_i8(M * K, 1).reshape(M, K)
    out = torch.zeros((N, M), dtype=torch.int32, device="cuda")      # column-major M x N
    try:
        sp.dense_cublas_gemm(dev(np.ascontiguousarray(X.T)), dev(W), out, M, K, N)
    except sp.SptmmError as e:
        if e.code == -3:
            pytest.skip("cuBLAS declined the int8 shape: " + e.message)
        raise
    torch.cuda.synchronize()
    assert (out.cpu().numpy().T == O.gemv_i8_dense(X, W)).all()


def test_cublas_fp16_comparator_agrees_with_the_ternary_kernel():
    M, K, N = 8, 2560, 640
    W = sp.gen_ternary_iid(K, N, 0.5, 3)
    Xh = np.random.default_rng(4).standard_normal((M, K)).astype(np.float16)
    out = torch.zeros((N, M), dtype=torch.float32, device="cuda")    # column-major M x N
    sp.dense_cublas_gemm_f16(dev(np.ascontiguousarray(Xh.T)), dev(W.astype(np.float16)), out, M, K, N)
    ours = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    sp.Weights(W, sp.FMT_U16_V256).upload().gemv(dev(Xh), M, ours, sp.F16)
    torch.cuda.synchronize()
    want = Xh.astype(np.float64) @ W.T.astype(np.float64)
    scale = np.abs(Xh.astype(np.float64)) @ np.abs(W.T.astype(np.float64))
    assert (np.abs(out.cpu().numpy().T - want) <= FP16_RTOL * scale + 1e-30).all()
    assert (np.abs(ours.cpu().numpy() - want) <= FP16_RTOL * scale + 1e-30).all()


# ---------------------------------------------------------------- golden fixtures

def _golden_cases():
    path = os.path.join(GOLD, "manifest.json")
    if not os.path.exists(path):
        return []
    seen = []
    for e in json.load(open(path)):
        if e["case"] not in seen:
            seen.append(e["case"])
    return seen


@pytest.mark.parametrize("case", _golden_cases() or [pytest.param("none", marks=pytest.mark.skip(reason="no golden fixtures yet"))])
def test_against_reference_kernel_outputs(case):
    """Same W (reference generator), same X: the library's result equals what the reference's
    own kernel wrote on a B200."""
    from test_oracle import _parse, _load
    d = _parse(case)
    M, K, N, S, split = d["m"], d["k"], d["n"], d["s"], d["sp"]
    X = _load(case, "X", np.int8)
    Cgold = _load(case, "C", np.int32)
    W = sp.gen_ternary_fixed(K, N, S)
    if d["mode"] == "s3":
        w = sp.Weights(W, sp.FMT_U16_DIV, split=split, S=S).upload()
    else:
        w = sp.Weights(W, sp.FMT_DELTA_DIV256, S=S).upload()
    assert (run_i8(w, X, M) == Cgold).all()
    wn = sp.Weights(W, sp.FMT_U16_V256).upload()
    assert (run_i8(wn, X, M) == Cgold).all()
