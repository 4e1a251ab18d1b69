"""GPU parity of the steps either side of the matmul in a quantised layer: the per-row absmax
quantiser as a kernel of its own (sptmm_quantize_absmax) against the oracle's quantiser, and the
de-quantising epilogue of the per-call kernel (sptmm_gemv_scaled) against the same arithmetic in
numpy float32 and against a double-precision product."""
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


@pytest.mark.parametrize("M,K", [(1, 2560), (4, 6912), (16, 333), (3, 1)])
def test_quantize_absmax_matches_oracle(M, K):
    rng = np.random.default_rng(M * 1000 + K)
    A = rng.integers(-400000, 400000, size=(M, K), dtype=np.int32)
    if M > 1:
        A[1] = 0                                               # a row of zeros: zeros out, scale 0
    want_q, want_s = O.quant_absmax_i8(A)
    q = torch.full((M, K), 99, dtype=torch.int8, device="cuda")
    s = torch.full((M,), -1.0, dtype=torch.float32, device="cuda")
    sp.quantize_absmax(dev(A), M, K, q, s)
    torch.cuda.synchronize()
    assert (q.cpu().numpy() == want_q).all()
    assert (s.cpu().numpy() == want_s).all()


def test_quantize_absmax_row_stride_pairs_and_shards():
    rng = np.random.default_rng(7)
    M, K, ld = 5, 384, 1000
    big = rng.integers(-90000, 90000, size=(M, ld), dtype=np.int32)
    # a column range of wider rows
    q = torch.zeros((M, K), dtype=torch.int8, device="cuda")
    sp.quantize_absmax(dev(big)[:, 100:], M, K, q, None, ldx=ld)
    torch.cuda.synchronize()
    assert (q.cpu().numpy() == O.quant_absmax_i8(np.ascontiguousarray(big[:, 100:100 + K]))[0]).all()
    # pair sums of interleaved columns: value k = X[2k] + X[2k+1]
    inter = np.ascontiguousarray(big[:, :2 * K])
    sp.quantize_absmax(dev(inter), M, K, q, None, pair=True)
    torch.cuda.synchronize()
    assert (q.cpu().numpy() == O.quant_absmax_i8(np.ascontiguousarray(inter[:, 0::2]), np.ascontiguousarray(inter[:, 1::2]))[0]).all()
    # the layout an all-gather of four ranks' column shards leaves: [rank][M][shard]
    shard = K // 4
    rows = np.ascontiguousarray(big[:, :K])
    gathered = np.ascontiguousarray(rows.reshape(M, 4, shard).transpose(1, 0, 2))
    s = torch.zeros(M, dtype=torch.float32, device="cuda")
    sp.quantize_absmax(dev(gathered), M, K, q, s, shard=shard)
    torch.cuda.synchronize()
    want_q, want_s = O.quant_absmax_i8(rows)
    assert (q.cpu().numpy() == want_q).all() and (s.cpu().numpy() == want_s).all()
    # the leading columns only (a reader of part of the gathered row)
    sp.quantize_absmax(dev(gathered), M, K - 100, q[:, :K - 100].contiguous(), None, shard=shard)
    qq = torch.zeros((M, K - 100), dtype=torch.int8, device="cuda")
    sp.quantize_absmax(dev(gathered), M, K - 100, qq, None, shard=shard)
    torch.cuda.synchronize()
    assert (qq.cpu().numpy() == O.quant_absmax_i8(np.ascontiguousarray(rows[:, :K - 100]))[0]).all()
    with pytest.raises(sp.SptmmError):
        sp.quantize_absmax(dev(gathered), M, K // 2, q, None, shard=7, pair=True)


@pytest.mark.parametrize("fmt", [sp.FMT_U16_V256, sp.FMT_DELTA_LANE])
@pytest.mark.parametrize("M", [1, 4, 16])
def test_gemv_scaled_dequantises_in_the_epilogue(M, fmt):
    K, N = 1024, 384
    W = sp.gen_ternary_iid(K, N, 1 / 3, 21)
    w = sp.Weights(W, fmt).upload()
    X = O.gen_x_i8(M * K, 3)
    rs = (np.arange(M, dtype=np.float32) + 1.0) * np.float32(0.0131)
    w_scale = 0.0473
    out = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    w.gemv_scaled(dev(X), M, out, dev(rs), w_scale)
    torch.cuda.synchronize()
    sums = O.gemv_i8_dense(X, W).reshape(M, N)
    sc = rs * np.float32(w_scale)                                   # one fp32 product of the two scales
    want = sums.astype(np.float32) * sc[:, None]                    # one fp32 product with the exact sum
    got = out.cpu().numpy()
    assert (got == want).all()
    exact = sums.astype(np.float64) * rs.astype(np.float64)[:, None] * w_scale
    assert np.max(np.abs(got - exact) / np.maximum(np.abs(exact), 1e-30)) <= 2e-7      # two roundings to fp32
    out.zero_()
    w.gemv_scaled(dev(X), M, out, None, 1.0)                         # no scales: the sums as floats
    torch.cuda.synchronize()
    assert (out.cpu().numpy() == sums.astype(np.float32)).all()
    assert w.status() == 0
