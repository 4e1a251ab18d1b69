"""CPU tests of the oracle itself: internal consistency (list path == dense product), the
reference's structural invariants, and -- once present -- the golden fixtures produced by the
reference's own kernels (tests/golden/)."""
import json
import os

import numpy as np
import pytest

import oracle_lib as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_fixed_generator_invariants():
    # main.cu:251-256, 276: exactly S/2 entries of each sign in every column
    K, N, S = 256, 32, 128
    W = O.gen_fixed(K, N, S)
    assert ((W == 1).sum(axis=1) == S // 2).all()
    assert ((W == -1).sum(axis=1) == S // 2).all()
    assert set(np.unique(W)) <= {-1, 0, 1}
    # columns are seeded differently (0xCAFEBABE ^ col)
    assert not (W[0] == W[1]).all()
    # deterministic
    assert (O.gen_fixed(K, N, S) == W).all()


def test_xorshift_known_answer():
    # three steps of macro.cuh:69-76 from state 1, worked by hand
    # x=1: x^=x<<13 -> 8193; x^=x>>17 -> 8193; x^=x<<5 -> 8193^262176 = 270369
    x = 1
    def step(x):
        x ^= (x << 13) & 0xFFFFFFFF
        x ^= x >> 17
        x ^= (x << 5) & 0xFFFFFFFF
        return x
    assert step(1) == 270369
    # the oracle's activation stream uses the same recurrence
    s = 12345
    want = []
    for _ in range(8):
        s = step(s)
        want.append((s % 255) - 127)
    assert O.gen_x_i8(8, 12345).tolist() == want


def test_iid_generator_density():
    W = O.gen_iid(2048, 64, 1 / 3, 0)
    frac0 = (W == 0).mean()
    assert abs(frac0 - 1 / 3) < 0.01
    assert abs((W == 1).mean() - (W == -1).mean()) < 0.01
    assert (O.gen_iid(2048, 64, 1 / 3, 0) == W).all()
    assert not (O.gen_iid(2048, 64, 1 / 3, 1) == W).all()
    assert (O.gen_iid(64, 16, 1.0, 0) == 0).all()
    assert (O.gen_iid(64, 16, 0.0, 0) != 0).all()


@pytest.mark.parametrize("split", [8, 16, 32])
@pytest.mark.parametrize("M", [1, 4])
def test_div_path_equals_dense(split, M):
    K, N, S = 512, 48, 256
    W = O.gen_fixed(K, N, S)
    X = O.gen_x_i8(M * K, 7)
    pos, neg, npos, nneg = O.build_lists(W, S // 2, K)
    assert (npos == S // 2).all() and (nneg == S // 2).all()
    # lists are sorted ascending (main.cu:267-274 scans rows upward)
    assert (np.diff(pos.astype(np.int32), axis=1) > 0).all()
    got = O.gemv_i8_div(X, O.encode_div(pos, split), O.encode_div(neg, split), M, K, N, S, split)
    want = O.gemv_i8_dense(X, W)
    assert (got == want).all()
    assert (want == (X.reshape(M, K).astype(np.int64) @ W.T.astype(np.int64))).all()
    assert (O.gemv_i8_lists(X, pos, neg, npos, nneg, K) == want).all()
    assert (O.gemv_i8_div_mt(X, O.encode_div(pos, split), O.encode_div(neg, split), M, K, N, S, split, 3) == want).all()


def test_div_layout_offsets():
    # element (entry e, column c) at (e/split)*(split*N) + c*split + e%split  (main.cu:345-351)
    N, half, split = 16, 64, 32
    lst = (np.arange(N * half, dtype=np.uint32) % 60000).astype(np.uint16).reshape(N, half)
    out = O.encode_div(lst, split)
    for c in (0, 5, 15):
        for e in (0, 1, 31, 32, 63):
            assert out[(e // split) * (split * N) + c * split + e % split] == lst[c, e]


@pytest.mark.parametrize("S", [512, 384])
def test_delta_path_equals_dense(S):
    K, N, M = 1024, 32, 2
    W = O.gen_fixed(K, N, S)
    X = O.gen_x_i8(M * K, 9)
    pos, neg, _, _ = O.build_lists(W, S // 2, K)
    gp, lossy_p = O.delta_lists(pos)
    gn, lossy_n = O.delta_lists(neg)
    assert lossy_p == 0 and lossy_n == 0
    got = O.gemv_i8_delta256(X, O.encode_delta_div256(gp), O.encode_delta_div256(gn), M, K, N, S)
    assert (got == O.gemv_i8_dense(X, W)).all()


def test_delta_truncation_is_reproduced():
    # main.cu:377-383 stores the first index and every gap in 8 bits; a gap > 255 makes the
    # reference rebuild a wrong index.  The oracle must reproduce that, not repair it.
    K, N = 1024, 16
    W = np.zeros((N, K), dtype=np.int8)
    W[:, 300] = 1; W[:, 310] = 1          # first index 300 -> stored as 44
    W[:, 5] = -1; W[:, 6] = -1
    X = O.gen_x_i8(K, 3)
    pos, neg, _, _ = O.build_lists(W, 2, K)
    gp, lossy = O.delta_lists(pos)
    assert lossy == N and gp[0, 0] == 300 - 256
    gn, _ = O.delta_lists(neg)
    got = O.gemv_i8_delta256(X, O.encode_delta_div256(gp), O.encode_delta_div256(gn), 1, K, N, 4)
    wrong = int(X[44]) + int(X[54]) - int(X[5]) - int(X[6])
    assert (got == wrong).all()


def test_float_path_matches_double():
    K, N, M = 512, 32, 3
    W = O.gen_iid(K, N, 0.4, 5)
    rng = np.random.default_rng(0)
    X = rng.standard_normal((M, K)).astype(np.float16).astype(np.float32)
    cap = int(max((W == 1).sum(1).max(), (W == -1).sum(1).max()))
    pos, neg, npos, nneg = O.build_lists(W, cap, K)
    ref, dbl, ab = O.gemv_f32_lists(X, pos, neg, npos, nneg, K)
    want = X.astype(np.float64) @ W.T.astype(np.float64)
    assert np.allclose(dbl, want, rtol=0, atol=1e-9)
    assert (np.abs(ref - dbl) <= 1e-5 * ab + 1e-12).all()
    assert np.allclose(ab, np.abs(X).astype(np.float64) @ np.abs(W.T).astype(np.float64))


def test_i2s_bit_positions():
    # bitnet_kernels.cuh:57-71: output byte e comes from bits 8*(e%4)+2*(e/4); code = w+2
    for e in range(16):
        w = np.zeros(16, dtype=np.int8)
        w[e] = 1
        word = O.i2s_pack16(w)
        zero = O.i2s_pack16(np.zeros(16, dtype=np.int8))
        assert word ^ zero == (3 ^ 2) << (8 * (e % 4) + 2 * (e // 4))
    rng = np.random.default_rng(1)
    w = rng.integers(-1, 2, 16).astype(np.int8)
    assert (O.i2s_unpack16(O.i2s_pack16(w)) == w).all()


# ---- golden fixtures from the reference's own kernels --------------------------------------

def _manifest():
    path = os.path.join(GOLD, "manifest.json")
    if not os.path.exists(path):
        return []
    with open(path) as f:
        return json.load(f)


def _cases():
    seen = []
    for e in _manifest():
        if e["case"] not in seen:
            seen.append(e["case"])
    return seen


def _parse(case):
    # s3_m1_k256_n32_s128_sp8 / dl_m1_k1024_n32_s512
    parts = case.split("_")
    d = {"mode": parts[0]}
    for p in parts[1:]:
        for key in ("sp", "m", "k", "n", "s"):
            if p.startswith(key) and p[len(key):].isdigit():
                d[key] = int(p[len(key):])
                break
    d.setdefault("sp", 32)
    return d


def _entry(case, array):
    for e in _manifest():
        if e["case"] == case and e["array"] == array:
            return e
    raise KeyError((case, array))


def _load(case, array, dtype):
    return np.fromfile(os.path.join(GOLD, "%s.%s.bin" % (case, array)), dtype=dtype)


@pytest.mark.parametrize("case", _cases() or [pytest.param("none", marks=pytest.mark.skip(reason="no golden fixtures yet"))])
def test_oracle_against_reference_golden(case):
    """Generator, list builder, encoders and matmul of the oracle reproduce, byte for byte, what
    the reference's prepareW_map and SpTMM kernels produced on a B200."""
    d = _parse(case)
    M, K, N, S, split = d["m"], d["k"], d["n"], d["s"], d["sp"]
    X = _load(case, "X", np.int8)
    Cgold = _load(case, "C", np.int32).reshape(M, N)
    W = O.gen_fixed(K, N, S)
    assert O.fnv1a64(W) == _entry(case, "W_dense")["fnv1a64"]
    pos, neg, _, _ = O.build_lists(W, S // 2, K)
    assert O.fnv1a64(pos) == _entry(case, "W_map")["fnv1a64"]
    assert O.fnv1a64(neg) == _entry(case, "W_map_negative")["fnv1a64"]
    for sp in (8, 16, 32):
        if (S // 2) % sp == 0:
            assert O.fnv1a64(O.encode_div(pos, sp)) == _entry(case, "W_map_%d_div" % sp)["fnv1a64"]
            assert O.fnv1a64(O.encode_div(neg, sp)) == _entry(case, "W_map_negative_%d_div" % sp)["fnv1a64"]
    gp, _ = O.delta_lists(pos)
    gn, _ = O.delta_lists(neg)
    dp, dn = O.encode_delta_div256(gp), O.encode_delta_div256(gn)
    assert O.fnv1a64(dp) == _entry(case, "W_map_delta2_div256")["fnv1a64"]
    assert O.fnv1a64(dn) == _entry(case, "W_map_negative_delta2_div256")["fnv1a64"]
    if d["mode"] == "s3":
        got = O.gemv_i8_div(X, O.encode_div(pos, split), O.encode_div(neg, split), M, K, N, S, split)
    else:
        got = O.gemv_i8_delta256(X, dp, dn, M, K, N, S)
    assert (got == Cgold).all()
    if _entry(case, "W_map")["file"]:
        assert (_load(case, "W_map", np.uint16).reshape(N, S // 2) == pos).all()
        assert (_load(case, "W_dense", np.int8).reshape(N, K) == W).all()
