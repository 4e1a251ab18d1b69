"""Real-valued weights -> ternary (absmean, BitNet b1.58): the library's host routine against the
oracle's restatement and against the rule written out in numpy; fp16 input; the encoder tool's
-f32 path.  No checkpoint is involved: seeded Gaussian tensors stand in for a model's weights."""
import os
import subprocess

import numpy as np
import pytest

import oracle_lib as O
import sptmm_b200 as sp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _weights(N, K, seed, dtype=np.float32):
    rng = np.random.default_rng(seed)
    W = (rng.standard_normal((N, K)) * 0.02).astype(dtype)
    W[0, :8] = [0.0, 1.0, -1.0, 5.0, -5.0, 1e-9, -1e-9, 0.0]          # clamps and tiny values
    return W


@pytest.mark.parametrize("N,K", [(48, 256), (7, 33), (1, 1)])
def test_matches_the_oracle_and_the_rule(N, K):
    W = _weights(N, K, N * 100 + K) if K >= 8 else np.full((N, K), 0.3, dtype=np.float32)
    got, scale = sp.ternarise_absmean(W)
    want, want_scale = O.ternarise_absmean(W)
    assert (got == want).all() and scale == want_scale
    mean = np.float32(np.abs(W.astype(np.float64)).sum(axis=1).sum() / W.size) if N * K > 1 else np.float32(abs(float(W[0, 0])))
    rule = np.clip(np.rint(W * (np.float32(1.0) / (mean + np.float32(1e-5)))), -1, 1).astype(np.int8)
    assert (got == rule).all()
    assert set(np.unique(got)) <= {-1, 0, 1}
    assert abs(scale - float(np.abs(W.astype(np.float64)).mean())) <= 1e-6 * max(scale, 1e-30)


def test_half_precision_input_and_the_share_of_zeros():
    W32 = _weights(64, 512, 3)
    W16 = W32.astype(np.float16)
    got16, s16 = sp.ternarise_absmean(W16)
    want, s32 = O.ternarise_absmean(W16.astype(np.float32))            # fp16 -> fp32 is exact
    assert (got16 == want).all() and s16 == s32
    # for Gaussian weights the rule leaves about P(|w| < mean/2) = 31 % zeros
    assert 0.25 < float((got16 == 0).mean()) < 0.40
    # subnormal and special halves convert like numpy does
    odd = np.array([[6e-8, -6e-8, 65504.0, -65504.0, 0.0, 1e-4, -2e-5, 3e-5]], dtype=np.float16)
    g, s = sp.ternarise_absmean(odd)
    w, ws = O.ternarise_absmean(odd.astype(np.float32))
    assert (g == w).all() and s == ws


def test_rejects_bad_input():
    with pytest.raises(ValueError):
        sp.ternarise_absmean(np.zeros((4, 4), dtype=np.int8))
    bad = np.zeros((2, 8), dtype=np.float32); bad[1, 3] = np.nan
    with pytest.raises(sp.SptmmError):
        sp.ternarise_absmean(bad)


def test_encoder_tool_takes_real_weights(tmp_path):
    tool = os.path.join(ROOT, "sptmm_b200", "bin", "sptmm_encode")
    if not os.path.exists(tool):
        pytest.skip("bin/sptmm_encode is not built")
    N, K = 40, 128
    W = _weights(N, K, 11)
    raw, out = str(tmp_path / "w.f32"), str(tmp_path / "w.sptmm")
    W.tofile(raw)
    r = subprocess.run([tool, "-K", str(K), "-N", str(N), "-f32", raw, "-o", out], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    want, scale = O.ternarise_absmean(W)
    assert abs(float(r.stdout.split("absmean scale")[1].split()[0]) - scale) <= 1e-7 * scale
    loaded = sp.Weights.load(out)
    direct = sp.Weights(want, sp.FMT_U16_V256)
    assert loaded.info.nnz == direct.info.nnz == int((want != 0).sum())
    for i in range(direct.info.n_arrays):
        assert (loaded.array(i)[1] == direct.array(i)[1]).all()
