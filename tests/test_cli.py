"""The rcr / ccc programs: flag handling and the reference's error messages on CPU; on a GPU the
reference README's commands (README.md:23-27) with -check, and the stdout contract
(main.cu:813-832, 1459): 'make_X done', 'Compiled on ...', 'Start: ...', then ms per iteration."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RCR = os.path.join(ROOT, "sptmm_b200", "bin", "rcr")
CCC = os.path.join(ROOT, "sptmm_b200", "bin", "ccc")


def run(binary, *args):
    return subprocess.run([binary] + list(args), capture_output=True, text=True, timeout=600)


def test_binaries_exist():
    assert os.access(RCR, os.X_OK) and os.access(CCC, os.X_OK)


def test_unknown_flag_is_rejected():
    r = run(RCR, "-bogus", "1")
    assert r.returncode != 0 and "unknown command line flag 'bogus'" in r.stderr


@pytest.mark.parametrize("args,msg", [
    (["-row_split3_small", "12", "-M=1", "-K=256", "-N=32", "-S=128"], "Wrong split size"),      # main.cu:1039
    (["-row_split_delta2", "16", "-M=1", "-K=256", "-N=32", "-S=128"], "Wrong split size"),      # main.cu:1837
    (["-row_split3_small", "32", "-M=1", "-K=256", "-N=32", "-S=96"], "Wrong SPLIT Size"),       # main.cu:564
    (["-row_split3_small", "32", "-M=1", "-K=256", "-N=32", "-S=127"], "S mod 2 must be 0"),     # main.cu:90
    (["-row_split3_small", "32", "-M=1", "-K=65536", "-N=32", "-S=128"], "K should be fit"),      # main.cu:89
    (["-row_split3_small", "32", "-M=1", "-K=64", "-N=32", "-S=128"], "K should be bigger than S"),  # main.cu:91
    (["-cu_blas", "-M=1", "-K=256", "-N=32", "-S=128"], "Wrong layout"),                          # main.cu:843
])
def test_rcr_guards(args, msg):
    r = run(RCR, *args)
    assert r.returncode != 0 and msg in r.stderr


def test_ccc_rejects_i2s():
    r = run(CCC, "-i2s", "-M=1", "-K=256", "-N=32", "-S=128")
    assert r.returncode != 0 and "must be row-major" in r.stderr              # main.cu:1852-1854


README_COMMANDS = [
    (RCR, ["-row_split3_small", "32", "-M=1"]),
    (RCR, ["-row_split3_small", "32", "-M=4"]),
    (RCR, ["-row_split_delta2", "32", "-M=1"]),
    (CCC, ["-cu_blas", "-M=4"]),
    (RCR, ["-i2s", "-M=1"]),
    (RCR, ["-row_split3_small", "8", "-M=1", "-native=0"]),
    (RCR, ["--row_split3_small=16", "--M=8", "-native", "0"]),
]


@pytest.mark.gpu
@pytest.mark.parametrize("binary,args", README_COMMANDS)
def test_readme_commands(binary, args):
    r = run(binary, *args, "-K=6912", "-N=2560", "-S=4096", "-iter=50", "-check", "-seed=7", "-json")
    if "-cu_blas" in args and "cublasGemmEx" in r.stderr:
        pytest.skip("cuBLAS declined the int8 shape: " + r.stderr.strip().splitlines()[-1])
    assert r.returncode == 0, r.stderr
    lines = r.stdout.strip().splitlines()
    assert lines[0] == "make_X done"
    assert lines[1].startswith("Compiled on ")
    m = re.match(r"Start: M=(\d+) K=6912 N=2560 ITER=50 S=4096 \(40\.7407% Sparsity\) L=1 B=8 X_MAJOR=(ROW|COL) W_MAJOR=COL C_MAJOR=(ROW|COL)$", lines[2])
    assert m, lines[2]
    assert float(lines[3]) > 0
    assert "check: OK" in r.stderr


# ---------------------------------------------------------------- offline encoder

ENC = os.path.join(ROOT, "sptmm_b200", "bin", "sptmm_encode")


@pytest.mark.parametrize("fmt_name,fmt_flag", [("u16_v256", []), ("delta_lane", []), ("u16_div", ["-split", "32"]), ("i2s", [])])
def test_offline_encoder_writes_what_the_library_encodes(tmp_path, fmt_name, fmt_flag):
    import numpy as np
    import sptmm_b200 as sp
    path = str(tmp_path / "w.sptmm")
    r = run(ENC, "-K", "256", "-N", "48", "-S", "128", "-format", fmt_name, "-o", path, *fmt_flag)
    assert r.returncode == 0, r.stderr
    assert "K=256 N=48" in r.stdout
    fmt = {"u16_v256": sp.FMT_U16_V256, "delta_lane": sp.FMT_DELTA_LANE, "u16_div": sp.FMT_U16_DIV, "i2s": sp.FMT_I2S}[fmt_name]
    want = sp.Weights(sp.gen_ternary_fixed(256, 48, 128), fmt, split=32, S=128 if fmt == sp.FMT_U16_DIV else 0)
    got = sp.Weights.load(path)
    assert got.info.n_arrays == want.info.n_arrays and got.info.nnz == want.info.nnz
    for i in range(want.info.n_arrays):
        assert (got.array(i)[1] == want.array(i)[1]).all()


def test_offline_encoder_reads_a_dense_matrix_and_checks_its_size(tmp_path):
    import numpy as np
    import sptmm_b200 as sp
    W = sp.gen_ternary_iid(128, 20, 0.5, 9)
    dense, path = str(tmp_path / "W.i8"), str(tmp_path / "w.sptmm")
    W.tofile(dense)
    r = run(ENC, "-K", "128", "-N", "20", "-dense", dense, "-o", path)
    assert r.returncode == 0, r.stderr
    want = sp.Weights(W, sp.FMT_U16_V256)
    assert (sp.Weights.load(path).array(0)[1] == want.array(0)[1]).all()
    r = run(ENC, "-K", "128", "-N", "21", "-dense", dense, "-o", path)
    assert r.returncode != 0 and "exactly K*N bytes" in r.stderr
    r = run(ENC, "-K", "128", "-N", "20", "-o", path)
    assert r.returncode != 0 and "-S" in r.stderr
    r = run(ENC, "-K", "128", "-N", "20", "-S", "64", "-format", "nope", "-o", path)
    assert r.returncode != 0 and "unknown -format" in r.stderr


@pytest.mark.gpu
def test_rcr_runs_an_encoded_weights_file(tmp_path):
    path = str(tmp_path / "w.sptmm")
    assert run(ENC, "-K", "6912", "-N", "2560", "-S", "4096", "-format", "u16_v256", "-o", path).returncode == 0
    r = run(RCR, "-row_split3_small", "32", "-M=4", "-K=6912", "-N=2560", "-S=4096", "-iter=5", "-check", "-seed=3", "-weights", path)
    assert r.returncode == 0, r.stderr
    assert "check: OK" in r.stderr
    r = run(RCR, "-row_split3_small", "32", "-M=1", "-K=256", "-N=2560", "-S=128", "-iter=1", "-weights", path)
    assert r.returncode != 0 and "-weights file" in r.stderr
