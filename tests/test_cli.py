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
