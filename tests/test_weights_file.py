"""Encoded weights on disk (sptmm_weights_save / sptmm_weights_load): round trips of every format,
rejection of damaged, truncated and inconsistent files, and -- on a GPU -- that a loaded matrix
multiplies like the one it was saved from."""
import os
import struct

import numpy as np
import pytest

import oracle_lib as O
import sptmm_b200 as sp

FORMATS = [(sp.FMT_U16_V256, 0), (sp.FMT_DELTA_LANE, 0), (sp.FMT_U16_DIV, 128), (sp.FMT_DELTA_DIV256, 128), (sp.FMT_I2S, 0)]


def _matrix(fmt):
    if fmt in (sp.FMT_U16_DIV, sp.FMT_DELTA_DIV256):
        return sp.gen_ternary_fixed(256, 48, 128)            # the reference layouts need equal list lengths
    return sp.gen_ternary_iid(256, 48, 0.4, 3)


@pytest.mark.parametrize("fmt,S", FORMATS)
def test_save_load_round_trip(tmp_path, fmt, S):
    w = sp.Weights(_matrix(fmt), fmt, split=32, S=S)
    path = str(tmp_path / "w.sptmm")
    w.save(path)
    r = sp.Weights.load(path)
    for f in ("K", "N", "format", "split", "S", "max_count", "nnz", "stream_bytes", "lossy_entries", "n_arrays"):
        assert getattr(r.info, f) == getattr(w.info, f), f
    for i in range(w.info.n_arrays):
        (na, da, _), (nb, db, _) = w.array(i), r.array(i)
        assert na == nb and (da == db).all()
    assert os.path.getsize(path) % 8 == 0


def test_load_rejects_damage(tmp_path):
    w = sp.Weights(sp.gen_ternary_iid(256, 48, 0.4, 3), sp.FMT_U16_V256)
    path = str(tmp_path / "w.sptmm")
    w.save(path)
    blob = bytearray(open(path, "rb").read())

    def attempt(data, needle):
        p = str(tmp_path / "bad.sptmm")
        open(p, "wb").write(bytes(data))
        with pytest.raises(sp.SptmmError) as e:
            sp.Weights.load(p)
        assert needle in e.value.message, e.value.message

    flipped = bytearray(blob); flipped[len(blob) // 2] ^= 0x40
    attempt(flipped, "checksum")
    attempt(blob[: len(blob) // 2], "checksum")                       # truncated
    attempt(b"NOTSPTMM" + bytes(blob[8:]), "bad magic")
    attempt(b"", "too short")
    with pytest.raises(sp.SptmmError):
        sp.Weights.load(str(tmp_path / "missing.sptmm"))


def _rehash(blob: bytearray) -> bytearray:
    h = 1469598103934665603
    for b in blob[:-8]:
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    blob[-8:] = struct.pack("<Q", h)
    return blob


def test_load_rejects_consistent_looking_but_wrong_files(tmp_path):
    """A file with a valid checksum whose contents would make a kernel read out of range."""
    w = sp.Weights(sp.gen_ternary_iid(256, 48, 0.4, 3), sp.FMT_U16_V256)
    path = str(tmp_path / "w.sptmm")
    w.save(path)
    blob = bytearray(open(path, "rb").read())
    _, idx, _ = w.array(0)
    first = bytes(idx[:16].tobytes())
    at = bytes(blob).find(first)                                       # start of the index array in the file
    assert at > 0
    bad = bytearray(blob); bad[at:at + 2] = struct.pack("<H", 60000)    # a row index far beyond K
    p = str(tmp_path / "bad.sptmm"); open(p, "wb").write(bytes(_rehash(bad)))
    with pytest.raises(sp.SptmmError) as e:
        sp.Weights.load(p)
    assert "beyond K" in e.value.message
    bad = bytearray(blob); bad[16:20] = struct.pack("<I", 70000)        # K in the header
    open(p, "wb").write(bytes(_rehash(bad)))
    with pytest.raises(sp.SptmmError):
        sp.Weights.load(p)
    for at_, v in ((48, 7), (44, 128)):                                  # blocks per list / entries per block the table does not bear out
        bad = bytearray(blob); bad[at_:at_ + 4] = struct.pack("<I", v)
        open(p, "wb").write(bytes(_rehash(bad)))
        with pytest.raises(sp.SptmmError) as e:
            sp.Weights.load(p)
        assert "disagrees" in e.value.message
    bad = bytearray(blob); bad[8:12] = struct.pack("<I", 9)             # a future file version
    open(p, "wb").write(bytes(_rehash(bad)))
    with pytest.raises(sp.SptmmError) as e:
        sp.Weights.load(p)
    assert "version" in e.value.message


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,S", FORMATS)
def test_loaded_weights_multiply_like_the_original(tmp_path, fmt, S):
    torch = pytest.importorskip("torch")
    torch.cuda.set_device(0)
    W = _matrix(fmt)
    path = str(tmp_path / "w.sptmm")
    sp.Weights(W, fmt, split=32, S=S).save(path)
    w = sp.Weights.load(path).upload()
    M = 3
    X = O.gen_x_i8(M * 256, 5)
    out = torch.zeros(M * 48, dtype=torch.int32, device="cuda")
    w.gemv(torch.from_numpy(X).cuda(), M, out, sp.I8)
    torch.cuda.synchronize()
    assert (out.cpu().numpy().reshape(M, 48) == O.gemv_i8_dense(X, W)).all()
