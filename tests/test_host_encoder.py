"""CPU tests of the library's host side through the C ABI: generators and encoder against the
oracle byte for byte, error behaviour, and that libsptmm.so exports what include/sptmm.h declares.
No compute call is made here (no GPU)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import oracle_lib as O
import sptmm_b200 as sp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "sptmm.h")).read()
    declared = sorted(set(re.findall(r"\b(sptmm_[a-z0-9_]+)\s*\(", header)))
    assert declared, "no declarations found"
    raw = C.CDLL(sp.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), "libsptmm.so does not export %s" % name
    assert sorted(sp.EXPORTS) == declared
    assert sp.lib.sptmm_version() >= 100


@pytest.mark.parametrize("K,N,S", [(256, 32, 128), (512, 48, 256), (6912, 64, 4096)])
def test_fixed_generator_matches_oracle(K, N, S):
    assert (sp.gen_ternary_fixed(K, N, S) == O.gen_fixed(K, N, S)).all()


@pytest.mark.parametrize("p0,seed", [(1 / 3, 0), (0.5, 7), (0.75, 123456789)])
def test_iid_generator_matches_oracle(p0, seed):
    assert (sp.gen_ternary_iid(1000, 80, p0, seed) == O.gen_iid(1000, 80, p0, seed)).all()


@pytest.mark.parametrize("split", [8, 16, 32])
def test_u16_div_encoding_is_reference_layout(split):
    K, N, S = 512, 64, 256
    W = sp.gen_ternary_fixed(K, N, S)
    w = sp.Weights(W, sp.FMT_U16_DIV, split=split, S=S)
    pos, neg, _, _ = O.build_lists(W, S // 2, K)
    name0, a0, _ = w.array(0)
    name1, a1, _ = w.array(1)
    assert name0 == "W_map_%d_div" % split and name1 == "W_map_negative_%d_div" % split
    assert (a0.view(np.uint16) == O.encode_div(pos, split)).all()
    assert (a1.view(np.uint16) == O.encode_div(neg, split)).all()
    assert w.info.S == S and w.info.nnz == S * N and w.info.stream_bytes == 2 * S * N
    assert w.info.max_count == S // 2


@pytest.mark.parametrize("S", [512, 384])
def test_delta_div256_encoding_is_reference_layout(S):
    K, N = 1024, 32
    W = sp.gen_ternary_fixed(K, N, S)
    w = sp.Weights(W, sp.FMT_DELTA_DIV256, S=S)
    pos, neg, _, _ = O.build_lists(W, S // 2, K)
    gp, _ = O.delta_lists(pos)
    gn, _ = O.delta_lists(neg)
    assert (w.array(0)[1] == O.encode_delta_div256(gp)).all()
    assert (w.array(1)[1] == O.encode_delta_div256(gn)).all()
    assert w.info.lossy_entries == 0
    assert w.info.stream_bytes == S * N          # the padded tail of the last block is never read


def test_delta_div256_reports_lossy_entries():
    K, N = 1024, 16
    W = np.zeros((N, K), dtype=np.int8)
    W[:, 300] = 1; W[:, 310] = 1
    W[:, 5] = -1; W[:, 700] = -1
    w = sp.Weights(W, sp.FMT_DELTA_DIV256)
    assert w.info.lossy_entries == 2 * N         # first +1 index 300 and the -1 gap 695


def _decode_v256(w: sp.Weights, K: int):
    """Invert the native layout: position 8*lane+t of a block holds entry 32*t+lane."""
    _, idx, _ = w.array(0)
    _, off, _ = w.array(1)
    idx = idx.view(np.uint16).reshape(-1, 32, 8)
    off = off.view(np.uint32)
    lists = []
    for l in range(len(off) - 1):
        blocks = idx[off[l]:off[l + 1]]                      # (nb, lane, t)
        entries = blocks.transpose(0, 2, 1).reshape(-1)      # entry = b*256 + 32*t + lane
        lists.append(entries[entries != K])
    return lists


@pytest.mark.parametrize("p0", [1 / 3, 0.75, 1.0])
def test_v256_encoding_roundtrip(p0):
    K, N = 700, 40
    W = sp.gen_ternary_iid(K, N, p0, 11)
    w = sp.Weights(W, sp.FMT_U16_V256)
    lists = _decode_v256(w, K)
    for c in range(N):                  # same entries as the sorted lists; their order is the encoder's choice
        assert (np.sort(lists[2 * c]) == np.nonzero(W[c] == 1)[0]).all()
        assert (np.sort(lists[2 * c + 1]) == np.nonzero(W[c] == -1)[0]).all()
    _, off, _ = w.array(1)
    total_blocks = int(off.view(np.uint32)[-1])
    assert w.info.stream_bytes == total_blocks * 512 + (2 * N + 1) * 4
    assert w.info.nnz == int((W != 0).sum())


def _decode_delta_lane(w: sp.Weights):
    """Invert the lane-delta layout: 304-byte blocks = 256 offsets (byte 8*lane + t), eight 32-bit
    bases, eight counts; entry `lane` of step t is base[t] + offset for lane < count[t]."""
    _, raw, _ = w.array(0)
    _, off, _ = w.array(1)
    blocks = raw.view(np.uint8).reshape(-1, 304)
    off = off.view(np.uint32)
    lists = []
    for l in range(len(off) - 1):
        rows = []
        for blk in blocks[off[l]:off[l + 1]]:
            offs = blk[:256].reshape(32, 8)
            bases = blk[256:288].copy().view(np.uint32)
            counts = blk[288:296]
            assert (blk[296:] == 0).all()
            for t in range(8):
                rows.extend(int(bases[t]) + int(offs[lane, t]) for lane in range(counts[t]))
        lists.append(np.array(rows, dtype=np.int64))
    return lists


@pytest.mark.parametrize("p0", [1 / 3, 0.75, 0.97, 1.0])
def test_delta_lane_encoding_roundtrip(p0):
    K, N = 1500, 24
    W = sp.gen_ternary_iid(K, N, p0, 12)
    w = sp.Weights(W, sp.FMT_DELTA_LANE)
    lists = _decode_delta_lane(w)
    for c in range(N):                                   # exact and in ascending order, whatever the gaps
        assert (lists[2 * c] == np.nonzero(W[c] == 1)[0]).all()
        assert (lists[2 * c + 1] == np.nonzero(W[c] == -1)[0]).all()
    _, off, _ = w.array(1)
    assert w.info.stream_bytes == int(off.view(np.uint32)[-1]) * 304 + (2 * N + 1) * 4
    assert w.info.nnz == int((W != 0).sum()) and w.info.lossy_entries == 0


def test_delta_lane_is_about_0_6_of_the_u16_stream():
    W = sp.gen_ternary_fixed(6912, 16, 4096)
    d, u = sp.Weights(W, sp.FMT_DELTA_LANE), sp.Weights(W, sp.FMT_U16_V256)
    assert 0.55 < d.info.stream_bytes / u.info.stream_bytes < 0.70


def _bank_cycles(step_rows: np.ndarray, rb: int) -> int:
    """Shared-memory cycles of one 32-lane gather of `rb`-byte rows: accesses of up to 4 bytes go
    in one phase of 32 lanes, 8-byte ones in half warps, 16-byte ones in quarter warps; a phase
    costs as many cycles as the fullest bank holds distinct words."""
    lanes = 32 if rb <= 4 else 128 // rb
    total = 0
    for p in range(0, 32, lanes):
        rows = np.unique(step_rows[p:p + lanes].astype(np.int64))
        units = np.unique((rows * rb) >> 2) if rb <= 4 else rows
        banks = units % (32 if rb <= 4 else lanes)
        total += int(np.bincount(banks).max())
    return total


def test_v256_entry_order_avoids_bank_conflicts():
    """The native format orders a list's entries so that the rows a warp gathers together fall
    into different shared-memory banks for 4-, 8- and 16-byte tile rows, without giving up the
    conflict-free byte gathers of M=1 (sorted order: about 1.1 / 2.9 / 5.1 / 9.1 cycles)."""
    K, N, S = 6912, 8, 4096
    W = sp.gen_ternary_fixed(K, N, S)
    w = sp.Weights(W, sp.FMT_U16_V256)
    _, idx, _ = w.array(0)
    steps = idx.view(np.uint16).reshape(-1, 32, 8).transpose(0, 2, 1).reshape(-1, 32)     # (step, lane)
    steps = steps[(steps != K).all(axis=1)]
    mean = {rb: np.mean([_bank_cycles(s, rb) for s in steps]) for rb in (1, 4, 8, 16)}
    assert mean[1] < 1.15 and mean[4] < 1.7 and mean[8] < 2.9 and mean[16] < 5.0, mean
    again = sp.Weights(W, sp.FMT_U16_V256).array(0)[1]
    assert (again == idx).all()                                      # deterministic


def test_i2s_encoding_matches_oracle_packing():
    K, N = 64, 16
    W = sp.gen_ternary_iid(K, N, 0.4, 3)
    w = sp.Weights(W, sp.FMT_I2S)
    words = w.array(0)[1].view(np.uint32).reshape(N, K // 16)
    for c in (0, 7, 15):
        for j in range(K // 16):
            assert int(words[c, j]) == O.i2s_pack16(W[c, 16 * j:16 * j + 16])
    assert w.info.stream_bytes == K * N // 4


def test_encode_errors():
    W = sp.gen_ternary_fixed(256, 32, 128)
    with pytest.raises(sp.SptmmError) as e:
        sp.Weights(W, sp.FMT_U16_DIV, split=12)
    assert "Wrong split size" in e.value.message and e.value.code == -1     # main.cu:1039
    with pytest.raises(sp.SptmmError):
        sp.Weights(W, sp.FMT_U16_DIV, split=32, S=64)                       # a column has more than S/2
    with pytest.raises(sp.SptmmError):
        sp.Weights(W, sp.FMT_U16_DIV, split=32, S=129)                      # S odd (main.cu:90)
    bad = W.copy(); bad[3, 5] = 2
    with pytest.raises(sp.SptmmError):
        sp.Weights(bad, sp.FMT_U16_V256)
    with pytest.raises(sp.SptmmError):
        sp.Weights(np.zeros((4, 65536), dtype=np.int8), sp.FMT_U16_V256)    # K < 65536 (main.cu:89)
    iid = sp.gen_ternary_iid(256, 32, 0.5, 0)
    with pytest.raises(sp.SptmmError) as e:
        sp.Weights(iid, sp.FMT_DELTA_DIV256)                                # ragged lists: no padding value
    assert e.value.code == -3
    with pytest.raises(sp.SptmmError):
        sp.Weights(W[:, :250], sp.FMT_I2S)                                  # K % 16


def test_gemv_without_upload_fails_loudly():
    W = sp.gen_ternary_fixed(256, 32, 128)
    w = sp.Weights(W, sp.FMT_U16_V256)
    x = np.zeros(256, dtype=np.int8)
    out = np.zeros(32, dtype=np.int32)
    with pytest.raises(sp.SptmmError) as e:
        w.gemv(x, 1, out)
    assert e.value.code == -6 and "not uploaded" in e.value.message


def test_k_tiled_encoding_partitions_the_rows(tmp_path):
    """sptmm_encode_ktiled: every tile is a native matrix of its own K range; together they hold
    every non-zero once; tiles come out as handles; the parent cannot be saved as one file."""
    K, N, kt = 400, 24, 128                                       # the last tile is shorter (16 rows)
    W = sp.gen_ternary_iid(K, N, 0.4, 5)
    w = sp.Weights(W, sp.FMT_U16_V256, k_tile=kt)
    assert (w.info.k_tile, w.info.n_tiles, w.info.K, w.info.N) == (kt, 4, K, N)
    assert w.info.nnz == int((W != 0).sum())
    total = 0
    for t in range(4):
        tile = w.tile(t)
        k0, k1 = t * kt, min(K, (t + 1) * kt)
        ref = sp.Weights(np.ascontiguousarray(W[:, k0:k1]), sp.FMT_U16_V256)
        assert (tile.info.K, tile.info.N, tile.info.nnz) == (k1 - k0, N, ref.info.nnz)
        for i in range(ref.info.n_arrays):
            assert (tile.array(i)[1] == ref.array(i)[1]).all()
        total += tile.info.stream_bytes
    assert total == w.info.stream_bytes
    with pytest.raises(sp.SptmmError):
        w.tile(4)
    with pytest.raises(sp.SptmmError):
        w.save(str(tmp_path / "w.sptmm"))
    w.tile(1).save(str(tmp_path / "t1.sptmm"))                    # single tiles are ordinary matrices
    assert sp.Weights.load(str(tmp_path / "t1.sptmm")).info.K == kt
    with pytest.raises(sp.SptmmError):
        sp.Weights(W, sp.FMT_U16_V256, k_tile=100)                # not a multiple of 16


def test_status_and_wait_entry_points_validate_their_arguments():
    """Host plumbing of the per-call status word (no GPU, no kernel): null pointers and weights that
    were never uploaded are refused with the right codes."""
    import ctypes as C
    w = sp.Weights(sp.gen_ternary_iid(64, 16, 0.5, 1), sp.FMT_U16_V256)
    word = C.c_uint32(7)
    assert sp.lib.sptmm_gemv_status(None, C.byref(word)) == -1
    assert sp.lib.sptmm_gemv_status(w._h, None) == -1
    assert sp.lib.sptmm_gemv_status(w._h, C.byref(word)) == -6          # not uploaded
    assert b"not uploaded" in sp.lib.sptmm_last_error()
    assert sp.lib.sptmm_gemv_host_wait(w._h, 99) == -1                   # no such slot
    assert sp.lib.sptmm_gemv_host_wait(w._h, 0) == 0                     # an idle slot has nothing to wait for
    assert sp.lib.sptmm_seq_set_wait_limit(None, 1) == -1
    assert sp.lib.sptmm_seq_shared_bytes_for(None, 3, 1) == 0
