"""The allocation-free sequence call, sptmm_seq_run_static.

Some callers cannot allocate device memory when they need a matmul (a closed, pre-sized memory
pool; a loop that may not block on the allocator; a framework that owns the whole device), so this
entry point keeps the sequence kernel's scratch in a fixed array inside the library.  The test
calls it through the C ABI twice in a row -- the array keeps the previous call's contents, so the
second call proves the per-call clearing -- and checks every output against the allocating entry
points (sptmm_seq_create / sptmm_seq_run) bit for bit (int32 results: the tolerance is zero).
Kept in a file that pytest collects last, so that a failure here cannot hide other results.
"""
import numpy as np
import pytest

import oracle_lib as O
import sptmm_b200 as sp

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _case(M):
    K1, N1, H, N3 = 512, 384, 320, 200
    Ws = [sp.gen_ternary_iid(K1, N1, 0.4, 1), sp.gen_ternary_iid(N1, 2 * H, 0.5, 2), sp.gen_ternary_iid(H, N3, 1 / 3, 3)]
    ws = [sp.Weights(W, sp.FMT_U16_V256).upload() for W in Ws]          # uploading allocates; running will not
    x = torch.from_numpy(O.gen_x_i8(M * K1, 4)).cuda()

    def buffers():
        return (torch.zeros((M, N1), dtype=torch.int32, device="cuda"),
                torch.zeros((M, 2 * H), dtype=torch.int32, device="cuda"),
                torch.zeros((M, N3), dtype=torch.int32, device="cuda"),
                torch.zeros(M, dtype=torch.float32, device="cuda"))

    def steps(c1, c2, c3, s3):
        return [{"w": ws[0], "X": x, "C": c1},
                {"w": ws[1], "X": c1, "C": c2, "x_kind": 1, "dep": 0},
                {"w": ws[2], "X": c2, "X2": c2[:, H:], "ldx": 2 * H, "ldx2": 2 * H, "C": c3, "x_kind": 1, "dep": 1,
                 "scale_out": s3}]
    return buffers, steps


@pytest.mark.parametrize("M", [1, 4])
def test_static_scratch_call_matches_allocating_path(M):
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    buffers, steps = _case(M)
    ref = buffers()
    seq = sp.Sequence(steps(*ref), M=M)
    seq.run()
    assert seq.status() == 0
    want = [t.cpu().numpy().copy() for t in ref]
    for call in range(2):                                   # two calls in a row share the fixed array
        got = buffers()
        for t in got[:3]:
            t.fill_(-1)
        before = torch.cuda.memory_allocated()
        status = sp.run_sequence_static(steps(*got), M=M)
        assert status == 0
        assert torch.cuda.memory_allocated() == before      # torch's allocator was not touched either
        for g, w in zip(got, want):
            assert np.array_equal(g.cpu().numpy(), w), "call %d differs from the allocating path" % call


def test_static_scratch_call_rejects_what_does_not_fit():
    torch.cuda.set_device(0)
    W = sp.gen_ternary_iid(256, 64, 0.5, 0)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    x = torch.from_numpy(O.gen_x_i8(256, 1)).cuda()
    c = torch.zeros(64, dtype=torch.int32, device="cuda")
    with pytest.raises(sp.SptmmError) as e:
        sp.run_sequence_static([{"w": w, "X": x, "C": c}] * 17)
    assert e.value.code == -1 and "at most 16" in e.value.message
    with pytest.raises(sp.SptmmError):
        sp.run_sequence_static([{"w": w, "X": x, "C": c}], M=17)
    assert sp.run_sequence_static([{"w": w, "X": x, "C": c}]) == 0      # still usable afterwards
    assert np.array_equal(c.cpu().numpy(), O.gemv_i8_dense(O.gen_x_i8(256, 1), W).reshape(-1))


def test_static_scratch_call_refuses_a_capturing_stream():
    """The call copies its step tables from host memory that dies with the call, so it must not be
    recorded into a CUDA graph: on a stream under capture it returns an error and records nothing;
    the capture itself stays valid and the entry point keeps working afterwards."""
    torch.cuda.set_device(0)
    W = sp.gen_ternary_iid(256, 64, 0.5, 0)
    w = sp.Weights(W, sp.FMT_U16_V256).upload()
    x = torch.from_numpy(O.gen_x_i8(256, 1)).cuda()
    c = torch.zeros(64, dtype=torch.int32, device="cuda")
    assert sp.run_sequence_static([{"w": w, "X": x, "C": c}]) == 0      # the first call on the device: outside any capture
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
        with pytest.raises(sp.SptmmError) as e:
            sp.run_sequence_static([{"w": w, "X": x, "C": c}], stream=torch.cuda.current_stream().cuda_stream, wait=False)
        assert e.value.code == -6 and "captured" in e.value.message
        c.add_(0)                                                        # something harmless so the graph is not empty
    graph.replay()
    torch.cuda.synchronize()
    c.zero_()
    assert sp.run_sequence_static([{"w": w, "X": x, "C": c}]) == 0
    assert np.array_equal(c.cpu().numpy(), O.gemv_i8_dense(O.gen_x_i8(256, 1), W).reshape(-1))
