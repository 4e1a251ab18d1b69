#!/usr/bin/env python
"""Benchmark of the ternary GEMV hot path (6912 x 2560, M=1, int8 -> int32) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = `--calls` GEMV calls, rotating over enough distinct copies of the encoded weights
that their total exceeds L2 (cold-cache, HBM-bound).  The calls are independent of one another,
as the iterations of the reference's timing loop are, so they are issued round-robin on
`--streams` streams (ordered, with programmatic-dependent-launch edges, inside each stream).
The step is captured once in a CUDA graph and replayed; timing is by CUDA events on the stream
the graph is launched on, max over ranks.  `single_stream` in the output is the same step with
every call on one stream.  Prints ONE JSON line on rank 0.

`--impl reference` times the CPU restatement of the reference's loop (the reference has no CPU
path and its GPU kernels print only a time) on all host threads, same metric and unit.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

K, N, S, M = 6912, 2560, 4096, 1
L2_BYTES = 126 * 1024 * 1024
METRIC = "effective_hbm_GBps_ternary_gemv_6912x2560_M1"
WORKLOAD = "C1 ternary GEMV M=1 K=6912 N=2560, reference generator -S=4096, int8 activations, int32 sums"
# DRAM bytes (read + write) per launch of the GEMV kernel on exactly this workload, from one ncu
# capture of two launches (21.0092 MB each); not measured by the run that prints it.
NCU_TRAFFIC_BYTES = 21009200
# the same in both arms of the bench (the GPU arm's copy count and launch mode, and each arm's weight layout, are in "detail")
CONFIG = {"workload": WORKLOAD,
          "l2": "GPU arm: cold, the calls rotate over weight copies totalling more than the 126 MB L2; host arm: one 21 MB copy"}


def algorithmic_bytes(stream_bytes: int, m: int, act_size: int) -> int:
    """encoded weights + M*K activations + M*N int32/float32 outputs, per call."""
    return stream_bytes + m * K * act_size + m * N * 4


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the benchmark runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.thread = [], None, None
        self.cmd = ["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "50"]

    def start(self):
        try:
            self.proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        def pump():
            for line in self.proc.stdout:
                self.rows.append((time.time(), line.strip()))
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self, t0: float, t1: float) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, n = [], None, set(), 0
        for t, line in self.rows:
            if t < t0 or t > t1 + 0.05:
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx = float(f[1])
            except ValueError:
                continue
            n += 1
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": n}


def cpu_baseline(budget_s: float = 8.0, blocks: int = 7):
    """Scalar add/sub loop over the reference's chunk-interleaved u16 layout on the host cores.
    The budget is split into `blocks` equal parts and the MEDIAN block is reported: other work on
    the box moves single timings by tens of per cent."""
    import oracle_lib as O
    W = O.gen_fixed(K, N, S)
    X = O.gen_x_i8(M * K, 1)
    pos, neg, _, _ = O.build_lists(W, S // 2, K)
    wp, wn = O.encode_div(pos, 32), O.encode_div(neg, 32)
    cores = os.cpu_count() or 1
    nbytes = algorithmic_bytes(2 * S * N, M, 1)
    O.gemv_i8_div_mt(X, wp, wn, M, K, N, S, 32, cores)
    per_call, calls = [], 0
    for _ in range(blocks):
        n, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < budget_s / blocks:
            O.gemv_i8_div_mt(X, wp, wn, M, K, N, S, 32, cores)
            n += 1
        per_call.append((time.perf_counter() - t0) / n)
        calls += n
    dt = statistics.median(per_call)
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "us_per_call": dt * 1e6, "us_per_call_min_max": [min(per_call) * 1e6, max(per_call) * 1e6],
            "sample": "%d calls of the same M=1 6912x2560 S=4096 GEMV in %d blocks over ~%.0f s, %d threads; median block" % (calls, blocks, budget_s, cores)}, (X, wp, wn)


def run_reference(args):
    """CPU port of the reference loop, all host threads; step = 4 calls."""
    import oracle_lib as O
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, (X, wp, wn) = cpu_baseline(budget_s=2.0)
    cores = base["cores"]
    per_step = 4
    for _ in range(min(args.warmup, 20)):
        O.gemv_i8_div_mt(X, wp, wn, M, K, N, S, 32, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for _ in range(per_step):
            O.gemv_i8_div_mt(X, wp, wn, M, K, N, S, 32, cores)
    dt = time.perf_counter() - t0
    nbytes = algorithmic_bytes(2 * S * N, M, 1)
    value = nbytes * per_step * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "us_per_call": dt / (args.steps * per_step) * 1e6, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "i8", "data": "synthetic",
        "config": CONFIG,
        "detail": {"layout": "reference u16 lists, split 32 (W_map_32_div)", "calls_per_step": per_step},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "%d steps x %d calls, scalar add/sub loop over W_map_32_div, %d threads" % (args.steps, per_step, cores)},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    import sptmm_b200 as sp
    import oracle_lib as O

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    # ---- workload: every rank owns an independent 2560-column shard (weak scaling over N)
    W = sp.gen_ternary_fixed(K, N, S)
    w = sp.Weights(W, sp.FMT_U16_V256)
    per_copy = w.stream_bytes
    replicas = max(2, -(-int(2.5 * L2_BYTES) // per_copy))
    w.upload(replicas)
    nbytes = algorithmic_bytes(per_copy, M, 1)
    Xh = O.gen_x_i8(M * K, 1)
    xd = torch.from_numpy(Xh).cuda()
    out = torch.zeros(replicas, M * N, dtype=torch.int32, device="cuda")
    calls = args.calls
    st = torch.cuda.Stream()
    nstreams = max(1, args.streams)
    side = [torch.cuda.Stream() for _ in range(nstreams)] if nstreams > 1 else [st]

    def issue_step(stream, lanes=None):
        """`calls` GEMVs.  No call depends on another (as in the reference's timing loop), so they go
        round-robin to `lanes` streams forked from and joined back into `stream`; inside a lane the
        calls are ordered, with programmatic-dependent-launch edges."""
        lanes = side if lanes is None else lanes
        if lanes[0] is not stream:
            fork = torch.cuda.Event()
            fork.record(stream)
            for s in lanes:
                s.wait_event(fork)
        for i in range(calls):
            r = i % replicas
            w.gemv(xd, M, out[r], sp.I8, sp.LAUNCH_PDL, replica=r, stream=lanes[i % len(lanes)].cuda_stream)
        if lanes[0] is not stream:
            for s in lanes:
                join = torch.cuda.Event()
                join.record(s)
                stream.wait_event(join)

    # parity first: a fast wrong kernel is not a result
    with torch.cuda.stream(st):
        issue_step(st)
    st.synchronize()
    want = O.gemv_i8_dense(Xh, W).reshape(-1)
    for r in range(replicas):
        if not np.array_equal(out[r].cpu().numpy(), want):
            raise SystemExit("parity failure on replica %d" % r)

    graph, mode = None, "direct launches"
    if not args.no_graph:
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st, capture_error_mode="thread_local"):
                issue_step(st)
            graph, mode = g, "CUDA graph replay"
        except Exception as e:                      # keep going with plain launches
            mode = "direct launches (graph capture failed: %s)" % str(e).splitlines()[0][:80]
            torch.cuda.synchronize()

    def one_step():
        if graph is not None:
            graph.replay()
        else:
            issue_step(st)

    sampler = ClockSampler(local) if rank == 0 else None
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(st):
        if sampler:
            sampler.start()
        t_load0 = time.time()
        for _ in range(max(3, args.warmup)):
            one_step()
        st.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ev0.record(st)
        for _ in range(args.steps):
            one_step()
        ev1.record(st)
        st.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t_load1 = time.time()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.stop(t_load0, t_load1) if sampler else None

    total_calls = args.steps * calls
    us_per_call = ms * 1e3 / total_calls
    per_gpu = nbytes / (us_per_call * 1e-6) / 1e9
    value = per_gpu * world

    # ---- the same calls on ONE stream: every call then waits for the previous one to finish
    # (what a caller with a true data dependence between calls gets)
    single = None
    if nstreams > 1 and not args.no_graph:
        try:
            g1 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g1, stream=st, capture_error_mode="thread_local"):
                issue_step(st, [st])
            reps = max(4, args.steps // 8)
            with torch.cuda.stream(st):
                for _ in range(3):
                    g1.replay()
                st.synchronize()
                s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s0.record(st)
                for _ in range(reps):
                    g1.replay()
                s1.record(st)
                st.synchronize()
            sus = s0.elapsed_time(s1) * 1e3 / (reps * calls)
            single = {"us_per_call": sus, "GBps": nbytes / sus / 1e3, "steps_timed": reps}
            del g1
        except Exception as e:
            single = {"error": str(e).splitlines()[0][:120]}
            torch.cuda.synchronize()

    # ---- end to end through the host-buffer entry points: every call brings its activations from
    # host memory (copy to the device inside the timed region) and delivers its result to host
    # memory.  The calls are independent, as in the device-timed part, so `e2e_slots` of them are
    # in flight at once (sptmm_gemv_host_async / _wait); `one_at_a_time` is the same through the
    # blocking call.
    e2e_calls = max(64, min(4000, total_calls // 4))
    e2e_slots = max(1, min(16, args.e2e_slots))
    Xh2 = np.ascontiguousarray(Xh.reshape(M, K))
    Chs = [np.empty((M, N), dtype=np.int32) for _ in range(e2e_slots)]
    Ch = np.empty((M, N), dtype=np.int32)
    for i in range(8):
        w.gemv_host(Xh, sp.I8, replica=i % replicas, out=Ch)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_calls // 4):
        w.gemv_host(Xh, sp.I8, replica=i % replicas, out=Ch)
    e2e_sync_us = (time.perf_counter() - t0) / (e2e_calls // 4) * 1e6
    if not np.array_equal(Ch.reshape(-1), want):
        raise SystemExit("parity failure in the host-buffer call")
    # at most one issuing thread per host core this rank can count on
    e2e_threads = max(1, min(e2e_slots, args.e2e_threads, (os.cpu_count() or 1) // world))
    per_thread = e2e_slots // e2e_threads
    e2e_slots = per_thread * e2e_threads
    e2e_calls -= e2e_calls % e2e_threads

    def host_calls(t, n):
        # one host thread, its own slots: issue the next call while earlier ones are in flight
        torch.cuda.set_device(local)          # the current device is per host thread
        # its list of n independent requests goes to the library in one sptmm_gemv_host_batch call
        # (every request still copies its own X in and gets its own result out)
        s0 = t * per_thread
        xa = Xh2.ctypes.data
        ca = [Chs[s0 + j].ctypes.data for j in range(per_thread)]
        w.gemv_host_batch([xa] * n, [ca[i % per_thread] for i in range(n)],
                          [(i * e2e_threads + t) % replicas for i in range(n)], sp.I8, 0, s0, per_thread, M=M)

    def host_round(n):
        if e2e_threads == 1:
            host_calls(0, n)
            return
        th = [threading.Thread(target=host_calls, args=(t, n // e2e_threads)) for t in range(e2e_threads)]
        for x in th:
            x.start()
        for x in th:
            x.join()

    host_round(4 * e2e_slots)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    host_round(e2e_calls)
    e2e_s = time.perf_counter() - t0
    if not all(np.array_equal(c.reshape(-1), want) for c in Chs[:e2e_slots]):
        raise SystemExit("parity failure in the asynchronous host-buffer calls")
    if world > 1:
        t = torch.tensor([e2e_s, e2e_sync_us], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s, e2e_sync_us = float(t[0].item()), float(t[1].item())
    e2e_us = e2e_s / e2e_calls * 1e6
    e2e_value = nbytes / (e2e_us * 1e-6) / 1e9 * world

    # ---- the same GEMVs as one persistent-kernel sequence (sptmm_seq_*): `chain` makes every
    # step wait for the previous one device-wide (a layer stack), `independent` does not
    seq_info = {}
    if not args.no_seq:
        nseq = min(calls, 512)
        for name, dep in (("chain", True), ("independent", False)):
            steps = [{"w": w, "replica": i % replicas, "X": xd, "C": out[i % replicas], "dep": (i - 1 if dep else -1)}
                     for i in range(nseq)]
            seq = sp.Sequence(steps, M=M)
            with torch.cuda.stream(st):
                out.zero_()
                seq.run(st.cuda_stream)
                st.synchronize()
                if seq.status() != 0 or not all(np.array_equal(out[r].cpu().numpy(), want) for r in range(replicas)):
                    raise SystemExit("parity failure in the sequence kernel (%s)" % name)
                for _ in range(3):
                    seq.run(st.cuda_stream)
                st.synchronize()
                reps = max(4, args.steps // 8)
                s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s0.record(st)
                for _ in range(reps):
                    seq.run(st.cuda_stream)
                s1.record(st)
                st.synchronize()
            sus = s0.elapsed_time(s1) * 1e3 / (reps * nseq)
            seq_info[name] = {"us_per_gemv": sus, "GBps": nbytes / sus / 1e3, "steps_per_launch": nseq, "launches_timed": reps}
            seq.close()

    # ---- BitNet-2B-shaped layer stack (30 x {qkv, o, gate|up, down}), one persistent kernel per
    # pass, column-sharded over all ranks with the fused peer-store exchange when world > 1
    stack_info = {}
    if not args.no_stack:
        w.close()                                   # free the GEMV replicas first
        del out
        torch.cuda.empty_cache()
        stack_info = stack_leg(args, sp, O, torch, dist, st, rank, world)

    large_info = large_sweep(args, sp, O, torch, dist, rank, world) if args.large else None

    line = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "us_per_call": us_per_call,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "i8", "data": "synthetic",
            "pct_of_8000GBps": per_gpu / 8000.0 * 100.0,
            "config": CONFIG,
            "detail": {"layout": "native u16 lists (256-entry blocks)", "calls_per_step": calls, "weight_copies": replicas,
                       "l2": "cold: rotating %d weight copies (%.0f MB) > 126 MB L2" % (replicas, replicas * per_copy / 1e6),
                       "launch": mode + ", %d concurrent streams (independent calls, round-robin), programmatic dependent launch inside a stream" % nstreams,
                       "per_rank": "each GPU runs the same independent 2560-column shard"},
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                         "peak_kind": peak_kind, "algorithmic_bytes_per_launch": nbytes, "traffic": NCU_TRAFFIC_BYTES,
                         "traffic_source": "ncu capture of this kernel on this workload (two launches); a constant here, not measured by this run",
                         "single_stream_frac": (single["GBps"] / peak) if single and "GBps" in single else None},
            "e2e": {"value": e2e_value, "unit": "GB/s", "us_per_call": e2e_us,
                    "h2d_bytes_per_step": M * K * calls, "d2h_bytes_per_step": M * N * 4 * calls,
                    "calls_timed": e2e_calls, "calls_in_flight": e2e_slots, "host_threads": e2e_threads,
                    "one_at_a_time_us_per_call": e2e_sync_us,
                    "how": "sptmm_gemv_host_batch (a list of independent calls, each through sptmm_gemv_host_async/_wait) from host_threads threads: host X -> pinned -> device copy, kernel storing C into mapped pinned host memory, stream poll, copy out"},
            "single_stream": single,
            "sequence": seq_info,
            "stack": stack_info,
            "gpu_launches": total_calls,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"], _ = cpu_baseline()
        if world == 1 and not args.no_reference_gpu:
            torch.cuda.synchronize()
            line["reference_gpu"] = reference_gpu_leg()
        if args.extra:
            line["extra"] = extra_workloads(sp, O, torch, st)
        if large_info is not None:
            line["large"] = large_info
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()



README_COMMANDS = [          # the reference's README.md:23-27 (cu_blas is broken as shipped: it passes a null W)
    ("rcr", ["-row_split3_small", "32", "-M=1", "-K=6912", "-N=2560", "-S=4096"]),
    ("rcr", ["-row_split3_small", "32", "-M=4", "-K=6912", "-N=2560", "-S=4096"]),
    ("rcr", ["-row_split_delta2", "32", "-M=1", "-K=6912", "-N=2560", "-S=4096"]),
    ("rcr", ["-i2s", "-M=1", "-K=6912", "-N=2560", "-S=4096"]),       # M=1 only: the reference's M>1 launch writes out of bounds when K>N
]


def reference_gpu_leg(iters: int = 20000):
    """Not part of the timed metric: where the reference's own GPU program was built beside the
    oracle, run its README commands (launch + device synchronise per iteration, its own protocol)
    and this library's drop-in for the same commands, alternately, and record both ms/iter."""
    harness = os.path.join(ROOT, "oracle", "_ref", "ref_harness")
    ours = os.path.join(ROOT, "sptmm_b200", "bin")
    if not os.path.exists(harness):
        return {"unavailable": "the reference program is not built here"}

    def last_number(cmd):
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=180)
        except (OSError, subprocess.TimeoutExpired) as e:
            return None, str(e)[:100]
        lines = [l.strip() for l in r.stdout.splitlines() if l.strip()]
        try:
            return float(lines[-1]), None
        except (IndexError, ValueError):
            return None, ("rc %d: " % r.returncode) + (r.stdout + r.stderr)[-120:]

    rows = []
    for prog, flags in README_COMMANDS:
        flags = flags + ["-iter=%d" % iters]
        row = {"command": prog + " " + " ".join(flags), "protocol": "launch + device synchronise per iteration, weights stay in L2"}
        ref, ours_t = [], []
        for _ in range(3):                                        # alternate, keep the best of three
            v, err = last_number([harness, "readme"] + flags)
            if v is None:
                row["reference_error"] = err
                break
            ref.append(v)
            v, err = last_number([os.path.join(ours, prog)] + flags)
            if v is None:
                row["ours_error"] = err
                break
            ours_t.append(v)
        if ref:
            row["reference_us_per_iter"] = min(ref) * 1e3
        if ours_t:
            row["ours_us_per_iter"] = min(ours_t) * 1e3
        rows.append(row)
    return {"rows": rows, "iterations": iters}


def stack_leg(args, sp, O, torch, dist, st, rank, world):
    """The 30-layer stack at M = 1, 4, 16: one persistent kernel per pass, every matrix sharded by
    columns over the ranks (fused exchange).  With several ranks also, per M: a parity pass against
    the single-GPU stack on the same input (every rank, the last layer's four buffers, bit for bit
    -- a mismatch ends the run), the same GPUs as independent replicas, and the NCCL variant
    (per-call kernels + ncclAllGather + quantiser kernel in one CUDA graph)."""
    from sptmm_b200 import stack as SM
    shape = (args.stack_layers, 2560, 6912, 640)
    wts = SM.StackWeights(*shape, p_zero=1 / 3, seed=0, rank=rank, world=world)
    wts1 = wts if world == 1 else SM.StackWeights(*shape, p_zero=1 / 3, seed=0, rank=0, world=1)
    passes = 20
    names = ("qkv", "o", "gu", "down")
    info = {}

    def timed(forward, sync_ranks=True):
        with torch.cuda.stream(st):
            for _ in range(3):
                if world > 1 and sync_ranks:
                    dist.barrier()
                forward()
                st.synchronize()
            if world > 1:
                dist.barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record(st)
            for _ in range(passes):
                forward()
            s1.record(st)
            st.synchronize()
        ms = s0.elapsed_time(s1) / passes
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms * 1e3

    def all_ranks(flag: bool) -> bool:
        if world == 1:
            return flag
        t = torch.tensor([0.0 if flag else 1.0], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) == 0.0

    for m_rows in (1, 4, 16):
        x = O.gen_x_i8(m_rows * 2560, 5).reshape(m_rows, 2560)
        stk = SM.TernaryStack(*shape, M=m_rows, rank=rank, world=world, weights=wts, settled=True if args.stack_settled else None,
                              tagged=True if args.stack_tagged else None,
                              exchange=SM.SETTLED_HALVES if (args.stack_halves and m_rows % 2 == 0) else None)
        stk.set_input(x)
        us = timed(lambda: stk.forward(st.cuda_stream))
        ok = all_ranks(stk.status() == 0)
        total_bytes = float(stk.stream_bytes)
        if world > 1:
            tb = torch.tensor([total_bytes], dtype=torch.float64, device="cuda")
            dist.all_reduce(tb)
            total_bytes = float(tb.item())
        entry = {"us_per_pass": us, "tokens_per_s": m_rows / (us * 1e-6), "encoded_GB": total_bytes / 1e9,
                 "GBps_all_gpus": total_bytes / (us * 1e-6) / 1e9, "status_ok": ok, "layers": args.stack_layers,
                 "steps_per_pass": stk.n_steps,
                 "exchange": {1: "step counters", 2: "tagged words polled by every reader", 3: "step counters + row maxima",
                              4: "producer-side quantiser", 5: "settled (one watcher per word, local counters)",
                              6: "settled, two half-batches with alternating steps"}.get(stk.exchange, str(stk.exchange))}
        info["M%d" % m_rows] = entry
        # the same weights as launch-per-matmul: per-call kernels + (NCCL all-gather) + quantiser kernel, one CUDA graph per pass
        ns = SM.NcclStack(wts, M=m_rows)
        ns.set_input(x)
        with torch.cuda.stream(st):
            nccl_us = timed(ns.forward)
        nccl_out = ns.result()
        if world > 1:
            # ---- parity, visible in this record: the 1-GPU stack on the SAME input
            rep = SM.TernaryStack(*shape, M=m_rows, rank=0, world=1, weights=wts1)
            rep.set_input(x)
            with torch.cuda.stream(st):
                dist.barrier()
                stk.forward(st.cuda_stream)
                rep.forward(st.cuda_stream)
                st.synchronize()
                dist.barrier()
            same = all(np.array_equal(stk.buffer(n), rep.buffer(n)) for n in names) and stk.status() == 0 and rep.status() == 0
            if not all_ranks(same):
                raise SystemExit("parity failure: the sharded stack (M=%d, %d GPUs) differs from the single-GPU stack" % (m_rows, world))
            entry["parity"] = "bit-exact vs 1 GPU: qkv, o, gu, down of the last layer, on every rank"
            if not all_ranks(np.array_equal(nccl_out, rep.buffer("down"))):
                raise SystemExit("parity failure: the NCCL stack (M=%d, %d GPUs) differs from the single-GPU stack" % (m_rows, world))
            # ---- the same hardware used as replicas: every rank runs the whole stack on its own M rows
            rep.set_input(O.gen_x_i8(m_rows * 2560, 5 + rank).reshape(m_rows, 2560))
            rus = timed(lambda: rep.forward(st.cuda_stream), sync_ranks=False)
            entry["replicas"] = {"us_per_pass": rus, "tokens_per_s_all_gpus": world * m_rows / (rus * 1e-6), "status_ok": all_ranks(rep.status() == 0)}
            entry["sharded_speedup"] = rus / us
            entry["nccl"] = {"us_per_pass": nccl_us, "sharded_speedup": rus / nccl_us, "parity": "bit-exact vs 1 GPU (final output)",
                             "how": "per step: sptmm_gemv on the rank's columns, ncclAllGather of the int32 results, sptmm_quantize_absmax; one CUDA graph per pass"}
            del rep
        else:
            same = np.array_equal(nccl_out, stk.buffer("down"))
            if not same:
                raise SystemExit("parity failure: launch-per-matmul stack (M=%d) differs from the persistent kernel" % m_rows)
            entry["launch_per_matmul"] = {"us_per_pass": nccl_us, "parity": "bit-exact vs the persistent kernel (final output)",
                                          "how": "per step: sptmm_gemv + sptmm_quantize_absmax; one CUDA graph per pass"}
        del stk, ns
        torch.cuda.empty_cache()
    return info

def extra_workloads(sp, O, torch, st, nstreams=4):
    """The same matrix at M=1/4/16 (int8, fp16) in the native format, the reference layouts and the
    i2s comparator: us/call, cold L2 (rotating weight copies), timed like the headline -- 256
    independent calls per CUDA graph over `nstreams` streams (`us_per_call`) and on one stream
    (`us_single_stream`)."""
    res = {}
    W = sp.gen_ternary_fixed(K, N, S)
    rng = np.random.default_rng(2)
    side = [torch.cuda.Stream() for _ in range(nstreams)]
    ncalls = 256

    def timeit(call, lanes, n=12):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st, capture_error_mode="thread_local"):
            if lanes[0] is not st:
                fork = torch.cuda.Event()
                fork.record(st)
                for s in lanes:
                    s.wait_event(fork)
            for i in range(ncalls):
                call(i, lanes[i % len(lanes)])
            if lanes[0] is not st:
                for s in lanes:
                    join = torch.cuda.Event()
                    join.record(s)
                    st.wait_event(join)
        with torch.cuda.stream(st):
            for _ in range(3):
                g.replay()
            st.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            for _ in range(n):
                g.replay()
            e1.record(st)
            st.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (n * ncalls)

    def cold_replicas(w):
        r = max(2, -(-int(2.5 * L2_BYTES) // max(1, w.stream_bytes)))
        return min(r, 160)

    cases = [("u16_v256", sp.FMT_U16_V256, 32, 0), ("delta_lane", sp.FMT_DELTA_LANE, 32, 0), ("u16_div32", sp.FMT_U16_DIV, 32, S),
             ("delta_div256", sp.FMT_DELTA_DIV256, 32, S), ("i2s", sp.FMT_I2S, 0, 0)]
    for name, fmt, split, s_arg in cases:
        w = sp.Weights(W, fmt, split=split, S=s_arg)
        reps = cold_replicas(w)
        w.upload(reps)
        for m, dt in ((1, sp.I8), (4, sp.I8), (4, sp.F16), (16, sp.I8)):
            if fmt == sp.FMT_I2S and dt != sp.I8:
                continue
            if dt == sp.I8:
                x = torch.from_numpy(O.gen_x_i8(m * K, 1)).cuda()
                o = torch.zeros(nstreams, m * N, dtype=torch.int32, device="cuda")
            else:
                x = torch.from_numpy(rng.standard_normal((m, K)).astype(np.float16)).cuda()
                o = torch.zeros(nstreams, m * N, dtype=torch.float32, device="cuda")
            def call(i, stream):
                w.gemv(x, m, o[i % nstreams], dt, sp.LAUNCH_PDL, replica=i % reps, stream=stream.cuda_stream)
            us = timeit(call, side)
            us1 = timeit(call, [st])
            nb = algorithmic_bytes(w.stream_bytes, m, 1 if dt == sp.I8 else 2)
            res["%s_M%d_%s" % (name, m, "i8" if dt == sp.I8 else "f16")] = {
                "us_per_call": us, "GBps": nb / us / 1e3, "us_single_stream": us1, "bytes": nb, "copies": reps}
        w.close()

    # the delta layout's sparsity sweep: P(0) = 0.33 / 0.5 / 0.75 as fixed counts S = 4608 / 3456 / 1728
    # per column (the reference generator), M=1 int8, beside the native u16 format on the same matrix
    x = torch.from_numpy(O.gen_x_i8(K, 1)).cuda()
    o = torch.zeros(nstreams, N, dtype=torch.int32, device="cuda")
    for s_sweep in (4608, 3456, 1728):
        Ws = sp.gen_ternary_fixed(K, N, s_sweep)
        for name, fmt, s_arg in (("delta_lane", sp.FMT_DELTA_LANE, 0), ("delta_div256", sp.FMT_DELTA_DIV256, s_sweep),
                                 ("u16_v256", sp.FMT_U16_V256, 0)):
            w = sp.Weights(Ws, fmt, split=32, S=s_arg)
            reps = cold_replicas(w)
            w.upload(reps)
            def call(i, stream):
                w.gemv(x, 1, o[i % nstreams], sp.I8, sp.LAUNCH_PDL, replica=i % reps, stream=stream.cuda_stream)
            us = timeit(call, side)
            us1 = timeit(call, [st])
            nb = algorithmic_bytes(w.stream_bytes, 1, 1)
            res["%s_S%d_M1_i8" % (name, s_sweep)] = {
                "us_per_call": us, "GBps": nb / us / 1e3, "us_single_stream": us1, "bytes": nb, "copies": reps}
            w.close()
    return res


def large_sweep(args, sp, O, torch, dist, rank, world):
    """Large ternary matrices (P(0)=0.5, fp16 activations, fp32 sums) at M = 1, 8, 64, over all
    ranks two ways: columns sharded (each rank its N/world columns, X replicated, no exchange) and
    K split (each rank its K/world rows; partial sums reduce-scattered -- fused into the kernel's
    epilogue, and through NCCL for comparison).  Times are per matmul, max over ranks; on one
    rank the 2-bit i2s comparator (int8 activations) runs on the same matrix."""
    from sptmm_b200 import splitk as SK
    shapes = [(8192, 28672), (28672, 8192), (16384, 53248)] if args.large == "all" else [(8192, 28672)]
    res = {}
    st = torch.cuda.current_stream()

    def timed(fn, n=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(n):
            fn()
        e1.record(st)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / n
        if world > 1:
            t = torch.tensor([us], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us = float(t.item())
        return us

    def all_ranks(flag: bool) -> bool:
        if world == 1:
            return flag
        t = torch.tensor([0.0 if flag else 1.0], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) == 0.0

    for Kl, Nl in shapes:
        W = sp.gen_ternary_iid(Kl, Nl, 0.5, 7)
        rng = np.random.default_rng(8)
        key = "%dx%d" % (Kl, Nl)
        res[key] = {}
        c0, c1 = SK.col_range(Nl, rank, world)
        wn = sp.Weights(np.ascontiguousarray(W[c0:c1]), sp.FMT_U16_V256).upload()
        wk = sp.Weights(np.ascontiguousarray(W[c0:c1]), sp.FMT_U16_V256, k_tile=4096).upload()
        k0, k1 = SK.k_range(Kl, rank, world)
        ws = sp.Weights(np.ascontiguousarray(W[:, k0:k1]), sp.FMT_U16_V256).upload()      # this rank's K range, encoded once
        for m in (1, 8, 64):
            X = rng.standard_normal((m, Kl)).astype(np.float16)
            xd = torch.from_numpy(X).cuda()
            # two fp16 results of the same product may differ by the tolerance each has against the
            # exact sum: 1e-3 of the sum of |x| over the row, as in the parity tests
            scale = np.abs(X.astype(np.float64)).sum(axis=1)[:, None]
            out = torch.zeros(m, c1 - c0, dtype=torch.float32, device="cuda")
            entry = {"n_sharded_us": timed(lambda: wn.gemv(xd, m, out, sp.F16, sp.LAUNCH_PDL, stream=st.cuda_stream)),
                     "encoded_MB_per_rank": wn.stream_bytes / 1e6}
            base = out.cpu().numpy().astype(np.float64)
            outk = torch.zeros_like(out)
            entry["n_sharded_k_tiles_4096_us"] = timed(lambda: wk.gemv(xd, m, outk, sp.F16, sp.LAUNCH_PDL, stream=st.cuda_stream))
            mm = SK.SplitKMatmul(W, m, sp.F16, rank, world, weights=ws)
            xs = torch.from_numpy(np.ascontiguousarray(X[:, mm.k0:mm.k1])).cuda()
            entry["split_k_fused_us"] = timed(lambda: mm.forward(xs))
            torch.cuda.synchronize()
            same = (np.abs(outk.cpu().numpy() - base) <= 2e-3 * scale).all() and \
                   (np.abs(mm.out.cpu().numpy() - base) <= 2e-3 * scale).all()
            if world > 1 and Nl % world == 0:
                entry["split_k_nccl_us"] = timed(lambda: mm.forward_nccl(xs))
                torch.cuda.synchronize()
                same = same and (np.abs(mm.rs_out.cpu().numpy() - base) <= 2e-3 * scale).all()
            if not all_ranks(bool(same)):
                raise SystemExit("parity failure in the large sweep (%s, M=%d): K-tiled, split-K and column-sharded results disagree" % (key, m))
            entry["parity"] = "column-sharded, K-tiled and split-K results agree within 2e-3 of sum|x| (fp16), on every rank"
            del mm
            res[key]["M%d" % m] = entry
        wn.close()
        wk.close()
        ws.close()
        if world == 1:
            wi = sp.Weights(W, sp.FMT_I2S).upload()
            for m in (1, 8):
                xi = torch.from_numpy(O.gen_x_i8(m * Kl, 9)).cuda()
                oi = torch.zeros(m * Nl, dtype=torch.int32, device="cuda")
                res[key]["M%d" % m]["i2s_int8_us"] = timed(lambda: wi.gemv(xi, m, oi, sp.I8, stream=st.cuda_stream))
            wi.close()
            wd = torch.from_numpy(W).cuda().to(torch.float16)          # dense K x N, column-major: 2 bytes per weight
            for m in (1, 8, 64):
                xc = torch.from_numpy(np.ascontiguousarray(rng.standard_normal((m, Kl)).astype(np.float16).T)).cuda()
                oc = torch.zeros(Nl, m, dtype=torch.float32, device="cuda")
                res[key]["M%d" % m]["cublas_fp16_dense_us"] = timed(
                    lambda: sp.dense_cublas_gemm_f16(xc, wd, oc, m, Kl, Nl, stream=st.cuda_stream))
            del wd
        del W
    return res


def run_case(args):
    """A short run of ONE configuration, for a profiler to capture: `--case` names it
    (m1_i8, m4_i8, m4_f16, m16_i8: the per-call kernel on the 6912x2560 matrix over rotating weight
    copies; stack_m1, stack_m4, stack_m16: a six-layer stack through the persistent kernel).
    Prints the case and the time per call or pass; nothing here is a bench value."""
    import torch
    import sptmm_b200 as sp
    import oracle_lib as O
    torch.cuda.set_device(0)
    name = args.case
    st = torch.cuda.Stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if name.startswith("stack_m"):
        from sptmm_b200 import stack as SM
        m = int(name[len("stack_m"):])
        stk = SM.TernaryStack(6, 2560, 6912, 640, M=m, p_zero=1 / 3, seed=0)
        stk.set_input(O.gen_x_i8(m * 2560, 5).reshape(m, 2560))
        with torch.cuda.stream(st):
            for _ in range(3):
                stk.forward(st.cuda_stream)
            e0.record(st)
            for _ in range(4):
                stk.forward(st.cuda_stream)
            e1.record(st)
            st.synchronize()
        assert stk.status() == 0
        print(json.dumps({"case": name, "exchange": stk.exchange, "us_per_pass_of_6_layers": e0.elapsed_time(e1) * 1e3 / 4}))
        return
    m, dt = {"m1_i8": (1, sp.I8), "m4_i8": (4, sp.I8), "m4_f16": (4, sp.F16), "m16_i8": (16, sp.I8)}[name]
    W = sp.gen_ternary_fixed(K, N, S)
    w = sp.Weights(W, sp.FMT_U16_V256).upload(16)
    if dt == sp.I8:
        x = torch.from_numpy(O.gen_x_i8(m * K, 1)).cuda()
        out = torch.zeros(4, m * N, dtype=torch.int32, device="cuda")
    else:
        x = torch.from_numpy(np.random.default_rng(2).standard_normal((m, K)).astype(np.float16)).cuda()
        out = torch.zeros(4, m * N, dtype=torch.float32, device="cuda")
    n = 64
    with torch.cuda.stream(st):
        for i in range(16):
            w.gemv(x, m, out[i % 4], dt, sp.LAUNCH_PDL, replica=i % 16, stream=st.cuda_stream)
        e0.record(st)
        for i in range(n):
            w.gemv(x, m, out[i % 4], dt, sp.LAUNCH_PDL, replica=i % 16, stream=st.cuda_stream)
        e1.record(st)
        st.synchronize()
    info = {"case": name, "us_per_call_launch_bound_from_python": e0.elapsed_time(e1) * 1e3 / n, "launches": n + 16}
    # parity of what was just computed: int8 exact; floats against the double-precision product, as a
    # fraction of the sum of |x| over each column's non-zero rows (the tolerance is 1e-3 of that for fp16)
    Wd = W.T.astype(np.float64)
    xh = x.cpu().numpy().reshape(m, K).astype(np.float64)
    got = out[(n - 1) % 4].cpu().numpy().reshape(m, N).astype(np.float64)
    if dt == sp.I8:
        info["mismatches"] = int((got != xh @ Wd).sum())
    else:
        info["max_err_over_sum_abs_x"] = float((np.abs(got - xh @ Wd) / np.maximum(np.abs(xh) @ np.abs(Wd), 1e-30)).max())
    print(json.dumps(info))


def run_timeline(args):
    """Where a step of the 30-layer stack spends its time, from timestamps every CTA records inside
    the persistent kernel (the TUNING build of the library: python sptmm_b200/build.py --tuning).
    For the four steps of layer 25 and every rank: minimum / median / maximum over the CTAs of the
    moments they finished the previous gather, saw their input arrive, passed the local counters,
    had the tile staged and finished the gather, in ns after the rank's LAST CTA finished the
    previous gather.  Works under torchrun (one rank per GPU); not a bench value."""
    os.environ["SPTMM_B200_TUNING"] = "1"
    import torch
    import torch.distributed as dist
    import sptmm_b200 as sp
    import oracle_lib as O
    from sptmm_b200 import stack as SM
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    m = args.timeline
    stk = SM.TernaryStack(30, 2560, 6912, 640, M=m, p_zero=1 / 3, seed=0, rank=rank, world=world,
                          settled=True if args.stack_settled else None, tagged=True if args.stack_tagged else None,
                          exchange=SM.SETTLED_HALVES if args.stack_halves else None)
    stk.set_input(O.gen_x_i8(m * 2560, 5).reshape(m, 2560))
    for _ in range(3):
        if world > 1:
            dist.barrier()
        stk.forward()
        torch.cuda.synchronize()
    assert stk.status() == 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    e0.record()
    for _ in range(10):
        stk.forward()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / 10
    trace = torch.zeros(16384, dtype=torch.int64, device="cuda")
    stk.seq.set_trace(trace)
    if world > 1:
        dist.barrier()
    stk.forward()
    torch.cuda.synchronize()
    stk.seq.set_trace(None)
    t = trace.cpu().numpy()
    G = torch.cuda.get_device_properties(local).multi_processor_count

    def arr(base):
        return t[base:base + 1024].reshape(4, 256)[:, :G].astype(np.int64)

    wait, staged, gathered = arr(2048), arr(3072), arr(4096)
    marks = [arr(5120), arr(6144), arr(7168)]
    lines = ["rank %d of %d, M=%d, exchange %d: %.1f us per pass (%.2f us per step)" % (rank, world, m, stk.exchange, us, us / 120),
             "  step  prev-gather-end | past-wait | input arrived | counter 1 | counter 2 / row loaded | staged | gathered   (min/median/max over %d CTAs, ns)" % G]
    names = ((1, "gu B"), (2, "down A"), (3, "down B")) if stk.exchange == SM.SETTLED_HALVES else ((1, "o"), (2, "gu"), (3, "down"))
    for i, name in names:
        ref = gathered[i - 1].max()

        def q(a):
            if a.max() == 0:
                return "-"
            a = a - ref
            return "%d/%d/%d" % (a.min(), np.median(a), a.max())

        lines.append("  %-6s  %s | %s | %s | %s | %s | %s | %s" % (name, q(gathered[i - 1]), q(wait[i]), q(marks[0][i]), q(marks[1][i]),
                                                                  q(marks[2][i]), q(staged[i]), q(gathered[i])))
    if args.timeline_warps:
        # the consumer warps of two CTAs: start and end of the gather after the CTA's tile was staged, time spent waiting for ring slots
        wv = t[8192:8192 + 512].reshape(2, 4, 16, 4).astype(np.int64)
        for ci, cta in enumerate((0, 100)):
            for i, name in names:
                w = wv[ci, i]
                if w[:, 0].max() == 0:
                    continue
                t0 = staged[i][cta]
                lines.append("  CTA %3d %-6s warps: start %s | end %s | waited for slots %s | slots %s" % (
                    cta, name, " ".join("%d" % (x - t0) for x in w[:, 0]), " ".join("%d" % (x - t0) for x in w[:, 2]),
                    " ".join("%d" % x for x in w[:, 1]), " ".join("%d" % x for x in w[:, 3])))
    for r in range(world):
        if r == rank:
            print("\n".join(lines), flush=True)
        if world > 1:
            dist.barrier()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--calls", type=int, default=1024, help="GEMV calls per step")
    ap.add_argument("--streams", type=int, default=4, help="streams the independent calls of a step are spread over")
    ap.add_argument("--e2e-slots", type=int, default=16, help="host-buffer calls in flight in the e2e measurement (1..16)")
    ap.add_argument("--e2e-threads", type=int, default=4, help="host threads issuing those calls (each owns slots/threads of them)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-seq", action="store_true", help="skip the persistent-sequence measurement")
    ap.add_argument("--no-stack", action="store_true", help="skip the layer-stack measurement")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip running the reference's own GPU program (README commands)")
    ap.add_argument("--stack-layers", type=int, default=30)
    ap.add_argument("--stack-tagged", action="store_true", help="layer stack hands activations on as tagged words (x_kind 2)")
    ap.add_argument("--stack-halves", action="store_true", help="layer stack runs its rows as two interleaved half-batches (pipelined settled exchange)")
    ap.add_argument("--stack-settled", action="store_true", help="layer stack uses the settled exchange (x_kind 5) at every M and GPU count")
    ap.add_argument("--extra", action="store_true", help="also time M=4, the reference layouts and the comparators")
    ap.add_argument("--large", nargs="?", const="one", default=None, choices=["one", "all"],
                    help="also run the large-matrix sweep (column-sharded and split-K over all ranks); 'all' = three shapes")
    ap.add_argument("--case", default=None, choices=["m1_i8", "m4_i8", "m4_f16", "m16_i8", "stack_m1", "stack_m4", "stack_m16"],
                    help="run one configuration briefly (for a profiler) instead of the benchmark")
    ap.add_argument("--timeline", type=int, default=0, metavar="M",
                    help="print the per-step timeline of the 30-layer stack at M rows (needs the tuning build of the library)")
    ap.add_argument("--timeline-warps", action="store_true", help="with --timeline: also the consumer warps of two CTAs (gather start/end, time waiting for ring slots)")
    args = ap.parse_args()
    if args.timeline:
        run_timeline(args)
    elif args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
