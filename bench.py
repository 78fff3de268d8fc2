#!/usr/bin/env python3
"""Benchmark of the IMEX hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload (BASELINE config 5): row-sharded GEMM, bf16
A[65536,8192] . B[8192,8192] -> f32 C with the silu epilogue fused, A split by
rows over the N ranks with the reference's block-partition rule, B resident on
rank 0 and replicated by NCCL broadcast inside the step.  One "step" is one
pass over the whole A (strong scaling: the job is fixed, ranks share it).
`value` is whole-job TFLOP/s with inputs resident in HBM; `e2e` is the same
metric through the C ABI with host buffers (pinned host -> device copies of A
and B and the device -> host copy of C inside the timed region).

At N=1 the line also carries `kernels`: the other BASELINE configs (softmax
4096x1024, GEMM 4096^3 + relu, row reduce 32768x8192, transpose 8192^2) timed
cold (L2 flushed before every launch) with their own roofline fractions, and
`cpu_baseline`: the reference's CPU GEMM timed on a bounded sample.

--impl reference times the reference's own CPU implementation of the path
(its in-tree runner-utils GEMM compiled into oracle/_ref, else the oracle
port) on the host cores, same metric and config.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_TOTAL, N_DIM, K_DIM = 65536, 8192, 8192
SEED_A, SEED_B = 7, 8
METRIC = "bf16 GEMM throughput (row-sharded A[65536,8192].B[8192,8192]->f32, fused silu)"
UNIT = "TFLOP/s"
WORKLOAD = ("config 5: row-sharded linalg.matmul bf16 A[65536,8192].B[8192,8192] -> f32 C, "
            "fused silu, A,B ~ N(0,0.02) rounded to bf16 (seeds 7,8)")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


def ncu_traffic():
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of each kernel, taken
    from ncu captures: a text table `key bytes_read bytes_written` kept with the other profiler
    summaries.  A key without a capture maps to None."""
    table = {}
    path = os.path.join(ROOT, "profiles", "ncu_dram_traffic.txt")
    if os.path.exists(path):
        with open(path) as f:
            for line in f:
                p = line.split("#")[0].split()
                if len(p) >= 3:
                    try:
                        table[p[0]] = float(p[1]) + float(p[2])
                    except ValueError:
                        pass
    return table


NCU_TRAFFIC = ncu_traffic()


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device_index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    p = [x.strip() for x in line.split(",")]
                    if len(p) < 9:
                        continue
                    try:
                        sm.append(float(p[1]))
                        mx.append(float(p[2]))
                    except ValueError:
                        continue
                    for name, v in zip(("hw_slowdown", "hw_thermal_slowdown",
                                        "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                        if v.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)),
                       reasons=sorted(reasons), samples=len(sm))
        return out


# ----------------------------------------------------------------------------
# reference arm / CPU baseline
def cpu_gemm_sample(rows_per_thread, threads, steps, warmup):
    """The reference's CPU GEMM (oracle/_ref: lib/ExecutionEngine/ImexRunnerUtils.cpp
    _mlir_ciface_gemmBF16BF16F32; the oracle port when _ref was not built) on a
    bounded sample of config 5: `threads` independent blocks of `rows_per_thread`
    rows of A against the full B.  Returns (TFLOP/s, seconds per step, kind)."""
    from oracle import oracle
    kind = "reference" if oracle.ref_lib() is not None else "port"
    rng = np.random.default_rng(SEED_B)
    Bm = oracle.to_bf16_bits((rng.standard_normal((K_DIM, N_DIM), dtype=np.float32) * 0.02))
    blocks = []
    for t in range(threads):
        a = np.random.default_rng(SEED_A + t).standard_normal((rows_per_thread, K_DIM),
                                                              dtype=np.float32) * 0.02
        blocks.append(oracle.to_bf16_bits(a))

    def work(t):
        if kind == "reference":
            c = oracle.ref_gemm_x16_f32(blocks[t], Bm, True)
        else:
            c = oracle.matmul_x16_f32(blocks[t], Bm, True, loops=True)
        oracle.silu(c)

    def one_step():
        ths = [threading.Thread(target=work, args=(t,)) for t in range(threads)]
        for th in ths:
            th.start()
        for th in ths:
            th.join()

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    flops = 2.0 * rows_per_thread * threads * N_DIM * K_DIM
    return flops / dt / 1e12, dt, kind


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = min(os.cpu_count() or 1, 32)
    rows = 64
    tf, dt, kind = cpu_gemm_sample(rows, threads, args.steps, min(args.warmup, 1))
    sample = (f"{threads} threads x {rows} rows of A against the full B[8192,8192] per step "
              f"({rows * threads} of 65536 rows), + silu; the reference GEMM is single-threaded, "
              "row blocks are independent so one runs per host thread")
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": tf, "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": sample},
        "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def graph_back_to_back(torch, stream, sess, kernel, ptr_sets, rounds=9):
    """ms per launch of `kernel` when launches follow each other without the host in
    between: one launch per entry of ptr_sets (distinct buffers, together larger than L2, so
    every launch reads cold data) captured into ONE CUDA graph on `stream`, the graph
    replayed `rounds` times with an event pair around each replay.  A Python-side launch
    costs ~10 us of host time, more than these kernels run, so without the graph a loop of
    launches measures the host.  Returns (median ms per launch, min ms per launch)."""
    return graph_replay_ms(torch, stream, sess, [lambda ptrs=ptrs: sess.launch(kernel, ptrs, wait=False)
                                                 for ptrs in ptr_sets], rounds)


def graph_replay_ms(torch, stream, sess, launches, rounds=9):
    """The same timing for any list of enqueue functions (one graph node each)."""
    ptr_sets = launches
    for fn in launches[:2]:
        fn()                                       # everything lazy happens before the capture
    sess.wait()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for fn in launches:
            fn()
    per = []
    for i in range(rounds + 2):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        g.replay()
        b.record(stream)
        b.synchronize()
        if i >= 2:
            per.append(a.elapsed_time(b) / len(ptr_sets))
    return float(np.median(per)), float(np.min(per))


# ----------------------------------------------------------------------------
# single small cases for profiler captures: a few launches, a few GB at most
CASES = {
    "gemm8192_silu": "bf16 GEMM 8192x8192x8192 + silu (the config-5 kernel on 1/8 of the rows)",
    "gemm4096_relu": "bf16 GEMM 4096^3 + relu (config 3)",
    "gemm8192_none": "bf16 GEMM 8192x8192x8192, no epilogue",
    "softmax": "softmax 4096x1024 (config 2)",
    "softmax_big": "softmax 65536x1024 (config-2 kernel on a 512 MiB problem, larger than L2)",
    "softmax_graph": "softmax 4096x1024 (config 2): 16 launches on 16 buffer pairs as one CUDA graph",
    "reduce": "row reduce 32768x8192 (config 4a)",
    "reduce_shard8": "row reduce 4096x8192 (one rank's rows of config 4a at 8 GPUs)",
    "transpose": "transpose 8192x8192 (config 4b)",
    "attention": "attention forward, 4 heads x 4096 keys x d 64, f16 (the reference test's shape)",
    "loop_fusion": "fused elementwise chain (log, absf, addf, subf) on 8192x8192 f32",
    "loop_fusion_f16": "the same chain on 8192x8192 f16 (packed 16-bit arithmetic)",
    "loop_fusion_bf16": "the same chain on 8192x8192 bf16 (packed 16-bit arithmetic)",
}


def run_case(name, iters):
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    B = pkg.blob
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    sess = pkg.Session(device=0, adopt_stream=stream.cuda_stream)
    if name.startswith("gemm"):
        n = 8192 if name.startswith("gemm8192") else 4096
        epi = {"silu": B.EPI_SILU, "relu": B.EPI_RELU, "none": B.EPI_NONE}[name.split("_")[1]]
        A = torch.empty((n, n), dtype=torch.bfloat16, device=dev)
        Bm = torch.empty((n, n), dtype=torch.bfloat16, device=dev)
        Cm = torch.empty((n, n), dtype=torch.float32, device=dev)
        sess.run(B.fill_normal("fa", n * n, B.BF16, SEED_A, 0.0, 0.02), [A.data_ptr()])
        sess.run(B.fill_normal("fb", n * n, B.BF16, SEED_B, 0.0, 0.02), [Bm.data_ptr()])
        k, ptrs = sess.kernel(B.gemm(name, n, n, n, B.BF16, epi)), [A.data_ptr(), Bm.data_ptr(), Cm.data_ptr()]
        work, unit = 2.0 * n ** 3 / 1e12, "TFLOP/s"
    elif name == "softmax_graph":
        pairs = [(torch.empty((4096, 1024), dtype=torch.float32, device=dev).normal_(0.0, 3.0),
                  torch.empty((4096, 1024), dtype=torch.float32, device=dev)) for _ in range(16)]
        k = sess.kernel(B.softmax(name, 4096, 1024))
        med, mn = graph_back_to_back(torch, stream, sess, k, [[a.data_ptr(), b.data_ptr()] for a, b in pairs],
                                     rounds=max(iters, 5))
        nbytes = 2 * 4096 * 1024 * 4
        print(json.dumps({"case": name, "what": CASES[name], "ms_per_launch_median": med, "ms_per_launch_min": mn,
                          "gbs_median": nbytes / (med * 1e-3) / 1e9, "gbs_best": nbytes / (mn * 1e-3) / 1e9}), flush=True)
        sess.close()
        return
    elif name.startswith("softmax"):
        rows = 65536 if name == "softmax_big" else 4096
        X = torch.empty((rows, 1024), dtype=torch.float32, device=dev).normal_(0.0, 3.0)
        Y = torch.empty_like(X)
        k, ptrs = sess.kernel(B.softmax(name, rows, 1024)), [X.data_ptr(), Y.data_ptr()]
        work, unit = 2 * X.numel() * 4 / 1e9, "GB/s"
    elif name == "attention":
        heads, n_ctx = 4, 4096
        Q, Kt, Vt = [(torch.rand((heads * n_ctx, 64), device=dev) * 2 - 1).to(torch.float16) for _ in range(3)]
        Ot = torch.empty_like(Q)
        k = sess.kernel(B.attention_fwd(name, heads, n_ctx, 64, B.F16, 0.5))
        ptrs = [Q.data_ptr(), Kt.data_ptr(), Vt.data_ptr(), Ot.data_ptr()]
        work, unit = 4.0 * heads * n_ctx * n_ctx * 64 / 1e12, "TFLOP/s"
    elif name.startswith("loop_fusion"):
        tdt, bdt = {"loop_fusion": (torch.float32, B.F32), "loop_fusion_f16": (torch.float16, B.F16),
                    "loop_fusion_bf16": (torch.bfloat16, B.BF16)}[name]
        X = torch.empty((8192, 8192), dtype=tdt, device=dev).uniform_(0.5, 4.0)
        X1 = torch.empty((8192, 8192), dtype=tdt, device=dev).uniform_(-2.0, 2.0)
        Y = torch.empty_like(X)
        k = sess.kernel(B.expr(name, 8192, 8192, "in0 log in1 abs add in0 sub", bdt))
        ptrs = [X.data_ptr(), X1.data_ptr(), Y.data_ptr()]
        work, unit = 3 * X.numel() * X.element_size() / 1e9, "GB/s"
    elif name.startswith("reduce"):
        nrows = 32768 if name == "reduce" else 4096
        X = torch.empty((nrows, 8192), dtype=torch.float32, device=dev).uniform_(0.0, 1.0)
        Y = torch.empty(nrows, dtype=torch.float32, device=dev)
        k, ptrs = sess.kernel(B.reduce_rows(name, nrows, 8192)), [X.data_ptr(), Y.data_ptr()]
        work, unit = (X.numel() + Y.numel()) * 4 / 1e9, "GB/s"
    else:
        X = torch.empty((8192, 8192), dtype=torch.float32, device=dev).uniform_(-1.0, 1.0)
        Y = torch.empty_like(X)
        k, ptrs = sess.kernel(B.transpose2d(name, 8192, 8192)), [X.data_ptr(), Y.data_ptr()]
        work, unit = 2 * X.numel() * 4 / 1e9, "GB/s"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ms = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        sess.launch(k, ptrs, wait=False)
        b.record()
        b.synchronize()
        ms.append(a.elapsed_time(b))
    sess.wait()
    print(json.dumps({"case": name, "what": CASES[name], "ms": ms,
                      "best": work / (min(ms) * 1e-3), "unit": unit}), flush=True)
    sess.close()


# ----------------------------------------------------------------------------
# our arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel section")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-gather", action="store_true", help="N>1: skip the optional all-gather of C")
    ap.add_argument("--rows", type=int, default=M_TOTAL, help="total rows of A (small runs)")
    ap.add_argument("--e2e-chunks", type=int, default=16, help="row chunks of the host-buffer pipeline")
    ap.add_argument("--e2e-full-b", action="store_true",
                    help="N>1: every rank uploads all of B itself (default: 1/N each, the rest over NVLink)")
    ap.add_argument("--sm-margin", type=int, default=None,
                    help="SMs the GEMM leaves to the NCCL broadcast when N > 1")
    ap.add_argument("--timeline", type=int, default=0,
                    help="N>1: after the timed region run this many more steps with timing events around "
                         "every broadcast and every step's GEMM launches and report the intervals")
    ap.add_argument("--comm-ms", type=float, default=0.5,
                    help="N>1, --overlap calls: how long the first GEMM launch (NCCL beside it) should last")
    ap.add_argument("--overlap", default=os.environ.get("IMEX_BENCH_OVERLAP", "ce"),
                    choices=["slabs", "calls", "ce"],
                    help="N>1: hide the replication of B inside a call (column slabs) or across calls")
    ap.add_argument("--case", default=None, choices=sorted(CASES),
                    help="run ONE small kernel case --iters times and exit (ncu captures)")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--repeats", type=int, default=5,
                    help="how many times the K-step region runs in all (the first one gives `value`)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.case:
        run_case(args.case, args.iters)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()  # raises when the CUDA library is missing: no fallback
    rt, B = pkg.runtime, pkg.blob

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    peaks = measured_peaks()
    M_total = args.rows
    rows = rt.imexShardSize(rank, world, M_total)
    row0 = rt.imexShardOffset(rank, world, M_total)

    # torch owns the device buffers and the stream; the session adopts the stream so
    # that NCCL, torch events and the library's launches are ordered on one stream
    stream = torch.cuda.Stream(device=dev)  # a real handle: the default stream's is NULL
    torch.cuda.set_stream(stream)
    sess = pkg.Session(device=local_rank, adopt_stream=stream.cuda_stream)
    assert rt.imexStreamNative(sess.stream) == stream.cuda_stream
    A = torch.empty((rows, K_DIM), dtype=torch.bfloat16, device=dev)
    Bm = torch.empty((K_DIM, N_DIM), dtype=torch.bfloat16, device=dev)
    Cm = torch.empty((rows, N_DIM), dtype=torch.float32, device=dev)
    sess.run(B.fill_normal("fill_a", rows * K_DIM, B.BF16, SEED_A, 0.0, 0.02, first=row0 * K_DIM),
             [A.data_ptr()])
    if rank == 0:
        sess.run(B.fill_normal("fill_b", K_DIM * N_DIM, B.BF16, SEED_B, 0.0, 0.02), [Bm.data_ptr()])
    epi = {"silu": B.EPI_SILU, "relu": B.EPI_RELU, "none": B.EPI_NONE}[
        os.environ.get("IMEX_BENCH_EPILOGUE", "silu")]  # experiments only; the metric is silu
    from mlir_extensions_b200.dist import RowShardedGemm
    gemm = RowShardedGemm(sess, rank, world, M_total, N_DIM, K_DIM, B.BF16, epi, src=0,
                          sm_margin=args.sm_margin, device=dev, overlap=args.overlap, comm_ms=args.comm_ms)
    assert (gemm.row0, gemm.rows) == (row0, rows)
    if world > 1 and args.overlap == "ce":
        gemm.register_b(Bm)  # B enters the copy-engine replication once; every step replicates it again

    def step():
        # world > 1: B lives on rank 0; its column slabs are NCCL-broadcast on a side
        # stream and land in local HBM, each slab's GEMM starts when its slab is in
        return gemm(A, Bm, Cm, b_ready=True)  # B is resident on rank 0 before the step

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # samples cover warm-up + timed region (same work, back to back)
        time.sleep(0.05)
    for _ in range(args.warmup):
        step()
    barrier()
    launches0 = rt.imexLaunchCount()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k_events = []
    barrier()
    e0.record()
    for _ in range(args.steps):
        if world == 1:
            ka, kb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ka.record()
            step()
            kb.record()
            k_events.append((ka, kb))
        else:
            step()
    e1.record()
    barrier()
    sess.wait()
    gemm.check()
    launches = rt.imexLaunchCount() - launches0
    gemm_kernel_name = sess.last_kernel()
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    ms_per_step = total_ms / args.steps
    # the same K-step region again, a few times: how much one region's figure moves (short
    # regions do not reach the power cap, long ones do); `value` stays the first region's
    region_ms = [ms_per_step]
    for _ in range(max(0, args.repeats - 1)):
        barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(args.steps):
            step()
        r1.record()
        barrier()
        region_ms.append(max_over_ranks(r0.elapsed_time(r1)) / args.steps)
    sess.wait()
    clocks = sampler.stop() if rank == 0 else None
    if world == 1:
        kernel_ms = float(np.mean([a.elapsed_time(b) for a, b in k_events]))
    else:
        # the GEMM launches of one step, timed alone (B already replicated), max over ranks
        barrier()
        ka, kb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ka.record()
        gemm.launch_gemms(A, Cm)
        kb.record()
        kb.synchronize()
        kernel_ms = max_over_ranks(ka.elapsed_time(kb))
    flops_job = 2.0 * M_total * N_DIM * K_DIM
    value = flops_job / (ms_per_step * 1e-3) / 1e12

    # optional: when does each broadcast run relative to the GEMMs (ms since the first event)
    timeline = None
    if world > 1 and args.timeline > 0 and args.overlap in ("calls", "slabs"):
        barrier()
        base = torch.cuda.Event(enable_timing=True)
        base.record()
        gemm.trace = []
        for _ in range(args.timeline):
            step()
        torch.cuda.synchronize()
        mine = [{"step": i, "broadcast": [base.elapsed_time(e[0]), base.elapsed_time(e[1])],
                 "gemm": [base.elapsed_time(e[2]), base.elapsed_time(e[3])]} for i, e in enumerate(gemm.trace)]
        gemm.trace = None
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        timeline = {"rank0": gathered[0], "rank%d" % (world - 1): gathered[-1],
                    "note": "each rank's own clock; broadcast[0] = the moment it may start"}

    # optional last step, outside the timed region and reported on its own: every rank
    # gets all rows of C (NCCL all-gather of the row shards)
    gather = None
    if world > 1 and not args.no_gather:
        from mlir_extensions_b200.dist import all_gather_rows
        c_full = torch.empty((M_total, N_DIM), dtype=torch.float32, device=dev)
        ms_list = []
        for i in range(4):
            barrier()
            ga, gb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ga.record()
            all_gather_rows(Cm, c_full, rank, world, M_total)
            gb.record()
            gb.synchronize()
            if i:
                ms_list.append(max_over_ranks(ga.elapsed_time(gb)))
        same = bool(torch.equal(c_full[row0:row0 + rows], Cm))
        g_ms = float(np.median(ms_list))
        recv = (M_total - rows) * N_DIM * 4
        gather = {"ms": g_ms, "bytes_received_per_rank": recv, "gbs_per_rank": recv / (g_ms * 1e-3) / 1e9,
                  "own_block_intact": same, "note": "NCCL all-gather of the f32 row shards of C, not in ms_per_step"}
        del c_full

    # parity guard (enforced): rows of this rank's shard against the CPU oracle: the first
    # and the last row, one row of the last 256-row block (where a k-split tail lands) and
    # random ones; at N > 1 the whole shard against ONE plain launch over the same rows
    from oracle import oracle
    rng = np.random.default_rng(rank)
    fixed = {0, rows - 1, max(0, rows - 1 - int(rng.integers(0, min(256, rows))))}
    extra = rng.choice(rows, size=min(8, rows), replace=False)
    sample_rows = np.array(sorted(fixed | set(int(r) for r in extra)))
    a_bits = A[torch.as_tensor(sample_rows, device=dev)].view(torch.int16).cpu().numpy().view(np.uint16)
    if world > 1:
        dist.broadcast(Bm, src=0)  # only for this check: non-root ranks hold B as slabs
    b_bits = Bm.view(torch.int16).cpu().numpy().view(np.uint16)
    got = Cm[torch.as_tensor(sample_rows, device=dev)].cpu().numpy()
    ref = oracle.silu(oracle.matmul_x16_f32(a_bits, b_bits, True))
    frob_local = oracle.rel_frobenius(got, ref)
    frob = max_over_ranks(frob_local if np.isfinite(frob_local) else 1e30)
    shard_check = None
    if world > 1:
        plain = sess.kernel(B.gemm("whole_shard_one_launch", rows, N_DIM, K_DIM, B.BF16, epi))
        C_one = torch.empty_like(Cm)
        sess.launch(plain, [A.data_ptr(), Bm.data_ptr(), C_one.data_ptr()])
        diff = (Cm - C_one).abs().max().item()
        scale = C_one.abs().max().item()
        shard_check = {"max_abs_diff_vs_one_launch": max_over_ranks(diff), "max_abs": max_over_ranks(scale),
                       "bitwise_equal": bool(max_over_ranks(0.0 if torch.equal(Cm, C_one) else 1.0) == 0.0),
                       "tolerance": "max abs diff <= 1e-5 x max abs (k-split tails sum in another order)"}
        del C_one
        if not (shard_check["max_abs_diff_vs_one_launch"] <= 1e-5 * shard_check["max_abs"]):
            frob = 1e30  # every rank holds the same maxima, so every rank takes this branch
    if not (frob <= 1e-3):
        print("bench.py: PARITY FAILURE on rank %d: rel. Frobenius of sampled rows %.3e (this rank), "
              "worst rank %.3e, shard check %s; tolerance 1e-3" % (rank, frob_local, frob, shard_check),
              file=sys.stderr, flush=True)
        sess.close()
        if world > 1:
            dist.destroy_process_group()
        sys.exit(3)

    # ---- end to end through the C ABI with host buffers ----------------------
    e2e = None
    if not args.no_e2e:
        e2e_steps = max(1, min(args.steps, 3))
        hA = torch.empty((rows, K_DIM), dtype=torch.bfloat16, pin_memory=True)
        hB = torch.empty((K_DIM, N_DIM), dtype=torch.bfloat16, pin_memory=True)
        hC = torch.empty((rows, N_DIM), dtype=torch.float32, pin_memory=True)
        hA.copy_(A)
        hB.copy_(Bm)
        # the public host-buffer call: rows of A in chunks, three host threads (upload /
        # launch+wait / download), every transfer a blocking gpuMemCopy through the C ABI
        from mlir_extensions_b200.pipeline import HostPipelinedGemm
        b_gather, gsess = None, None
        if world > 1 and not args.e2e_full_b:
            # the ranks share the upload of B: each sends its own block of rows over PCIe and
            # fetches the other blocks from its peers over NVLink (copy engines)
            from mlir_extensions_b200.dist import PeerAllGather
            gsess = pkg.Session(device=local_rank)
            b_gather = PeerAllGather(gsess, rank, world, K_DIM, N_DIM * 2)
        own = HostPipelinedGemm(local_rank, rows, N_DIM, K_DIM, B.BF16, B.EPI_SILU, chunks=args.e2e_chunks,
                                b_gather=b_gather)

        def e2e_step():
            own(hA.data_ptr(), hB.data_ptr(), hC.data_ptr())

        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / e2e_steps
        # same products, but the two runs cut the work into different launches, and a k-split tile
        # sums its parts in another order than a whole one: equal to the last bits, not bit for bit
        assert torch.allclose(hC[:64], Cm[:64].cpu(), rtol=1e-4, atol=1e-6), \
            "e2e result differs from the resident run"
        b_up = b_gather.own_block()[1] if b_gather is not None else hB.numel() * 2
        h2d, d2h = int(hA.numel() * 2 + b_up), int(hC.numel() * 4)
        e2e = {"value": flops_job / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
               "steps": e2e_steps, "chunks": len(own.bounds),
               "host_link_gbs_per_rank": {"h2d": h2d / (e2e_ms * 1e-3) / 1e9, "d2h": d2h / (e2e_ms * 1e-3) / 1e9},
               "host_link_gbs_node": {"h2d": world * h2d / (e2e_ms * 1e-3) / 1e9,
                                      "d2h": world * d2h / (e2e_ms * 1e-3) / 1e9},
               "note": "per rank; every rank uploads its A shard and " +
                       ("its 1/%d of B (the other rows of B come from the peers over NVLink)" % world
                        if b_gather is not None else "B") +
                       ", downloads its C shard; uploads, GEMMs on row chunks and downloads overlap "
                       "(host threads, blocking gpuMemCopy / gpuLaunchKernel / gpuWait only)"}
        own.close()
        if b_gather is not None:
            barrier()
            b_gather.close()
            barrier()
            gsess.close()
        del hA, hB, hC

    # ---- the other configs, cold-cache, rank 0 -----------------------------------
    kernels = None
    if rank == 0 and world == 1 and not args.no_kernels:
        kernels = bench_kernels(torch, pkg, sess, dev, peaks, stream)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        tf, dt, kind = cpu_gemm_sample(256, 1, 1, 0)
        cpu = {"value": tf, "unit": UNIT, "cores": 1, "kind": kind,
               "sample": "256 of 65536 rows of A against the full B (%.1f s), + silu; the reference's "
                         "CPU GEMM (runner-utils _mlir_ciface_gemmBF16BF16F32) is single-threaded" % dt,
               "host_cores": os.cpu_count()}

    sharded = None
    if world > 1 and not args.no_kernels:
        sharded = bench_sharded_rows(torch, pkg, sess, dev, peaks, rank, world, barrier,
                                     max_over_ranks, stream)

    if rank == 0:
        flops_launch = 2.0 * rows * N_DIM * K_DIM
        achieved = flops_launch / (kernel_ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops"]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_total": M_total, "rows_per_rank": rows,
                       "partition": "block rows, last extent%N shards one longer",
                       "collective": ("none" if world == 1 else
                                      "B replicated from rank 0 inside every step by the copy engines over NVLink "
                                      "(buffers shared over CUDA IPC: each rank pulls its slice from rank 0, a "
                                      "stream-ordered barrier, then the other slices from their holders), beside "
                                      "the previous step's GEMM; one GEMM launch on all SMs, no NCCL kernel"
                                      if gemm.overlap == "ce" else
                                      "NCCL broadcast of B from rank 0 inside every step, " +
                                      ("in column slabs %s overlapped with the slab GEMMs; every GEMM launch "
                                       "leaves %d SMs free" if gemm.overlap == "slabs" else
                                       "as one slab %s into one of two replica buffers, overlapped with the "
                                       "previous step's GEMM, whose first launch leaves %d SMs free and whose "
                                       "second uses all SMs") % ([w for _, w in gemm.slabs], gemm.margin)),
                       "gemm_launch_columns": [int(k_.dims[1]) for k_ in gemm.launch_descs],
                       "l2": "inputs (%d MiB A shard + 128 MiB B) and the %d MiB C shard exceed the 126 MB L2"
                             % (rows * K_DIM * 2 >> 20, rows * N_DIM * 4 >> 20)},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         "traffic": (NCU_TRAFFIC["gemm_cfg5_per_8192_rows"] * rows / 8192.0
                                     if NCU_TRAFFIC.get("gemm_cfg5_per_8192_rows") else None),
                         "traffic_note": "ncu capture on 8192 rows scaled by rows/8192",
                         "kernel": gemm_kernel_name, "kernel_ms": kernel_ms,
                         "launches_per_step": len(gemm.launches),
                         "peak_source": peaks["source"] + " (cuBLAS bf16 burst)",
                         "frac_of_sustained": (achieved / peaks["bf16_tflops_sustained"])
                         if peaks.get("bf16_tflops_sustained") else None,
                         "frac_of_nominal_2250": achieved / 2250.0},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "parity": {"rel_frobenius_sampled_rows": frob, "tolerance": 1e-3, "enforced": True,
                       "rows_checked_per_rank": int(len(sample_rows)), "whole_shard_vs_one_launch": shard_check},
            "cpu_baseline": cpu, "sharded_rows": sharded, "all_gather_c": gather, "timeline": timeline,
            "repeats": {"regions": len(region_ms), "tflops": [flops_job / (m * 1e-3) / 1e12 for m in region_ms],
                        "median": flops_job / (float(np.median(region_ms)) * 1e-3) / 1e12,
                        "min": flops_job / (max(region_ms) * 1e-3) / 1e12,
                        "max": flops_job / (min(region_ms) * 1e-3) / 1e12,
                        "ms_per_step_x_sm_mhz": (ms_per_step * clocks["sm_mhz"]) if clocks and clocks.get("sm_mhz") else None},
            "kernels_detail": kernels,
        }
        # last, and short, so that a reader who keeps only the end of the line still has every
        # kernel's roofline: name -> [achieved, unit, fraction of the measured peak, ms]
        if kernels:
            line["kernels"] = {k: {"achieved": round(v["roofline"]["achieved"], 1), "unit": v["roofline"]["unit"],
                                   "frac": round(v["roofline"]["frac"], 3), "ms": round(v["roofline_ms"], 5),
                                   "bound": v["roofline"]["bound"], "traffic": v["roofline"].get("traffic")}
                               for k, v in kernels.items()}
        print(json.dumps(line), flush=True)
    gemm.close()
    sess.close()
    if world > 1:
        dist.destroy_process_group()


def bench_sharded_rows(torch, pkg, sess, dev, peaks, rank, world, barrier, max_over_ranks, stream,
                       iters=20):
    """Configs 4a and 2 row-sharded over the ranks: no exchange step, every rank
    reduces / normalises its own block of rows; aggregate GB/s = all bytes / max time."""
    B, rt = pkg.blob, pkg.runtime
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    out = {}
    for name, total_rows, cols, make in (
            ("reduce_rows_32768x8192", 32768, 8192, lambda r, c: B.reduce_rows("reduce", r, c)),
            ("softmax_4096x1024", 4096, 1024, lambda r, c: B.softmax("softmax", r, c))):
        rows = rt.imexShardSize(rank, world, total_rows)
        X = torch.empty((rows, cols), dtype=torch.float32, device=dev).uniform_(0.0, 1.0)
        is_reduce = name.startswith("reduce")
        Y = torch.empty(rows if is_reduce else (rows, cols), dtype=torch.float32, device=dev)
        k = sess.kernel(make(rows, cols))
        ms = []
        for i in range(iters + 3):
            barrier()
            flush.zero_()  # the launch queues behind the flush: no idle-GPU launch latency in the timing
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            sess.launch(k, [X.data_ptr(), Y.data_ptr()], wait=False)
            b.record()
            b.synchronize()
            t = max_over_ranks(a.elapsed_time(b))
            if i >= 3:
                ms.append(t)
        nbytes = total_rows * cols * 4 + (total_rows * 4 if is_reduce else total_rows * cols * 4)
        med = float(np.median(ms))
        ach = nbytes / (med * 1e-3) / 1e9
        out[name] = {"value": ach, "unit": "GB/s", "ms_cold_median": med, "n_gpus": world,
                     "rows_per_rank": rows, "algorithmic_bytes": nbytes,
                     "frac_of_measured_hbm_per_gpu": ach / world / peaks["hbm_gbs"],
                     "collective": "none (rows are independent)"}
        # a shard this small is timed mostly by the event pair around one launch: the launch
        # duration proper shows when launches on distinct buffers (together larger than L2)
        # follow each other inside one CUDA graph
        per_set = X.numel() * 4 + Y.numel() * 4
        n_sets = int(min(16, max(2, -(-(512 << 20) // per_set))))
        try:
            sets = [(torch.empty_like(X).uniform_(0.0, 1.0), torch.empty_like(Y)) for _ in range(n_sets)]
            barrier()
            b2b, _ = graph_back_to_back(torch, stream, sess, k, [[a.data_ptr(), b.data_ptr()] for a, b in sets])
            b2b = max_over_ranks(b2b)
            ach2 = nbytes / (b2b * 1e-3) / 1e9
            out[name].update(ms_back_to_back=b2b, value_back_to_back=ach2, buffer_sets=n_sets,
                             frac_of_measured_hbm_per_gpu_back_to_back=ach2 / world / peaks["hbm_gbs"])
            del sets
        except Exception as e:  # noqa: BLE001 - reported, the flushed figure stays
            out[name]["graph_timing_error"] = repr(e)[:200]
        del X, Y
    return out


def bench_kernels(torch, pkg, sess, dev, peaks, stream, iters=30):
    """Configs 2, 3, 4a, 4b on one GPU: every launch preceded by an L2 flush
    (a 512 MiB buffer is overwritten), timed with CUDA events on the launch stream."""
    B = pkg.blob
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    hbm = peaks["hbm_gbs"]
    out = {}

    def timed(kernel, ptrs, cold=True):
        ms = []
        for i in range(iters + 3):
            if cold:
                flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            sess.launch(kernel, ptrs, wait=False)
            b.record()
            b.synchronize()
            if i >= 3:
                ms.append(a.elapsed_time(b))
        return float(np.median(ms)), float(np.min(ms))

    def copy_floor_ms(nbytes):
        """A plain device copy moving the same bytes (read half, write half), timed the same
        way: context for problems too small to reach the streaming rate."""
        n = max(nbytes // 2, 4)
        src = torch.empty(n, dtype=torch.uint8, device=dev)
        dst = torch.empty_like(src)
        ms = []
        for i in range(iters + 3):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            dst.copy_(src)
            b.record()
            b.synchronize()
            if i >= 3:
                ms.append(a.elapsed_time(b))
        return float(np.median(ms))

    def hbm_entry(name, key, nbytes, kernel, ptrs, note, ptr_sets=None, tensor_pairs=None):
        med, mn = timed(kernel, ptrs, cold=True)
        wmed, _ = timed(kernel, ptrs, cold=False)
        ach = nbytes / (med * 1e-3) / 1e9
        floor = copy_floor_ms(nbytes)
        out[name] = {"value": ach, "unit": "GB/s", "ms_cold_median": med, "ms_cold_min": mn,
                     "ms_warm_median": wmed, "algorithmic_bytes": nbytes,
                     "ms_copy_of_same_bytes": floor, "speed_vs_copy_of_same_bytes": floor / med,
                     "roofline": {"bound": "hbm", "achieved": ach, "peak": hbm, "unit": "GB/s",
                                  "frac": ach / hbm, "traffic": NCU_TRAFFIC.get(key),
                                  "peak_source": peaks["source"] + " (copy)",
                                  "frac_of_nominal_8000": ach / 8000.0},
                     "roofline_ms": med, "note": note}
        if ptr_sets:
            # an event pair around ONE launch adds 5-10 us (all of a 32 MiB problem's time, a tenth
            # of a 512 MiB problem's; a plain copy timed that way loses as much); the launch
            # duration proper shows when launches on distinct buffers follow each other inside
            # one CUDA graph, which is also how a streaming peak is measured
            try:
                b2b, b2b_min = graph_back_to_back(torch, stream, sess, kernel, ptr_sets)
            except Exception as e:  # noqa: BLE001 - reported, the flushed figure stays
                out[name]["graph_timing_error"] = repr(e)[:200]
                return
            ach2 = nbytes / (b2b * 1e-3) / 1e9
            out[name].update(ms_back_to_back=b2b, ms_back_to_back_min=b2b_min, gbs_flushed_single_launch=ach,
                             roofline_ms=b2b)
            if tensor_pairs:
                # the yardstick at this size: plain device copies of the same buffers (the same
                # bytes read and written), one graph node each, timed the same way
                try:
                    cp, _ = graph_replay_ms(torch, stream, sess,
                                            [lambda a=a, b=b: b.copy_(a) for a, b in tensor_pairs])
                    out[name].update(ms_copy_back_to_back=cp, speed_vs_copy_back_to_back=cp / b2b)
                except Exception as e:  # noqa: BLE001
                    out[name]["copy_graph_timing_error"] = repr(e)[:200]
            out[name]["roofline"].update(achieved=ach2, frac=ach2 / hbm, frac_of_nominal_8000=ach2 / 8000.0,
                                         timing="%d launches on %d distinct buffer sets (%d MiB in all, larger "
                                                "than L2) replayed as one CUDA graph, one event pair around the "
                                                "replay; the flushed single-launch figure is "
                                                "gbs_flushed_single_launch"
                                                % (len(ptr_sets), len(ptr_sets), len(ptr_sets) * nbytes >> 20))
            out[name]["value"] = ach2

    # config 2: softmax 4096 x 1024
    X = torch.empty((4096, 1024), dtype=torch.float32, device=dev).normal_(0.0, 3.0)
    Y = torch.empty_like(X)
    pairs = [(torch.empty_like(X).normal_(0.0, 3.0), torch.empty_like(X)) for _ in range(16)]
    hbm_entry("softmax_4096x1024", "softmax", 2 * X.numel() * 4,
              sess.kernel(B.softmax("softmax", 4096, 1024)), [X.data_ptr(), Y.data_ptr()],
              "config 2; 32 MiB moved, fits L2: cold = flushed before each launch",
              ptr_sets=[[a.data_ptr(), b.data_ptr()] for a, b in pairs], tensor_pairs=pairs)
    del pairs
    # config 4a: row reduce 32768 x 8192
    R = torch.empty((32768, 8192), dtype=torch.float32, device=dev).uniform_(0.0, 1.0)
    S = torch.empty(32768, dtype=torch.float32, device=dev)
    more = [(torch.empty_like(R).uniform_(0.0, 1.0), torch.empty_like(S)) for _ in range(2)]
    hbm_entry("reduce_rows_32768x8192", "reduce_rows", R.numel() * 4 + S.numel() * 4,
              sess.kernel(B.reduce_rows("reduce", 32768, 8192)), [R.data_ptr(), S.data_ptr()],
              "config 4a", ptr_sets=[[a.data_ptr(), b.data_ptr()] for a, b in more])
    del R, S, more
    # config 4b: transpose 8192 x 8192
    T = torch.empty((8192, 8192), dtype=torch.float32, device=dev).uniform_(-1.0, 1.0)
    U = torch.empty_like(T)
    more = [(torch.empty_like(T).uniform_(-1.0, 1.0), torch.empty_like(U)) for _ in range(3)]
    hbm_entry("transpose_8192x8192", "transpose2d", 2 * T.numel() * 4,
              sess.kernel(B.transpose2d("transpose", 8192, 8192)), [T.data_ptr(), U.data_ptr()],
              "config 4b", ptr_sets=[[a.data_ptr(), b.data_ptr()] for a, b in more], tensor_pairs=more)
    del T, U, more
    # the reference's fusion benchmark chain (log, absf, addf, subf: kLoopFusion), scaled up to
    # 8192 x 8192 so that it streams from HBM; its own 512 x 1024 shape moves 6 MiB
    for tag, tdt, bdt, esz in (("f32", torch.float32, B.F32, 4), ("f16", torch.float16, B.F16, 2),
                               ("bf16", torch.bfloat16, B.BF16, 2)):
        F0 = torch.empty((8192, 8192), dtype=tdt, device=dev).uniform_(0.5, 4.0)
        F1 = torch.empty((8192, 8192), dtype=tdt, device=dev).uniform_(-2.0, 2.0)
        F2 = torch.empty_like(F0)
        hbm_entry("loop_fusion_8192x8192_" + tag, "expr_" + tag, 3 * F0.numel() * esz,
                  sess.kernel(B.expr("loop_fusion", 8192, 8192, "in0 log in1 abs add in0 sub", bdt)),
                  [F0.data_ptr(), F1.data_ptr(), F2.data_ptr()],
                  "four elementwise generics fused into one pass: two reads (x0 is read twice, the "
                  "second time from cache) and one write per element")
        del F0, F1, F2
    # attention forward at the reference test's size: Z*H = 4 heads, 4096 keys, d 64, f16
    heads, n_ctx = 4, 4096
    Q = (torch.rand((heads * n_ctx, 64), device=dev) * 2 - 1).to(torch.float16)
    Kt = (torch.rand((heads * n_ctx, 64), device=dev) * 2 - 1).to(torch.float16)
    Vt = (torch.rand((heads * n_ctx, 64), device=dev) * 2 - 1).to(torch.float16)
    Ot = torch.empty_like(Q)
    ak = sess.kernel(B.attention_fwd("attention", heads, n_ctx, 64, B.F16, 0.5))
    med, mn = timed(ak, [Q.data_ptr(), Kt.data_ptr(), Vt.data_ptr(), Ot.data_ptr()], cold=True)
    aflops = 4.0 * heads * n_ctx * n_ctx * 64
    out["attention_fwd_4x4096x64"] = {
        "value": aflops / (med * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_cold_median": med, "ms_cold_min": mn,
        "algorithmic_flops": aflops, "roofline_ms": med,
        "roofline": {"bound": "tensor", "achieved": aflops / (med * 1e-3) / 1e12, "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": aflops / (med * 1e-3) / 1e12 / peaks["bf16_tflops"], "traffic": None},
        "note": "the reference's flash-attention test shape; 128 CTAs of 128 query rows, 17 GFLOP in all"}

    def tensor_graph_timing(name, kernel, ptr_sets, flops, what):
        """The launch duration proper of a 40-100 us kernel: launches on distinct buffer sets
        (together larger than L2) replayed as one CUDA graph; an event pair around one launch
        adds 5-10 us.  The flushed single-launch figure stays in ms_cold_median."""
        try:
            b2b, b2b_min = graph_back_to_back(torch, stream, sess, kernel, ptr_sets)
        except Exception as e:  # noqa: BLE001 - reported, the flushed figure stays
            out[name]["graph_timing_error"] = repr(e)[:200]
            return
        ach = flops / (b2b * 1e-3) / 1e12
        out[name].update(ms_back_to_back=b2b, ms_back_to_back_min=b2b_min, roofline_ms=b2b,
                         tflops_flushed_single_launch=out[name]["value"], value=ach)
        out[name]["roofline"].update(achieved=ach, frac=ach / peaks["bf16_tflops"], timing=what)

    asets = [[(torch.rand((heads * n_ctx, 64), device=dev) * 2 - 1).to(torch.float16) for _ in range(3)]
             + [torch.empty_like(Q)] for _ in range(32)]
    tensor_graph_timing("attention_fwd_4x4096x64", ak, [[t.data_ptr() for t in ts] for ts in asets], aflops,
                        "32 launches on 32 distinct sets of Q, K, V, O (256 MiB in all) replayed as one CUDA graph")
    del Q, Kt, Vt, Ot, asets
    # config 3: GEMM 4096^3 + relu
    n = 4096
    A = torch.empty((n, n), dtype=torch.bfloat16, device=dev)
    Bm = torch.empty((n, n), dtype=torch.bfloat16, device=dev)
    sess.run(B.fill_uniform("cfg3_a", n * n, B.BF16, 3, -1.0, 1.0), [A.data_ptr()])   # seeds 3, 4: the inputs of
    sess.run(B.fill_uniform("cfg3_b", n * n, B.BF16, 4, -1.0, 1.0), [Bm.data_ptr()])  # the config-3 parity test
    Cm = torch.empty((n, n), dtype=torch.float32, device=dev)
    k = sess.kernel(B.gemm("gemm_relu", n, n, n, B.BF16, B.EPI_RELU))
    med, mn = timed(k, [A.data_ptr(), Bm.data_ptr(), Cm.data_ptr()], cold=True)
    wmed, _ = timed(k, [A.data_ptr(), Bm.data_ptr(), Cm.data_ptr()], cold=False)
    fl = 2.0 * n ** 3
    ach = fl / (med * 1e-3) / 1e12
    out["gemm_4096_relu"] = {
        "value": ach, "unit": "TFLOP/s", "ms_cold_median": med, "ms_cold_min": mn,
        "ms_warm_median": wmed, "algorithmic_flops": fl, "roofline_ms": med,
        "roofline": {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"],
                     "traffic": NCU_TRAFFIC.get("gemm_cfg3"),
                     "peak_source": peaks["source"] + " (cuBLAS bf16 burst)",
                     "frac_of_nominal_2250": ach / 2250.0},
        "note": "config 3"}
    gsets = []
    for i in range(2):   # with the first set: 3 x (32 + 32 + 64 MiB), larger than L2
        a2, b2 = torch.empty_like(A), torch.empty_like(Bm)
        sess.run(B.fill_uniform("cfg3_a%d" % i, n * n, B.BF16, 13 + 2 * i, -1.0, 1.0), [a2.data_ptr()])
        sess.run(B.fill_uniform("cfg3_b%d" % i, n * n, B.BF16, 14 + 2 * i, -1.0, 1.0), [b2.data_ptr()])
        gsets.append((a2, b2, torch.empty_like(Cm)))
    gsets.append((A, Bm, Cm))
    tensor_graph_timing("gemm_4096_relu", k, [[t.data_ptr() for t in ts] for ts in gsets], fl,
                        "3 launches on 3 distinct sets of A, B, C (384 MiB in all) replayed as one CUDA graph")
    out["gemm_4096_relu"]["roofline"]["frac_of_nominal_2250"] = out["gemm_4096_relu"]["value"] / 2250.0
    return out


if __name__ == "__main__":
    main()
