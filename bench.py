#!/usr/bin/env python
"""Benchmark of the int4 GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

One "step" is one int4 GEMM with M = K = 8192 and N = 8192 columns PER GPU: at N GPUs the problem
is C[8192, 8192*N] = A[8192, 8192] * B[8192*N, 8192]^T with B split by output columns, A replicated
and no collective on the data path (weak scaling).  Inputs are seeded synthetic nibbles, uniform on
[-8, 7].  The metric is TOPS = 2*M*N*K / time, whole job.

The line printed by rank 0 carries, beside the base keys:
  roofline      the GEMM kernel against the dense int8 tensor peak (2 x the measured bf16 rate)
  cpu_baseline  the CPU oracle timed on a bounded row slab of the same product (N=1 only)
  e2e           the same metric through the host-buffer C-ABI call, copies included
  clocks        SM clock and throttle reasons sampled during the timed region
  verified      the C that is timed, compared with the CPU oracle before the timed region (full rows + sampled points);
                a mismatch aborts the run without a number (the reference checks before it times, test.py:39-43)
  extra         (1 GPU) further shapes of the target list, each verified and timed in a CUDA graph that rotates its
                buffers past the L2: the decode shapes against the HBM roofline, the M = 2048 prefill shapes and
                32768^3 against the tensor roofline
  sharded_check, large   (2+ GPUs, after the timed region) the column-sharded product with the NCCL gather and with
                the fused peer-store gather checked against the oracle on rank 0, and 32768^3 strong scaling:
                compute only, with NCCL gather, with fused gather

`--impl reference` times the reference's own CPU implementation of the path (its compiled
cpu_gemm_int8 + unpack_int4_matrix where that build exists, else the oracle port) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M = K = 8192
N_PER_GPU = 8192
METRIC = "int4 GEMM TOPS at M=N=K=8192"
UNIT = "TOPS"
INT8_PEAK_NOMINAL_TOPS = 4500.0  # NVIDIA's dense int8 figure for B200
FALLBACK_BF16_TFLOPS = 1590.0    # earlier measurement on this pool, used only if MEASURED_PEAKS.json is absent
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the headline kernel at 8192^3, from an ncu capture of this
# command (`--steps 2 --warmup 3 --no-cpu-baseline --no-e2e --no-extra`, one launch captured): 164.1 MB read + 221.0 MB written
DRAM_TRAFFIC_BYTES_PER_LAUNCH = 385.1e6


def config(n_gpus: int) -> dict:
    return {
        "workload": f"int4 GEMM M={M} K={K}, N={N_PER_GPU} per GPU ({N_PER_GPU * n_gpus} total; B column-sharded, A replicated)",
        "m": M,
        "n_total": N_PER_GPU * n_gpus,
        "k": K,
        "values": "uniform on [-8, 7], seeded",
        "parallelism": f"n-shard x{n_gpus}, no data-path collective",
        "l2": "working set 320 MiB per GPU exceeds the 126 MB L2; the 256 MiB C is rewritten every step",
    }


def measured_peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            bf16 = float(json.load(f)["bf16_tflops"])
        return 2.0 * bf16, "2 x measured bf16_tflops (burst) from MEASURED_PEAKS.json; int8 issues at twice the bf16 rate (of measured)"
    except Exception:
        return 2.0 * FALLBACK_BF16_TFLOPS, "2 x fallback bf16 figure, MEASURED_PEAKS.json absent (of fallback)"


def measured_hbm() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured hbm_gbs (copy) from MEASURED_PEAKS.json (of measured)"
    except Exception:
        return 6650.0, "fallback HBM figure (MEASURED_PEAKS.json absent) (of fallback)"


# ------------------------------------------------------------------------------------------
# clocks: read-only NVML polling in a thread
# ------------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index: int):
        self.index = index
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._ok = False
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self._ok = True
        except Exception:
            self._ok = False

    _REASONS = {
        "hw_slowdown": 0x8,
        "sw_power_cap": 0x4,
        "sw_thermal_slowdown": 0x20,
        "hw_thermal_slowdown": 0x40,
        "hw_power_brake_slowdown": 0x80,
    }

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                for name, bit in self._REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self._ok:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self) -> dict:
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


# ------------------------------------------------------------------------------------------
# CPU legs (the only places that touch oracle/)
# ------------------------------------------------------------------------------------------
def cpu_baseline_port(rows: int = 8192) -> dict:
    """The oracle (CPU restatement, OpenMP) on rows [0, rows) of the 8192^3 product."""
    from oracle import oracle as o

    a = o.fill_packed(rows, K, 1002)
    b = o.fill_packed(N_PER_GPU, K, 2002)
    o.gemm(a[:8], b)  # warm the threads
    t0 = time.perf_counter()
    o.gemm(a, b)
    dt = time.perf_counter() - t0
    return {
        "value": 2.0 * rows * N_PER_GPU * K / dt / 1e12,
        "unit": UNIT,
        "cores": o.threads(),
        "kind": "port",
        "sample": f"rows 0..{rows - 1} of the 8192^3 product ({rows}/8192 of the work), {dt:.2f} s",
    }


def reference_arm(args) -> None:
    """The reference's CPU implementation of the path on the host cores, one bounded slab per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import concurrent.futures as cf

    import numpy as np

    from oracle import oracle as o

    threads = os.cpu_count() or 1
    use_ref = o.ref_lib() is not None
    rows_per_thread = 2 if use_ref else 16
    rows = rows_per_thread * threads
    ap = o.fill_packed(rows, K, 1002)
    bp = o.fill_packed(N_PER_GPU, K, 2002)
    if use_ref:
        # kernel.cu:389-408 then kernel.cu:291-306, as compiled from the reference's sources; the
        # reference code is single-threaded, so row slabs run on a thread pool (ctypes drops the GIL)
        bu = o.ref_unpack(bp)

        def one(i):
            sl = ap[i * rows_per_thread : (i + 1) * rows_per_thread]
            return o.ref_cpu_gemm(o.ref_unpack(sl), bu)

        pool = cf.ThreadPoolExecutor(max_workers=threads)

        def step():
            list(pool.map(one, range(threads)))

        kind = "reference"
    else:
        o.set_threads(threads)

        def step():
            o.gemm(ap, bp)

        kind = "port"
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = 2.0 * rows * N_PER_GPU * K / dt / 1e12
    sample = f"{rows} rows of the 8192^3 product per step ({rows_per_thread} per thread, {threads} threads)"
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": dt * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "s4 x s4 -> s32 (CPU int32 multiply-add)",
        "data": "synthetic",
        "config": config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)



# ------------------------------------------------------------------------------------------
# verification against the CPU oracle (checker only: never inside a timed region)
# ------------------------------------------------------------------------------------------
def verify_against_oracle(torch, a, b, c, m, n, k, seams=(), rows_full=2, points=4096, seed=1):
    """Compare C (a device tensor [m, >= n]; its columns [0, n) hold A x B^T for the given packed device operands) with the
    oracle: `rows_full` whole rows (first and last), `points` sampled positions with tile seams (multiples of 192 and 256,
    and the given extra seam columns) mixed in.  Returns a description; raises SystemExit on the first difference."""
    import numpy as np

    from oracle import oracle as o

    ap = a.cpu().numpy().view(np.uint8)
    bp = b.cpu().numpy().view(np.uint8)
    rng = np.random.default_rng(seed)
    row_ids = sorted({0, m - 1} if rows_full >= 2 else {m // 2})
    for r in row_ids:
        want = o.gemm(ap[r : r + 1], bp)[0]
        got = c[r, :n].cpu().numpy()
        if not np.array_equal(got, want):
            bad = np.flatnonzero(got != want)
            raise SystemExit(f"bench.py: row {r} of the {m}x{n}x{k} product differs from the oracle at {bad.size} columns "
                             f"(first {bad[:4].tolist()}); no number reported")
    seam_cols = [x for step in (192, 256) for x in list(range(step - 1, n, step))[:32] + list(range(step, n, step))[:32]]
    seam_cols += [x for x in seams if 0 <= x < n]
    cols = np.concatenate([rng.integers(0, n, max(points - len(seam_cols), 0)), np.asarray(seam_cols, dtype=np.int64)]) if n > 0 else np.zeros(0, np.int64)
    rows = np.concatenate([rng.integers(0, m, len(cols) - min(len(cols), 64)), np.full(min(len(cols), 64), m - 1)])
    got = c[torch.from_numpy(rows).to(c.device), torch.from_numpy(cols).to(c.device)].cpu().numpy().astype(np.int64)
    want = o.gemm_points(ap, bp, rows, cols)
    if not np.array_equal(got, want):
        bad = np.flatnonzero(got != want)
        raise SystemExit(f"bench.py: {bad.size} of {len(cols)} sampled outputs of the {m}x{n}x{k} product differ from the oracle "
                         f"(first at row {int(rows[bad[0]])}, column {int(cols[bad[0]])}); no number reported")
    return {"ok": True, "full_rows": len(row_ids), "points": int(len(cols)), "against": "CPU oracle (int64 accumulate)"}


def time_graph_of_launches(torch, qm, m, n, k, per_graph, replays):
    """One shape through qm.gemm in a CUDA graph of `per_graph` launches over rotating operand buffers (so that a small
    problem is streamed from HBM, not served from L2).  Returns (min, median) milliseconds per launch and the tensors of
    buffer 0 for verification."""
    per_launch_bytes = m * k // 2 + n * k // 2 + 4 * m * n
    rotate = 1 if per_launch_bytes > 200e6 else min(64, int(2 * 126e6 // per_launch_bytes) + 2)
    a = qm.fill_packed(m, k, 1002)
    bs = [qm.fill_packed(n, k, 3002 + 17 * i) for i in range(rotate)]
    cs = [torch.empty((m, n), dtype=torch.int32, device="cuda") for _ in range(rotate)]
    qm.gemm(a, bs[0], cs[0], m, n, k)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(per_graph):
            qm.gemm(a, bs[i % rotate], cs[i % rotate], m, n, k)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / per_graph)
    times.sort()
    return times[0], times[len(times) // 2], (a, bs[0], cs[0]), rotate


EXTRA_SHAPES = [  # (m, n, k, kind): the decode and prefill shapes of the target list, and the large square
    (16, 4096, 4096, "decode"), (16, 11008, 4096, "decode"), (16, 28672, 8192, "decode"),
    (2048, 12288, 4096, "prefill"), (2048, 4096, 4096, "prefill"), (2048, 22016, 4096, "prefill"), (2048, 4096, 11008, "prefill"),
    (32768, 32768, 32768, "large"),
]


def time_prelaid(torch, qm, m, n, k, per_graph, replays):
    """The same product through qm_gemm_s4_prelaid: B rearranged once (untimed, as a weight loader would) into the load
    order of the register-resident decode kernel."""
    per_launch_bytes = m * k // 2 + n * k // 2 + 4 * m * n
    rotate = min(64, int(2 * 126e6 // per_launch_bytes) + 2)
    a = qm.fill_packed(m, k, 1002)
    bs = [qm.fill_packed(n, k, 3002 + 17 * i) for i in range(rotate)]
    bps = [qm.prelayout_b(b, n, k) for b in bs]
    cs = [torch.empty((m, n), dtype=torch.int32, device="cuda") for _ in range(rotate)]
    qm.gemm_prelaid(a, bps[0], cs[0], m, n, k)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(per_graph):
            qm.gemm_prelaid(a, bps[i % rotate], cs[i % rotate], m, n, k)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / per_graph)
    times.sort()
    return times[0], times[len(times) // 2], (a, bs[0], cs[0]), rotate


def extra_legs(torch, qm) -> list:
    """Further shapes, each verified against the oracle and then timed; not part of the headline number."""
    out = []
    peak_t, _ = measured_peaks()
    peak_h, _ = measured_hbm()
    for m, n, k, kind in EXTRA_SHAPES:
        nbytes = m * k // 2 + n * k // 2 + 4 * m * n
        if kind == "large" and torch.cuda.mem_get_info()[0] < 8 * 2**30:
            continue
        per_graph, replays = (20, 7) if kind == "decode" else ((10, 5) if kind == "prefill" else (2, 3))
        t_min, t_med, (a, b, c), rotate = time_graph_of_launches(torch, qm, m, n, k, per_graph, replays)
        ver = verify_against_oracle(torch, a, b, c, m, n, k, points=1024, seed=m + n + k)
        code, where = qm.device_status()
        if code != 0:
            raise SystemExit(f"bench.py: in-kernel wait expired in the extra leg {m}x{n}x{k} (site {where & 0xFF}); no number reported")
        ops = 2.0 * m * n * k
        e = {"shape": [m, n, k], "kind": kind, "us_min": t_min * 1e3, "us_median": t_med * 1e3, "verified": ver["ok"],
             "buffers_in_rotation": rotate, "cuda_graph_launches": per_graph}
        if kind == "decode":
            e.update({"bound": "hbm", "gbs": nbytes / (t_med * 1e-3) / 1e9, "frac": nbytes / (t_med * 1e-3) / 1e9 / peak_h,
                      "algorithmic_bytes": nbytes})
        else:
            e.update({"bound": "tensor", "tops": ops / (t_med * 1e-3) / 1e12, "frac": ops / (t_med * 1e-3) / 1e12 / peak_t,
                      "frac_nominal": ops / (t_med * 1e-3) / 1e12 / INT8_PEAK_NOMINAL_TOPS})
        out.append(e)
        del a, b, c
        torch.cuda.empty_cache()
        if kind == "decode" and k <= 8192 and n * k <= 64 * 2**20:
            # the optional offline weight layout (qm_prelayout_b): same product, same bytes, verified against the PLAIN B
            t_min, t_med, (a, b, c), rotate = time_prelaid(torch, qm, m, n, k, per_graph, replays)
            ver = verify_against_oracle(torch, a, b, c, m, n, k, points=1024, seed=m + n + k + 1)
            gbs = nbytes / (t_med * 1e-3) / 1e9
            out.append({"shape": [m, n, k], "kind": "decode, pre-laid-out weights (qm_gemm_s4_prelaid)", "us_min": t_min * 1e3,
                        "us_median": t_med * 1e3, "verified": ver["ok"], "buffers_in_rotation": rotate, "cuda_graph_launches": per_graph,
                        "bound": "hbm", "gbs": gbs, "frac": gbs / peak_h, "algorithmic_bytes": nbytes})
            del a, b, c
            torch.cuda.empty_cache()
    return out


def multi_gpu_legs(torch, dist, qm, world: int, rank: int, steps: int = 2) -> dict:
    """After the headline: (a) the column-sharded product with both gathers, checked on rank 0 against the oracle;
    (b) 32768^3 strong scaling: compute only, with NCCL gather, with fused peer-store gather (device-timed, max over
    ranks).  Raises SystemExit on any mismatch or in-kernel time-out."""
    import numpy as np

    from oracle import oracle as o
    from quadmul_b200.sharded import NShardedGemm, SymmetricC

    def max_over_ranks(ms: float) -> float:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, n_steps):
        fn()  # warm
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1) / n_steps)

    # ---- (a) correctness of the two gather paths on a shape whose shards are uneven and cut tiles ----
    m, n, k = 1024, 128 * (4 * world + 3), 2048
    sh = NShardedGemm(n, world=world, rank=rank)
    a = qm.fill_packed(m, k, 4001)
    b_full = qm.fill_packed(n, k, 4002)
    b = sh.shard_of(b_full).contiguous()
    seams = sorted({x for r in range(world) for x in (sh.ranges[r][0] - 1, sh.ranges[r][0], sh.ranges[r][0] + sh.ranges[r][1] - 1)
                    if 0 <= x < n})
    slab = sh.local(a, b, m, k)
    full = sh.gather(slab, m)
    csym = SymmetricC(m, n)
    csym.local.fill_(-3)
    torch.cuda.synchronize()
    dist.barrier()
    sh.local_into(a, b, m, k, csym, dst=0)
    if rank == 0:
        csym.wait_all()
    torch.cuda.synchronize()
    ok_local = True
    if rank == 0:
        ap_host = a.cpu().numpy().view(np.uint8)
        bp_host = b_full.cpu().numpy().view(np.uint8)
        for name, cmat in (("NCCL gather", full), ("fused peer-store gather", csym.local)):
            verify_against_oracle(torch, a, b_full, cmat, m, n, k, seams=seams, points=4096, seed=world)
            for col in seams:  # every shard seam as a whole column
                want = o.gemm(ap_host, bp_host[col : col + 1])[:, 0]
                if not np.array_equal(cmat[:, col].cpu().numpy(), want):
                    raise SystemExit(f"bench.py: {name}: column {col} (a shard seam) differs from the oracle; no number reported")
    else:
        ok_local = bool((csym.local == -3).all())  # nobody may write into the other ranks' copies
    code, where = qm.device_status()
    flag = torch.tensor([0 if (ok_local and code == 0) else 1], dtype=torch.int32, device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if int(flag.item()) != 0:
        raise SystemExit("bench.py: sharded check failed on some rank (stray writes or an in-kernel time-out); no number reported")
    result = {"sharded_check": {"ok": True, "world": world, "shape": [m, n, k], "paths": ["nccl_gather", "fused_gather"],
                                "checked": "rank 0: 2 full rows, 4096 points and every shard-seam column against the CPU oracle, both paths"}}
    del full, csym, slab, a, b, b_full
    torch.cuda.empty_cache()

    # ---- (b) 32768^3, B column-sharded, A replicated ----
    m = n = k = 32768
    sh = NShardedGemm(n, world=world, rank=rank)
    a = qm.fill_packed(m, k, 1005)
    b = qm.fill_packed(sh.count, k, 2005 + 7919 * rank)
    c_local = torch.empty((m, sh.count), dtype=torch.int32, device="cuda")
    compute_ms = timed(lambda: sh.local(a, b, m, k, out=c_local), steps + 1)
    full_c = torch.empty((m, n), dtype=torch.int32, device="cuda")

    def with_nccl():
        sh.local(a, b, m, k, out=c_local)
        sh.gather(c_local, m, out=full_c)

    nccl_ms = timed(with_nccl, steps)

    def with_nccl_to_rank0():
        sh.local(a, b, m, k, out=c_local)
        sh.gather_to(c_local, m, dst=0, out=full_c if rank == 0 else None)

    nccl_to0_ms = timed(with_nccl_to_rank0, steps)
    del full_c
    torch.cuda.empty_cache()
    csym = SymmetricC(m, n)

    def with_fused():
        sh.local_into(a, b, m, k, csym, dst=0)
        if rank == 0:
            csym.wait_all()

    fused_ms = timed(with_fused, steps)
    dist.barrier()
    if rank == 0:  # the gathered matrix, sampled: own slab and every other rank's
        bp_rows = {}
        rng = np.random.default_rng(5)
        rows = rng.integers(0, m, 512)
        cols = np.concatenate([rng.integers(0, n, 512 - 2 * world), np.asarray([sh.ranges[r][0] for r in range(world)] + [sh.ranges[r][0] + sh.ranges[r][1] - 1 for r in range(world)])])
        got = csym.local[torch.from_numpy(rows).cuda(), torch.from_numpy(cols).cuda()].cpu().numpy().astype(np.int64)
        ap = a.cpu().numpy().view(np.uint8)
        want = np.empty(len(cols), dtype=np.int64)
        for i, (r, cidx) in enumerate(zip(rows, cols)):
            owner = next(q for q in range(world) if sh.ranges[q][0] <= cidx < sh.ranges[q][0] + sh.ranges[q][1])
            if owner not in bp_rows:
                bp_rows[owner] = o.fill_packed(sh.ranges[owner][1], k, 2005 + 7919 * owner)
            want[i] = o.gemm_points(ap[r : r + 1], bp_rows[owner][cidx - sh.ranges[owner][0] : cidx - sh.ranges[owner][0] + 1], np.zeros(1, np.int64), np.zeros(1, np.int64))[0]
        if not np.array_equal(got, want):
            raise SystemExit("bench.py: 32768^3 fused gather: sampled outputs on rank 0 differ from the oracle; no number reported")
    code, where = qm.device_status()
    flag = torch.tensor([0 if code == 0 else 1], dtype=torch.int32, device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if int(flag.item()) != 0:
        raise SystemExit("bench.py: in-kernel time-out in the 32768^3 legs; no number reported")
    ops = 2.0 * m * n * k
    result["large"] = {"shape": [m, n, k], "world": world, "scaling": "strong", "steps": steps,
                       "compute_ms": compute_ms, "compute_tops": ops / (compute_ms * 1e-3) / 1e12,
                       "nccl_gather_ms": nccl_ms, "nccl_gather_to_rank0_ms": nccl_to0_ms, "fused_gather_ms": fused_ms,
                       "note": "B column-sharded, A replicated; *_gather_ms = GEMM + bringing the full int32 C together (nccl_gather: all-gather, to "
                               "every rank; nccl_gather_to_rank0: NCCL gather, to rank 0 only; fused: to rank 0 only); "
                               "fused: GEMM epilogues store into rank 0's C over NVLink, completion flags with a bounded wait; "
                               "rank 0's gathered C sampled against the CPU oracle"}
    del csym, a, b, c_local
    torch.cuda.empty_cache()
    return result


# ------------------------------------------------------------------------------------------
# native arm
# ------------------------------------------------------------------------------------------
def bind_host_to_gpu_numa_node(torch, device_index: int):
    """Restrict this process to the CPUs next to the GPU (sysfs `local_cpulist` of its PCI function), so that host buffers
    allocated from now on land on that NUMA node (first touch).  Returns (node, previous affinity) or (None, None) when sysfs
    does not say; undo with os.sched_setaffinity(0, previous)."""
    try:
        props = torch.cuda.get_device_properties(device_index)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        base = f"/sys/bus/pci/devices/{bdf}"
        node = int(open(f"{base}/numa_node").read().strip())
        cpus = set()
        for part in open(f"{base}/local_cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        previous = os.sched_getaffinity(0)
        cpus &= previous
        if node < 0 or not cpus:
            return None, None
        os.sched_setaffinity(0, cpus)
        return node, previous
    except (OSError, ValueError, AttributeError):
        return None, None


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def native_arm(args) -> None:
    import torch
    import torch.distributed as dist

    import quadmul_b200 as qm
    from quadmul_b200.sharded import NShardedGemm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the native arm has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    qm.init()

    custom = args.shape is not None
    large = args.workload == "large"
    if custom:
        if world != 1:
            raise SystemExit("bench.py: --shape is a single-GPU option")
        m, n_total, k = (int(x) for x in args.shape.split(","))
    elif large:
        m = n_total = k = 32768
    else:
        m, n_total, k = M, N_PER_GPU * world, K
    forced = dict(tile_n=args.tile_n, swap_ab=args.swap_ab, cta_pair=args.cta_pair, split_k=args.split_k, a_tmem=args.a_tmem)
    forced = {kk: v for kk, v in forced.items() if v}
    sh = NShardedGemm(n_total, world=world, rank=rank)
    n_local = sh.count
    a = qm.fill_packed(m, k, 1002)  # replicated
    # B buffers: one for tensor-bound shapes; for small (HBM-bound) ones enough distinct copies that
    # consecutive launches cannot be served from the 126 MB L2
    b_bytes = n_local * (k // 2)
    per_launch_bytes = m * k // 2 + b_bytes + 4 * m * n_local
    rotate = 1 if (per_launch_bytes > 200e6 or args.l2_resident) else min(64, int(2 * 126e6 // max(per_launch_bytes, 1)) + 2)
    bs = [qm.fill_packed(n_local, k, 2002 + 7919 * rank + 31 * i) for i in range(rotate)]
    cs = [torch.empty((m, n_local), dtype=torch.int32, device="cuda") for _ in range(rotate)]
    c = cs[0]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    counter = [0]
    csym = full_c = None
    if large and args.gather == "fused" and world > 1:
        from quadmul_b200.sharded import SymmetricC

        csym = SymmetricC(m, n_total)
    if large and args.gather == "nccl" and world > 1:
        full_c = torch.empty((m, n_total), dtype=torch.int32, device="cuda")

    dq = None
    if args.dequant:
        # fused dequantising epilogue (qm_gemm_s4_dequant_bf16): bf16 output, per-row and per-column scales
        if world != 1 or forced or large:
            raise SystemExit("bench.py: --dequant is a single-GPU option without forced tiles")
        dq = (torch.rand(m, device="cuda") * 0.01 + 1e-3, torch.rand(n_local, device="cuda") * 0.01 + 1e-3,
              [torch.empty((m, n_local), dtype=torch.bfloat16, device="cuda") for _ in range(rotate)])
        per_launch_bytes = m * k // 2 + b_bytes + 2 * m * n_local + 4 * (m + n_local)

    bps = None
    if args.prelaid:
        # the optional offline weight layout: B rearranged once, outside every timed region, as a weight loader would
        if world != 1 or forced or large or dq is not None:
            raise SystemExit("bench.py: --prelaid is a single-GPU option without forced tiles")
        bps = [qm.prelayout_b(b_i, n_local, k) for b_i in bs]

    def launch():
        i = counter[0] % rotate
        counter[0] += 1
        if bps is not None:
            qm.gemm_prelaid(a, bps[i], cs[i], m, n_local, k)
        elif dq is not None:
            qm.gemm_dequant(a, bs[i], dq[0], dq[1], dq[2][i], m, n_local, k, workspace=cs[i].view(-1))
        elif forced:
            qm.gemm_ex(a, bs[i], cs[i], m, n_local, k, kernel=1, **forced)
        elif csym is not None:
            sh.local_into(a, bs[i], m, k, csym, dst=0)  # epilogue stores go to rank 0's C over NVLink
            if rank == 0:
                csym.wait_all()  # completion flags, bounded wait
        elif full_c is not None:
            sh.local(a, bs[i], m, k, out=cs[i])
            sh.gather(cs[i], m, out=full_c)
        else:
            sh.local(a, bs[i], m, k, out=cs[i])

    launches_per_step = 1
    if args.graph > 0:
        launches_per_step = args.graph
        launch()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(launches_per_step):
                launch()

        def step():
            graph.replay()
    else:
        step = launch

    # the C that is about to be timed, against the CPU oracle (the reference checks before it times: test.py:39-43)
    verified = None
    if dq is None and csym is None:
        launch()
        torch.cuda.synchronize()
        counter[0] = 0
        verified = verify_against_oracle(torch, a, bs[0], cs[0], m, n_local, k, seed=rank + 1)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    launches_before = qm.launch_count()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for i in range(args.steps):
        step()
        ev[i + 1].record()
    barrier()
    clocks = sampler.stop()
    gpu_launches = (qm.launch_count() - launches_before) if args.graph == 0 else args.steps * launches_per_step
    total_ms = ev[0].elapsed_time(ev[-1])
    per_step_ms = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps))
    t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    code, where = qm.device_status()
    if code != 0:
        raise SystemExit(f"bench.py: in-kernel wait expired (site {where & 0xFF}); no number reported")

    ops_per_launch = 2.0 * m * n_local * k
    ms_per_step = total_ms / args.steps
    value = ops_per_launch * launches_per_step * world / (ms_per_step * 1e-3) / 1e12

    line = None
    if rank == 0:
        plan = qm.plan(m, n_local, k)
        plan.update(forced)
        avg_launch_ms = sum(per_step_ms) / len(per_step_ms) / launches_per_step
        tensor_bound = (ops_per_launch / per_launch_bytes) > 700  # machine balance of B200, int8 ops per HBM byte
        if tensor_bound:
            peak, peak_note = measured_peaks()
            achieved = ops_per_launch / (avg_launch_ms * 1e-3) / 1e12
            roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s", "frac": achieved / peak,
                        "peak_nominal": INT8_PEAK_NOMINAL_TOPS, "frac_nominal": achieved / INT8_PEAK_NOMINAL_TOPS}
        else:
            peak, peak_note = measured_hbm()
            achieved = per_launch_bytes / (avg_launch_ms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak}
        roofline.update({
            "kernel": ("gemm_rmma_kernel<pre-laid-out weights into registers, mma.sync s8>" if bps is not None else
                       "gemv_kernel<dp4a, weight streaming>" if plan.get("kernel") == 3 and not forced else
                       "gemm_rmma_kernel<weights into registers, mma.sync s8>" if plan.get("kernel") == 4 and not forced else
                       f"gemm_dec_kernel<tile_n={plan['tile_n']}, B rows through TMEM, " +
                       ("balanced shares" if plan.get("stream_k") == 2 else f"split_k={plan['split_k']}") + ">"
                       if plan.get("a_tmem") == 2 and plan.get("swap_ab") == 2 else
                       "gemm_tc2_kernel<256x256 pair tile, A in TMEM>" if plan.get("a_tmem") == 2 else
                       f"gemm_tc_kernel<tile_n={plan['tile_n']}, swap_ab={plan['swap_ab'] - 1}, cta_pair={plan['cta_pair']}>"),
            "traffic": DRAM_TRAFFIC_BYTES_PER_LAUNCH if not custom and not forced else None,
            "peak_note": peak_note,
            "launch_ms_min": per_step_ms[0] / launches_per_step,
            "launch_ms_median": per_step_ms[len(per_step_ms) // 2] / launches_per_step,
            "launch_ms_avg": avg_launch_ms,
            "algorithmic_ops_per_launch": ops_per_launch,
            "algorithmic_bytes_per_launch": per_launch_bytes,
        })
        cfg = config(world)
        if large:
            cfg.update({"workload": f"int4 GEMM M=N=K=32768, B column-sharded over {world} GPU(s), A replicated; gather: {args.gather}",
                        "m": m, "n_total": n_total, "k": k, "parallelism": f"n-shard x{world}, gather={args.gather}",
                        "l2": "working set exceeds the 126 MB L2 many times over"})
        if custom:
            cfg.update({"workload": f"int4 GEMM M={m} N={n_total} K={k} (single GPU, not the headline case)", "m": m,
                        "n_total": n_total, "k": k})
            if args.l2_resident:
                cfg["l2"] = "one B and C buffer reused by every launch: served from L2, not an HBM figure"
            if rotate > 1:
                cfg["l2"] = f"{rotate} distinct B and C buffers in rotation ({rotate * per_launch_bytes / 1e6:.0f} MB) exceed the 126 MB L2"
        if args.graph:
            cfg["cuda_graph_launches_per_step"] = launches_per_step
        if dq is not None:
            cfg["epilogue"] = "fused dequantisation to bf16 (row and column scales), not the int32 store of the headline metric"
        line = {
            "metric": (METRIC if not (custom or large) else f"int4 GEMM TOPS at M={m} N={n_total} K={k}") + (" (bf16 dequant epilogue)" if dq is not None else ""),
            "value": value,
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": warmup,
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "strong" if large else "weak",
            "vs_baseline": None,
            "dtype": "s4 x s4 -> s32 (tcgen05 kind::i8, exact)",
            "data": "synthetic",
            "config": cfg,
            "pct_int8_peak_nominal": 100.0 * value / (INT8_PEAK_NOMINAL_TOPS * world),
            "roofline": roofline,
            "gpu_launches": gpu_launches,
            "clocks": clocks,
        }
        if verified is not None:
            line["verified"] = verified

    # ---- end to end through the host-buffer C-ABI call, copies inside the timed region ----
    if not args.no_e2e and not large:
        numa_node, previous_affinity = (None, None) if args.no_numa_bind else bind_host_to_gpu_numa_node(torch, torch.cuda.current_device())
        ha = a.cpu().pin_memory()
        hb = bs[0].cpu().pin_memory()
        hc = torch.empty((m, n_local), dtype=torch.int32).pin_memory()
        e2e_steps = max(3, min(10, args.steps))
        qm.gemm_host(ha, hb, hc, m, n_local, k)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            qm.gemm_host(ha, hb, hc, m, n_local, k)
        torch.cuda.synchronize()
        dt = torch.tensor([(time.perf_counter() - t0) / e2e_steps], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        if previous_affinity:
            os.sched_setaffinity(0, previous_affinity)
        if rank == 0:
            import numpy as np

            from oracle import oracle as o

            pos = np.arange(0, m * n_local, 65537, dtype=np.int64)
            expected = int(o.gemm_points(ha.numpy().view(np.uint8), hb.numpy().view(np.uint8), pos // n_local, pos % n_local).sum())
            checksum = int(hc.view(-1)[:: 65537].to(torch.int64).sum())
            if checksum != expected:
                raise SystemExit(f"bench.py: end-to-end result checksum {checksum} != {expected} (oracle); no number reported")
            line["e2e"] = {
                "value": ops_per_launch * world / float(dt.item()) / 1e12,
                "unit": UNIT,
                "h2d_bytes_per_step": int(ha.numel() + hb.numel()),
                "d2h_bytes_per_step": int(hc.numel() * 4),
                "ms_per_step": float(dt.item()) * 1e3,
                "steps": e2e_steps,
                # what bounds this figure: the bytes that cross PCIe per step, per GPU, over the step time (max over ranks)
                "pcie_gbs_per_gpu": (ha.numel() + hb.numel() + hc.numel() * 4) / float(dt.item()) / 1e9,
                "api": "qm_gemm_s4_host (pinned host A, B in; int32 C out; per GPU)",
                "host_numa_node": numa_node,  # rank 0's; every rank binds its host buffers to the node of its own GPU (None: not bound)
                "result_checksum": checksum,
                "result_checksum_expected": expected,
                "result_checksum_of": f"every 65537th element of the host C ({len(pos)} elements), expected value from the CPU oracle",
            }
            line["gpu_launches"] += e2e_steps + 1

    headline = not custom and not large and not forced and dq is None and args.graph == 0 and bps is None
    if headline and not args.no_extra:
        del bs, cs, c, a
        torch.cuda.empty_cache()
        if world == 1:
            line["extra"] = extra_legs(torch, qm)
        else:
            legs = multi_gpu_legs(torch, dist, qm, world, rank)
            if rank == 0:
                line.update(legs)
    if rank == 0 and world == 1 and not custom and not large and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_port()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def byte_kernel_arm(args) -> None:
    """pack / unpack against the HBM roof: 1.5 bytes of traffic per element."""
    import torch

    import quadmul_b200 as qm
    from quadmul_b200 import _lib

    rows, k = (int(x) for x in (args.shape or "16384,16384").split(","))
    torch.cuda.set_device(0)
    packed = qm.fill_packed(rows, k, 7)
    full = qm.unpack(packed)
    out_p = torch.empty_like(packed)
    out_u = torch.empty_like(full)
    stream = torch.cuda.current_stream().cuda_stream
    if args.op == "pack":
        fn = lambda: _lib.check(_lib.LIB.qm_pack_s4(full.data_ptr(), out_p.data_ptr(), rows, k, stream), "pack")
    else:
        fn = lambda: _lib.check(_lib.LIB.qm_unpack_s4(packed.data_ptr(), out_u.data_ptr(), rows, k, stream), "unpack")
    for _ in range(max(args.warmup, 3)):
        fn()
    torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(0))
    sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for i in range(args.steps):
        fn()
        ev[i + 1].record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    per = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps))
    avg = ev[0].elapsed_time(ev[-1]) / args.steps
    nbytes = 1.5 * rows * k
    peak, note = measured_hbm()
    ok = torch.equal(out_p, packed) if args.op == "pack" else torch.equal(out_u, full)
    print(json.dumps({
        "metric": f"{args.op} GB/s ({rows} x {k} elements)", "value": nbytes / (avg * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": avg, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": f"{args.op} of a {rows} x {k} signed-int4 matrix", "l2": f"{nbytes / 1e6:.0f} MB per launch exceeds the 126 MB L2"},
        "roofline": {"bound": "hbm", "achieved": nbytes / (avg * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": nbytes / (avg * 1e-3) / 1e9 / peak, "traffic": None, "peak_note": note,
                     "launch_ms_min": per[0], "launch_ms_median": per[len(per) // 2], "algorithmic_bytes_per_launch": nbytes,
                     "kernel": f"{args.op}_kernel"},
        "gpu_launches": args.steps, "clocks": clocks, "round_trip_ok": bool(ok)}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-numa-bind", action="store_true", help="end-to-end leg: leave the host buffers wherever the process happens to run")
    ap.add_argument("--no-extra", action="store_true", help="skip the further shapes (1 GPU) and the sharded check / 32768^3 legs (2+ GPUs)")
    ap.add_argument("--shape", default=None, help="M,N,K of a single-GPU case other than the headline one (profiling, sweeps)")
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--swap-ab", type=int, default=0)
    ap.add_argument("--cta-pair", type=int, default=0)
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--a-tmem", type=int, default=0)
    ap.add_argument("--graph", type=int, default=0, help="capture this many launches per step in one CUDA graph")
    ap.add_argument("--workload", choices=["headline", "large"], default="headline",
                    help="large: M=N=K=32768 with B column-sharded over the GPUs (strong scaling)")
    ap.add_argument("--gather", choices=["none", "nccl", "fused"], default="none",
                    help="with --workload large: also bring the full C to every rank (nccl) or to rank 0 (fused) inside each step")
    ap.add_argument("--l2-resident", action="store_true",
                    help="with --shape: reuse one B and C buffer so that a small problem is served from L2 (the latency floor of "
                         "the launch; never the roofline number)")
    ap.add_argument("--prelaid", action="store_true",
                    help="with --shape (a decode shape): time qm_gemm_s4_prelaid on weights rearranged once by qm_prelayout_b")
    ap.add_argument("--dequant", action="store_true",
                    help="time qm_gemm_s4_dequant_bf16 (bf16 output with row and column scales) instead of the int32 GEMM")
    ap.add_argument("--op", choices=["gemm", "pack", "unpack"], default="gemm",
                    help="pack / unpack: time the HBM-bound byte kernels on a --shape ROWS,K matrix instead of the GEMM")
    args = ap.parse_args()

    if args.impl == "reference":
        reference_arm(args)
        return
    if args.op != "gemm":
        byte_kernel_arm(args)
        return
    if args.gpus > 1 and "RANK" not in os.environ:
        # started by hand without a launcher: re-enter under torch.distributed.run
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    native_arm(args)


if __name__ == "__main__":
    main()
