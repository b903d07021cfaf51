"""Sweep of the tensor-path variants over a list of shapes; prints one JSON line per (shape, variant).

    python -m quadmul_b200.tune [--shapes M,N,K;M,N,K;...] [--iters 20]

The plan rules in csrc/qm_tile_table.h are written from these measurements (the reference shipped
its A40 table without the tuner that produced it; reference README.md:13).  Timing: CUDA events
around CUDA graphs of back-to-back launches, B buffers rotated so that small problems are not
served from L2, minimum over `iters` replays.
"""
from __future__ import annotations

import argparse
import json

DEFAULT_SHAPES = [
    (1024, 1024, 1024), (8192, 8192, 8192),
    (1, 4096, 4096), (16, 4096, 4096), (64, 4096, 4096), (1, 11008, 4096), (16, 11008, 4096), (64, 11008, 4096),
    (2048, 12288, 4096), (2048, 4096, 4096), (2048, 22016, 4096), (2048, 4096, 11008),
]


def variants(m: int, n: int):
    out = []
    if m <= 4:
        out.append(dict(kernel=3))  # dp4a row kernel
    if m <= 64:
        out.append(dict(kernel=4))  # register-resident mma.sync kernel (k <= 8192)
    if m <= 256:
        for tn in (16, 32, 64, 128):
            if tn >= min(m, 128) or tn == 128:
                for sk in ((1, 2, 3, 4, 6, 8, 16) if m <= 64 else (1, 2, 4)):
                    out.append(dict(tile_n=tn, swap_ab=2, cta_pair=1, split_k=sk))
    if m <= 64:  # decode kernel: B rows through TMEM
        for tn in (16, 32, 64):
            if tn >= m:
                for sk in (1, 2, 3, 4, 5, 6, 8):
                    out.append(dict(tile_n=tn, swap_ab=2, cta_pair=1, split_k=sk, a_tmem=2))
                out.append(dict(tile_n=tn, swap_ab=2, cta_pair=1, a_tmem=2, stream_k=2))
                for sk in (2, 3, 4):  # the K partitions of a tile as one cluster
                    out.append(dict(tile_n=tn, swap_ab=2, cta_pair=1, split_k=sk, a_tmem=2, stream_k=3))
                if tn == 16:  # two smaller CTAs per SM
                    for sk in (1, 2, 3, 4):
                        out.append(dict(tile_n=tn, swap_ab=2, cta_pair=1, split_k=sk, a_tmem=2, ctas_per_sm=2))
                    out.append(dict(tile_n=tn, swap_ab=2, cta_pair=1, a_tmem=2, stream_k=2, ctas_per_sm=2))
    if m > 64:
        for tn in (128, 256):
            out.append(dict(tile_n=tn, swap_ab=1, cta_pair=1, split_k=1))
            out.append(dict(tile_n=tn, swap_ab=1, cta_pair=2, split_k=1))
        for sk in (1, 2, 3, 4, 6, 8):  # pair tile with A through TMEM; K partitions add into C with TMA reduce
            out.append(dict(tile_n=256, swap_ab=1, cta_pair=2, split_k=sk, a_tmem=2))
    return out


def time_variant(qm, torch, m, n, k, opts, iters, per_graph):
    per_launch_bytes = m * k // 2 + n * k // 2 + 4 * m * n
    rotate = 1 if per_launch_bytes > 200e6 else min(64, int(2 * 126e6 // per_launch_bytes) + 2)
    a = qm.fill_packed(m, k, 1)
    bs = [qm.fill_packed(n, k, 2 + i) for i in range(rotate)]
    cs = [torch.empty((m, n), dtype=torch.int32, device="cuda") for _ in range(rotate)]
    opts = dict({"kernel": 1}, **opts)
    qm.gemm_ex(a, bs[0], cs[0], m, n, k, **opts)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(per_graph):
            qm.gemm_ex(a, bs[i % rotate], cs[i % rotate], m, n, k, **opts)
    g.replay()
    torch.cuda.synchronize()
    best = 1e30
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / per_graph)
    code, where = qm.device_status()
    return best, code


# Shapes of the kernel-family sweep behind the decode cost model: rows of A x (N, K) of common layer shapes.
FAMILY_M = [1, 2, 4, 8, 16, 24, 32, 48, 64]
FAMILY_NK = [(2048, 4096), (4096, 4096), (6144, 4096), (8192, 4096), (11008, 4096), (12288, 4096), (14336, 4096), (16384, 4096), (22016, 4096), (28672, 4096), (2048, 8192),
             (4096, 8192), (8192, 8192), (10240, 8192), (28672, 8192), (57344, 8192), (4096, 2048), (4096, 11008), (4096, 14336)]
FAMILIES = {"rmma": dict(kernel=4), "gemv": dict(kernel=3), "dec": dict(kernel=1)}  # dec: the tensor path with the table's K cut


def family_sweep(qm, torch, iters, out):
    """One line per (shape, kernel family): the register-resident kernel, the row kernel and the TMA/TMEM decode kernel, each
    in the form the table would run it.  These lines are what `--emit` fits the cost model to."""
    for n, k in FAMILY_NK:
        for m in FAMILY_M:
            for fam, opts in FAMILIES.items():
                try:
                    ms, code = time_variant(qm, torch, m, n, k, opts, iters, 50 if n * k < 64e6 else 20)
                except qm.QuadmulError as exc:
                    if exc.status in (3, 7, 8):  # this family does not take the shape
                        continue
                    raise
                if code != 0:
                    raise SystemExit(f"tune: in-kernel wait expired for {m}x{n}x{k} {fam}; stopping")
                line = json.dumps({"family": fam, "m": m, "n": n, "k": k, "us": round(ms * 1e3, 2)})
                print(line, flush=True)
                if out:
                    out.write(line + "\n")
                    out.flush()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--families", action="store_true", help="sweep the decode kernel families (input of --emit)")
    ap.add_argument("--out", default=None, help="with --families: also append the lines to this file")
    ap.add_argument("--emit", action="store_true", help="no GPU: fit the cost model to the committed sweep and write csrc/tile_table.inc")
    ap.add_argument("--check", action="store_true", help="with --emit: do not write, exit 1 if csrc/tile_table.inc would change")
    args = ap.parse_args()
    if args.emit:
        from . import tile_table_gen

        raise SystemExit(tile_table_gen.main(check=args.check))
    import torch

    import quadmul_b200 as qm

    if args.families:
        qm.init()
        with (open(args.out, "a") if args.out else open("/dev/null", "w")) as out:
            family_sweep(qm, torch, args.iters, out if args.out else None)
        return
    shapes = DEFAULT_SHAPES if not args.shapes else [tuple(int(x) for x in s.split(",")) for s in args.shapes.split(";")]
    qm.init()
    for m, n, k in shapes:
        ops = 2.0 * m * n * k
        nbytes = m * k // 2 + n * k // 2 + 4 * m * n
        per_graph = 10 if ops > 1e11 else 50
        rows = []
        for opts in variants(m, n):
            try:
                ms, code = time_variant(qm, torch, m, n, k, opts, args.iters, per_graph)
            except qm.QuadmulError as exc:
                if exc.status in (3, 7, 8):  # variant not built or not for this shape, or scratch too small for this split
                    continue
                raise
            if code != 0:
                raise SystemExit(f"tune: in-kernel wait expired for {m}x{n}x{k} {opts}; stopping")
            rows.append((ms, opts))
            print(json.dumps({"m": m, "n": n, "k": k, **opts, "us": round(ms * 1e3, 2), "tops": round(ops / ms / 1e9, 1),
                              "gbs": round(nbytes / ms / 1e6, 1), "status": code}), flush=True)
        if rows:
            ms, opts = min(rows, key=lambda r: r[0])
            print(json.dumps({"best": [m, n, k], **opts, "us": round(ms * 1e3, 2)}), flush=True)


if __name__ == "__main__":
    main()
