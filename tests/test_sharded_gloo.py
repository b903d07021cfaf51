"""Host logic of the column-sharded driver under torch.distributed (gloo, world size 2 and 3, CPU).

The CUDA entry points are replaced by CPU stand-ins (the oracle as the per-shard GEMM, a torch
gather as the un-interleave), so what is tested is the driver: partition, padding of uneven slabs,
all-gather layout and assembly of the full C."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, m, n, k, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from oracle import oracle as o
    from quadmul_b200.sharded import NShardedGemm

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        def cpu_gemm(a, b, out, mm, nn, kk):
            c = o.gemm(a.numpy().view(np.uint8), b.numpy().view(np.uint8))
            out[:, :nn] = torch.from_numpy(c)

        def cpu_unshard(slabs, out, mm, nn, w, stride):
            from quadmul_b200 import nshard_range

            for r in range(w):
                b, c = nshard_range(nn, w, r)
                out[:, b : b + c] = slabs[r, :, :c]

        ap = o.fill_packed(m, k, 5)
        bp = o.fill_packed(n, k, 6)
        a = torch.from_numpy(ap).view(torch.int8)
        b_full = torch.from_numpy(bp).view(torch.int8)
        sh = NShardedGemm(n, gemm_fn=cpu_gemm, unshard_fn=cpu_unshard)
        assert (sh.world, sh.rank) == (world, rank)
        slab = sh.local(a, sh.shard_of(b_full).contiguous(), m, k)
        assert tuple(slab.shape) == (m, sh.count)
        full = sh.gather(slab, m)
        want = o.gemm(ap, bp)
        ok = bool(np.array_equal(full.numpy(), want)) and bool(np.array_equal(slab.numpy(), want[:, sh.begin : sh.begin + sh.count]))
        # the gather to one rank only: the last rank gets the full C, the others nothing
        dst = world - 1
        only = sh.gather_to(slab, m, dst=dst)
        ok = ok and ((only is None) if rank != dst else bool(np.array_equal(only.numpy(), want)))
        q.put((rank, ok, sh.begin, sh.count))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,m,n,k", [(2, 24, 512, 64), (2, 5, 300, 96), (3, 8, 1000, 32)])
def test_sharded_driver_gloo(world, m, n, k):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, m, n, k, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _, _ in results), results
    covered = sorted((b, c) for _, _, b, c in results)
    pos = 0
    for b, c in covered:
        assert b == pos
        pos += c
    assert pos == n


def test_single_rank_is_identity():
    import torch

    from quadmul_b200.sharded import NShardedGemm

    sh = NShardedGemm(640, world=1, rank=0, gemm_fn=lambda a, b, out, m, n, k: out.fill_(3))
    assert (sh.begin, sh.count, sh.slab_stride) == (0, 640, 640)
    a = torch.zeros((4, 16), dtype=torch.int8); b = torch.zeros((640, 16), dtype=torch.int8)
    slab = sh.local(a, b, 4, 32)
    assert torch.equal(sh.gather(slab, 4), slab)
    with pytest.raises(ValueError):
        sh.local(a, b[:100], 4, 32)
    with pytest.raises(ValueError):
        NShardedGemm(640, world=2, rank=2)
