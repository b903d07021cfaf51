"""Column-sharded GEMM on real devices.

On one GPU the ranks are emulated one after another on the same device (each rank's slab written through
qm_gemm_s4_ldc into the full-width C, and the gather path through qm_unshard_c).  With two or more GPUs
the same check runs as one process per GPU over NCCL, including the optional all-gather of C."""
import os
import socket
import sys

import numpy as np
import pytest

from _util import to_dev

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world,m,n,k", [(2, 300, 1024, 512), (4, 64, 11008, 256), (8, 260, 2048, 384), (3, 16, 1000, 128)])
def test_shards_emulated_on_one_gpu(qm, cuda_clean, oracle, world, m, n, k):
    torch = cuda_clean
    from quadmul_b200.sharded import NShardedGemm

    ap = oracle.fill_packed(m, k, 21); bp = oracle.fill_packed(n, k, 22)
    want = oracle.gemm(ap, bp)
    a, b = to_dev(torch, ap), to_dev(torch, bp)
    full = torch.full((m, n), -9, dtype=torch.int32, device="cuda")
    shards = [NShardedGemm(n, world=world, rank=r) for r in range(world)]
    stride = shards[0].slab_stride
    slabs = torch.zeros((world, m, stride), dtype=torch.int32, device="cuda")
    for sh in shards:
        # (1) straight into the full-width C through the leading dimension
        sh.local(a, sh.shard_of(b), m, k, out=full[:, sh.begin : sh.begin + sh.count])
        # (2) into a padded slab, as a rank would before an all-gather
        sh.local(a, sh.shard_of(b), m, k, out=slabs[sh.rank])
    torch.cuda.synchronize()
    assert np.array_equal(full.cpu().numpy(), want)
    out = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    qm.unshard_c(slabs, out, m, n, world, stride)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("m,n,k,pitch,offset", [
    (300, 1024, 512, 1024, 0),      # ragged rows, large-shape kernel
    (1024, 2000, 1056, 2560, 256),  # ragged columns, a column slab of a wider C, K tail
    (520, 1022, 256, 1030, 4),      # row pitch that is not a multiple of 4 elements: no 16-byte vector stores
    (257, 513, 128, 513, 0),        # odd row pitch
])
def test_plain_store_epilogue_as_used_for_a_peer_destination(qm, cuda_clean, oracle, m, n, k, pitch, offset):
    """plain_stores = 1 (what a rank passes when C lives in another GPU's memory): the large-shape kernel writes C with ordinary
    stores (blocks transposed through shared memory into row segments) instead of TMA stores, here into local memory.  Ragged
    edges, a slab of a wider C whose other columns must stay untouched, pitches that rule out vector stores."""
    torch = cuda_clean
    from quadmul_b200.sharded import NShardedGemm

    ap = oracle.fill_packed(m, k, 31); bp = oracle.fill_packed(n, k, 32)
    want = oracle.gemm(ap, bp)
    a, b = to_dev(torch, ap), to_dev(torch, bp)
    wide = torch.full((m, pitch), -5, dtype=torch.int32, device="cuda")
    sh = NShardedGemm(n, world=1, rank=0)
    for _ in range(2):
        sh.local(a, b, m, k, out=wide[:, offset : offset + n], plain_stores=True)
    torch.cuda.synchronize()
    got = wide.cpu().numpy()
    assert np.array_equal(got[:, offset : offset + n], want)
    assert (got[:, :offset] == -5).all() and (got[:, offset + n :] == -5).all()
    assert qm.device_status() == (0, 0)


def test_call_on_a_device_that_is_not_current(qm, cuda_clean, oracle):
    """The reference launches on whichever device is current (extension.cpp:17-23 has no device guard); this mirror
    switches to the operands' device for the call."""
    torch = cuda_clean
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    m, n, k = 300, 520, 512
    ap = oracle.fill_packed(m, k, 31); bp = oracle.fill_packed(n, k, 32)
    a = torch.from_numpy(ap).view(torch.int8).to("cuda:1"); b = torch.from_numpy(bp).view(torch.int8).to("cuda:1")
    c = torch.zeros((m, n), dtype=torch.int32, device="cuda:1")
    assert torch.cuda.current_device() == 0
    qm.gemm(a, b, c, m, n, k)
    torch.cuda.synchronize(1)
    assert torch.cuda.current_device() == 0
    assert np.array_equal(c.cpu().numpy(), oracle.gemm(ap, bp))
    with torch.cuda.device(1):
        code, _ = qm.device_status()
    assert code == 0


def test_completion_flags_signal_then_wait(qm, cuda_clean):
    """qm_flag_signal / qm_flags_wait on one device: flags that were signalled (stream order) satisfy the wait at once."""
    torch = cuda_clean
    from quadmul_b200 import _lib

    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for step in (1, 2, 3):
        for r in range(4):
            assert _lib.LIB.qm_flag_signal(flags.data_ptr() + 4 * r, step, stream) == 0
        assert _lib.LIB.qm_flags_wait(flags.data_ptr(), 4, step, 1000, stream) == 0
    torch.cuda.synchronize()
    assert flags[:4].tolist() == [3, 3, 3, 3]
    assert _lib.LIB.qm_flags_wait(flags.data_ptr(), 4, 2, 1000, stream) == 0  # an older step is satisfied too
    assert _lib.LIB.qm_flags_wait(None, 4, 1, 1000, stream) == 1
    assert _lib.LIB.qm_flags_wait(flags.data_ptr(), 65, 1, 1000, stream) == 8
    assert _lib.LIB.qm_flags_wait(flags.data_ptr(), 4, 1, 0, stream) == 8


def test_completion_flag_that_nobody_raises_times_out(qm, oracle):
    """The wait of the fused gather is bounded: with a flag that no rank ever raises the kernel gives up after its limit,
    returns, and the status word reports QM_ERR_TIMEOUT at the peer-wait site; the context stays usable.  Nothing faults and
    nothing spins without end: the flag simply never arrives."""
    import time

    import torch

    from _util import run_gemm
    from quadmul_b200 import _lib

    qm.device_status(clear=True)
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert _lib.LIB.qm_flag_signal(flags.data_ptr(), 1, stream) == 0  # rank 0 arrives, rank 1 never does
    t0 = time.time()
    assert _lib.LIB.qm_flags_wait(flags.data_ptr(), 2, 1, 200, stream) == 0
    code, where = qm.device_status(clear=True)  # synchronises
    elapsed = time.time() - t0
    assert code == 5 and (where & 0xFF) == 8 and (where >> 8) == 1, (code, where)  # QM_ERR_TIMEOUT, peer wait, flag 1
    assert 0.15 < elapsed < 5.0, elapsed
    ap = oracle.fill_packed(16, 256, 1); bp = oracle.fill_packed(300, 256, 2)
    assert np.array_equal(run_gemm(qm, torch, ap, bp), oracle.gemm(ap, bp))
    assert qm.device_status(clear=True) == (0, 0)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _nccl_worker(rank, world, port, m, n, k, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import quadmul_b200 as qm
    from oracle import oracle as o
    from quadmul_b200.sharded import NShardedGemm

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ap = o.fill_packed(m, k, 5); bp = o.fill_packed(n, k, 6)
        a = torch.from_numpy(ap).view(torch.int8).cuda()
        sh = NShardedGemm(n)
        b = torch.from_numpy(bp[sh.begin : sh.begin + sh.count]).view(torch.int8).cuda()  # a rank holds only its rows of B
        slab = sh.local(a, b, m, k)
        full = sh.gather(slab, m)
        torch.cuda.synchronize()
        want = o.gemm(ap, bp)
        ok = bool(np.array_equal(full.cpu().numpy(), want))
        only = sh.gather_to(slab, m, dst=0)  # NCCL gather to rank 0 alone
        torch.cuda.synchronize()
        ok = ok and ((only is None) if rank != 0 else bool(np.array_equal(only.cpu().numpy(), want)))
        # fused gather: every rank's GEMM epilogue stores its slab into rank 0's C over NVLink
        from quadmul_b200.sharded import SymmetricC

        csym = SymmetricC(m, n)
        csym.local.fill_(-3)
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(2):  # twice: the step number of the completion flags advances
            sh.local_into(a, b, m, k, csym, dst=0)
            if rank == 0:
                csym.wait_all()  # completion flags in rank 0's memory, bounded wait
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            ok = ok and bool(np.array_equal(csym.local.cpu().numpy(), want))
        else:
            ok = ok and bool((csym.local == -3).all())  # nobody wrote into the other ranks' copies
        dist.barrier()
        code, _ = qm.device_status()
        q.put((rank, ok and code == 0))
    finally:
        dist.destroy_process_group()


def test_shards_over_nccl(qm, cuda_clean):
    torch = cuda_clean
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_nccl_worker, args=(r, world, port, 520, 4096 + 128, 1024, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok in results), results
