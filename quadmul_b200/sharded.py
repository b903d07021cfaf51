"""Column-sharded multi-GPU GEMM: one process per GPU, B split by output columns, A replicated.

The reference is single-GPU (one kernel launch, kernel.cu:268-289); this driver is the multi-GPU
form of the same product.  Output columns are independent, so rank r of `world` owns the contiguous
block of B rows [begin, begin + count) given by qm_nshard_range (no repacking: a block of rows of
the packed N x K/2 matrix is itself a packed matrix) and computes the column slab
C[:, begin:begin+count].  The GEMM needs no communication.  Only when the caller asks for the full
C does a collective run: an all-gather of the (padded) slabs over NCCL, followed by one kernel that
un-interleaves [world][m][stride] into row-major C[m][n].

`gemm_fn` / `unshard_fn` default to the CUDA entry points; the CPU tests inject stand-ins so the
partition, padding and assembly logic runs under the gloo backend.
"""
from __future__ import annotations

from typing import Callable, Optional


class NShardedGemm:
    def __init__(self, n: int, *, world: Optional[int] = None, rank: Optional[int] = None, group=None,
                 gemm_fn: Optional[Callable] = None, unshard_fn: Optional[Callable] = None):
        import torch.distributed as dist

        from . import nshard_range

        self.group = group
        if world is None or rank is None:
            if not dist.is_initialized():
                raise RuntimeError("NShardedGemm: pass world and rank, or initialise torch.distributed first")
            world = dist.get_world_size(group)
            rank = dist.get_rank(group)
        if not (0 <= rank < world):
            raise ValueError("NShardedGemm: rank outside [0, world)")
        self.n, self.world, self.rank = int(n), int(world), int(rank)
        self.ranges = [nshard_range(self.n, self.world, r) for r in range(self.world)]
        self.begin, self.count = self.ranges[self.rank]
        self.slab_stride = max(c for _, c in self.ranges) if self.ranges else 0
        self._gemm_fn = gemm_fn
        self._unshard_fn = unshard_fn

    # -- partition ---------------------------------------------------------------------
    def shard_of(self, b_full):
        """This rank's rows of a full packed B (a view, no copy)."""
        if b_full.shape[0] != self.n:
            raise ValueError(f"B has {b_full.shape[0]} rows, expected {self.n}")
        return b_full[self.begin : self.begin + self.count]

    # -- local product -----------------------------------------------------------------
    def local(self, a, b_shard, m: int, k: int, out=None, plain_stores: bool = False):
        """C[:, begin:begin+count] = A @ b_shard^T on this rank's device. `out` may be a padded
        [m, slab_stride] buffer; the slab is written into its first `count` columns.  `plain_stores`
        is for an `out` that is a view of ANOTHER GPU's memory (see SymmetricC)."""
        import torch

        if b_shard.shape[0] != self.count:
            raise ValueError(f"rank {self.rank}: B shard has {b_shard.shape[0]} rows, expected {self.count}")
        if out is None:
            out = torch.empty((m, self.count), dtype=torch.int32, device=a.device)
        if out.shape[0] != m or out.shape[1] < self.count:
            raise ValueError("output slab too small")
        if self.count == 0 or m == 0:
            return out
        if self._gemm_fn is not None:
            self._gemm_fn(a, b_shard, out, m, self.count, k)
        else:
            self._gemm_ldc(a, b_shard, out, m, k, plain_stores)
        return out

    def _gemm_ldc(self, a, b_shard, out, m, k, plain_stores=False):
        import ctypes

        import quadmul_b200 as qm
        from ._lib import LIB, GemmOpts, check

        if not (a.is_cuda and b_shard.is_cuda and out.is_cuda):
            raise ValueError("NShardedGemm.local: CUDA tensors required (there is no CPU path)")
        if out.stride(1) != 1 or not a.is_contiguous() or not b_shard.is_contiguous():
            raise ValueError("NShardedGemm.local: operands must be contiguous, out row-major")
        opts = GemmOpts(plain_stores=1 if plain_stores else 0)
        with qm._on_device(a):
            st = LIB.qm_gemm_s4_ldc_ex(a.data_ptr(), b_shard.data_ptr(), out.data_ptr(), m, self.count, k, out.stride(0),
                                       qm._stream_of(a), ctypes.byref(opts))
        check(st, f"sharded gemm rank {self.rank}")
        qm._launches += 1

    def gather_to(self, slab, m: int, dst: int = 0, out=None):
        """Full row-major C[m, n] on rank `dst` only (NCCL gather = grouped send / receive, then the un-interleave kernel on
        `dst`); returns None on the other ranks.  The library-collective counterpart of `local_into`."""
        import torch
        import torch.distributed as dist

        if self.world == 1:
            return self.gather(slab, m, out=out)
        if slab.shape[1] != self.slab_stride:
            padded = torch.zeros((m, self.slab_stride), dtype=slab.dtype, device=slab.device)
            padded[:, : self.count] = slab[:, : self.count]
            slab = padded
        slab = slab.contiguous()
        if self.rank != dst:
            dist.gather(slab, gather_list=None, dst=dst, group=self.group)
            return None
        slabs = torch.empty((self.world, m, self.slab_stride), dtype=slab.dtype, device=slab.device)
        dist.gather(slab, gather_list=[slabs[r] for r in range(self.world)], dst=dst, group=self.group)
        if out is None:
            out = torch.empty((m, self.n), dtype=slab.dtype, device=slab.device)
        if self._unshard_fn is not None:
            self._unshard_fn(slabs, out, m, self.n, self.world, self.slab_stride)
        else:
            from . import unshard_c

            unshard_c(slabs, out, m, self.n, self.world, self.slab_stride)
        return out

    # -- fused gather: the GEMM epilogue writes straight into the destination rank's C ------------
    def local_into(self, a, b_shard, m: int, k: int, c_sym: "SymmetricC", dst: int = 0):
        """Compute this rank's column slab and store it, from inside the GEMM kernel, into rank `dst`'s
        full-width C (peer-mapped memory, ordinary stores over NVLink; no staging, no NCCL), then raise
        this rank's completion flag on `dst` (stream-ordered after the GEMM).  A collective step: every
        rank calls it once per product.  Rank `dst` calls `c_sym.wait_all()` afterwards: its stream
        continues once every rank's slab has landed, or records a time-out (qm_device_status)."""
        target = c_sym.on_rank(dst)
        if tuple(target.shape) != (m, self.n):
            raise ValueError("SymmetricC shape does not match (m, n)")
        out = self.local(a, b_shard, m, k, out=target[:, self.begin : self.begin + self.count],
                         plain_stores=(dst != self.rank))
        c_sym.signal(dst, self.rank)
        return out

    # -- optional collective -------------------------------------------------------------
    def gather(self, slab, m: int, out=None):
        """Full row-major C[m, n] on every rank from the per-rank column slabs (all-gather + one
        un-interleave kernel).  `slab` is [m, count] or a padded [m, slab_stride] buffer."""
        import torch
        import torch.distributed as dist

        if self.world == 1:
            full = slab[:, : self.count]
            if out is not None:
                out.copy_(full)
                return out
            return full.contiguous()
        if slab.shape[1] != self.slab_stride:
            padded = torch.zeros((m, self.slab_stride), dtype=slab.dtype, device=slab.device)
            padded[:, : self.count] = slab[:, : self.count]
            slab = padded
        slab = slab.contiguous()
        slabs = torch.empty((self.world, m, self.slab_stride), dtype=slab.dtype, device=slab.device)
        dist.all_gather_into_tensor(slabs.view(-1), slab.view(-1), group=self.group)
        if out is None:
            out = torch.empty((m, self.n), dtype=slab.dtype, device=slab.device)
        if self._unshard_fn is not None:
            self._unshard_fn(slabs, out, m, self.n, self.world, self.slab_stride)
        else:
            from . import unshard_c

            unshard_c(slabs, out, m, self.n, self.world, self.slab_stride)
        return out


class SymmetricC:
    """A full-width C [m, n] (int32) allocated collectively so that every rank can address every rank's copy.

    Uses torch's symmetric memory (CUDA virtual-memory handles exchanged inside one node).  `local` is this
    rank's copy, `on_rank(r)` a tensor view of rank r's copy mapped into this process."""

    def __init__(self, m: int, n: int, group=None, device=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        self.m, self.n = int(m), int(n)
        self.group = group if group is not None else dist.group.WORLD
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.local = symm.empty((self.m, self.n), dtype=torch.int32, device=device)
        self.handle = symm.rendezvous(self.local, self.group)
        # one completion word per rank, in every rank's memory; `step` counts the products stored into this buffer
        self.world = dist.get_world_size(self.group)
        self.flags = symm.empty((64,), dtype=torch.int32, device=device)
        self.flags.zero_()
        self.flags_handle = symm.rendezvous(self.flags, self.group)
        self.step = 0
        torch.cuda.synchronize(device)
        self.flags_handle.barrier()  # set-up only: every rank's flags are zero before anyone signals

    def on_rank(self, r: int):
        import torch

        return self.handle.get_buffer(int(r), (self.m, self.n), torch.int32)

    def signal(self, dst: int, rank: int):
        """Stream-ordered: this rank's earlier kernels are complete, system-wide, before word `rank` of rank `dst`'s flags
        takes the new step number (qm_flag_signal).  Advances the step; every rank calls it once per product."""
        import torch

        from ._lib import LIB, check

        self.step += 1
        peer = self.flags_handle.get_buffer(int(dst), (64,), torch.int32)
        check(LIB.qm_flag_signal(peer.data_ptr() + 4 * int(rank), self.step, torch.cuda.current_stream().cuda_stream), "flag_signal")

    def wait_all(self, timeout_ms: int = 5000):
        """On the destination rank: a kernel on the current stream that waits, for at most `timeout_ms`, until every rank
        has signalled the current step (qm_flags_wait).  A time-out is reported by qm_device_status, not by a hang."""
        import torch

        from ._lib import LIB, check

        check(LIB.qm_flags_wait(self.flags.data_ptr(), self.world, self.step, int(timeout_ms),
                                torch.cuda.current_stream().cuda_stream), "flags_wait")

    def barrier(self):
        """Set-up and tests only (torch's symmetric-memory barrier): all ranks' earlier work on the current streams is
        complete when this returns on the stream.  The data path uses signal / wait_all."""
        self.handle.barrier()
