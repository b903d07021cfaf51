"""qm_gemm_s4_static_scratch: the split-K GEMM for callers that cannot allocate device memory.

Some users of this library run where cudaMalloc is off limits: inside a host framework that owns
all device memory, under a fixed memory budget, or in a loop that cannot afford an allocation's
stall.  For them the library carries its split-K scratch as built-in device arrays.  This test calls
that entry point through the C ABI twice in a row and requires both results to equal, bit for bit,
the CPU oracle and what the ordinary entry point (qm_gemm_s4_ex, scratch from cudaMalloc) gives for
the same operands and the same number of K partitions.  It also checks that the free device memory
does not move across the calls after the first, that the entry point's own status word stays clear,
and that a request beyond the built-in capacity is refused with QM_ERR_WORKSPACE rather than run."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_bytes(torch):
    # cudaMemGetInfo through torch: (free, total) of the current device
    return torch.cuda.mem_get_info()[0]


@pytest.mark.parametrize("m,n,k,split_k", [(16, 4096, 4096, 4), (64, 1280, 2048, 3), (1, 11008, 4096, 2), (128, 1024, 2048, 2),
                                           (200, 520, 1056, 3)])
def test_static_scratch_matches_oracle_and_allocating_entry_point(qm, cuda_clean, oracle, m, n, k, split_k):
    torch = cuda_clean
    from quadmul_b200 import _lib

    ap = oracle.fill_packed(m, k, 91); bp = oracle.fill_packed(n, k, 92)
    want_cpu = oracle.gemm(ap, bp)
    a = torch.from_numpy(ap).view(torch.int8).cuda(); b = torch.from_numpy(bp).view(torch.int8).cuda()
    want = torch.empty((m, n), dtype=torch.int32, device="cuda")
    plan = qm.plan(m, n, k)
    tile_n = plan["tile_n"] if plan["swap_ab"] == 2 else 128
    qm.gemm_ex(a, b, want, m, n, k, kernel=1, tile_n=tile_n, swap_ab=plan["swap_ab"], cta_pair=1, split_k=split_k)
    torch.cuda.synchronize()
    assert np.array_equal(want.cpu().numpy(), want_cpu)
    stream = torch.cuda.current_stream().cuda_stream
    outs = [torch.full((m, n), -77, dtype=torch.int32, device="cuda") for _ in range(3)]  # allocated before the calls
    free_before = None
    for call, got in enumerate(outs):
        st = _lib.LIB.qm_gemm_s4_static_scratch(a.data_ptr(), b.data_ptr(), got.data_ptr(), m, n, k, split_k, stream)
        assert st == 0, _lib.LIB.qm_status_string(st)
        torch.cuda.synchronize()
        if call == 0:
            free_before = _free_bytes(torch)  # the first call on a device may load the module and resolve the symbols
        else:
            assert _free_bytes(torch) == free_before, "device memory moved across a call that must not allocate"
        assert torch.equal(got, want), f"call {call}: {(got != want).sum().item()} outputs differ from the allocating entry point"
        assert np.array_equal(got.cpu().numpy(), want_cpu), f"call {call}: differs from the oracle"
    assert qm.static_scratch_status(clear=True) == (0, 0)


def test_static_scratch_rejects_what_does_not_fit(qm, cuda_clean):
    torch = cuda_clean
    from quadmul_b200 import _lib

    m, n, k = 128, 8192, 4096  # 64 tiles x 8 partitions x 64 KiB = 32 MiB of partial tiles > 8 MiB
    a = qm.fill_packed(m, k, 1); b = qm.fill_packed(n, k, 2)
    c = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    st = _lib.LIB.qm_gemm_s4_static_scratch(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, 8, None)
    assert st == 7  # QM_ERR_WORKSPACE
    assert _lib.LIB.qm_gemm_s4_static_scratch(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, 30, 1, None) == 3  # QM_ERR_ALIGN
    assert _lib.LIB.qm_gemm_s4_static_scratch(None, b.data_ptr(), c.data_ptr(), m, n, k, 1, None) == 1
    torch.cuda.synchronize()
    assert int(c.abs().max()) == 0  # nothing ran
    code, where = ctypes.c_int(-1), ctypes.c_int(-1)
    assert _lib.LIB.qm_static_scratch_status(ctypes.byref(code), ctypes.byref(where), 1) == 0
    assert (code.value, where.value) == (0, 0)
