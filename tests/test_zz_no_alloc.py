"""qm_gemm_s4_static_scratch: the split-K GEMM for callers that cannot allocate device memory.

Some users of this library run where cudaMalloc is off limits: inside a host framework that owns
all device memory, under a fixed memory budget, or in a loop that cannot afford an allocation's
stall.  For them the library carries its split-K scratch as built-in device arrays.  This test calls that entry point through the C ABI twice in a row and
requires both results to equal, bit for bit, what the ordinary entry point (qm_gemm_s4_ex, scratch
from cudaMalloc) gives for the same operands and the same number of K partitions; it also checks
that a request beyond the built-in capacity is refused with QM_ERR_WORKSPACE rather than run."""
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k,split_k", [(16, 4096, 4096, 4), (64, 1280, 2048, 3), (1, 11008, 4096, 2)])
def test_static_scratch_matches_allocating_entry_point(qm, cuda_clean, m, n, k, split_k):
    torch = cuda_clean
    from quadmul_b200 import _lib

    a = qm.fill_packed(m, k, 91)
    b = qm.fill_packed(n, k, 92)
    want = torch.empty((m, n), dtype=torch.int32, device="cuda")
    plan = qm.plan(m, n, k)
    qm.gemm_ex(a, b, want, m, n, k, kernel=1, tile_n=plan["tile_n"], swap_ab=plan["swap_ab"], cta_pair=1, split_k=split_k)
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        got = torch.full((m, n), -77, dtype=torch.int32, device="cuda")
        st = _lib.LIB.qm_gemm_s4_static_scratch(a.data_ptr(), b.data_ptr(), got.data_ptr(), m, n, k, split_k, stream)
        assert st == 0, _lib.LIB.qm_status_string(st)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}: {(got != want).sum().item()} outputs differ"


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
