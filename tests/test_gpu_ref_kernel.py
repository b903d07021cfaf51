"""Bit-exact agreement with the REFERENCE'S OWN CUDA kernel, where it was compiled (oracle/_ref).

The reference binary is built from the unmodified reference sources; these tests are skipped
where it is absent.  Shapes: one from the reference's dispatch table (kernel.cu:343-384) through its
own `wrapper`, and sizes it does not list through extra instantiations of its kernel template."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _ref(oracle):
    L = oracle.ref_lib()
    if L is None:
        pytest.skip("reference build (oracle/_ref) not present")
    return L


def test_reference_dispatch_table_shape(qm, cuda_clean, oracle):
    torch = cuda_clean
    L = _ref(oracle)
    m, n, k = 256, 6144, 4096  # configs.cu: quadmul_256_6144_4096
    a = qm.fill_packed(m, k, 71); b = qm.fill_packed(n, k, 72)
    c_ref = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    c = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    L.qm_ref_wrapper(a.data_ptr(), b.data_ptr(), c_ref.data_ptr(), m, n, k, None)
    qm.gemm(a, b, c, m, n, k)
    torch.cuda.synchronize()
    assert int(c_ref.abs().max()) > 0, "the reference kernel wrote nothing"
    assert torch.equal(c, c_ref)


@pytest.mark.parametrize("m,n,k", [(1024, 1024, 1024), (16, 4096, 4096), (64, 11008, 4096)])
def test_reference_kernel_extra_instantiations(qm, cuda_clean, oracle, m, n, k):
    torch = cuda_clean
    L = _ref(oracle)
    a = qm.fill_packed(m, k, 73); b = qm.fill_packed(n, k, 74)
    c_ref = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    c = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    assert L.qm_ref_gpu_gemm(a.data_ptr(), b.data_ptr(), c_ref.data_ptr(), m, n, k, None) == 0
    qm.gemm(a, b, c, m, n, k)
    torch.cuda.synchronize()
    assert torch.equal(c, c_ref)
    ap = a.cpu().numpy().view(np.uint8); bp = b.cpu().numpy().view(np.uint8)
    assert np.array_equal(c_ref[:8].cpu().numpy(), oracle.gemm(ap, bp, rows=(0, 8)))
