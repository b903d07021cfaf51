"""The reference's own pybind file, extension.cpp, compiled UNCHANGED against this library.

The drop-in claim is that a maintainer of the reference removes kernel.cu, configs.cu and helpers.cu from
setup.py:10-13, links -lquadmul_b200 instead, and changes no source line: `wrapper` (declared at
extension.cpp:6, called at extension.cpp:17-23) then resolves to this library's symbol of the same signature.
oracle.build_ref_extension does exactly that build, from the sources where they lie (never copied), into
oracle/_ref/ext/quadmul.so.  The CPU test builds and imports it; the GPU test calls its `gemm` (the
reference's call, extension.cpp:8) on a golden fixture, on the reference's own 1024^3 smoke size and on a shape
the reference's dispatch table never had, against the oracle."""
import numpy as np
import pytest


def test_reference_extension_builds_and_imports_unchanged(oracle, qm):
    if oracle.reference_dir() is None and oracle.ref_extension() is None:
        pytest.skip("the reference's sources are not on this machine and no earlier build is present")
    path = oracle.build_ref_extension()
    assert path is not None
    mod = oracle.ref_extension()
    assert mod is not None and callable(mod.gemm)
    assert "Int4xInt4" in (mod.gemm.__doc__ or "")  # the doc string of extension.cpp:28


@pytest.mark.gpu
def test_reference_extension_runs_on_this_library(oracle, qm, cuda_clean, golden):
    torch = cuda_clean
    mod = oracle.ref_extension()
    if mod is None:
        pytest.skip("oracle/_ref/ext/quadmul.so was not built (the reference's sources were absent at build time)")
    g = golden["block_128x256x256"]
    cases = [(g["a_packed"], g["b_packed"], g["c"])]
    for m, n, k in [(1024, 1024, 1024), (300, 520, 1056), (16, 4096, 4096)]:
        ap = oracle.fill_packed(m, k, 71); bp = oracle.fill_packed(n, k, 72)
        cases.append((ap, bp, oracle.gemm(ap, bp)))
    for ap, bp, want in cases:
        m, n, k = ap.shape[0], bp.shape[0], ap.shape[1] * 2
        a = torch.from_numpy(np.ascontiguousarray(ap)).view(torch.int8).cuda()
        b = torch.from_numpy(np.ascontiguousarray(bp)).view(torch.int8).cuda()
        c = torch.full((m, n), -5, dtype=torch.int32, device="cuda")
        assert mod.gemm(a, b, c, m, n, k) is None  # the reference's call returns nothing (extension.cpp:8)
        torch.cuda.synchronize()
        assert np.array_equal(c.cpu().numpy(), want), (m, n, k)
