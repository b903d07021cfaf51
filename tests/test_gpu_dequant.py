"""GPU parity of the fused dequantising GEMM (qm_gemm_s4_dequant_bf16) against the oracle, bit for bit.

The oracle is the exact int32 product (oracle.gemm) followed by oracle.dequant_bf16, the restatement of the epilogue
contract: float32(sum) * scale_a[row] * scale_b[col] -> bfloat16, round to nearest even at every step."""
import ctypes

import numpy as np
import pytest

from _util import to_dev

pytestmark = pytest.mark.gpu


def _scales(rng, count):
    return rng.uniform(1e-3, 0.5, size=count).astype(np.float32)


def _run(qm, torch, ap, bp, sa, sb, out=None, workspace=None):
    m, n, k = ap.shape[0], bp.shape[0], ap.shape[1] * 2
    a, b = to_dev(torch, ap), to_dev(torch, bp)
    if out is None:
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    qm.gemm_dequant(a, b, None if sa is None else torch.from_numpy(sa).cuda(), None if sb is None else torch.from_numpy(sb).cuda(),
                    out, m, n, k, workspace=workspace)
    torch.cuda.synchronize()
    return out


def _bits(t):
    import torch

    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("m,n,k,fused", [
    (512, 512, 512, True),       # the 256 x 256 pair kernel converts in its epilogue
    (300, 520, 1056, True),      # ragged rows and columns, K tail inside a stage
    (1000, 1000, 2048, True),
    (257, 136, 64, True),        # one row and eight columns into the second tile
    (300, 516, 512, False),      # row pitch not a multiple of 8 elements: int32 product + second pass
    (16, 1024, 1024, True),      # register-resident mma.sync kernel
    (16, 2048, 8448, True),      # decode kernel, K partitions through scratch, converts when the last partition sums
    (64, 4096, 512, True),       # decode kernel, K partitions as one cluster
    (7, 11008, 1024, True),      # decode kernel, two CTAs per SM, ragged tokens
    (40, 300, 96, True),         # decode kernel, unsplit
    (1, 4096, 1024, True),       # dp4a row kernel
    (3, 1001, 256, True),
    (5, 38016, 512, True),       # decode kernel, equal shares
    (200, 100, 512, False),      # narrow output: single-CTA tile + second pass
    (33, 47, 30, False),         # dp4a kernel + second pass
])
def test_dequant_matches_the_oracle(qm, cuda_clean, oracle, m, n, k, fused):
    torch = cuda_clean
    rng = np.random.default_rng(m * 7 + n)
    ap, bp = oracle.fill_packed(m, k, 81), oracle.fill_packed(n, k, 82)
    sa, sb = _scales(rng, m), _scales(rng, n)
    from quadmul_b200._lib import LIB

    assert (LIB.qm_gemm_s4_dequant_workspace_bytes(m, n, k, n, 0) == 0) == fused
    acc = oracle.gemm(ap, bp)
    for use_a, use_b in ((True, True), (False, True), (True, False), (False, False)):
        got = _bits(_run(qm, torch, ap, bp, sa if use_a else None, sb if use_b else None))
        want = oracle.dequant_bf16(acc, sa if use_a else None, sb if use_b else None)
        bad = np.argwhere(got != want)
        assert bad.size == 0, f"{len(bad)} of {got.size} differ, first {bad[:3].tolist()}: got {got[tuple(bad[0])]:#06x} want {want[tuple(bad[0])]:#06x}"


def test_dequant_writes_a_column_slab_and_leaves_the_rest(qm, cuda_clean, oracle):
    torch = cuda_clean
    rng = np.random.default_rng(3)
    m, n, k, wide, off = 384, 256, 512, 1024, 512
    ap, bp = oracle.fill_packed(m, k, 83), oracle.fill_packed(n, k, 84)
    sa, sb = _scales(rng, m), _scales(rng, n)
    full = torch.full((m, wide), 7.0, dtype=torch.bfloat16, device="cuda")
    _run(qm, torch, ap, bp, sa, sb, out=full[:, off : off + n])
    want = oracle.dequant_bf16(oracle.gemm(ap, bp), sa, sb)
    assert np.array_equal(_bits(full[:, off : off + n]), want)
    rest = torch.cat([full[:, :off], full[:, off + n :]], dim=1)
    assert bool((rest == 7.0).all())


def test_dequant_large_fused_against_the_second_pass(qm, cuda_clean, oracle):
    """4096 x 4096 x 4096: the fused kernel against the oracle on row slabs, and against the composed path everywhere."""
    torch = cuda_clean
    rng = np.random.default_rng(11)
    m = n = k = 4096
    ap, bp = oracle.fill_packed(m, k, 85), oracle.fill_packed(n, k, 86)
    sa, sb = _scales(rng, m), _scales(rng, n)
    got = _run(qm, torch, ap, bp, sa, sb)
    a, b = to_dev(torch, ap), to_dev(torch, bp)
    c = torch.empty((m, n), dtype=torch.int32, device="cuda")
    qm.gemm(a, b, c, m, n, k)
    ref = ((c.to(torch.float32) * torch.from_numpy(sa).cuda()[:, None]) * torch.from_numpy(sb).cuda()[None, :]).to(torch.bfloat16)
    assert torch.equal(got.view(torch.int16), ref.view(torch.int16))
    for r0 in (0, 1900, 4096 - 64):
        acc = oracle.gemm(ap, bp, rows=(r0, r0 + 64))
        want = oracle.dequant_bf16(acc, sa[r0 : r0 + 64], sb)
        assert np.array_equal(_bits(got[r0 : r0 + 64]), want)


def test_dequant_reports_a_missing_workspace(qm, cuda_clean, oracle):
    torch = cuda_clean
    from quadmul_b200._lib import LIB

    m, n, k = 200, 100, 256  # narrow output: no fused epilogue, the int32 product needs the workspace
    a, b = to_dev(torch, oracle.fill_packed(m, k, 1)), to_dev(torch, oracle.fill_packed(n, k, 2))
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    st = LIB.qm_gemm_s4_dequant_bf16(a.data_ptr(), b.data_ptr(), None, None, out.data_ptr(), m, n, k, n, None, 0, None)
    assert st == 7  # QM_ERR_WORKSPACE
    small = torch.empty(m * n - 1, dtype=torch.int32, device="cuda")
    st = LIB.qm_gemm_s4_dequant_bf16(a.data_ptr(), b.data_ptr(), None, None, out.data_ptr(), m, n, k, n, small.data_ptr(),
                                     small.numel() * 4, None)
    assert st == 7
    torch.cuda.synchronize()
