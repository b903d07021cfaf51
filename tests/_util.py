"""Helpers shared by the GPU parity tests."""
import numpy as np


def to_dev(torch, arr):
    """numpy uint8/int8/int32 array -> CUDA tensor (packed bytes travel as int8, like the reference's pack_b output)."""
    t = torch.from_numpy(np.ascontiguousarray(arr))
    if t.dtype == torch.uint8:
        t = t.view(torch.int8)
    return t.cuda()


def run_gemm(qm, torch, ap, bp, m=None, n=None, k=None, **opts):
    """Run the product GEMM on packed numpy operands; returns C as numpy int32.
    C is pre-filled with a sentinel so unwritten outputs show."""
    m = ap.shape[0] if m is None else m
    n = bp.shape[0] if n is None else n
    k = ap.shape[1] * 2 if k is None else k
    a, b = to_dev(torch, ap), to_dev(torch, bp)
    c = torch.full((m, n), -123456789, dtype=torch.int32, device="cuda")
    if opts:
        qm.gemm_ex(a, b, c, m, n, k, **opts)
    else:
        qm.gemm(a, b, c, m, n, k)
    torch.cuda.synchronize()
    return c.cpu().numpy()


def mismatch_report(got, want, limit=5):
    bad = np.argwhere(got != want)
    head = [(tuple(i), int(got[tuple(i)]), int(want[tuple(i)])) for i in bad[:limit]]
    return f"{len(bad)} of {got.size} outputs differ; first (index, got, want): {head}"
