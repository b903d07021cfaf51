"""The reference's own shape list (test.py:130-187: eight (N, K) blocks x M in 128 ... 4096, the nine rows it comments
out included) through the drop-in call `quadmul.gemm`, bit for bit.

The reference checks each shape against cuBLASLt int8 with a tolerance of 1 before it times it (test.py:39-43).  Here
every shape is compared (a) with the CPU oracle on two full rows and 2048 sampled points, tile seams included, and (b)
in full with an independent GPU computation: the unpack kernel followed by cuBLASLt int8 (torch._int_mm).  Inputs are the
counter-based generator's nibbles, uniform on [-8, 7] (the reference draws from [-8, 6], test.py:22-24)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NK = [(10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672), (6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]
MS = [128, 256, 512, 1024, 2048, 4096]


@pytest.mark.parametrize("n,k", NK)
def test_reference_shape_block(qm, cuda_clean, oracle, n, k):
    torch = cuda_clean
    import quadmul  # the reference's module name (setup.py:8,11)

    b = qm.fill_packed(n, k, 7000 + n % 97)
    bp = b.cpu().numpy().view(np.uint8)
    ub = qm.unpack(b).t()
    rng = np.random.default_rng(n + k)
    for m in MS:
        a = qm.fill_packed(m, k, 6000 + m)
        c = torch.full((m, n), -3, dtype=torch.int32, device="cuda")
        quadmul.gemm(a, b, c, m, n, k)
        ref = torch._int_mm(qm.unpack(a), ub)
        torch.cuda.synchronize()
        assert torch.equal(c, ref), f"{m}x{n}x{k}: {int((c != ref).sum())} outputs differ from unpack + cuBLASLt int8"
        ap = a.cpu().numpy().view(np.uint8)
        # two full rows (first and last) and sampled points: seams of 192- and 256-wide tiles, the last row and column
        for r in (0, m - 1):
            assert np.array_equal(c[r].cpu().numpy(), oracle.gemm(ap[r : r + 1], bp)[0]), f"{m}x{n}x{k}: row {r} differs from the oracle"
        rows = np.concatenate([rng.integers(0, m, 1792), np.full(256, m - 1)])
        seams = np.concatenate([np.arange(191, n, 192)[:64], np.arange(192, n, 192)[:64], np.arange(255, n, 256)[:64], np.arange(256, n, 256)[:64]])
        cols = np.concatenate([rng.integers(0, n, 2048 - len(seams)), seams])
        got = c[torch.from_numpy(rows).cuda(), torch.from_numpy(cols).cuda()].cpu().numpy().astype(np.int64)
        assert np.array_equal(got, oracle.gemm_points(ap, bp, rows, cols)), f"{m}x{n}x{k}: sampled points differ from the oracle"
        del a, c, ref
