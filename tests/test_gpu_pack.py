"""Parity of the pack / unpack / fill / unshard kernels with the oracle (bit-exact), through the C ABI."""
import numpy as np
import pytest

from _util import to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,k", [(1, 2), (3, 34), (128, 256), (257, 1000), (1024, 4096), (5, 16384 + 6)])
def test_pack_unpack_vs_oracle(qm, cuda_clean, oracle, rows, k):
    torch = cuda_clean
    x = oracle.random_s4(rows, k, rows + k)
    x[0, 0], x[-1, -1] = -8, 7
    p = qm.pack(to_dev(torch, x))
    assert p.dtype == torch.int8 and tuple(p.shape) == (rows, k // 2)
    assert np.array_equal(p.cpu().numpy().view(np.uint8), oracle.pack(x))
    u = qm.unpack(p)
    assert np.array_equal(u.cpu().numpy(), x)
    assert np.array_equal(u.cpu().numpy(), oracle.unpack(oracle.pack(x)))


def test_golden_pack_unpack(qm, cuda_clean, golden):
    torch = cuda_clean
    for name, g in golden.items():
        for op in ("a", "b"):
            p = qm.pack(to_dev(torch, g[op]))
            assert np.array_equal(p.cpu().numpy().view(np.uint8), g[op + "_packed"]), name
            u = qm.unpack(to_dev(torch, g[op + "_packed"]))
            assert np.array_equal(u.cpu().numpy(), g[op + "_unpacked"]), name


def test_unaligned_views_take_the_scalar_path(qm, cuda_clean, oracle):
    torch = cuda_clean
    from quadmul_b200 import _lib

    rows, k = 7, 70
    x = oracle.random_s4(rows, k, 3)
    buf = torch.zeros(rows * k + 32, dtype=torch.int8, device="cuda")
    xin = buf[3 : 3 + rows * k]
    xin.copy_(to_dev(torch, x).flatten())
    out = torch.zeros(rows * k // 2 + 8, dtype=torch.int8, device="cuda")
    assert _lib.LIB.qm_pack_s4(xin.data_ptr(), out.data_ptr() + 1, rows, k, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out[1 : 1 + rows * k // 2].cpu().numpy().view(np.uint8).reshape(rows, k // 2), oracle.pack(x))


def test_all_256_byte_values_unpack(qm, cuda_clean, oracle):
    torch = cuda_clean
    p = np.arange(256, dtype=np.uint8).reshape(1, 256).repeat(4, 0)
    u = qm.unpack(to_dev(torch, p))
    assert np.array_equal(u.cpu().numpy(), oracle.unpack(p))
    assert np.array_equal(qm.pack(u).cpu().numpy().view(np.uint8), p)


def test_fill_matches_oracle_generator(qm, cuda_clean, oracle):
    for rows, k, seed in [(64, 256, 1), (3, 38, 99), (1000, 1024, 2**40 + 5)]:
        got = qm.fill_packed(rows, k, seed).cpu().numpy().view(np.uint8)
        assert np.array_equal(got, oracle.fill_packed(rows, k, seed))


def test_large_roundtrip_properties(qm, cuda_clean):
    torch = cuda_clean
    rows, k = 8192, 8192
    p = qm.fill_packed(rows, k, 5)
    u = qm.unpack(p)
    assert int(u.min()) == -8 and int(u.max()) == 7
    assert torch.equal(qm.pack(u), p)  # pack(unpack(p)) = p for every byte
    # checksum of nibbles: sum over elements equals sum over low + high nibbles sign-extended
    lo = (p.to(torch.int16) << 12 >> 12).sum(dtype=torch.int64)
    hi = (p.to(torch.int16) >> 4).sum(dtype=torch.int64)
    assert int(u.sum(dtype=torch.int64)) == int(lo + hi)


@pytest.mark.parametrize("m,n,world", [(16, 1024, 2), (5, 11008, 4), (3, 1000, 3), (8, 256, 8)])
def test_unshard(qm, cuda_clean, m, n, world):
    torch = cuda_clean
    full = torch.arange(m * n, dtype=torch.int32, device="cuda").view(m, n)
    ranges = [qm.nshard_range(n, world, r) for r in range(world)]
    stride = max(c for _, c in ranges)
    slabs = torch.full((world, m, stride), -1, dtype=torch.int32, device="cuda")
    for r, (b, c) in enumerate(ranges):
        slabs[r, :, :c] = full[:, b : b + c]
    out = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    qm.unshard_c(slabs, out, m, n, world, stride)
    torch.cuda.synchronize()
    assert torch.equal(out, full)
