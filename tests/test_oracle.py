"""The oracle against the reference's own outputs (CPU only).

tests/golden/*.npz were produced by the reference's compiled cpu_gemm_int8 / unpack_int4_matrix and
its Python pack_b (see tests/golden/make_golden.py); here the C oracle and its numpy twin have to
reproduce them bit for bit."""
import numpy as np
import pytest


def test_golden_pack_unpack(oracle, golden):
    for name, g in golden.items():
        for op in ("a", "b"):
            x, xp = g[op], g[op + "_packed"]
            assert np.array_equal(oracle.pack(x), xp), name
            assert np.array_equal(oracle.np_pack(x), xp), name
            assert np.array_equal(oracle.unpack(xp), g[op + "_unpacked"]), name
            assert np.array_equal(oracle.np_unpack(xp), g[op + "_unpacked"]), name


def test_golden_gemm(oracle, golden):
    for name, g in golden.items():
        c = oracle.gemm(g["a_packed"], g["b_packed"])
        assert c.dtype == np.int32 and np.array_equal(c, g["c"]), name
        assert np.array_equal(oracle.np_gemm(g["a_packed"], g["b_packed"]), g["c"]), name


def test_golden_extremes_values(golden):
    g = golden["extremes_16x24x256"]
    assert g["c"].max() == 64 * 256 and g["c"].min() == -56 * 256
    ap = golden["allpairs_16x16x32"]
    v = np.arange(-8, 8)
    assert np.array_equal(ap["c"], 32 * np.outer(v, v))


def test_row_slab_and_points(oracle):
    a = oracle.pack(oracle.random_s4(40, 96, 1))
    b = oracle.pack(oracle.random_s4(24, 96, 2))
    full = oracle.gemm(a, b)
    assert np.array_equal(oracle.gemm(a, b, rows=(8, 31)), full[8:31])
    rows = np.array([0, 5, 39, 17]); cols = np.array([23, 0, 11, 11])
    assert np.array_equal(oracle.gemm_points(a, b, rows, cols), full[rows, cols].astype(np.int64))


def test_nibble_rules(oracle):
    # kernel.cu:387: nibble x > 7 means x - 16; test.py:14: even element in the low nibble
    p = np.array([[0x8F, 0x70, 0x07]], dtype=np.uint8)
    assert oracle.unpack(p).tolist() == [[-1, -8, 0, 7, 7, 0]]
    assert oracle.pack(np.array([[-1, -8, 0, 7, 7, 0]], dtype=np.int8)).tolist() == [[0x8F, 0x70, 0x07]]
    with pytest.raises(ValueError):
        oracle.pack(np.array([[8, 0]], dtype=np.int8))


def test_generator(oracle):
    p = oracle.fill_packed(64, 256, 1234)
    u = oracle.unpack(p)
    assert u.min() == -8 and u.max() == 7
    assert all(oracle.value(1234, r, c, 256) == u[r, c] for r, c in [(0, 0), (3, 5), (63, 255), (17, 128)])
    hist = np.bincount(u.ravel() + 8, minlength=16) / u.size
    assert abs(hist - 1 / 16).max() < 0.01


def test_int64_accumulate_matches_int32_where_defined(oracle):
    # the largest magnitude the reference's int32 accumulator sees at K = 32768 is 64 * K = 2^21
    a = np.full((2, 32768), -8, np.int8); b = np.full((3, 32768), -8, np.int8)
    assert (oracle.gemm(oracle.pack(a), oracle.pack(b)) == 64 * 32768).all()


def test_against_reference_binary_if_present(oracle):
    if oracle.ref_lib() is None:
        pytest.skip("reference build (oracle/_ref) not present")
    for seed, (m, n, k) in enumerate([(7, 9, 34), (64, 48, 256), (33, 130, 1000)]):
        a = oracle.random_s4(m, k, 10 + seed); b = oracle.random_s4(n, k, 20 + seed)
        ap, bp = oracle.pack(a), oracle.pack(b)
        assert np.array_equal(oracle.ref_unpack(ap), a) and np.array_equal(oracle.ref_unpack(bp), b)
        assert np.array_equal(oracle.ref_cpu_gemm(a, b), oracle.gemm(ap, bp))


def test_dequant_restatement_rounds_like_torch(oracle):
    """int32 -> float32 -> two float32 products -> bfloat16 (nearest even): numpy restatement against torch on the CPU."""
    import torch

    rng = np.random.default_rng(5)
    acc = rng.integers(-(2**31), 2**31 - 1, size=(37, 53), dtype=np.int64).astype(np.int32)
    acc[0, :8] = [0, 1, -1, 2**24 + 1, -(2**24) - 1, 2**31 - 1, -(2**31), 12345678]
    sa = rng.uniform(1e-3, 2.0, size=37).astype(np.float32)
    sb = rng.uniform(1e-3, 2.0, size=53).astype(np.float32)
    got = oracle.dequant_bf16(acc, sa, sb)
    t = (torch.from_numpy(acc).to(torch.float32) * torch.from_numpy(sa)[:, None]) * torch.from_numpy(sb)[None, :]
    want = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got, want)
    ones = oracle.dequant_bf16(acc, None, None)
    want1 = torch.from_numpy(acc).to(torch.float32).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(ones, want1)
