"""The C-ABI library loads without a GPU, exports what include/quadmul_b200.h declares, and rejects
bad arguments before touching CUDA (CPU only; no compute calls)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "quadmul_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qm_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(qm):
    from quadmul_b200 import _lib

    names = _declared()
    assert len(names) >= 14
    for n in names:
        assert hasattr(_lib.LIB, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert hasattr(_lib.LIB, _lib.WRAPPER_MANGLED), "C++ symbol wrapper(void*,void*,void*,int,int,int,cudaStream_t) missing"


def test_status_strings(qm):
    from quadmul_b200 import _lib

    assert _lib.LIB.qm_status_string(0) == b"QM_OK"
    for s in range(1, 9):
        assert _lib.LIB.qm_status_string(s).startswith(b"QM_ERR_")
    assert _lib.LIB.qm_version() >= 100


def test_argument_errors_do_not_need_a_gpu(qm):
    from quadmul_b200 import _lib

    L = _lib.LIB
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    assert L.qm_gemm_s4(p, p, p, 4, 4, 7, None) == 2      # k odd
    assert L.qm_gemm_s4(p, p, p, -1, 4, 8, None) == 2     # negative m
    assert L.qm_gemm_s4(None, p, p, 4, 4, 8, None) == 1   # NULL A
    assert L.qm_gemm_s4(p, p, None, 4, 4, 8, None) == 1   # NULL C
    assert L.qm_gemm_s4(p, p, p, 0, 4, 8, None) == 0      # empty product: nothing to do
    assert L.qm_gemm_s4(p, p, p, 4, 0, 8, None) == 0
    assert L.qm_gemm_s4_ldc(p, p, p, 4, 4, 8, 3, None) == 2  # ldc < n
    assert L.qm_pack_s4(p, p, 2, 3, None) == 2
    assert L.qm_pack_s4(None, p, 2, 4, None) == 1
    assert L.qm_pack_s4(None, None, 0, 4, None) == 0
    assert L.qm_unpack_s4(p, None, 2, 4, None) == 1
    assert L.qm_fill_s4(None, 2, 4, 1, None) == 1
    assert L.qm_gemm_s4_host(p, p, p, 2, 2, 3) == 2


def test_nshard_range_partitions(qm):
    for n, world in [(32768, 1), (32768, 2), (32768, 8), (11008, 4), (4096, 8), (1000, 3), (256, 8), (7, 8), (0, 2)]:
        pos = 0
        for r in range(world):
            b, c = qm.nshard_range(n, world, r)
            assert b == pos and c >= 0
            pos += c
        assert pos == n
    b, c = qm.nshard_range(32768, 8, 3)
    assert (b, c) == (12288, 4096)
    # whole 128-column units where n allows
    assert all(qm.nshard_range(11008, 4, r)[1] % 128 == 0 for r in range(4))
    with pytest.raises(qm.QuadmulError):
        qm.nshard_range(128, 4, 4)


def test_plan(qm):
    from quadmul_b200 import _lib

    p = qm.plan(8192, 8192, 8192)
    assert p["kernel"] == _lib.QM_KERNEL_TC and p["tile_n"] == 256 and p["swap_ab"] == 1 and p["cta_pair"] == 2 and p["a_tmem"] == 2
    assert qm.plan(128, 4096, 4096)["a_tmem"] == 2 and qm.plan(128, 4096, 4096)["split_k"] == 4
    d = qm.plan(16, 4096, 16384)  # decode shape beyond the K limit of the register-resident kernel
    assert d["kernel"] == _lib.QM_KERNEL_TC and d["swap_ab"] == 2 and d["tile_n"] >= 16 and d["a_tmem"] == 2
    assert d["stream_k"] == 1 and d["ctas_per_sm"] == 1 and d["split_k"] == 4
    big = qm.plan(16, 57344, 8192)  # more tiles than CTA slots: equal shares, two CTAs per SM
    assert big["stream_k"] == 2 and big["ctas_per_sm"] == 2
    assert qm.plan(16, 11008, 16384)["ctas_per_sm"] == 2 and qm.plan(16, 11008, 16384)["split_k"] == 3  # K above the register kernel's limit
    wide = qm.plan(64, 4096, 8192)  # wide token tile (K above the register kernel's limit): K partitions as one cluster
    assert wide["stream_k"] == 3 and wide["split_k"] == 4 and wide["tile_n"] == 64
    # which decode family takes a swept shape is the sweep's business (test_plan_follows_the_sweep_and_the_cost_model);
    # here only what the families' limits force
    assert qm.plan(65, 4096, 4096)["kernel"] == _lib.QM_KERNEL_TC and qm.plan(33, 4096, 8192)["kernel"] == _lib.QM_KERNEL_TC
    assert qm.plan(1, 4096, 4096)["kernel"] in (_lib.QM_KERNEL_RMMA, _lib.QM_KERNEL_GEMV)
    # clusters of K partitions: the largest size of which the device holds as many as there are tiles
    assert qm.plan(64, 6144, 8192)["stream_k"] == 3 and qm.plan(64, 6144, 8192)["split_k"] == 2   # 48 tiles: 3 would not fit
    assert qm.plan(64, 5120, 8192)["split_k"] == 3 and qm.plan(64, 4608, 8192)["split_k"] == 3    # 40 and 36 tiles
    # 160 tiles on 74 CTA pairs: the 12 tiles of the third round run as K partitions; 8192^3 (62 tiles in the last round) does not
    assert qm.plan(1024, 10240, 8192)["stream_k"] == 2 and qm.plan(1024, 10240, 8192)["split_k"] == 1
    assert qm.plan(8192, 8192, 8192)["stream_k"] == 1 and qm.plan(2048, 4096, 4096)["stream_k"] == 1
    assert qm.plan(5, 7, 30)["kernel"] == _lib.QM_KERNEL_SIMT      # k % 32 != 0
    assert qm.plan(8, 8, 131072)["kernel"] == _lib.QM_KERNEL_SIMT  # 256 x sum would leave int32
    with pytest.raises(qm.QuadmulError):
        qm.plan(4, 4, 3)


def test_plan_is_consistent_over_a_grid_of_shapes(qm):
    """Every plan the table produces must be launchable: known tile widths, K partitions no more than K blocks,
    the pair tile only at 256 columns, decode tiles wide enough for m."""
    from quadmul_b200 import _lib

    for m in (1, 7, 16, 17, 33, 64, 65, 100, 128, 129, 300, 1024, 5000):
        for n in (1, 8, 100, 128, 129, 1000, 4096, 11008, 57344):
            for k in (32, 128, 512, 4096, 28672):
                p = qm.plan(m, n, k)
                # decode shapes: the generated table picks among the families whose limits admit the shape
                allowed = {_lib.QM_KERNEL_TC}
                if m <= 64 and k <= (8192 if m <= 16 else 4096):
                    allowed.add(_lib.QM_KERNEL_RMMA)  # register-resident kernel
                if m <= 4:
                    allowed.add(_lib.QM_KERNEL_GEMV)  # dp4a row kernel
                assert p["kernel"] in allowed, (m, n, k, p)
                assert p["tile_n"] in (16, 32, 64, 128, 256)
                swap, pair, tm = p["swap_ab"] == 2, p["cta_pair"] == 2, p["a_tmem"] == 2
                blocks = (k + 255) // 256 if tm else (k + 127) // 128
                assert 1 <= p["split_k"] <= max(1, blocks)
                if swap:
                    assert m <= 64 and p["tile_n"] in (16, 32, 64) and p["tile_n"] >= m and not pair and tm
                    assert p["stream_k"] in (1, 3) or p["split_k"] == 1
                    if p["stream_k"] == 3:  # cluster form: wide token tiles, 2..4 partitions, one CTA per SM
                        assert p["tile_n"] >= 32 and 2 <= p["split_k"] <= 4 and p["ctas_per_sm"] == 1
                    assert p["ctas_per_sm"] == 1 or (p["ctas_per_sm"] == 2 and p["tile_n"] == 16)
                else:
                    assert p["ctas_per_sm"] == 1
                    # the large-shape kernel may cut a short last round of whole tiles into K partitions (reported as stream_k = 2)
                    assert p["stream_k"] == 1 or (p["stream_k"] == 2 and tm and pair and p["split_k"] == 1)
                if tm and not swap:
                    assert pair and p["tile_n"] == 256
                if pair:
                    assert p["tile_n"] in (128, 256)
                if not tm:
                    assert p["split_k"] == 1 or swap


def test_python_mirror_checks_arguments(qm):
    import torch

    a = torch.zeros((4, 4), dtype=torch.int8)
    c = torch.zeros((4, 4), dtype=torch.int32)
    with pytest.raises((ValueError, qm.QuadmulError)):
        qm.gemm(a, a, c, 4, 4, 8)  # CPU tensors are not accepted: there is no CPU path


def test_drop_in_module_name():
    import quadmul

    assert callable(quadmul.gemm) and callable(quadmul.pack_b)


def test_generated_tile_table_matches_the_committed_sweep():
    """csrc/tile_table.inc is generated (`python -m quadmul_b200.tune --emit`) from the committed B200 sweep
    quadmul_b200/tune_sweep_b200.jsonl: regenerating it must reproduce the committed file byte for byte."""
    from quadmul_b200 import tile_table_gen as gen

    assert open(gen.INC_PATH).read() == gen.render(gen.load_sweep())


def test_plan_follows_the_sweep_and_the_cost_model(qm):
    """Every swept decode shape resolves to the kernel family that was fastest in the sweep; a shape between swept points
    resolves to one of the families, never to nothing (the reference does nothing for an unknown shape, kernel.cu:340-385)."""
    from quadmul_b200 import tile_table_gen as gen

    kernel_of_family = {0: 4, 1: 3, 2: 1}  # QM_KERNEL_RMMA, QM_KERNEL_GEMV, QM_KERNEL_TC
    for m, n, k, fam, _ in gen.best_per_shape(gen.load_sweep()):
        assert qm.plan(m, n, k)["kernel"] == kernel_of_family[fam], (m, n, k)
    for m, n, k in [(3, 5000, 4096), (12, 7168, 4096), (20, 12288, 4096), (40, 3072, 8192), (16, 100000, 4096), (1, 512, 2048), (64, 64, 64)]:
        assert qm.plan(m, n, k)["kernel"] in (1, 3, 4)
    assert qm.plan(16, 4096, 16384)["kernel"] == 1   # K beyond the register-resident kernel's limit
    assert qm.plan(16, 200000, 4096)["kernel"] == 1  # far beyond the sweep: the streaming kernel's slope wins
