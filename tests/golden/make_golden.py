"""Generates tests/golden/*.npz from the REFERENCE ITSELF (run where the reference sources exist).

  python tests/golden/make_golden.py [/path/to/reference]

For every case it stores
  a, b            int8 operands with values in [-8, 7]
  a_packed, ...   produced by the reference's Python packer `pack_b` (test.py:6-15), whose source
                  is read from the reference's test.py and executed unchanged on CPU tensors
  a_unpacked, ... produced by the reference's compiled `unpack_int4_matrix` (kernel.cu:389-408)
                  from those packed bytes
  c               produced by the reference's compiled `cpu_gemm_int8` (kernel.cu:291-306)
The compiled functions come from oracle/_ref (built by `make -C oracle ref`).  Nothing here
uses this repository's own oracle or kernels, so the fixtures pin them from outside.
"""
from __future__ import annotations

import ast
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def load_reference_pack_b(ref_dir: str):
    """Return the reference's pack_b function object, compiled from its own source text."""
    import torch  # noqa: F401  (pack_b uses torch.where)

    path = os.path.join(ref_dir, "test.py")
    tree = ast.parse(open(path).read(), filename=path)
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "pack_b"]
    assert len(fn) == 1, "pack_b not found in the reference's test.py"
    mod = ast.Module(body=fn, type_ignores=[])
    ns: dict = {"torch": __import__("torch")}
    exec(compile(mod, path, "exec"), ns)
    return ns["pack_b"]


def cases():
    rng = np.random.default_rng(20240611)

    def rnd(r, k):
        return rng.integers(-8, 8, size=(r, k), dtype=np.int8)

    out = {}
    out["tiny_8x8x32"] = (rnd(8, 32), rnd(8, 32))
    out["ragged_5x13x64"] = (rnd(5, 64), rnd(13, 64))
    out["decode_1x64x128"] = (rnd(1, 128), rnd(64, 128))
    out["ktail_96x136x416"] = (rnd(96, 416), rnd(136, 416))
    out["block_128x256x256"] = (rnd(128, 256), rnd(256, 256))
    out["twotile_160x288x384"] = (rnd(160, 384), rnd(288, 384))
    # extremes: every product is +64, -56, +49 or the sign-alternating mix
    a = np.full((16, 256), -8, np.int8)
    b = np.full((24, 256), -8, np.int8)
    b[8:16] = 7
    b[16:, 0::2] = 7
    b[16:, 1::2] = -8
    a[8:, 1::2] = 7
    out["extremes_16x24x256"] = (a, b)
    # every (a, b) value pair appears: row i of A is constant i-8, row j of B is constant j-8
    a = np.repeat(np.arange(-8, 8, dtype=np.int8)[:, None], 32, axis=1)
    out["allpairs_16x16x32"] = (a.copy(), a.copy())
    return out


def main():
    import torch

    from oracle import oracle as o

    ref_dir = sys.argv[1] if len(sys.argv) > 1 else o.reference_dir()
    if ref_dir is None:
        raise SystemExit("make_golden.py: pass the reference's directory (or set QUADMUL_REFERENCE_DIR)")

    assert o.build_ref(ref_dir), "reference build missing"
    assert o.ref_lib() is not None
    pack_b = load_reference_pack_b(ref_dir)

    for name, (a, b) in cases().items():
        ap = pack_b(torch.from_numpy(a)).numpy().view(np.uint8)
        bp = pack_b(torch.from_numpy(b)).numpy().view(np.uint8)
        au = o.ref_unpack(ap)
        bu = o.ref_unpack(bp)
        c = o.ref_cpu_gemm(au, bu)
        assert (au == a).all() and (bu == b).all(), name  # the reference round-trips its own packing
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, a=a, b=b, a_packed=ap, b_packed=bp, a_unpacked=au, b_unpacked=bu, c=c)
        print(f"{name}: A{a.shape} B{b.shape} C{c.shape} -> {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
