"""Drop-in module name: `import quadmul; quadmul.gemm(a, b, c, m, n, k)` as with the reference's
extension (setup.py:8-11, extension.cpp:26-29), served by quadmul_b200."""
from quadmul_b200 import gemm, pack, unpack  # noqa: F401
from quadmul_b200 import pack as pack_b  # the reference test's name for the packer (test.py:6)  # noqa: F401
