"""ctypes front end of the CPU oracle (oracle/qm_oracle.c) plus a numpy restatement.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline
leg of bench.py.  The product package never imports this module.

Every function cites the reference line it follows (carsonpo/quadmul):
  pack        test.py:6-15
  unpack      kernel.cu:387-408
  gemm        kernel.cu:291-306 (int64 accumulate here, int32 there)
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libqm_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libquadmul_ref.so")

_i64 = ctypes.c_int64
_vp = ctypes.c_void_p


def build(force: bool = False) -> str:
    """Compile the C oracle if the shared object is missing or stale."""
    src = os.path.join(_HERE, "qm_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "libqm_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def reference_dir() -> str | None:
    """Where the reference's sources lie: $QUADMUL_REFERENCE_DIR, else a directory named `reference` beside this
    repository; None where neither exists (a machine without the reference)."""
    cand = os.environ.get("QUADMUL_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isfile(os.path.join(cand, "kernel.cu")) else None


_REF_EXT_PATH = os.path.join(_HERE, "_ref", "ext", "quadmul.so")


def build_ref_extension(ref_dir: str | None = None) -> str | None:
    """Compile the reference's own pybind file, extension.cpp, UNCHANGED and from where it lies, against the product
    library: `wrapper` (declared at extension.cpp:6) resolves to libquadmul_b200.so instead of the reference's kernel.cu.
    This is the drop-in claim put to the test: the reference's setup.py:10-13 minus its three CUDA sources plus
    -lquadmul_b200.  Output: oracle/_ref/ext/quadmul.so (module name `quadmul`, as setup.py:8,11).  Returns the path, or
    the existing build where the reference is absent, or None."""
    import shutil
    import sysconfig

    ref_dir = ref_dir or reference_dir()
    if ref_dir is None or not os.path.isfile(os.path.join(ref_dir, "extension.cpp")):
        return _REF_EXT_PATH if os.path.exists(_REF_EXT_PATH) else None
    import torch
    from torch.utils import cpp_extension as ce

    pkg = os.path.join(os.path.dirname(_HERE), "quadmul_b200")
    os.makedirs(os.path.dirname(_REF_EXT_PATH), exist_ok=True)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cuda_home = os.path.dirname(os.path.dirname(nvcc))
    cmd = [cxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-w", "-DTORCH_EXTENSION_NAME=quadmul", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]:
        cmd += ["-isystem", inc]
    cmd += [os.path.join(ref_dir, "extension.cpp"), "-o", _REF_EXT_PATH, f"-L{pkg}", "-lquadmul_b200",
            "-Wl,-rpath,$ORIGIN/../../../quadmul_b200"]
    for lib_dir in ce.library_paths():
        cmd += [f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}"]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", f"-L{os.path.join(cuda_home, 'lib64')}",
            "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("building the reference's extension.cpp against libquadmul_b200.so failed:\n" + res.stderr[-2000:])
    return _REF_EXT_PATH


def ref_extension():
    """The module built by build_ref_extension (the reference's `quadmul` with this library behind it), or None."""
    import importlib.util

    if not os.path.exists(_REF_EXT_PATH):
        return None
    import torch  # noqa: F401  (the module links libtorch)

    spec = importlib.util.spec_from_file_location("quadmul", _REF_EXT_PATH)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def build_ref(ref_dir: str) -> str | None:
    """Compile the reference from its own sources (only where they exist). Returns the path or None."""
    if not os.path.isdir(ref_dir):
        return _REF_PATH if os.path.exists(_REF_PATH) else None
    subprocess.run(["make", "-C", _HERE, "ref", f"REF_DIR={ref_dir}"], check=True, capture_output=True)
    return _REF_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        L.qm_oracle_threads.restype = ctypes.c_int
        L.qm_oracle_set_threads.argtypes = [ctypes.c_int]
        L.qm_oracle_unpack.argtypes = [_vp, _vp, _i64, _i64]
        L.qm_oracle_unpack.restype = None
        L.qm_oracle_pack.argtypes = [_vp, _vp, _i64, _i64]
        L.qm_oracle_pack.restype = _i64
        L.qm_oracle_gemm_s4.argtypes = [_vp, _vp, _vp, _i64, _i64, _i64]
        L.qm_oracle_gemm_s4.restype = _i64
        L.qm_oracle_gemm_s4_rows.argtypes = [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64]
        L.qm_oracle_gemm_s4_rows.restype = _i64
        L.qm_oracle_gemm_s4_points.argtypes = [_vp, _vp, _i64, _vp, _vp, _i64, _vp]
        L.qm_oracle_gemm_s4_points.restype = None
        L.qm_oracle_value.argtypes = [ctypes.c_uint64, _i64, _i64, _i64]
        L.qm_oracle_value.restype = ctypes.c_int
        L.qm_oracle_fill_packed.argtypes = [_vp, _i64, _i64, ctypes.c_uint64]
        L.qm_oracle_fill_packed.restype = None
        _lib = L
    return _lib


def threads() -> int:
    return int(lib().qm_oracle_threads())


def set_threads(n: int) -> None:
    lib().qm_oracle_set_threads(int(n))


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def _packed2d(p: np.ndarray) -> np.ndarray:
    p = np.ascontiguousarray(p)
    if p.dtype != np.uint8:
        p = p.view(np.uint8)
    assert p.ndim == 2
    return p


# ---------------------------------------------------------------------------------------
# C oracle
# ---------------------------------------------------------------------------------------
def pack(x: np.ndarray) -> np.ndarray:
    """int8 [rows, K] in [-8, 7] -> uint8 [rows, K/2]; follows test.py:6-15."""
    x = np.ascontiguousarray(x, dtype=np.int8)
    rows, K = x.shape
    if K % 2:
        raise ValueError("K must be even")
    out = np.empty((rows, K // 2), dtype=np.uint8)
    bad = lib().qm_oracle_pack(_ptr(x), _ptr(out), rows, K)
    if bad:
        raise ValueError(f"{bad} values outside [-8, 7]")
    return out


def unpack(p: np.ndarray) -> np.ndarray:
    """uint8 [rows, K/2] -> int8 [rows, K]; follows kernel.cu:387-408."""
    p = _packed2d(p)
    rows, kb = p.shape
    out = np.empty((rows, kb * 2), dtype=np.int8)
    lib().qm_oracle_unpack(_ptr(p), _ptr(out), rows, kb * 2)
    return out


def gemm(a_packed: np.ndarray, b_packed: np.ndarray, rows: tuple[int, int] | None = None) -> np.ndarray:
    """C = A * B^T on packed operands (kernel.cu:291-306), int64 accumulate, int32 result.

    rows=(m0, m1) computes only that row slab and returns an array of m1-m0 rows."""
    a = _packed2d(a_packed)
    b = _packed2d(b_packed)
    M, kb = a.shape
    N, kb2 = b.shape
    if kb != kb2:
        raise ValueError("A and B disagree on K")
    m0, m1 = rows if rows is not None else (0, M)
    c = np.empty((m1 - m0, N), dtype=np.int32)
    ov = lib().qm_oracle_gemm_s4_rows(_ptr(a), _ptr(b), _ptr(c), M, N, kb * 2, m0, m1, m0, N)
    if ov < 0:
        raise MemoryError("oracle could not allocate its unpack buffers")
    if ov:
        raise OverflowError(f"{ov} outputs do not fit int32")
    return c


def gemm_points(a_packed: np.ndarray, b_packed: np.ndarray, rows: np.ndarray, cols: np.ndarray) -> np.ndarray:
    """C[rows[i], cols[i]] as int64 for a list of positions."""
    a = _packed2d(a_packed)
    b = _packed2d(b_packed)
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    cols = np.ascontiguousarray(cols, dtype=np.int64)
    out = np.empty(rows.shape[0], dtype=np.int64)
    lib().qm_oracle_gemm_s4_points(_ptr(a), _ptr(b), a.shape[1] * 2, _ptr(rows), _ptr(cols), rows.shape[0], _ptr(out))
    return out


def fill_packed(rows: int, K: int, seed: int) -> np.ndarray:
    """The counter-based generator the CUDA fill kernel also implements."""
    out = np.empty((rows, K // 2), dtype=np.uint8)
    lib().qm_oracle_fill_packed(_ptr(out), rows, K, seed)
    return out


def value(seed: int, row: int, col: int, K: int) -> int:
    return int(lib().qm_oracle_value(seed, row, col, K))


# ---------------------------------------------------------------------------------------
# numpy restatement (independent second statement of the same rules; small sizes)
# ---------------------------------------------------------------------------------------
def np_pack(x: np.ndarray) -> np.ndarray:
    """test.py:8 (negatives + 16) and test.py:14 (even | odd << 4)."""
    u = np.where(x < 0, x.astype(np.int16) + 16, x.astype(np.int16)).astype(np.uint8)
    return (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)


def np_unpack(p: np.ndarray) -> np.ndarray:
    """kernel.cu:387 and kernel.cu:395-396."""
    p = _packed2d(p)
    lo = (p & 0xF).astype(np.int16)
    hi = (p >> 4).astype(np.int16)
    lo = np.where(lo > 7, lo - 16, lo)
    hi = np.where(hi > 7, hi - 16, hi)
    out = np.empty((p.shape[0], p.shape[1] * 2), dtype=np.int8)
    out[:, 0::2] = lo
    out[:, 1::2] = hi
    return out


def np_gemm(a_packed: np.ndarray, b_packed: np.ndarray) -> np.ndarray:
    """kernel.cu:301 with an int64 accumulator."""
    a = np_unpack(a_packed).astype(np.int64)
    b = np_unpack(b_packed).astype(np.int64)
    c = a @ b.T
    assert np.all(np.abs(c) < 2**31)
    return c.astype(np.int32)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even (finite inputs)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def dequant_bf16(acc: np.ndarray, scale_a: np.ndarray | None, scale_b: np.ndarray | None) -> np.ndarray:
    """The fused epilogue of qm_gemm_s4_dequant_bf16 restated: bf16(float32(acc) * scale_a[r] * scale_b[c]) as uint16 bit
    patterns; int32 -> float32 rounds to nearest even, the two products are separate float32 multiplications in this
    order.  The reference has no such epilogue (its store is kernel.cu:155-184); this defines the contract of the added
    entry point."""
    f = acc.astype(np.float32)
    if scale_a is not None:
        f = f * np.asarray(scale_a, dtype=np.float32)[:, None]
    else:
        f = f * np.float32(1.0)
    if scale_b is not None:
        f = f * np.asarray(scale_b, dtype=np.float32)[None, :]
    return bf16_bits(f)


def random_s4(rows: int, K: int, seed: int) -> np.ndarray:
    """Uniform on [-8, 7] (both ends included), int8."""
    return np.random.default_rng(seed).integers(-8, 8, size=(rows, K), dtype=np.int8)


# ---------------------------------------------------------------------------------------
# the reference itself, where it was compiled (oracle/_ref)
# ---------------------------------------------------------------------------------------
_ref = None


def ref_lib() -> ctypes.CDLL | None:
    """The reference's own compiled host functions, or None where that build is absent."""
    global _ref
    if _ref is None and os.path.exists(_REF_PATH):
        try:
            L = ctypes.CDLL(_REF_PATH)
        except OSError:
            return None
        L.qm_ref_cpu_gemm_int8.argtypes = [_vp, _vp, _vp, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.qm_ref_cpu_gemm_int8.restype = None
        L.qm_ref_unpack_int4_matrix.argtypes = [_vp, _vp, ctypes.c_int, ctypes.c_int]
        L.qm_ref_unpack_int4_matrix.restype = None
        L.qm_ref_wrapper.argtypes = [_vp, _vp, _vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, _vp]
        L.qm_ref_wrapper.restype = None
        L.qm_ref_gpu_gemm.argtypes = [_vp, _vp, _vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, _vp]
        L.qm_ref_gpu_gemm.restype = ctypes.c_int
        _ref = L
    return _ref


def ref_unpack(p: np.ndarray) -> np.ndarray:
    """The reference's unpack_int4_matrix (kernel.cu:389-408), run as compiled."""
    L = ref_lib()
    assert L is not None
    p = _packed2d(p)
    out = np.empty((p.shape[0], p.shape[1] * 2), dtype=np.int8)
    L.qm_ref_unpack_int4_matrix(_ptr(p), _ptr(out), p.shape[0], p.shape[1] * 2)
    return out


def ref_cpu_gemm(a_unpacked: np.ndarray, b_unpacked: np.ndarray) -> np.ndarray:
    """The reference's cpu_gemm_int8 (kernel.cu:291-306), run as compiled, on unpacked int8."""
    L = ref_lib()
    assert L is not None
    a = np.ascontiguousarray(a_unpacked, dtype=np.int8)
    b = np.ascontiguousarray(b_unpacked, dtype=np.int8)
    c = np.empty((a.shape[0], b.shape[0]), dtype=np.int32)
    L.qm_ref_cpu_gemm_int8(_ptr(a), _ptr(b), _ptr(c), a.shape[0], b.shape[0], a.shape[1])
    return c
