"""In-tree build of the CUDA library: nvcc, sm_100a only, no torch involved.

    python -m quadmul_b200.build [--force] [--verbose]

Produces quadmul_b200/libquadmul_b200.so (the C ABI declared in include/quadmul_b200.h).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libquadmul_b200.so")
SOURCES = ["qm_api.cu", "qm_gemm_tc.cu", "qm_gemm_tc2.cu", "qm_gemm_dec.cu", "qm_gemv.cu", "qm_gemm_rmma.cu", "qm_gemm_simt.cu", "qm_pack.cu", "qm_dequant.cu", "qm_static_scratch.cu", "qm_peer_flags.cu"]
HEADERS = ["qm_internal.h", "qm_ptx.cuh", "qm_tile_table.h", "qm_tc_common.cuh", "qm_epilogue.cuh", "tile_table.inc", os.path.join("..", "..", "include", "quadmul_b200.h")]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def sources() -> list[str]:
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = sources() + [os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    cmd = [
        nvcc_path(),
        "-std=c++17",
        "-O3",
        "-gencode",
        "arch=compute_100a,code=sm_100a",
        "-lineinfo",
        "--expt-relaxed-constexpr",
        "-Xcompiler",
        "-fPIC,-O3,-Wall",
        "-shared",
        "-o",
        LIB_PATH,
    ]
    cmd += os.environ.get("QM_NVCC_FLAGS", "").split()  # e.g. -DNAME for a development build
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += sources()
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libquadmul_b200.so")
    return LIB_PATH


TORCH_EXT_PATH = os.path.join(PKG_DIR, "_quadmul_torch.so")


def build_torch_binding(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/torch_binding.cpp into quadmul_b200/_quadmul_torch.so (pybind11 + ATen; links the C-ABI library).

    Optional: the package works through ctypes without it; the compiled binding only shortens the host-side path
    of every call."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce

    src = os.path.join(CSRC, "torch_binding.cpp")
    if not force and os.path.exists(TORCH_EXT_PATH) and os.path.getmtime(TORCH_EXT_PATH) >= max(
            os.path.getmtime(src), os.path.getmtime(LIB_PATH)):
        return TORCH_EXT_PATH
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")
    cuda_home = os.path.dirname(os.path.dirname(nvcc_path()))
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-w", "-DTORCH_EXTENSION_NAME=_quadmul_torch",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]:
        cmd += ["-isystem", inc]
    cmd += [src, "-o", TORCH_EXT_PATH, f"-L{PKG_DIR}", "-lquadmul_b200", "-Wl,-rpath,$ORIGIN"]
    for lib in ce.library_paths():
        cmd += [f"-L{lib}", f"-Wl,-rpath,{lib}"]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", f"-L{os.path.join(cuda_home, 'lib64')}",
            "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("g++ failed building _quadmul_torch.so")
    return TORCH_EXT_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--torch" in sys.argv:
        print(build_torch_binding(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
