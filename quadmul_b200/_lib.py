"""ctypes binding of libquadmul_b200.so (the C ABI in include/quadmul_b200.h).

Loading never falls back to anything else: if the shared object is missing and cannot be built
with nvcc, importing the package raises.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

_vp = ctypes.c_void_p
_i = ctypes.c_int
_i64 = ctypes.c_int64
_u64 = ctypes.c_uint64


class GemmOpts(ctypes.Structure):
    """Mirror of qm_gemm_opts_t."""

    _fields_ = [
        ("kernel", _i),
        ("tile_n", _i),
        ("swap_ab", _i),
        ("split_k", _i),
        ("cta_pair", _i),
        ("a_tmem", _i),
        ("plain_stores", _i),
        ("stream_k", _i),
        ("ctas_per_sm", _i),
    ]


# name -> (restype, argtypes); every symbol include/quadmul_b200.h declares with C linkage
SIGNATURES = {
    "qm_status_string": (ctypes.c_char_p, [_i]),
    "qm_version": (_i, []),
    "qm_last_cuda_error": (ctypes.c_char_p, []),
    "qm_init": (_i, [_i]),
    "qm_gemm_s4": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "qm_gemm_s4_ex": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, ctypes.POINTER(GemmOpts)]),
    "qm_gemm_s4_ldc": (_i, [_vp, _vp, _vp, _i, _i, _i, _i64, _vp]),
    "qm_gemm_s4_ldc_ex": (_i, [_vp, _vp, _vp, _i, _i, _i, _i64, _vp, ctypes.POINTER(GemmOpts)]),
    "qm_gemm_s4_host": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "qm_pack_s4": (_i, [_vp, _vp, _i64, _i64, _vp]),
    "qm_unpack_s4": (_i, [_vp, _vp, _i64, _i64, _vp]),
    "qm_fill_s4": (_i, [_vp, _i64, _i64, _u64, _vp]),
    "qm_nshard_range": (_i, [_i, _i, _i, ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "qm_unshard_c": (_i, [_vp, _vp, _i, _i, _i, _i64, _vp]),
    "qm_device_status": (_i, [ctypes.POINTER(_i), ctypes.POINTER(_i), _i]),
    "qm_plan": (_i, [_i, _i, _i, ctypes.POINTER(GemmOpts)]),
    "qm_selftest_wait_timeout": (_i, [_vp]),
    "qm_gemm_s4_dequant_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _vp, ctypes.c_size_t, _vp]),
    "qm_gemm_s4_dequant_workspace_bytes": (ctypes.c_size_t, [_i, _i, _i, _i64, _vp]),
    "qm_gemm_s4_static_scratch": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "qm_static_scratch_status": (_i, [ctypes.POINTER(_i), ctypes.POINTER(_i), _i]),
    "qm_selftest_stale_counters": (_i, [_vp]),
    "qm_stream_release": (_i, [_vp]),
    "qm_prelayout_b_bytes": (ctypes.c_size_t, [_i, _i]),
    "qm_prelayout_b": (_i, [_vp, _vp, _i, _i, _vp]),
    "qm_gemm_s4_prelaid": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "qm_flag_signal": (_i, [_vp, _i, _vp]),
    "qm_flags_wait": (_i, [_vp, _i, _i, _i, _vp]),
}

# the reference's C++ entry point `wrapper(void*, void*, void*, int, int, int, cudaStream_t)`
WRAPPER_MANGLED = "_Z7wrapperPvS_S_iiiP11CUstream_st"

QM_OK = 0
QM_KERNEL_AUTO, QM_KERNEL_TC, QM_KERNEL_SIMT, QM_KERNEL_GEMV, QM_KERNEL_RMMA = 0, 1, 2, 3, 4


class QuadmulError(RuntimeError):
    def __init__(self, status: int, detail: str = ""):
        self.status = status
        super().__init__(detail)


def load() -> ctypes.CDLL:
    path = _build.LIB_PATH
    if not os.path.exists(path) or _build.is_stale():
        try:
            _build.build()
        except Exception as exc:  # no nvcc on this machine: use the prebuilt object if there is one
            if not os.path.exists(path):
                raise ImportError(
                    f"quadmul_b200: {path} is missing and could not be built ({exc}); there is no fallback path"
                ) from exc
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    w = getattr(lib, WRAPPER_MANGLED)
    w.restype = None
    w.argtypes = [_vp, _vp, _vp, _i, _i, _i, _vp]
    return lib


LIB = load()


def check(status: int, what: str) -> None:
    if status != QM_OK:
        msg = LIB.qm_status_string(status).decode()
        detail = LIB.qm_last_cuda_error().decode()
        raise QuadmulError(status, f"{what}: {msg}" + (f" [{detail}]" if detail and status == 4 else ""))
