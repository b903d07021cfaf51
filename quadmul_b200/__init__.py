"""quadmul_b200: B200 (sm_100a) packed signed-int4 GEMM, a drop-in for carsonpo/quadmul's GEMM path.

Host-side mirror of the reference's Python surface:

  gemm(a, b, c, m, n, k)   the reference's only extension function (extension.cpp:8-24, registered
                           at extension.cpp:26-29): packed A (m x k/2), packed B (n x k/2), int32 C
                           (m x n), launched on the current stream of a's device, returns None.
  pack(x)                  the reference test's `pack_b` (test.py:6-15) as a CUDA kernel.
  unpack(p)                the reference's host `unpack_int4_matrix` (kernel.cu:389-408) as a CUDA kernel.

Everything runs through the C ABI in include/quadmul_b200.h (libquadmul_b200.so, built in-tree
with nvcc).  torch is used for device memory and streams only.  There is no CPU or library
fallback: without the shared object the import fails, and every error status raises.
"""
from __future__ import annotations

import ctypes

from . import _lib
from ._lib import LIB, GemmOpts, QuadmulError, check

__all__ = [
    "gemm",
    "gemm_ex",
    "gemm_host",
    "pack",
    "unpack",
    "fill_packed",
    "plan",
    "device_status",
    "init",
    "nshard_range",
    "unshard_c",
    "QuadmulError",
    "launch_count",
]

_launches = 0  # kernels this package launched (one per call below; split-K adds none)

# The compiled binding (csrc/torch_binding.cpp, built by `python -m quadmul_b200.build --torch`) shortens the host side
# of gemm(); without it the same C-ABI entry point is reached through ctypes.  Either way the work is qm_gemm_s4.
try:
    from . import _quadmul_torch as _EXT  # noqa: F401
except Exception:  # not built, or built against another torch
    _EXT = None


def launch_count() -> int:
    return _launches


def _torch():
    import torch

    return torch


def _stream_of(t) -> int:
    return _torch().cuda.current_stream(t.device).cuda_stream


class _on_device:
    """Make t's device current for the duration of a call (the reference has no such guard:
    extension.cpp:23 takes the stream of a's device but launches on whichever device is current)."""

    def __init__(self, t):
        torch = _torch()
        self.idx = t.device.index if t.device.index is not None else torch.cuda.current_device()
        self.guard = None if self.idx == torch.cuda.current_device() else torch.cuda.device(self.idx)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)


def _check_gemm_tensors(a, b, c, m, n, k):
    torch = _torch()
    if not (a.is_cuda and b.is_cuda and c.is_cuda):
        raise ValueError("quadmul.gemm: a, b and c must be CUDA tensors")
    if not (a.device == b.device == c.device):
        raise ValueError("quadmul.gemm: a, b and c must be on the same device")
    if c.dtype != torch.int32:
        raise TypeError("quadmul.gemm: c must be int32")
    if a.element_size() != 1 or b.element_size() != 1:
        raise TypeError("quadmul.gemm: a and b must be 1-byte tensors holding two nibbles per byte")
    if not (a.is_contiguous() and b.is_contiguous() and c.is_contiguous()):
        raise ValueError("quadmul.gemm: tensors must be contiguous")
    if a.numel() < m * (k // 2) or b.numel() < n * (k // 2) or c.numel() < m * n:
        raise ValueError("quadmul.gemm: tensor smaller than m, n, k imply")


def gemm(a, b, c, m: int, n: int, k: int) -> None:
    """C[m, n] (int32) = A[m, k] (s4) @ B[n, k]^T (s4) on packed operands; same call as the
    reference's quadmul.gemm (extension.cpp:8-24).  Asynchronous on the current stream."""
    global _launches
    if _EXT is not None:
        try:
            _EXT.gemm(a, b, c, m, n, k)  # checks, device guard and status handling are in the binding
        except RuntimeError as exc:
            raise QuadmulError(-1, str(exc).split("\n")[0]) from exc
        _launches += 1
        return
    _check_gemm_tensors(a, b, c, m, n, k)
    with _on_device(a):
        st = LIB.qm_gemm_s4(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, _stream_of(a))
    check(st, f"quadmul.gemm(m={m}, n={n}, k={k})")
    _launches += 1


def gemm_ex(a, b, c, m: int, n: int, k: int, *, kernel: int = 0, tile_n: int = 0, swap_ab: int = 0, split_k: int = 0,
            cta_pair: int = 0, a_tmem: int = 0, stream_k: int = 0, ctas_per_sm: int = 0) -> None:
    """gemm with explicit kernel and tile choices (qm_gemm_s4_ex); for tuning and tests."""
    global _launches
    _check_gemm_tensors(a, b, c, m, n, k)
    opts = GemmOpts(kernel=kernel, tile_n=tile_n, swap_ab=swap_ab, split_k=split_k, cta_pair=cta_pair, a_tmem=a_tmem,
                    stream_k=stream_k, ctas_per_sm=ctas_per_sm)
    with _on_device(a):
        st = LIB.qm_gemm_s4_ex(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, _stream_of(a), ctypes.byref(opts))
    check(st, f"quadmul.gemm_ex(m={m}, n={n}, k={k}, tile_n={tile_n}, swap_ab={swap_ab}, split_k={split_k}, cta_pair={cta_pair}, a_tmem={a_tmem}, stream_k={stream_k}, ctas_per_sm={ctas_per_sm})")
    _launches += 1


def gemm_dequant(a, b, scale_a, scale_b, out, m: int, n: int, k: int, workspace=None):
    """out[m, n] (bfloat16) = bf16(float(A @ B^T) * scale_a[:, None] * scale_b[None, :]) (qm_gemm_s4_dequant_bf16).

    a, b: packed int4 as in `gemm`; scale_a [m] and scale_b [n]: float32 CUDA tensors or None (all ones); out: bfloat16,
    row-major with unit column stride (a column slab of a wider tensor is fine).  Large shapes convert inside the GEMM
    epilogue; the others need an int32 workspace of m * n elements, which is allocated here when not passed in."""
    global _launches
    torch = _torch()
    if not (a.is_cuda and b.is_cuda and out.is_cuda) or a.device != b.device or a.device != out.device:
        raise ValueError("gemm_dequant: a, b, out must be CUDA tensors on one device (there is no CPU path)")
    if a.dtype not in (torch.int8, torch.uint8) or b.dtype not in (torch.int8, torch.uint8) or out.dtype != torch.bfloat16:
        raise ValueError("gemm_dequant: a, b must be int8/uint8 (packed), out bfloat16")
    if not a.is_contiguous() or not b.is_contiguous() or out.dim() != 2 or out.stride(1) != 1:
        raise ValueError("gemm_dequant: a, b contiguous, out row-major")
    if a.numel() != m * (k // 2) or b.numel() != n * (k // 2) or tuple(out.shape) != (m, n) or k % 2:
        raise ValueError("gemm_dequant: shapes do not match (m, n, k)")
    for name, sc, cnt in (("scale_a", scale_a, m), ("scale_b", scale_b, n)):
        if sc is not None and (sc.dtype != torch.float32 or not sc.is_cuda or sc.device != a.device or not sc.is_contiguous()
                               or sc.numel() != cnt):
            raise ValueError(f"gemm_dequant: {name} must be a contiguous float32 CUDA tensor of {cnt} elements")
    ldc = out.stride(0) if m > 1 else max(out.stride(0), n)
    need = LIB.qm_gemm_s4_dequant_workspace_bytes(m, n, k, ldc, out.data_ptr())
    if (a.data_ptr() | b.data_ptr()) & 15:
        need = m * n * 4  # unaligned operands never take the fused kernel
    if need and workspace is None:
        workspace = torch.empty(need // 4, dtype=torch.int32, device=a.device)
    ws_ptr = workspace.data_ptr() if workspace is not None else None
    ws_bytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    with _on_device(a):
        st = LIB.qm_gemm_s4_dequant_bf16(a.data_ptr(), b.data_ptr(), scale_a.data_ptr() if scale_a is not None else None,
                                         scale_b.data_ptr() if scale_b is not None else None, out.data_ptr(), m, n, k, ldc,
                                         ws_ptr, ws_bytes, _stream_of(a))
    check(st, f"quadmul.gemm_dequant(m={m}, n={n}, k={k})")
    _launches += 1 if not need else 2
    return out


def gemm_host(a, b, c, m: int, n: int, k: int) -> None:
    """Host-buffer form (qm_gemm_s4_host): a, b, c are CPU tensors or numpy arrays; copies in, runs
    on the current device, copies out, synchronises."""
    global _launches

    def ptr(x):
        return x.data_ptr() if hasattr(x, "data_ptr") else x.ctypes.data

    st = LIB.qm_gemm_s4_host(ptr(a), ptr(b), ptr(c), m, n, k)
    check(st, f"quadmul.gemm_host(m={m}, n={n}, k={k})")
    _launches += 1


def prelayout_b(b, n: int, k: int):
    """B (packed, n x k/2) -> the pre-laid-out form in which the register-resident decode kernel's loads are contiguous
    (qm_prelayout_b).  Done once per weight matrix; returns a new 1-D int8 tensor."""
    global _launches
    torch = _torch()
    if not b.is_cuda or b.element_size() != 1 or not b.is_contiguous() or b.numel() < n * (k // 2):
        raise ValueError("prelayout_b: b must be a contiguous 1-byte CUDA tensor of n * k/2 bytes")
    out = torch.empty(LIB.qm_prelayout_b_bytes(n, k), dtype=torch.int8, device=b.device)
    with _on_device(b):
        st = LIB.qm_prelayout_b(b.data_ptr(), out.data_ptr(), n, k, _stream_of(b))
    check(st, f"prelayout_b(n={n}, k={k})")
    _launches += 1
    return out


def gemm_prelaid(a, b_pre, c, m: int, n: int, k: int) -> None:
    """C = A @ B^T with B given in the pre-laid-out form of prelayout_b (qm_gemm_s4_prelaid); m <= 16 with k <= 8192 or
    m <= 64 with k <= 4096."""
    global _launches
    torch = _torch()
    if not (a.is_cuda and b_pre.is_cuda and c.is_cuda) or c.dtype != torch.int32 or not (a.is_contiguous() and c.is_contiguous()):
        raise ValueError("gemm_prelaid: CUDA tensors, contiguous a and c, int32 c")
    if a.numel() < m * (k // 2) or c.numel() < m * n or b_pre.numel() < LIB.qm_prelayout_b_bytes(n, k):
        raise ValueError("gemm_prelaid: tensor smaller than m, n, k imply")
    with _on_device(a):
        st = LIB.qm_gemm_s4_prelaid(a.data_ptr(), b_pre.data_ptr(), c.data_ptr(), m, n, k, _stream_of(a))
    check(st, f"gemm_prelaid(m={m}, n={n}, k={k})")
    _launches += 1


def pack(x):
    """int8 tensor [rows, k] with values in [-8, 7] -> packed [rows, k/2] (dtype int8, like the
    reference's pack_b, test.py:6-15)."""
    global _launches
    torch = _torch()
    if x.dtype != torch.int8 or x.dim() != 2 or not x.is_cuda:
        raise TypeError("pack: expected a 2-D int8 CUDA tensor")
    rows, k = x.shape
    if k % 2:
        raise ValueError("pack: k must be even")
    x = x.contiguous()
    out = torch.empty((rows, k // 2), dtype=torch.int8, device=x.device)
    with _on_device(x):
        st = LIB.qm_pack_s4(x.data_ptr(), out.data_ptr(), rows, k, _stream_of(x))
    check(st, "pack")
    _launches += 1
    return out


def unpack(p):
    """packed [rows, k/2] (any 1-byte dtype) -> int8 [rows, k] (kernel.cu:387-408)."""
    global _launches
    torch = _torch()
    if p.element_size() != 1 or p.dim() != 2 or not p.is_cuda:
        raise TypeError("unpack: expected a 2-D 1-byte CUDA tensor")
    rows, kb = p.shape
    p = p.contiguous()
    out = torch.empty((rows, kb * 2), dtype=torch.int8, device=p.device)
    with _on_device(p):
        st = LIB.qm_unpack_s4(p.data_ptr(), out.data_ptr(), rows, kb * 2, _stream_of(p))
    check(st, "unpack")
    _launches += 1
    return out


def fill_packed(rows: int, k: int, seed: int, device="cuda"):
    """Packed [rows, k/2] int8 tensor of the counter-based generator (uniform on [-8, 7])."""
    global _launches
    torch = _torch()
    out = torch.empty((rows, k // 2), dtype=torch.int8, device=device)
    with _on_device(out):
        st = LIB.qm_fill_s4(out.data_ptr(), rows, k, seed, _stream_of(out))
    check(st, "fill_packed")
    _launches += 1
    return out


def init(device: int | None = None) -> None:
    """Per-device set-up (qm_init); call before capturing a CUDA graph."""
    if device is None:
        device = _torch().cuda.current_device()
    check(LIB.qm_init(int(device)), f"init({device})")


def plan(m: int, n: int, k: int) -> dict:
    o = GemmOpts()
    check(LIB.qm_plan(m, n, k, ctypes.byref(o)), "plan")
    return {"kernel": o.kernel, "tile_n": o.tile_n, "swap_ab": o.swap_ab, "split_k": o.split_k, "cta_pair": o.cta_pair,
            "a_tmem": o.a_tmem, "stream_k": o.stream_k, "ctas_per_sm": o.ctas_per_sm}


def selftest_wait_timeout() -> None:
    """Launch the one-warp kernel whose bounded wait must expire (qm_selftest_wait_timeout); afterwards device_status()
    reports (QM_ERR_TIMEOUT, wait site 9).  Takes the wait limit (0.2 s) of GPU time."""
    torch = _torch()
    check(LIB.qm_selftest_wait_timeout(torch.cuda.current_stream().cuda_stream), "selftest_wait_timeout")


def release_stream(stream) -> None:
    """Give back the split-K scratch slice a torch.cuda.Stream holds on the current device (qm_stream_release); call it
    once the stream's work is complete and before dropping the stream."""
    check(LIB.qm_stream_release(stream.cuda_stream), "release_stream")


def selftest_stale_counters() -> None:
    """Leave non-zero arrival counters in the current stream's scratch slice, as a launch whose wait expired would
    (qm_selftest_stale_counters); device_status(clear=True) must be called before the next split-K launch."""
    torch = _torch()
    check(LIB.qm_selftest_stale_counters(torch.cuda.current_stream().cuda_stream), "selftest_stale_counters")


def static_scratch_status(clear: bool = True) -> tuple[int, int]:
    """(code, where) of the launches made through qm_gemm_s4_static_scratch on the current device; allocates nothing."""
    code, where = ctypes.c_int(0), ctypes.c_int(0)
    check(LIB.qm_static_scratch_status(ctypes.byref(code), ctypes.byref(where), 1 if clear else 0), "static_scratch_status")
    return code.value, where.value


def device_status(clear: bool = True) -> tuple[int, int]:
    """(code, where) of the current device's in-kernel wait status; synchronises the device."""
    code, where = ctypes.c_int(0), ctypes.c_int(0)
    check(LIB.qm_device_status(ctypes.byref(code), ctypes.byref(where), 1 if clear else 0), "device_status")
    return code.value, where.value


def nshard_range(n: int, world: int, rank: int) -> tuple[int, int]:
    """(begin, count) of the C columns / B rows rank `rank` of `world` owns."""
    b, c = ctypes.c_int(0), ctypes.c_int(0)
    check(LIB.qm_nshard_range(n, world, rank, ctypes.byref(b), ctypes.byref(c)), "nshard_range")
    return b.value, c.value


def unshard_c(slabs, c, m: int, n: int, world: int, slab_stride: int) -> None:
    """slabs [world, m, slab_stride] int32 (rank-major column slabs) -> c [m, n]."""
    global _launches
    with _on_device(c):
        st = LIB.qm_unshard_c(slabs.data_ptr(), c.data_ptr(), m, n, world, slab_stride, _stream_of(c))
    check(st, "unshard_c")
    _launches += 1
