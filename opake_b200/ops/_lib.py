"""ctypes binding of ``libopake_kernels.so`` (the hand-written sm_100a kernels).

The library is built in-tree by :mod:`opake_b200._build`. On a machine with a GPU a missing library is a hard
error: no op silently falls back to eager PyTorch.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_double, c_float, c_int32, c_int64, c_void_p
from functools import lru_cache

import torch

import os

from .._build import KERNEL_LIB, KERNEL_LIB_DEBUG, build_kernels


class GemmArgs(Structure):
    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("C", c_void_p), ("R", c_void_p), ("bias", c_void_p),
        ("M", c_int32), ("N", c_int32), ("K", c_int32), ("batch", c_int32),
        ("a_mn", c_int32), ("b_mn", c_int32), ("epilogue", c_int32), ("b_batch_div", c_int32),
        ("lda", c_int64), ("ldb", c_int64), ("ldc", c_int64),
        ("strideA", c_int64), ("strideB", c_int64), ("strideC", c_int64),
        ("alpha", c_float), ("softcap", c_float),
        ("sumsq", c_void_p), ("act", c_void_p), ("ld_act", c_int64),
        ("labels", c_void_p), ("pmax", c_void_p), ("psum", c_void_p), ("tgt", c_void_p),
        ("lse", c_void_p), ("coef", c_void_p), ("err", c_void_p), ("max_ctas", c_int32),
        ("tile_group", c_void_p), ("n_groups", c_int32), ("group_k", c_void_p), ("sumsq_shared", c_int32),
        ("stage_dst", c_void_p), ("stage_ready", c_void_p),
    ]


class KernelLibraryError(RuntimeError):
    pass


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    # OPAKE_B200_DEBUG_KERNELS=1 loads the variant with index checks on data-dependent addresses (see debug_bounds_report)
    debug = os.environ.get("OPAKE_B200_DEBUG_KERNELS", "0") not in ("", "0")
    path = KERNEL_LIB_DEBUG if debug else KERNEL_LIB
    if not path.exists():
        try:
            build_kernels(debug_bounds=debug)
        except Exception as exc:  # pragma: no cover - build environment specific
            raise KernelLibraryError(f"{path} is missing and could not be built: {exc}") from exc
    L = ctypes.CDLL(str(path))
    L.opk_last_error.restype = c_char_p
    L.opk_gemm.argtypes = [POINTER(GemmArgs), c_void_p]
    L.opk_gemm.restype = c_int32
    L.opk_gemm_tiles_n.argtypes = [c_int32, c_int32]
    L.opk_gemm_tiles_n.restype = c_int32
    L.opk_num_sms.restype = c_int32
    L.opk_debug_bounds_read.argtypes = [POINTER(c_int64), c_char_p, c_int32, c_int32]
    L.opk_debug_bounds_read.restype = c_int32
    L.opk_gemm_set_pair_mode.argtypes = [c_int32]
    L.opk_gemm_set_pair_mode.restype = None
    L.opk_gemm_get_pair_mode.restype = c_int32
    _declare_optional(L)
    return L


def _declare_optional(L: ctypes.CDLL) -> None:
    """Attach prototypes for the non-GEMM kernels (declared in csrc/kernels/opk_api.h)."""
    from ._protos import PROTOTYPES

    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(L, name, None)
        if fn is None:
            raise KernelLibraryError(f"symbol {name} missing from {KERNEL_LIB}; rebuild with opake_b200._build")
        fn.restype = restype
        fn.argtypes = argtypes


LAUNCHES = [0]  # number of native kernel entry-point calls issued by this process


def check(code: int, what: str) -> None:
    LAUNCHES[0] += 1
    if code != 0:
        msg = lib().opk_last_error().decode("utf-8", "replace")
        raise KernelLibraryError(f"{what} failed (code {code}): {msg}")


def stream_ptr(device: torch.device | None = None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_ERR: dict[int, torch.Tensor] = {}


def err_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 that kernels set to 1 when one of their bounded waits expires."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _ERR.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _ERR[idx] = t
    return t


def debug_bounds_report(reset: bool = True) -> dict | None:
    """Record of the debug library's index checks: ``{"failures", "file", "line", "index", "bound"}`` (the first failing
    access since the last reset; such accesses were skipped, not performed). ``None`` when the release library is
    loaded. Synchronises the device."""
    out = (c_int64 * 4)()
    buf = ctypes.create_string_buffer(256)
    code = lib().opk_debug_bounds_read(out, buf, 256, 1 if reset else 0)
    if code == -3:
        return None
    if code != 0:
        raise KernelLibraryError(f"debug_bounds_read failed (code {code}): {lib().opk_last_error().decode()}")
    return {"failures": int(out[0]), "file": buf.value.decode("utf-8", "replace"), "line": int(out[1]), "index": int(out[2]),
            "bound": int(out[3])}


def raise_if_device_error(device: torch.device) -> None:
    """Synchronising check of the error word; raises :class:`KernelLibraryError` when a kernel gave up a wait."""
    t = err_word(device)
    if int(t.item()) != 0:
        t.zero_()
        raise KernelLibraryError("a device-side bounded wait expired (kernel aborted cleanly)")
