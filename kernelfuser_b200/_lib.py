"""ctypes binding of libkf_b200.so (the C ABI declared in include/kf_b200.h).

The shared object is loaded from this package directory.  If it is missing it
is built once with nvcc (``kernelfuser_b200.build``); if that is not possible
the import of the operator fails loudly -- there is no CPU or PyTorch
fallback for the kernels.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libkf_b200.so"

KF_BF16, KF_FP16 = 0, 1
EXPORTS = ("kf_version", "kf_last_error", "kf_prepare_rows", "kf_attention_fwd",
           "kf_static_scratch_bytes", "kf_optimized_attention_static", "kf_factored_attention",
           "kf_selftest_wait_timeout", "kf_optimized_attention", "kf_attention_full")

_lib = None


class KernelLibraryError(RuntimeError):
    pass


def _declare(lib):
    lib.kf_version.restype = c_int
    lib.kf_version.argtypes = []
    lib.kf_last_error.restype = c_char_p
    lib.kf_last_error.argtypes = []
    lib.kf_prepare_rows.restype = c_int
    lib.kf_prepare_rows.argtypes = ([c_void_p] * 5 + [c_int] * 6 + [c_float] + [c_int64] * 6 + [c_void_p])
    lib.kf_attention_fwd.restype = c_int
    lib.kf_attention_fwd.argtypes = ([c_void_p] * 7 + [c_int] * 9 + [c_float] * 2 + [c_int64] * 12 +
                                     [c_void_p, c_int, c_void_p])
    lib.kf_static_scratch_bytes.restype = ctypes.c_size_t
    lib.kf_static_scratch_bytes.argtypes = []
    lib.kf_optimized_attention_static.restype = c_int
    lib.kf_optimized_attention_static.argtypes = ([c_void_p] * 8 + [c_int] * 8 + [c_float] * 2 + [c_int64] * 12 +
                                                  [c_void_p, c_void_p])
    lib.kf_factored_attention.restype = c_int
    lib.kf_factored_attention.argtypes = ([c_void_p] * 7 + [c_int] * 7 + [c_float] * 2 + [c_int64] * 15 +
                                          [c_void_p, c_int, c_void_p])
    lib.kf_attention_full.restype = c_int
    lib.kf_attention_full.argtypes = ([c_void_p] * 8 + [c_int] * 8 + [c_float] * 2 + [c_int64] * 12 +
                                      [c_void_p, c_void_p])
    lib.kf_optimized_attention.restype = c_int
    lib.kf_optimized_attention.argtypes = ([c_void_p] * 9 + [c_int] * 8 + [c_float] * 2 + [c_int64] * 15 +
                                           [c_void_p, c_int, c_void_p])
    lib.kf_selftest_wait_timeout.restype = c_int
    lib.kf_selftest_wait_timeout.argtypes = [c_void_p, ctypes.c_longlong, c_void_p]
    return lib


def load(build_if_missing: bool = True):
    """Load (once) and return the ctypes handle of libkf_b200.so."""
    global _lib
    if _lib is not None:
        return _lib
    from . import build as _build
    if not LIB_PATH.exists():
        if not build_if_missing:
            raise KernelLibraryError(f"{LIB_PATH} is missing; run `python -m kernelfuser_b200.build`")
        _build.build()
    elif build_if_missing and _build.stale():
        # a kernel source or the header is newer than the library: never test or run an old binary silently
        if _build.have_nvcc():
            _build.build()
        else:
            import warnings
            warnings.warn(f"{LIB_PATH} is older than its sources and nvcc is not available to rebuild it")
    try:
        _lib = _declare(ctypes.CDLL(str(LIB_PATH)))
    except OSError as e:  # pragma: no cover - depends on the environment
        raise KernelLibraryError(f"cannot load {LIB_PATH}: {e}") from e
    return _lib


def last_error() -> str:
    return load().kf_last_error().decode("utf-8", "replace")
