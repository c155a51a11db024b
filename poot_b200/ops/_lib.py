"""ctypes loader for the native libraries (kernels and host runtime).

The libraries are built in-tree by :mod:`poot_b200.build`.  On a machine with a GPU a missing kernel
library is an error (there is no silent PyTorch fallback); on a CPU-only machine the kernel library can
still be loaded (the CUDA runtime is linked statically) but no launcher may be called.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
_lock = threading.Lock()
_kernels = None
_host = None


class NativeLibraryMissing(RuntimeError):
    pass


def _load(name: str, builder: str):
    path = _LIB_DIR / name
    if not path.exists():
        try:
            from poot_b200 import build as _build
            getattr(_build, builder)()
        except Exception as exc:  # pragma: no cover - depends on toolchain
            raise NativeLibraryMissing(
                f"{name} is not built and could not be built here ({exc}); run `python -m poot_b200.build`"
            ) from exc
    if not path.exists():
        raise NativeLibraryMissing(f"{name} missing after build")
    return ctypes.CDLL(str(path))


def kernels() -> ctypes.CDLL:
    """The CUDA kernel library: ``libpoot_kernels.so``, or its checked flavour ``libpoot_kernels_dbg.so`` (bounds
    checks on every data-dependent index, recorded for the host) when ``POOT_DEBUG_BOUNDS=1`` is set."""
    global _kernels
    if _kernels is None:
        with _lock:
            if _kernels is None:
                if os.environ.get("POOT_DEBUG_BOUNDS", "0") not in ("", "0"):
                    _kernels = _load("libpoot_kernels_dbg.so", "build_kernels_checked")
                else:
                    _kernels = _load("libpoot_kernels.so", "build_kernels")
    return _kernels


def host() -> ctypes.CDLL:
    """The host C++ runtime library (``libpoot_host.so``)."""
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                _host = _load("libpoot_host.so", "build_host")
    return _host


class KernelError(RuntimeError):
    """A launcher returned a CUDA error code."""


def check(code: int, what: str) -> None:
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")
