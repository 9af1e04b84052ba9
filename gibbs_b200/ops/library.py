"""Loads the compiled kernel libraries through ctypes.  There is no fallback:
if a library cannot be built or loaded, the call that needs it raises."""
from __future__ import annotations

import ctypes
import threading

from ..csrc import build as _build

_LOCK = threading.Lock()
_LOADED: dict[str, ctypes.CDLL] = {}


class KernelError(RuntimeError):
    pass


def library(name: str) -> ctypes.CDLL:
    lib = _LOADED.get(name)
    if lib is not None:
        return lib
    with _LOCK:
        lib = _LOADED.get(name)
        if lib is None:
            try:
                path = _build.build(name)
                lib = ctypes.CDLL(str(path))
            except (OSError, _build.BuildError) as e:
                raise KernelError(
                    f"the CUDA kernel library '{name}' of gibbs_b200 is not available ({e}); "
                    "there is no fallback path") from e
            _LOADED[name] = lib
    return lib


def ensure_built(names) -> None:
    """Build and load several libraries up front (an engine knows at start
    which ones its model and dtype need)."""
    for n in names:
        library(n)


def check(lib: ctypes.CDLL, status: int) -> None:
    if status != 0:
        fn = lib.gb_last_error
        fn.restype = ctypes.c_char_p
        raise KernelError(fn().decode(errors="replace"))
