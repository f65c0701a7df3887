"""ctypes binding of the built kernel libraries.

Each library exports ``extern "C"`` launchers that take device pointers, sizes
and a stream, return 0 on success, and keep the text of their last failure in
``<prefix>_last_error()``.  A launcher that fails raises ``KernelError`` here;
a library that cannot be built or loaded raises too: there is no fallback
path.  The binding manner follows the reference's
(pytorch/src/mini_llm/native.py:203-307: ``ctypes.CDLL`` plus declared
argument types).
"""

from __future__ import annotations

import ctypes
import os
import threading

from . import build


class KernelError(RuntimeError):
    pass


_libraries: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dependent_launch = os.environ.get("MLLM_DEPENDENT_LAUNCH", "1") != "0"


def set_dependent_launch(on: bool) -> None:
    """Whether kernels are launched as programmatic dependents of the kernel before them on
    their stream (they may be scheduled and set themselves up while it still runs, and wait
    for its end before they touch memory), in every library, loaded already or later.  On by
    default; off, every kernel starts after the one before it has ended."""
    global _dependent_launch
    with _lock:
        _dependent_launch = bool(on)
        for name, lib in _libraries.items():
            getattr(lib, f"mllm_{name}_set_dependent_launch")(int(_dependent_launch))



def load(name: str) -> ctypes.CDLL:
    """The loaded library ``name`` (built at the first call)."""
    lib = _libraries.get(name)
    if lib is not None:
        return lib
    with _lock:
        if name not in _libraries:
            path = build.library_path(name)
            try:
                _libraries[name] = ctypes.CDLL(path)
            except OSError as error:
                raise KernelError(f"cannot load kernel library {path}: {error}") from None
            last_error = getattr(_libraries[name], f"mllm_{name}_last_error")
            last_error.restype = ctypes.c_char_p
            switch = getattr(_libraries[name], f"mllm_{name}_set_dependent_launch")
            switch.argtypes, switch.restype = [ctypes.c_int], None
            switch(int(_dependent_launch))
        return _libraries[name]


class Function:
    """One exported launcher with declared argument types."""

    def __init__(self, library: str, symbol: str, argtypes):
        self.library = library
        self.symbol = symbol
        self.argtypes = argtypes
        self._fn = None
        self._err = None

    def _resolve(self):
        lib = load(self.library)
        fn = getattr(lib, self.symbol)
        fn.argtypes = self.argtypes
        fn.restype = ctypes.c_int
        self._err = getattr(lib, f"mllm_{self.library}_last_error")
        self._fn = fn

    def __call__(self, *args):
        if self._fn is None:
            self._resolve()
        status = self._fn(*args)
        if status != 0:
            text = self._err()
            raise KernelError(f"{self.symbol} failed ({status}): {text.decode() if text else 'no message'}")


P = ctypes.c_void_p
I = ctypes.c_int
L = ctypes.c_long
F = ctypes.c_float
