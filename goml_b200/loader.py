"""Library discovery, mirroring goml's backend/cuda/arch.go:57-101.

``libs_dir()`` follows ``LibsDir``: ``$GOML_LIBS_DIR``, ``./libs``, the
directory of the running program + ``/libs``, ``/usr/local/lib/goml`` — first
existing directory wins — with this package's own ``libs`` directory inserted
after the environment override so an in-tree build is found without setup.
``resolve_lib(name)`` follows ``resolveLib``: the full path when the file
exists in that directory, else the bare name for the OS loader.

There is no CPU or library fallback: when a library cannot be loaded the
caller gets a ``LibraryNotFound`` error.
"""
from __future__ import annotations

import ctypes
import os
import sys

_PKG_LIBS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libs")


class LibraryNotFound(OSError):
    pass


def libs_dir() -> str:
    candidates = [os.environ.get("GOML_LIBS_DIR", ""), _PKG_LIBS, os.path.join(os.getcwd(), "libs")]
    exe = sys.argv[0] if sys.argv and sys.argv[0] else ""
    if exe:
        candidates.append(os.path.join(os.path.dirname(os.path.abspath(exe)), "libs"))
    candidates.append("/usr/local/lib/goml")
    for d in candidates:
        if d and os.path.isdir(d):
            return d
    return ""


def resolve_lib(name: str) -> str:
    env = os.environ.get("GOML_LIBS_DIR", "")
    for d in ([env] if env else []) + [_PKG_LIBS, libs_dir()]:
        if d:
            full = os.path.join(d, name)
            if os.path.exists(full):
                return full
    return name


def dlopen(name_or_path: str, global_symbols: bool = False) -> ctypes.CDLL:
    mode = ctypes.RTLD_GLOBAL if global_symbols else ctypes.RTLD_LOCAL
    try:
        return ctypes.CDLL(name_or_path, mode=mode)
    except OSError as e:  # no fallback: fail loudly
        raise LibraryNotFound(
            f"{name_or_path}: cannot load ({e}). Build it with `python -m goml_b200.build` "
            f"or point GOML_LIBS_DIR at the directory that holds it.") from e
