"""Locates, builds on demand and loads the in-tree native libraries with ctypes."""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
LIB_DIR = PKG / "_lib"

_lock = threading.Lock()
_cache: dict[str, ctypes.CDLL] = {}


class NativeLibraryMissing(RuntimeError):
    """Raised when a native library is required but neither present nor buildable."""


def lib_path(name: str) -> Path:
    return LIB_DIR / name


def load(name: str, build: bool = True) -> ctypes.CDLL:
    """Loads `_lib/<name>`, building the native tree first when it is absent.

    There is no Python fallback for the kernels: a missing library is an error.
    """
    with _lock:
        if name in _cache:
            return _cache[name]
        path = lib_path(name)
        if not path.exists() and build and os.environ.get("TCPXB_NO_AUTOBUILD") != "1":
            from .. import _build
            if name == "libtcpxb_host.so":
                _build.build_host()
            else:
                _build.build_all()
        if not path.exists():
            raise NativeLibraryMissing(
                f"{path} is missing; run `python -m nccl_plugin_gpudirecttcpx_b200._build`")
        lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
        _cache[name] = lib
        return lib


def plugin_path() -> Path:
    """Path of the NCCL net plugin (`libnccl-net.so`), for NCCL_NET_PLUGIN."""
    return lib_path("libnccl-net.so")
