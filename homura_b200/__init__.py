"""homura_b200: a CUDA backend for NVIDIA B200 (sm_100a) for the elementwise / reduction hot path of the
homura tensor library, behind the C ABI of ``include/homura_cuda.h``.

``csrc/``   the kernels and the C ABI (``libhomura_cuda.so``), built by :mod:`homura_b200.build`
``ffi``     generated ctypes declarations of the ABI
``host``    the glue homura's Rust side keeps above its GPU boundary (dimension merging, descriptors,
            workspaces) and the backend functions on top of it
``caching`` binding of the native caching allocator

There is no CPU fallback: :func:`load` raises when the library is missing or cannot be loaded.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

from . import ffi

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libhomura_cuda.so"
SHARD_LIB_PATH = _PKG / "libhomura_cuda_shard.so"
_lib = None
_shard = None


class LibraryMissing(RuntimeError):
    pass


def load():
    """The CUDA library with its prototypes bound. Raises LibraryMissing if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise LibraryMissing(f"{LIB_PATH} is missing: build it with `python -m homura_b200.build` "
                                 "(there is no CPU fallback)")
        lib = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_GLOBAL)
        ffi.bind(lib)
        _lib = lib
    return _lib


def load_shard():
    """The multi-GPU library (NCCL); loads the core library first."""
    global _shard
    if _shard is None:
        load()
        if not SHARD_LIB_PATH.exists():
            raise LibraryMissing(f"{SHARD_LIB_PATH} is missing: build it with `python -m homura_b200.build`")
        lib = ctypes.CDLL(str(SHARD_LIB_PATH), mode=ctypes.RTLD_GLOBAL)
        ffi.bind(lib)
        _shard = lib
    return _shard
