"""Binding of the native caching allocator (``include/homura_cuda_alloc.h``), whose bookkeeping is that of
homura's ``src/backend/caching.rs``. The memory behind it is either the CUDA device of a context
(:class:`CudaMemory`) or any Python object with ``malloc/free/synchronize`` (the tests' fake device)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

from . import ffi

SMALL_MAX = 1 << 20
SMALL_ROUND = 512
SMALL_SEGMENT = 2 << 20
LARGE_ROUND = 2 << 20


class OutOfMemory(MemoryError):
    """homura's Error::OutOfMemory / PoolError::OutOfMemory."""


class PoolFailed(RuntimeError):
    """homura's PoolError::Failed."""


class MallocOutOfMemory(Exception):
    """Raised by a Python memory to say the device is full (MallocError::OutOfMemory)."""


@dataclass
class Block:
    ptr: int
    size: int
    allocator: "CachingAllocator"
    live: bool = True

    def release(self) -> None:
        if self.live:
            self.live = False
            self.allocator.release(self.ptr)

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class CudaMemory:
    """Marker: the allocator is created over the context of `backend` by the library itself."""

    def __init__(self, lib, device: int, backend):
        self.lib, self.device, self.backend = lib, device, backend


class CachingAllocator:
    def __init__(self, memory, lib=None):
        from . import load
        self.lib = lib or getattr(memory, "lib", None) or load()
        self.memory = memory
        handle = ctypes.c_void_p()
        if isinstance(memory, CudaMemory):
            self._check(self.lib.hmc_allocator_create_cuda(memory.backend.ctx, ctypes.byref(handle)))
        else:
            ops = ffi.hmc_memory_ops()
            fields = dict(ffi.hmc_memory_ops._fields_)

            def malloc_cb(_user, size, addr):
                try:
                    addr[0] = memory.malloc(size)
                    return ffi.HMC_MEM_OK
                except MallocOutOfMemory:
                    return ffi.HMC_MEM_OUT_OF_MEMORY
                except Exception as e:  # MallocError::Failed
                    self.lib.hmc_allocator_set_callback_error(str(e).encode())
                    return ffi.HMC_MEM_FAILED

            def free_cb(_user, addr):
                try:
                    memory.free(addr)
                    return ffi.HMC_MEM_OK
                except Exception as e:
                    self.lib.hmc_allocator_set_callback_error(str(e).encode())
                    return ffi.HMC_MEM_FAILED

            def sync_cb(_user):
                try:
                    memory.synchronize()
                    return ffi.HMC_MEM_OK
                except Exception as e:
                    self.lib.hmc_allocator_set_callback_error(str(e).encode())
                    return ffi.HMC_MEM_FAILED

            self._callbacks = (fields["malloc_fn"](malloc_cb), fields["free_fn"](free_cb), fields["synchronize_fn"](sync_cb))
            ops.user = None
            ops.malloc_fn, ops.free_fn, ops.synchronize_fn = self._callbacks
            self._check(self.lib.hmc_allocator_create(ctypes.byref(ops), ctypes.byref(handle)))
        self.handle = handle

    def _check(self, status: int) -> None:
        if status == ffi.HMC_OK:
            return
        message = self.lib.hmc_last_error().decode()
        if status == ffi.HMC_OUT_OF_MEMORY:
            raise OutOfMemory(message)
        raise PoolFailed(message)

    def allocate(self, nbytes: int) -> Block:
        """A block of at least `nbytes`; 0 bytes give a null block that owns nothing (src/storage.rs:253-270)."""
        if nbytes == 0:
            return Block(0, 0, self, live=False)
        addr, size = ctypes.c_uint64(), ctypes.c_uint64()
        self._check(self.lib.hmc_allocator_allocate(self.handle, nbytes, ctypes.byref(addr), ctypes.byref(size)))
        return Block(addr.value, size.value, self)

    def release(self, addr: int) -> None:
        if self.handle is not None:
            self._check(self.lib.hmc_allocator_release(self.handle, addr))

    def empty_cache(self) -> None:
        self._check(self.lib.hmc_allocator_empty_cache(self.handle))

    def memory_stats(self) -> dict:
        st = ffi.hmc_memory_stats()
        self._check(self.lib.hmc_allocator_stats(self.handle, ctypes.byref(st)))
        return {"allocated": st.allocated, "reserved": st.reserved, "peak": st.peak}

    def reset_peak_memory_stats(self) -> None:
        self._check(self.lib.hmc_allocator_reset_peak(self.handle))

    def destroy(self) -> None:
        if self.handle is not None:
            handle, self.handle = self.handle, None
            self._check(self.lib.hmc_allocator_destroy(handle))


def rounded(nbytes: int, lib=None):
    """(rounded size, small pool?) or None when rounding overflows (caching.rs:120-126)."""
    from . import load
    lib = lib or load()
    size, small = ctypes.c_uint64(), ctypes.c_int32()
    if lib.hmc_allocator_rounded(nbytes, ctypes.byref(size), ctypes.byref(small)) != ffi.HMC_OK:
        return None
    return size.value, bool(small.value)
