"""Contexts, memory and failure paths on a real GPU, after homura's src/backend/rocm/tests.rs:668-807 and
tests/rocm_memory.rs. Every failure is injected on the host: nothing here faults, traps or hangs the GPU."""
import ctypes

import numpy as np
import pytest

import homura_b200
from homura_b200 import ffi
from homura_b200.host import F32, BackendError, CudaBackend

pytestmark = pytest.mark.gpu


def test_device_properties_and_memory_info(cuda):
    lib = cuda.lib
    n = ctypes.c_int32()
    assert lib.hmc_device_count(ctypes.byref(n)) == 0 and n.value >= 1
    p = ffi.hmc_device_properties()
    assert lib.hmc_device_properties_get(0, ctypes.byref(p)) == 0
    assert b"B200" in p.name and p.arch == b"sm_100" and p.warp_size == 32 and p.multiprocessor_count == 148
    assert p.total_memory > 150 * 2**30
    free, total = ctypes.c_uint64(), ctypes.c_uint64()
    assert lib.hmc_mem_get_info(0, ctypes.byref(free), ctypes.byref(total)) == 0
    assert 0 < free.value <= total.value == p.total_memory
    assert lib.hmc_device_properties_get(n.value, ctypes.byref(p)) == ffi.HMC_INVALID


def test_failed_context_creation_leaks_nothing_and_can_be_retried(cuda):
    lib = cuda.lib
    before = lib.hmc_test_live_streams()
    ctx = ctypes.c_void_p()
    lib.hmc_test_fail_stream_create(1)
    assert lib.hmc_context_create(0, ctypes.byref(ctx)) == ffi.HMC_OUT_OF_MEMORY
    assert not ctx.value and lib.hmc_test_live_streams() == before
    lib.hmc_test_fail_after_probe(1)
    assert lib.hmc_context_create(0, ctypes.byref(ctx)) == ffi.HMC_OUT_OF_MEMORY
    assert lib.hmc_last_error() == b"out of host memory"
    assert not ctx.value and lib.hmc_test_live_streams() == before
    assert lib.hmc_context_create(0, ctypes.byref(ctx)) == 0
    assert lib.hmc_test_live_streams() == before + 1
    assert lib.hmc_context_destroy(ctx) == 0
    assert lib.hmc_test_live_streams() == before
    assert lib.hmc_context_create(99, ctypes.byref(ctx)) == ffi.HMC_INVALID
    lib.hmc_test_fail_properties(1)
    p = ffi.hmc_device_properties()
    assert lib.hmc_device_properties_get(0, ctypes.byref(p)) == ffi.HMC_CUDA_ERROR
    assert lib.hmc_device_properties_get(0, ctypes.byref(p)) == 0


def test_injected_data_failures_queue_nothing(cuda):
    lib = cuda.lib
    x = cuda.upload(np.arange(1000, dtype=np.float32), F32)
    out = cuda.upload(np.zeros(1000, dtype=np.float32), F32)
    for oom, status in ((1, ffi.HMC_OUT_OF_MEMORY), (0, ffi.HMC_CUDA_ERROR)):
        lib.hmc_test_fail_data(1, oom)
        with pytest.raises(BackendError) as e:
            cuda.unary(ffi.HMC_UNARY_NEG, out, x)
        assert e.value.status == status
        assert (cuda.download(out) == 0).all()
    cuda.unary(ffi.HMC_UNARY_NEG, out, x)
    assert (cuda.download(out) == -np.arange(1000, dtype=np.float32)).all()
    # the runtime's own last error stays clean after a refused launch
    d = ctypes.c_int32()
    assert lib.hmc_test_current_device(ctypes.byref(d)) == 0 and d.value == 0


def test_memset_and_host_copies(cuda):
    lib = cuda.lib
    t = cuda.empty((4096,), F32)
    assert lib.hmc_memset(cuda.ctx, t.storage.ptr, 0x3F, 4096 * 4) == 0
    assert (cuda.download(t).view(np.uint32) == 0x3F3F3F3F).all()
    src = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    u = cuda.upload(src, F32)
    assert lib.hmc_copy_device(cuda.ctx, t.storage.ptr, u.storage.ptr, 4096 * 4) == 0
    assert (cuda.download(t) == src).all()
    assert lib.hmc_copy_to_host(cuda.ctx, None, None, 0) == 0


def test_allocator_on_the_device_caches_and_reports(cuda):
    if cuda.debug:
        pytest.skip("guard bands round every block up: the byte counts below are those of a plain run")
    a = cuda.allocator
    a.empty_cache()
    before = a.memory_stats()
    t = cuda.empty((1 << 20,), F32)  # 4 MiB: a segment of its own
    s = a.memory_stats()
    assert s["allocated"] == before["allocated"] + (4 << 20) and s["reserved"] >= before["reserved"] + (4 << 20)
    ptr = t.storage.ptr
    del t
    assert a.memory_stats()["allocated"] == before["allocated"]
    assert a.memory_stats()["reserved"] == s["reserved"]      # cached
    t2 = cuda.empty((1 << 20,), F32)
    assert t2.storage.ptr == ptr                               # reused without asking the device
    del t2
    a.empty_cache()
    assert a.memory_stats()["reserved"] == before["reserved"]
    # a refused segment releases the cache and is tried once more
    keep = cuda.empty((1 << 20,), F32)
    del keep
    cuda.lib.hmc_test_fail_data(1, 1)
    again = cuda.empty((3 << 19,), F32)  # 6 MiB: no cached block fits
    assert again.storage.ptr != 0
    assert a.memory_stats()["reserved"] == before["reserved"] + (6 << 20)
    # twice refused: the PyTorch-style message
    cuda.lib.hmc_test_fail_data(2, 1)
    with pytest.raises(homura_b200.caching.OutOfMemory) as e:
        cuda.empty((1 << 22,), F32)
    msg = str(e.value)
    assert msg.startswith("CUDA out of memory. Tried to allocate 16.00 MiB. cuda:0 has a total capacity of")
    assert "is allocated by homura" in msg and "reserved but unallocated" in msg


def test_a_second_context_and_eight_submitting_threads(cuda):
    import threading
    other = CudaBackend(0)
    xs = [np.full(5000, float(i), dtype=np.float32) for i in range(8)]
    outs = [None] * 8
    lock = threading.Lock()  # homura holds one lock per device around each submission

    def work(i):
        be = cuda if i % 2 == 0 else other
        with lock:
            x = be.upload(xs[i], F32)
            o = be.empty((5000,), F32)
            be.unary(ffi.HMC_UNARY_EXP, o, x)
            outs[i] = be.download(o)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(8)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    for i in range(8):
        assert np.allclose(outs[i], np.exp(np.float32(i)), rtol=1e-6)
    other.close()
