"""hmc_reduce_noalloc, the reduction entry point for callers that cannot allocate a workspace (it keeps its
partial results in a fixed array inside the library instead): called through the C ABI twice in a row on
different data, its outputs must carry the bits of hmc_reduce with a caller-allocated workspace, since both
run the same plan. Collected last on purpose, so that a run that stops at the first failure has already run
every other test; it also passes alone in a fresh process."""
import ctypes

import numpy as np
import pytest

from homura_b200 import ffi
from homura_b200.host import F32, I32, I64, U8, describe, output_desc
from values import assert_same, words

pytestmark = pytest.mark.gpu


def normal(n, seed):
    w = words(seed, 2 * n)
    u1 = ((w[:n] >> np.uint64(11)).astype(np.float64) + 0.5) / float(1 << 53)
    u2 = (w[n:] >> np.uint64(11)).astype(np.float64) / float(1 << 53)
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)


def reduce_both(cuda, op, src, mask, out_dtype, out_shape):
    """(result of hmc_reduce with an allocated workspace, result of hmc_reduce_noalloc, workspace bytes)."""
    r = describe("reduce", src, mask)
    nbytes = ctypes.c_int64()
    assert cuda.lib.hmc_reduce_workspace(r.kept, r.red, 0, ctypes.byref(nbytes)) == ffi.HMC_OK
    want = cuda.empty(out_shape, out_dtype)
    ws = cuda.workspace(nbytes.value)
    cuda._check(cuda.lib.hmc_reduce(cuda.ctx, op, output_desc("reduce", r, want), r.kept, r.red,
                                    ws.ptr if ws else None, nbytes.value))
    got = cuda.empty(out_shape, out_dtype)
    cuda._check(cuda.lib.hmc_reduce_noalloc(cuda.ctx, op, output_desc("reduce", r, got), r.kept, r.red))
    return cuda.download(want), cuda.download(got), nbytes.value


def test_two_calls_in_a_row_match_the_workspace_entry_point(cuda):
    # first call: a full sum of 2^22 floats, whose plan cuts the range into chunks with partials
    a = cuda.upload(normal(1 << 22, 301), F32)
    want, got, nbytes = reduce_both(cuda, ffi.HMC_REDUCE_SUM, a, [True], F32, ())
    assert nbytes > 0, "the test must exercise the scratch array"
    assert_same(got, want, F32, "full sum through the built-in scratch")
    # second call, straight after, other data, other op, other plan (columns): what the first call left
    # in the array must not leak into it
    b = cuda.upload((words(302, 4096 * 1024) % np.uint64(2001)).astype(np.int64).astype(np.int32) - 1000, I32, (4096, 1024))
    want, got, nbytes = reduce_both(cuda, ffi.HMC_REDUCE_MAX, b, [True, False], I32, (1024,))
    assert nbytes > 0
    assert_same(got, want, I32, "column max through the built-in scratch")
    want, got, _ = reduce_both(cuda, ffi.HMC_REDUCE_SUM, b, [True, False], I64, (1024,))
    assert_same(got, want, I64, "column sum through the built-in scratch")
    assert (got == cuda.download(b).astype(np.int64).sum(axis=0)).all()
    # a plan without chunks needs no scratch and takes the same entry point
    want, got, nbytes = reduce_both(cuda, ffi.HMC_REDUCE_SUM, b, [False, True], I64, (4096,))
    assert nbytes == 0
    assert_same(got, want, I64, "row sum")


def test_a_reduction_beyond_the_built_in_scratch_is_refused(cuda):
    # 56000 adjacent u8 outputs folded over 2048 rows: two chunks of 16-byte partials, 1.8 MB
    k, r, o = ffi.hmc_tensor_desc(), ffi.hmc_tensor_desc(), ffi.hmc_tensor_desc()
    dummy = cuda.empty((16,), U8)
    for d, dt in ((k, U8), (r, U8), (o, I64)):
        d.data, d.dtype, d.ndim = dummy.storage.ptr, dt, 1
    k.sizes[0], k.strides[0] = 56000, 1
    r.sizes[0], r.strides[0] = 2048, 56000
    o.sizes[0], o.strides[0] = 56000, 1
    need = ctypes.c_int64()
    assert cuda.lib.hmc_reduce_workspace(ctypes.byref(k), ctypes.byref(r), 0, ctypes.byref(need)) == ffi.HMC_OK
    assert need.value > ffi.HMC_NOALLOC_SCRATCH_BYTES
    status = cuda.lib.hmc_reduce_noalloc(cuda.ctx, ffi.HMC_REDUCE_SUM, ctypes.byref(o), ctypes.byref(k), ctypes.byref(r))
    assert status == ffi.HMC_INVALID
    message = cuda.lib.hmc_last_error().decode()
    assert str(need.value) in message and str(ffi.HMC_NOALLOC_SCRATCH_BYTES) in message


def test_a_warmed_call_leaves_the_free_device_memory_unchanged(cuda):
    """Once the kernels of a reduction have run (the runtime loads a kernel's code at its first launch), further
    calls of the entry point take nothing from the device: free memory as the driver reports it is the same
    before and after, on the plans with and without partials."""
    a = cuda.upload(normal(1 << 22, 303), F32)
    r_full, r_rows = describe("reduce", a, [True]), describe("reduce", a.reshape(1 << 10, 1 << 12), [False, True])
    out_full, out_rows = cuda.empty((), F32), cuda.empty((1 << 10,), F32)

    def call():
        cuda._check(cuda.lib.hmc_reduce_noalloc(cuda.ctx, ffi.HMC_REDUCE_SUM, output_desc("reduce", r_full, out_full), r_full.kept, r_full.red))
        cuda._check(cuda.lib.hmc_reduce_noalloc(cuda.ctx, ffi.HMC_REDUCE_SUM, output_desc("reduce", r_rows, out_rows), r_rows.kept, r_rows.red))
        cuda.synchronize()

    def free_bytes():
        free, total = ctypes.c_uint64(), ctypes.c_uint64()
        cuda._check(cuda.lib.hmc_mem_get_info(cuda.device, ctypes.byref(free), ctypes.byref(total)))
        return free.value

    call()  # warm: module and kernels resident
    before = free_bytes()
    for _ in range(3):
        call()
    assert free_bytes() == before, "hmc_reduce_noalloc changed the device's free memory"


def test_sizes_whose_product_overflows_are_refused(cuda):
    k, r, o = ffi.hmc_tensor_desc(), ffi.hmc_tensor_desc(), ffi.hmc_tensor_desc()
    dummy = cuda.empty((16,), U8)
    for d, dt in ((k, U8), (r, U8), (o, I64)):
        d.data, d.dtype, d.ndim = dummy.storage.ptr, dt, 1
    k.ndim = 2
    k.sizes[0], k.strides[0], k.sizes[1], k.strides[1] = 1 << 40, 0, 1 << 40, 0
    r.sizes[0], r.strides[0] = 4, 1
    o.sizes[0], o.strides[0] = 4, 1
    assert cuda.lib.hmc_reduce_noalloc(cuda.ctx, ffi.HMC_REDUCE_SUM, ctypes.byref(o), ctypes.byref(k), ctypes.byref(r)) == ffi.HMC_INVALID
    assert b"too many outputs" in cuda.lib.hmc_last_error()
    k.ndim, k.sizes[0], k.strides[0] = 1, 4, 1
    r.ndim = 2
    r.sizes[0], r.strides[0], r.sizes[1], r.strides[1] = 1 << 40, 0, 1 << 40, 0
    assert cuda.lib.hmc_reduce_noalloc(cuda.ctx, ffi.HMC_REDUCE_SUM, ctypes.byref(o), ctypes.byref(k), ctypes.byref(r)) == ffi.HMC_INVALID
    assert b"too many reduced elements" in cuda.lib.hmc_last_error()
