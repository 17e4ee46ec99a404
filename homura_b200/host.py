"""Host-side glue above the C ABI: what homura's ``src/backend/rocm/{copy,elementwise,reduce}.rs`` do for
its ROCm layer, restated for ``libhomura_cuda.so``.

* :class:`TensorData`: a strided view (shape, element strides, element offset, dtype) of a storage, homura's
  ``TensorData`` / ``Layout`` (``src/tensor/mod.rs:83-336``), with the view constructors its tests use.
* :func:`merge_dims`, :func:`descs`: drop size-1 dimensions and merge neighbours that are contiguous in
  every operand (``src/backend/rocm/copy.rs:34-115``), giving the ``hmc_tensor_desc`` the kernels take.
* :func:`describe`, :func:`lines`: the kept/reduced split of a reduction and the rows of a softmax
  (``src/backend/rocm/reduce.rs:42-75, 216-256``).
* :class:`CudaBackend`: ``copy, fill, unary, binary, binary_constant, binary_scalar, fused, where_,
  where_constant, reduce, var, arg_reduce, softmax`` with the argument meaning of homura's
  ``backend::*`` functions (``src/backend/mod.rs:60-358``): outputs are allocated by the caller,
  workspaces are taken from the allocator before the call, failures raise :class:`BackendError` carrying
  the library's message (the Rust side panics or returns ``Error::OutOfMemory``).

The Rust host of a real integration keeps all of this in Rust; there is no Rust toolchain where this was
written, so the same logic is exercised from Python through ctypes. Only the CUDA path exists here: there is
no CPU fallback, and a missing or unloadable library is an error.
"""
from __future__ import annotations

import ctypes
import math
import os
import weakref
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

from . import ffi
from .ffi import hmc_tensor_desc

BOOL, U8, I8, I16, I32, I64, F16, BF16, F32, F64 = range(10)
DTYPE_NAMES = ["bool", "u8", "i8", "i16", "i32", "i64", "f16", "bf16", "f32", "f64"]
ALL_DTYPES = list(range(10))
FLOATS = [F16, BF16, F32, F64]
INTS = [U8, I8, I16, I32, I64]
# numpy type that holds the raw element (bool as a byte, f16/bf16 as their bit patterns)
STORAGE = [np.uint8, np.uint8, np.int8, np.int16, np.int32, np.int64, np.uint16, np.uint16, np.float32, np.float64]
SIZE = [1, 1, 1, 2, 4, 8, 2, 2, 4, 8]
MAX_DIMS = ffi.HMC_MAX_DIMS


def is_float(dt: int) -> bool:
    return dt >= F16


def is_int(dt: int) -> bool:
    return U8 <= dt <= I64


class BackendError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def contiguous_strides(shape: Sequence[int]) -> list[int]:
    st, acc = [], 1
    for n in reversed(shape):
        st.append(acc)
        acc *= max(n, 1)
    return st[::-1]


@dataclass
class Storage:
    """Device memory (``ptr`` on ``device``) or host memory (``array``)."""
    nbytes: int
    ptr: int = 0
    device: Optional[int] = None
    array: Optional[np.ndarray] = None
    owner: object = None  # the allocator block that frees the memory

    @property
    def address(self) -> int:
        return self.ptr if self.array is None else self.array.ctypes.data


@dataclass
class TensorData:
    storage: Storage
    dtype: int
    shape: tuple
    strides: tuple
    offset: int = 0

    @property
    def numel(self) -> int:
        return math.prod(self.shape)

    def is_contiguous(self) -> bool:
        expect = 1
        for n, s in zip(reversed(self.shape), reversed(self.strides)):
            if n != 1 and s != expect:
                return False
            expect *= n
        return True

    def _view(self, shape, strides, offset=None) -> "TensorData":
        return TensorData(self.storage, self.dtype, tuple(shape), tuple(strides), self.offset if offset is None else offset)

    # view constructors (no data movement)
    def reshape(self, *shape) -> "TensorData":
        shape = tuple(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else tuple(shape)
        assert self.is_contiguous() and math.prod(shape) == self.numel, "reshape of a non-contiguous view"
        return self._view(shape, contiguous_strides(shape))

    def transpose(self, a: int, b: int) -> "TensorData":
        sh, st = list(self.shape), list(self.strides)
        sh[a], sh[b] = sh[b], sh[a]
        st[a], st[b] = st[b], st[a]
        return self._view(sh, st)

    def t(self) -> "TensorData":
        return self.transpose(0, 1)

    def permute(self, *dims) -> "TensorData":
        dims = tuple(dims[0]) if len(dims) == 1 and isinstance(dims[0], (tuple, list)) else dims
        return self._view([self.shape[d] for d in dims], [self.strides[d] for d in dims])

    def narrow(self, dim: int, start: int, length: int) -> "TensorData":
        sh = list(self.shape)
        sh[dim] = length
        return self._view(sh, self.strides, self.offset + start * self.strides[dim])

    def select(self, dim: int, index: int) -> "TensorData":
        sh, st = list(self.shape), list(self.strides)
        off = self.offset + index * st[dim]
        del sh[dim], st[dim]
        return self._view(sh, st, off)

    def expand(self, *shape) -> "TensorData":
        shape = tuple(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else tuple(shape)
        pad = len(shape) - len(self.shape)
        sh = (1,) * pad + tuple(self.shape)
        st = (0,) * pad + tuple(self.strides)
        out = []
        for n, have, s in zip(shape, sh, st):
            if have == n:
                out.append(s)
            else:
                assert have == 1, f"cannot expand {self.shape} to {shape}"
                out.append(0)
        return self._view(shape, out)

    def unsqueeze(self, dim: int) -> "TensorData":
        sh, st = list(self.shape), list(self.strides)
        sh.insert(dim, 1)
        st.insert(dim, 0)
        return self._view(sh, st)


def merge_dims(shape: Sequence[int], strides: Sequence[Sequence[int]]):
    """``[(size, [stride per operand])]`` outermost first, or None for an empty shape.
    src/backend/rocm/copy.rs:34-57 (the CPU twin is Plan::new, src/backend/cpu/iter.rs:27-55)."""
    if 0 in shape:
        return None
    dims: list[tuple[int, list[int]]] = []
    for i, size in enumerate(shape):
        if size == 1:
            continue
        st = [s[i] for s in strides]
        if dims:
            outer_size, outer_st = dims[-1]
            if all(st[k] * size == outer_st[k] and st[k] * size < 2**63 for k in range(len(st))):
                dims[-1] = (outer_size * size, st)
                continue
        dims.append((size, st))
    return dims


# Debug runs (HOMURA_CUDA_DEBUG=1) check every description against its storage before the call: the last element a
# kernel can reach from it must lie inside the allocation. A description that reaches beyond is refused on the host
# with both numbers, instead of a kernel reading or writing beside its buffer.
CHECK_REACH = os.environ.get("HOMURA_CUDA_DEBUG", "") not in ("", "0")


def check_reach(kernel: str, t: TensorData, offset: int, dims, k: int, extra: int = 0) -> None:
    """`dims` as merge_dims gives them ([(size, strides per operand)]); `extra`: elements another description of the
    same operand adds to the farthest one of this (a reduction's kept and reduced parts)."""
    if any(size == 0 for size, _ in dims):
        return
    reach = offset + extra + sum((size - 1) * st[k] for size, st in dims)
    have = t.storage.nbytes // SIZE[t.dtype]
    if reach >= have or offset < 0:
        raise BackendError(ffi.HMC_INVALID, f"debug: {kernel}: an operand of {DTYPE_NAMES[t.dtype]} reaches element {reach} of a "
                                            f"storage of {have} elements")


def descs_with_dims(kernel: str, operands: Sequence[TensorData], offsets: Sequence[int], dims, check: bool = True) -> list[hmc_tensor_desc]:
    """src/backend/rocm/copy.rs:86-115. `check=False` for descriptions whose sizes are not the operand's own (the indexing
    kernels describe their source with the output's sizes and find its rows through the index)."""
    if len(dims) > MAX_DIMS:
        raise BackendError(ffi.HMC_INVALID, f"{kernel} on CUDA supports at most {MAX_DIMS} dimensions that can't be "
                                            f"merged, got {len(dims)}")
    out = []
    for k, t in enumerate(operands):
        if CHECK_REACH and check:
            check_reach(kernel, t, offsets[k], dims, k)
        d = hmc_tensor_desc()
        d.data = t.storage.address
        d.offset = offsets[k]
        d.dtype = t.dtype
        d.ndim = len(dims)
        for j, (size, st) in enumerate(dims):
            d.sizes[j] = size
            d.strides[j] = st[k]
        out.append(d)
    return out


def descs(kernel: str, operands: Sequence[TensorData]) -> Optional[list[hmc_tensor_desc]]:
    """Descriptions of same-shaped operands, None when they have no elements. copy.rs:59-84."""
    shape = operands[0].shape
    for t in operands[1:]:
        assert tuple(t.shape) == tuple(shape), "kernel operands must have the same shape"
    dims = merge_dims(shape, [t.strides for t in operands])
    if dims is None:
        return None
    return descs_with_dims(kernel, operands, [t.offset for t in operands], dims)


@dataclass
class Reduction:
    dims: list
    kept: hmc_tensor_desc
    red: hmc_tensor_desc


def describe(kernel: str, src: TensorData, mask: Sequence[bool]) -> Optional[Reduction]:
    """src/backend/rocm/reduce.rs:42-75."""
    strides = src.strides if src.numel > 0 else (0,) * len(src.strides)
    kept_shape, kept_strides, red_shape, red_strides = [], [], [], []
    for size, stride, reduced in zip(src.shape, strides, mask):
        if reduced:
            red_shape.append(size)
            red_strides.append(stride)
        else:
            kept_shape.append(size)
            kept_strides.append(stride)
    out_strides = contiguous_strides(kept_shape)
    dims = merge_dims(kept_shape, [out_strides, kept_strides])
    if dims is None:
        return None
    red_dims = merge_dims(red_shape, [red_strides])
    if red_dims is None:
        red_dims = [(0, [0])]  # nothing to fold
    src_dims = [(n, [st[1]]) for n, st in dims]
    if CHECK_REACH and src.numel > 0:
        check_reach(kernel, src, src.offset, src_dims, 0, extra=sum((n - 1) * st[0] for n, st in red_dims))
    # (each half alone says nothing about the reach: the check above covers both together)
    (kept,) = descs_with_dims(kernel, [src], [src.offset], src_dims, check=False)
    (red,) = descs_with_dims(kernel, [src], [0], red_dims, check=False)
    return Reduction(dims, kept, red)


def output_desc(kernel: str, r: Reduction, out: TensorData) -> hmc_tensor_desc:
    assert out.is_contiguous(), f"internal error: {kernel} into a strided tensor"
    dims = [(n, [st[0]]) for n, st in r.dims]
    (d,) = descs_with_dims(kernel, [out], [out.offset], dims)
    return d


def lines(kernel: str, out: TensorData, src: TensorData, dim: int, out_strides: Sequence[int]):
    """Rows along `dim`: (descs of the other dims for out and src, n, out stride, src stride).
    src/backend/rocm/reduce.rs:216-256."""
    assert tuple(out.shape) == tuple(src.shape), "kernel operands must have the same shape"
    if src.numel == 0:
        return None
    shape = src.shape
    others = lambda v: [s for d, s in enumerate(v) if d != dim]
    if len(shape) == 0:
        n, so, si = 1, 0, 0
    else:
        n, so, si = shape[dim], out_strides[dim], src.strides[dim]
    dims = merge_dims(others(shape), [others(out_strides), others(src.strides)])
    if dims is None:
        return None
    d = descs_with_dims(kernel, [out, src], [out.offset, src.offset], dims)
    return d, n, so, si


def scalar_bits(value, dtype: int) -> int:
    """The element of `dtype` holding `value` as the low bytes of a u64 (src/backend/rocm/copy.rs:256-270):
    floats are rounded as Sealed::from_f64 rounds them (half types through f32), integers wrap."""
    if dtype == BOOL:
        return int(bool(value))
    if is_int(dtype):
        v = int(value)  # trunc toward zero for floats
        return v & ((1 << (8 * SIZE[dtype])) - 1)
    if dtype == F64:
        return int(np.array([value], dtype=np.float64).view(np.uint64)[0])
    f = np.array([value], dtype=np.float64).astype(np.float32)
    if dtype == F32:
        return int(f.view(np.uint32)[0])
    return int(f32_to_half_bits(f, dtype)[0])


def f32_to_half_bits(f: np.ndarray, dtype: int) -> np.ndarray:
    """`half`'s f32 -> f16 / bf16 (round to nearest even; a NaN keeps its top payload bits, made quiet)."""
    x = f.astype(np.float32).view(np.uint32)
    if dtype == BF16:
        nan = (x & 0x7FFFFFFF) > 0x7F800000
        r = ((x.astype(np.uint64) + 0x7FFF + ((x >> 16) & 1)) >> 16).astype(np.uint16)
        return np.where(nan, ((x >> 16) | 0x40).astype(np.uint16), r)
    with np.errstate(over="ignore", invalid="ignore"):
        h = f.astype(np.float16).view(np.uint16)
    nan = (x & 0x7FFFFFFF) > 0x7F800000
    q = (((x >> 16) & 0x8000) | 0x7E00 | ((x >> 13) & 0x3FF)).astype(np.uint16)
    return np.where(nan, q, h)


def half_bits_to_f32(b: np.ndarray, dtype: int) -> np.ndarray:
    b = b.astype(np.uint16)
    if dtype == BF16:
        return (b.astype(np.uint32) << 16).view(np.float32)
    return b.view(np.float16).astype(np.float32)


class CudaBackend:
    """One device: its context (stream), a caching allocator over hmc_malloc/hmc_free, and homura's backend
    functions on :class:`TensorData` whose storage lives on that device."""

    name = "cuda"

    def __init__(self, device: int = 0, lib=None, allocator=None):
        from . import load
        self.lib = lib or load()
        self.device = device
        ctx = ctypes.c_void_p()
        self._check(self.lib.hmc_context_create(device, ctypes.byref(ctx)))
        self.ctx = ctx
        if allocator is None:
            from .caching import CachingAllocator, CudaMemory
            allocator = CachingAllocator(CudaMemory(self.lib, device, self))
        self.allocator = allocator
        self.debug = os.environ.get("HOMURA_CUDA_DEBUG", "") not in ("", "0")
        self._guarded, self.guard_failures = {}, []

    # ---- plumbing ----
    def _check(self, status: int) -> None:
        if status != ffi.HMC_OK:
            raise BackendError(status, self.lib.hmc_last_error().decode())

    def close(self) -> None:
        if self.ctx is not None:
            self.synchronize()
            self.check_guards()
            self.allocator.destroy()
            self._check(self.lib.hmc_context_destroy(self.ctx))
            self.ctx = None

    def synchronize(self) -> None:
        self._check(self.lib.hmc_context_synchronize(self.ctx))

    GUARD = 256          # bytes of guard band either side of a debug allocation
    GUARD_BYTE = 0xA5

    def storage(self, nbytes: int) -> Storage:
        """Device memory for a tensor or a workspace. In a debug run (environment variable HOMURA_CUDA_DEBUG=1) the
        memory is poisoned with 0xFF bytes, so that an element nothing wrote shows as NaN / -1 / true (what homura's
        debug builds do with their "uninit" memory, src/tensor/mod.rs:404-437), and sits between two guard bands
        that :meth:`check_guards` (called by :meth:`close`, and when a storage is dropped) finds intact or not: the
        stand-in for a memory checker on machines where none can run."""
        if not self.debug:
            block = self.allocator.allocate(nbytes)
            return Storage(nbytes, ptr=block.ptr, device=self.device, owner=block)
        g = self.GUARD
        padded = (nbytes + 15) // 16 * 16
        block = self.allocator.allocate(padded + 2 * g)
        lib, ctx = self.lib, self.ctx
        self._check(lib.hmc_memset(ctx, block.ptr, self.GUARD_BYTE, g))
        if padded:
            self._check(lib.hmc_memset(ctx, block.ptr + g, 0xFF, padded))
        self._check(lib.hmc_memset(ctx, block.ptr + g + padded, self.GUARD_BYTE, g))
        st = Storage(nbytes, ptr=block.ptr + g, device=self.device, owner=block)
        self._guarded[id(st)] = (block.ptr, padded)
        weakref.finalize(st, self._dropped, id(st))
        return st

    def _dropped(self, key: int) -> None:
        entry = self._guarded.pop(key, None)
        if entry is not None and self.ctx is not None:
            bad = self._guard_damage(*entry)
            if bad:
                self.guard_failures.append(bad)

    def _guard_damage(self, base: int, padded: int) -> str:
        g = self.GUARD
        band = np.empty(2 * g, dtype=np.uint8)
        self._check(self.lib.hmc_copy_to_host(self.ctx, band.ctypes.data, base, g))
        self._check(self.lib.hmc_copy_to_host(self.ctx, band.ctypes.data + g, base + g + padded, g))
        hit = np.nonzero(band != self.GUARD_BYTE)[0]
        if hit.size == 0:
            return ""
        first = int(hit[0])
        where = f"{g - first} bytes before its start" if first < g else f"{first - g} bytes past its end"
        return f"the allocation of {padded} bytes at {base + g:#x} was written {where} ({hit.size} guard bytes changed)"

    def check_guards(self) -> None:
        """Raises if a kernel wrote outside any live (or since dropped) debug allocation. No-op outside debug runs."""
        if not self.debug:
            return
        found = list(self.guard_failures)
        for base, padded in list(self._guarded.values()):
            bad = self._guard_damage(base, padded)
            if bad:
                found.append(bad)
        self.guard_failures.clear()
        if found:
            raise BackendError(ffi.HMC_INTERNAL_ERROR, "out-of-bounds write: " + "; ".join(found))

    def empty(self, shape, dtype: int) -> TensorData:
        shape = tuple(shape)
        return TensorData(self.storage(math.prod(shape) * SIZE[dtype]), dtype, shape, tuple(contiguous_strides(shape)))

    def workspace(self, nbytes: int) -> Optional[Storage]:
        return self.storage(nbytes) if nbytes > 0 else None

    def upload(self, array: np.ndarray, dtype: int, shape=None) -> TensorData:
        """A contiguous device tensor with the raw elements of `array` (storage dtype of `dtype`)."""
        array = np.ascontiguousarray(array, dtype=STORAGE[dtype])
        shape = tuple(array.shape if shape is None else shape)
        t = self.empty(shape, dtype)
        if array.nbytes:
            self._check(self.lib.hmc_copy_from_host(self.ctx, t.storage.ptr, array.ctypes.data, array.nbytes))
        return t

    def download_storage(self, t: TensorData) -> np.ndarray:
        """The whole storage behind `t` as a flat array of its storage dtype."""
        n = t.storage.nbytes // SIZE[t.dtype]
        out = np.empty(n, dtype=STORAGE[t.dtype])
        if out.nbytes:
            self._check(self.lib.hmc_copy_to_host(self.ctx, out.ctypes.data, t.storage.ptr, out.nbytes))
        return out

    def download(self, t: TensorData) -> np.ndarray:
        """The elements of `t` in row-major order (raw storage dtype), whatever its layout."""
        flat = self.download_storage(t)
        if t.numel == 0:
            return np.empty(t.shape, dtype=STORAGE[t.dtype])
        es = SIZE[t.dtype]
        view = np.lib.stride_tricks.as_strided(flat[t.offset:], shape=t.shape, strides=[s * es for s in t.strides],
                                               writeable=False)
        return np.ascontiguousarray(view).reshape(t.shape)

    # ---- homura's backend functions ----
    def copy(self, dst: TensorData, src: TensorData) -> None:
        src = src.expand(dst.shape)
        d = descs("copy", [dst, src])
        if d is None:
            return
        self._check(self.lib.hmc_copy(self.ctx, d[0], d[1]))

    def fill(self, dst: TensorData, value) -> None:
        d = descs("fill", [dst])
        if d is None:
            return
        self._check(self.lib.hmc_fill(self.ctx, d[0], scalar_bits(value, dst.dtype)))

    def unary(self, op: int, out: TensorData, src: TensorData) -> None:
        d = descs("unary", [out, src])
        if d is None:
            return
        self._check(self.lib.hmc_unary(self.ctx, op, d[0], d[1]))

    def binary(self, op: int, out: TensorData, a: TensorData, b: TensorData) -> None:
        d = descs("binary", [out, a, b])
        if d is None:
            return
        self._check(self.lib.hmc_binary(self.ctx, op, d[0], d[1], d[2]))

    def binary_promoted(self, op: int, out: TensorData, a: TensorData, b: TensorData) -> None:
        d = descs("binary_promoted", [out, a, b])
        if d is None:
            return
        self._check(self.lib.hmc_binary_promoted(self.ctx, op, d[0], d[1], d[2]))

    def unary_binary_binary(self, unary_op: int, first_op: int, second_op: int, out: TensorData, x: TensorData,
                            b: TensorData, c: TensorData) -> None:
        """out = (unary(x) first_op b) second_op c in one kernel with the three kernels' roundings; b and c
        broadcast to out's shape."""
        d = descs("unary_binary_binary", [out, x.expand(out.shape), b.expand(out.shape), c.expand(out.shape)])
        if d is None:
            return
        self._check(self.lib.hmc_unary_binary_binary(self.ctx, unary_op, first_op, second_op, d[0], d[1], d[2], d[3]))

    def binary_constant(self, op: int, out: TensorData, a: TensorData, value, constant_first: bool) -> None:
        bits = scalar_bits(value, a.dtype)
        d = descs("binary_constant", [out, a])
        if d is None:
            return
        self._check(self.lib.hmc_binary_constant(self.ctx, op, d[0], d[1], bits, int(constant_first)))

    def binary_scalar(self, op: int, out: TensorData, a: TensorData, s: float, scalar_first: bool) -> None:
        assert op in (ffi.HMC_BINARY_MUL, ffi.HMC_BINARY_DIV), "this op rounds its scalar to the dtype"
        d = descs("binary_scalar", [out, a])
        if d is None:
            return
        self._check(self.lib.hmc_binary_scalar(self.ctx, op, d[0], d[1], float(s), int(scalar_first)))

    def fused(self, op: int, value: float, out: TensorData, a: TensorData, b: TensorData,
              c: Optional[TensorData] = None) -> None:
        """`op` is an HMC_FUSED_* code, `value` homura's Fused payload (alpha, weight or value); the
        coefficient is computed here as the CPU computes it (src/backend/rocm/elementwise.rs:163-187)."""
        coefficient, small = fused_coefficient(op, value, out.dtype)
        ops = [out, a, b] + ([c] if c is not None else [])
        d = descs("fused", ops)
        if d is None:
            return
        self._check(self.lib.hmc_fused(self.ctx, op, d[0], d[1], d[2], d[3] if c is not None else None,
                                       coefficient, int(small)))

    def where_(self, out: TensorData, cond: TensorData, x: TensorData, y: TensorData) -> None:
        d = descs("where_", [out, cond, x, y])
        if d is None:
            return
        self._check(self.lib.hmc_where(self.ctx, d[0], d[1], d[2], d[3]))

    def where_constant(self, out: TensorData, cond: TensorData, x, y) -> None:
        """x / y: a TensorData, or a Python scalar for a constant branch."""
        xt, yt = isinstance(x, TensorData), isinstance(y, TensorData)
        if xt and yt:
            return self.where_(out, cond, x, y)
        ops = [out, cond] + ([x] if xt else []) + ([y] if yt else [])
        d = descs("where_constant", ops)
        if d is None:
            return
        xb = 0 if xt else scalar_bits(x, out.dtype)
        yb = 0 if yt else scalar_bits(y, out.dtype)
        xd = d[2] if xt else None
        yd = d[2] if (yt and not xt) else (d[3] if yt else None)
        self._check(self.lib.hmc_where_constant(self.ctx, d[0], d[1], xd, xb, yd, yb))

    def _plan_workspace(self, r: Reduction, var: bool) -> Optional[Storage]:
        nbytes = ctypes.c_int64()
        self._check(self.lib.hmc_reduce_workspace(r.kept, r.red, int(var), ctypes.byref(nbytes)))
        return self.workspace(nbytes.value)

    def reduce(self, op: int, out: TensorData, src: TensorData, mask: Sequence[bool]) -> None:
        r = describe("reduce", src, mask)
        if r is None:
            return
        o = output_desc("reduce", r, out)
        ws = self._plan_workspace(r, False)
        self._check(self.lib.hmc_reduce(self.ctx, op, o, r.kept, r.red, ws.ptr if ws else None, ws.nbytes if ws else 0))

    def var(self, out: TensorData, src: TensorData, mask: Sequence[bool], correction: float, take_sqrt: bool) -> None:
        r = describe("var", src, mask)
        if r is None:
            return
        o = output_desc("var", r, out)
        ws = self._plan_workspace(r, True)
        self._check(self.lib.hmc_var(self.ctx, o, r.kept, r.red, float(correction), int(take_sqrt),
                                     ws.ptr if ws else None, ws.nbytes if ws else 0))

    def arg_reduce(self, values: Optional[TensorData], indices: TensorData, src: TensorData, dim: int,
                   is_max: bool) -> None:
        nd = len(src.shape)
        mask = [d == dim for d in range(nd)]
        if nd > 0:
            assert src.shape[dim] > 0, "cannot compute the arg reduction of an empty dimension"
        r = describe("arg_reduce", src, mask)
        if r is None:
            return
        i = output_desc("arg_reduce", r, indices)
        v = output_desc("arg_reduce", r, values) if values is not None else None
        ws = self._plan_workspace(r, False)
        self._check(self.lib.hmc_arg_reduce(self.ctx, v, i, r.kept, r.red, int(is_max), ws.ptr if ws else None,
                                            ws.nbytes if ws else 0))

    # ---- sharded reductions (include/homura_cuda_shard.h) ----
    def reduce_partial(self, op: int, partial: Storage, src: TensorData, mask: Sequence[bool]) -> None:
        """f64 partial sums (products) of this shard, one per output, into `partial`."""
        r = describe("reduce_partial", src, mask)
        if r is None:
            return
        ws = self._plan_workspace(r, False)
        self._check(self.lib.hmc_reduce_partial(self.ctx, op, ctypes.cast(partial.ptr, ctypes.POINTER(ctypes.c_double)),
                                                r.kept, r.red, ws.ptr if ws else None, ws.nbytes if ws else 0))

    def shard_combine_float(self, op: int, out: TensorData, gathered: Storage, ranks: int, nout: int, count: int) -> None:
        d = _flat_desc(out)
        self._check(self.lib.hmc_shard_combine_float(self.ctx, op, d, ctypes.cast(gathered.ptr, ctypes.POINTER(ctypes.c_double)),
                                                     ranks, nout, count))

    def shard_combine_means(self, means: Storage, gathered: Storage, ranks: int, nout: int, count: int) -> None:
        f64p = ctypes.POINTER(ctypes.c_double)
        self._check(self.lib.hmc_shard_combine_means(self.ctx, ctypes.cast(means.ptr, f64p), ctypes.cast(gathered.ptr, f64p),
                                                     ranks, nout, count))

    def var_partial(self, partial: Storage, src: TensorData, mask: Sequence[bool], means: Storage) -> None:
        """f64 sums of this shard's squared deviations from the given f64 means, one per output."""
        r = describe("var_partial", src, mask)
        if r is None:
            return
        ws = self._plan_workspace(r, False)
        f64p = ctypes.POINTER(ctypes.c_double)
        self._check(self.lib.hmc_var_partial(self.ctx, ctypes.cast(partial.ptr, f64p), r.kept, r.red, ctypes.cast(means.ptr, f64p),
                                             ws.ptr if ws else None, ws.nbytes if ws else 0))

    def shard_combine_var(self, out: TensorData, gathered: Storage, ranks: int, nout: int, count: int, correction: float,
                          take_sqrt: bool) -> None:
        self._check(self.lib.hmc_shard_combine_var(self.ctx, _flat_desc(out), ctypes.cast(gathered.ptr, ctypes.POINTER(ctypes.c_double)),
                                                   ranks, nout, count, float(correction), int(take_sqrt)))

    def shard_combine_int(self, op: int, out: TensorData, gathered: Storage, ranks: int, nout: int) -> None:
        d = _flat_desc(out)
        self._check(self.lib.hmc_shard_combine_int(self.ctx, op, d, ctypes.cast(gathered.ptr, ctypes.POINTER(ctypes.c_int64)),
                                                   ranks, nout))

    def shard_combine_extreme(self, is_max: bool, values: Optional[TensorData], indices: Optional[TensorData],
                              gathered_values: Storage, dtype: int, gathered_indices: Optional[Storage],
                              offsets: Optional[Sequence[int]], ranks: int, nout: int) -> None:
        off = (ctypes.c_int64 * ranks)(*offsets) if offsets is not None else None
        gi = ctypes.cast(gathered_indices.ptr, ctypes.POINTER(ctypes.c_int64)) if gathered_indices is not None else None
        self._check(self.lib.hmc_shard_combine_extreme(
            self.ctx, int(is_max), _flat_desc(values) if values is not None else None,
            _flat_desc(indices) if indices is not None else None, gathered_values.ptr, dtype, gi, off, ranks, nout))

    def softmax(self, out: TensorData, src: TensorData, dim: int, log: bool) -> None:
        ln = lines("softmax", out, src, dim, out.strides)
        if ln is None:
            return
        (o, s), n, so, si = ln
        nbytes = ctypes.c_int64()
        self._check(self.lib.hmc_softmax_workspace(s, n, si, ctypes.byref(nbytes)))
        ws = self.workspace(nbytes.value)
        self._check(self.lib.hmc_softmax(self.ctx, o, s, n, so, si, int(log), ws.ptr if ws else None,
                                         ws.nbytes if ws else 0))

    # ---- the callers either side of the path: samplers, the mask builder, flip ----
    def random_uniform(self, out: TensorData, gen: "Generator", low: float, high: float) -> None:
        """`out` (contiguous, float) filled with uniform samples of [low, high): rocm_random_tensor's Uniform arm
        (src/ops/random.rs:303-311)."""
        assert out.is_contiguous() and out.dtype in FLOATS
        per_block = 2 if out.dtype == F64 else 4
        seed, start = gen.reserve(-(-out.numel // per_block))
        self._check(self.lib.hmc_random_uniform(self.ctx, _flat_desc(out), seed, start, float(low), float(high)))

    def random_normal(self, out: TensorData, gen: "Generator", mean: float, std: float) -> None:
        """src/ops/random.rs:312-317."""
        assert out.is_contiguous() and out.dtype in FLOATS
        seed, start = gen.reserve(-(-out.numel // 2))
        self._check(self.lib.hmc_random_normal(self.ctx, _flat_desc(out), seed, start, float(mean), float(std)))

    def random_int(self, out: TensorData, gen: "Generator", low: int, high: int) -> None:
        """`out` (contiguous, I64) filled with uniform integers of [low, high): the batches of rocm_random_tensor's
        Int arm (src/ops/random.rs:318-356): each reserves a block per two values still needed, the device reports
        how many words it accepted, and the tail of the last batch is dropped."""
        assert out.is_contiguous() and out.dtype == I64 and low < high
        n = out.numel
        rng, threshold = int_range(low, high)
        ws = None
        if threshold != 0 and n > 0:
            tiles = -(-(-(-n // 2)) // ffi.HMC_RANDOM_INT_TILE)
            ws = self.storage((2 * tiles + 1) * 8)
        flat = out.reshape(n) if n != 1 else out
        done = 0
        while done < n:
            needed = n - done
            blocks = -(-needed // 2)
            seed, start = gen.reserve(blocks)
            part = flat.narrow(0, done, needed) if n != 1 else flat
            self._check(self.lib.hmc_random_int(self.ctx, _flat_desc(part), seed, start, blocks, low, rng, threshold,
                                                ws.ptr if ws else None))
            if ws is None:
                done += needed
            else:
                tiles = -(-blocks // ffi.HMC_RANDOM_INT_TILE)
                accepted = np.empty(1, dtype=np.uint64)
                self._check(self.lib.hmc_copy_to_host(self.ctx, accepted.ctypes.data, ws.ptr + 2 * tiles * 8, 8))
                done += min(int(accepted[0]), needed)

    def triangle(self, out: TensorData, src: TensorData, diagonal: int, upper: bool) -> None:
        """tril / triu over the last two dimensions (src/backend/rocm/elementwise.rs, hmr_triangle): the batch
        dimensions are merged, the last two are passed as they are."""
        assert tuple(out.shape) == tuple(src.shape) and len(src.shape) >= 2 and out.dtype == src.dtype
        if src.numel == 0:
            return
        batch = merge_dims(src.shape[:-2], [out.strides[:-2], src.strides[:-2]])
        dims = list(batch) + [(src.shape[-2], [out.strides[-2], src.strides[-2]]), (src.shape[-1], [out.strides[-1], src.strides[-1]])]
        o, i = descs_with_dims("triangle", [out, src], [out.offset, src.offset], dims)
        self._check(self.lib.hmc_triangle(self.ctx, o, i, int(diagonal), int(bool(upper))))

    def flip(self, out: TensorData, src: TensorData, dims: Sequence[int]) -> None:
        """out = src flipped along `dims` (src/backend/rocm/copy.rs flip: the source is described with negative strides
        along the flipped dimensions and its offset at the element that comes first)."""
        assert tuple(out.shape) == tuple(src.shape) and out.dtype == src.dtype
        if src.numel == 0:
            return
        strides, offset = list(src.strides), src.offset
        for d in dims:
            offset += (src.shape[d] - 1) * strides[d]
            strides[d] = -strides[d]
        flipped = TensorData(src.storage, src.dtype, tuple(src.shape), tuple(strides), offset)
        o, i = descs("flip", [out, flipped])
        self._check(self.lib.hmc_flip(self.ctx, o, i))

    def index_check(self, index: TensorData, low: int, high: int, exempt=None):
        """(position, value) of the first index element outside [low, high) that is not `exempt`, or None."""
        if index.numel == 0:
            return None
        d, = descs("index_check", [index])
        slot = self.storage(16)
        self._check(self.lib.hmc_index_check(self.ctx, d, low, high, int(exempt is not None), exempt or 0,
                                             ctypes.cast(slot.ptr, ctypes.POINTER(ctypes.c_uint64))))
        words = np.empty(2, dtype=np.uint64)
        self._check(self.lib.hmc_copy_to_host(self.ctx, words.ctypes.data, slot.ptr, 16))
        return None if int(words[0]) == 2**64 - 1 else (int(words[0]), int(words[1:].view(np.int64)[0]))

    def index_select(self, out: TensorData, src: TensorData, dim: int, index: TensorData, wrap_negative: bool = False) -> None:
        if out.numel == 0:
            return
        o, s, i, at = index_select_descs("index_select", out, src, dim, index)
        self._check(self.lib.hmc_index_select(self.ctx, o, s, i, at, int(wrap_negative)))

    def gather(self, out: TensorData, src: TensorData, dim: int, index: TensorData) -> None:
        if out.numel == 0:
            return
        (o, s, i), at = around("gather", [out, src, index], tuple(out.shape), dim)
        s.sizes[at] = src.shape[dim]
        self._check(self.lib.hmc_gather(self.ctx, o, s, i, at))

    def index_overwrite(self, out: TensorData, dim: int, positions: TensorData, src: TensorData) -> None:
        """Slice i of src along dim -> slice positions[i] of out, the last of repeated positions winning
        (src/backend/rocm/index.rs:299-340)."""
        if src.numel == 0:
            return
        assert positions.is_contiguous() and positions.dtype == I64
        (s, o), at = around("index_overwrite", [src, out], tuple(src.shape), dim)
        o.sizes[at] = out.shape[dim]
        p = hmc_tensor_desc()
        p.data, p.offset, p.dtype, p.ndim = positions.storage.address, positions.offset, I64, 1
        p.sizes[0], p.strides[0] = positions.numel, 1
        nbytes = ctypes.c_int64()
        self._check(self.lib.hmc_index_overwrite_workspace(out.shape[dim], ctypes.byref(nbytes)))
        ws = self.workspace(nbytes.value)
        self._check(self.lib.hmc_index_overwrite(self.ctx, o, s, p, at, ws.ptr if ws else None, nbytes.value))

    def mask_coordinates(self, mask: TensorData) -> list:
        """One contiguous I64 tensor of coordinates per dimension of the Bool `mask`, for its true elements in row-major
        order (nonzero, transposed): count, read the count back, then place."""
        rank = len(mask.shape)
        if mask.numel == 0 or rank == 0:
            count = int(mask.numel and bool(self.download(mask)))
            return [self.empty((count,), I64) for _ in range(rank)]
        d = hmc_tensor_desc()
        d.data, d.offset, d.dtype, d.ndim = mask.storage.address, mask.offset, BOOL, rank
        for k in range(rank):
            d.sizes[k], d.strides[k] = mask.shape[k], mask.strides[k]
        nbytes, word = ctypes.c_int64(), ctypes.c_int64()
        self._check(self.lib.hmc_mask_workspace(mask.numel, ctypes.byref(nbytes), ctypes.byref(word)))
        ws = self.storage(nbytes.value)
        self._check(self.lib.hmc_mask_count(self.ctx, d, ws.ptr, nbytes.value))
        total = np.empty(1, dtype=np.uint64)
        self._check(self.lib.hmc_copy_to_host(self.ctx, total.ctypes.data, ws.ptr + 8 * word.value, 8))
        count = int(total[0])
        out = self.empty((rank, count), I64)
        if count:
            o = hmc_tensor_desc()
            o.data, o.offset, o.dtype, o.ndim = out.storage.address, out.offset, I64, 2
            o.sizes[0], o.strides[0], o.sizes[1], o.strides[1] = rank, count, count, 1
            self._check(self.lib.hmc_mask_coordinates(self.ctx, d, ws.ptr, nbytes.value, o))
        return [out.select(0, k) for k in range(rank)]

    def index_add(self, out: TensorData, dim: int, index: TensorData, src: TensorData) -> None:
        """Slice i of src along dim += into slice index[i] of the contiguous out, in f64 / wrapping i64, in the order of i
        (src/backend/rocm/index.rs:336-380)."""
        if src.numel == 0:
            return
        m, size = index.numel, out.shape[dim]
        (o, s), at = around("index_add", [out, src], tuple(out.shape), dim)
        s.sizes[at] = m
        i = hmc_tensor_desc()
        i.data, i.offset, i.dtype, i.ndim = index.storage.address, index.offset, index.dtype, 1
        i.sizes[0], i.strides[0] = m, index.strides[0] if index.shape else 1
        nbytes = ctypes.c_int64()
        self._check(self.lib.hmc_index_add_workspace(m, size, ctypes.byref(nbytes)))
        ws = self.workspace(nbytes.value)
        self._check(self.lib.hmc_index_add(self.ctx, o, s, i, at, ws.ptr if ws else None, nbytes.value))

    def scatter_add(self, out: TensorData, dim: int, index: TensorData, src: TensorData) -> None:
        """out[.., index[p], ..] += src[p] for every position p of the index, in row-major order
        (src/backend/rocm/index.rs:382-417)."""
        n = index.numel
        if n == 0:
            return
        (i, o, s), at = around("scatter_add", [index, out, src], tuple(index.shape), dim)
        o.sizes[at] = out.shape[dim]
        nbytes = ctypes.c_int64()
        self._check(self.lib.hmc_scatter_add_workspace(n, ctypes.byref(nbytes)))
        ws = self.workspace(nbytes.value)
        self._check(self.lib.hmc_scatter_add(self.ctx, o, s, i, at, ws.ptr if ws else None, nbytes.value))

    def index_positions(self, out: TensorData, coords: Sequence[TensorData], sizes: Sequence[int]) -> None:
        """The flat positions of advanced indexing: out (I64) = sum over k of wrapped coords[k] * contiguous stride k of
        `sizes`, each index broadcast to out's shape; one pass per index (src/backend/rocm/index.rs:618-668)."""
        if out.numel == 0:
            return
        strides = contiguous_strides(sizes)
        for k, c in enumerate(coords):
            d = descs("index_positions", [out, c.expand(out.shape)])
            self._check(self.lib.hmc_index_positions(self.ctx, d[0], d[1], sizes[k], strides[k], int(k == 0)))

    def addr(self, out: TensorData, v1: TensorData, v2: TensorData, input: Optional[TensorData], alpha, beta) -> None:
        """out = beta * input + alpha * outer(v1, v2) with the CPU kernel's steps (hmc_addr)."""
        d, a, b, ai, bi = addr_operands("addr", out, v1, v2, input, alpha, beta)
        if d is None:
            return
        self._check(self.lib.hmc_addr(self.ctx, d[0], d[1], d[2], d[3] if len(d) > 3 else None, a, b, ai, bi))

    def exclusive_cumprod(self, out: TensorData, src: TensorData, dim: int, reverse: bool) -> None:
        """hmc_exclusive_cumprod along `dim` (out contiguous, as the CPU kernel requires)."""
        ln = lines("exclusive_cumprod", out, src, dim, out.strides)
        if ln is None:
            return
        (o, s), n, so, si = ln
        self._check(self.lib.hmc_exclusive_cumprod(self.ctx, o, s, n, so, si, int(bool(reverse))))

    def adamw_step(self, param: TensorData, grad: TensorData, exp_avg: TensorData, exp_avg_sq: TensorData, *,
                   lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: float) -> None:
        """The fused AdamW update (hmc_adamw_step) with the scalars homura's optimizer derives
        (src/optim/adam.rs:139-170)."""
        d = descs("adamw_step", [param, grad, exp_avg, exp_avg_sq])
        if d is None:
            return
        sc = adamw_scalars(param.dtype, lr, beta1, beta2, eps, weight_decay, step)
        self._check(self.lib.hmc_adamw_step(self.ctx, d[0], d[1], d[2], d[3], ctypes.byref(sc)))


    def adamw_group(self, tensors: Sequence[Sequence[TensorData]], with_grad_sq: bool = False) -> "AdamWGroup":
        """The tensors of one parameter group, prepared for :meth:`AdamWGroup.step`."""
        return AdamWGroup(self, tensors, with_grad_sq)


class AdamWGroup:
    """One parameter group of an optimizer: (param, grad, exp_avg, exp_avg_sq) per parameter, all of one float
    dtype. Contiguous tensors are updated by one hmc_adamw_step_many launch; views with other strides go
    through hmc_adamw_step one by one (same bits). With `with_grad_sq` every step also leaves the f64 sums of
    the squared gradients, one per parameter in the order given (the contiguous ones first), in `grad_sq`."""

    def __init__(self, be: "CudaBackend", tensors: Sequence[Sequence[TensorData]], with_grad_sq: bool = False):
        self.be = be
        tensors = [tuple(t) for t in tensors]
        assert tensors, "an empty parameter group"
        self.dtype = tensors[0][0].dtype
        for t in tensors:
            assert len(t) == 4 and all(x.dtype == self.dtype and x.shape == t[0].shape for x in t)
        self.flat = [t for t in tensors if all(x.is_contiguous() for x in t)]
        self.strided = [t for t in tensors if not all(x.is_contiguous() for x in t)]
        assert not (with_grad_sq and self.strided), "gradient squares are summed for contiguous tensors only"
        n = len(self.flat)
        self.table = (ffi.hmc_adamw_tensor * max(n, 1))()
        es = SIZE[self.dtype]
        for i, (p, g, m, v) in enumerate(self.flat):
            e = self.table[i]
            e.param, e.grad = p.storage.ptr + p.offset * es, g.storage.ptr + g.offset * es
            e.exp_avg, e.exp_avg_sq = m.storage.ptr + m.offset * es, v.storage.ptr + v.offset * es
            e.n = p.numel
        nbytes = ctypes.c_int64()
        be._check(be.lib.hmc_adamw_step_many_workspace(self.dtype, self.table, n, int(with_grad_sq), ctypes.byref(nbytes)))
        self.workspace = be.workspace(nbytes.value)
        self.grad_sq = be.storage(8 * n) if with_grad_sq and n else None

    def step(self, *, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: float) -> None:
        be = self.be
        sc = adamw_scalars(self.dtype, lr, beta1, beta2, eps, weight_decay, step)
        if self.flat:
            gs = ctypes.cast(self.grad_sq.ptr, ctypes.POINTER(ctypes.c_double)) if self.grad_sq is not None else None
            be._check(be.lib.hmc_adamw_step_many(be.ctx, self.dtype, self.table, len(self.flat), ctypes.byref(sc), gs,
                                                 self.workspace.ptr if self.workspace else None,
                                                 self.workspace.nbytes if self.workspace else 0))
        for p, g, m, v in self.strided:
            d = descs("adamw_step", [p, g, m, v])
            if d is not None:
                be._check(be.lib.hmc_adamw_step(be.ctx, d[0], d[1], d[2], d[3], ctypes.byref(sc)))

    def grad_squares(self) -> np.ndarray:
        """The per-parameter f64 sums of the last step (a blocking copy)."""
        out = np.empty(len(self.flat), dtype=np.float64)
        if out.size:
            self.be._check(self.be.lib.hmc_copy_to_host(self.be.ctx, out.ctypes.data, self.grad_sq.ptr, out.nbytes))
        return out


def around(kernel: str, operands: Sequence[TensorData], shape: Sequence[int], dim: int):
    """Descriptions with the dimensions before `dim` and those after it merged, `dim` kept in between, and the position
    of `dim` among them (src/backend/rocm/index.rs:62-84). `shape` has elements."""
    strides = [t.strides for t in operands]
    part = lambda lo, hi: merge_dims(shape[lo:hi], [st[lo:hi] for st in strides]) or []
    dims = list(part(0, dim))
    at = len(dims)
    dims.append((shape[dim], [st[dim] for st in strides]))
    dims.extend(part(dim + 1, len(shape)))
    return descs_with_dims(kernel, operands, [t.offset for t in operands], dims, check=False), at


def index_select_descs(kernel: str, out: TensorData, src: TensorData, dim: int, index: TensorData):
    """(out, src, 1-D index, position of dim) as homura's glue passes them (src/backend/rocm/index.rs:221-270)."""
    shape = tuple(out.shape)
    strides = [0] * len(shape)
    strides[dim] = index.strides[0] if len(index.shape) else 0
    walk = TensorData(index.storage, index.dtype, shape, tuple(strides), index.offset)
    (o, s, w), at = around(kernel, [out, src, walk], shape, dim)
    s.sizes[at] = src.shape[dim]
    i = hmc_tensor_desc()
    i.data, i.offset, i.dtype, i.ndim = w.data, w.offset, w.dtype, 1
    i.sizes[0], i.strides[0] = w.sizes[at], w.strides[at]
    return o, s, i, at


def addr_operands(kernel: str, out: TensorData, v1: TensorData, v2: TensorData, input: Optional[TensorData], alpha, beta):
    """The descriptions and coefficients of addr as homura's glue passes them (src/backend/rocm/elementwise.rs, addr):
    v1 [n] and v2 [m] as [n, m] views with a stride of 0 along the other dimension, the input broadcast to [n, m] and left
    out when beta is zero; float coefficients rounded to the dtype, integer and Bool ones as integers."""
    n, m = out.shape
    assert tuple(v1.shape) == (n,) and tuple(v2.shape) == (m,)
    a_view = TensorData(v1.storage, v1.dtype, (n, m), (v1.strides[0], 0), v1.offset)
    b_view = TensorData(v2.storage, v2.dtype, (n, m), (0, v2.strides[0]), v2.offset)
    if out.dtype in FLOATS:
        round_to = lambda v: bits_to_float(scalar_bits(float(v), out.dtype), out.dtype)
        a, b, ai, bi = round_to(alpha), round_to(beta), 0, 0
        reads = b != 0.0
    else:
        a, b = 0.0, 0.0
        ai, bi = (int(bool(alpha)), int(bool(beta))) if out.dtype == BOOL else (int(alpha), int(beta))
        reads = bi != 0
    operands = [out, a_view, b_view] + ([input.expand(n, m)] if reads else [])
    return descs(kernel, operands), a, b, ai, bi


def bits_to_float(bits: int, dtype: int) -> float:
    """The value of a float element given by its bits."""
    if dtype == F64:
        return float(np.array([bits], dtype=np.uint64).view(np.float64)[0])
    if dtype == F32:
        return float(np.array([bits], dtype=np.uint32).view(np.float32)[0])
    if dtype == BF16:
        return float(np.array([bits << 16], dtype=np.uint32).view(np.float32)[0])
    return float(np.array([bits], dtype=np.uint16).view(np.float16)[0])


DEFAULT_SEED = 67280421310721  # PyTorch's default seed, as homura uses it (src/ops/random.rs:15-16)


class Generator:
    """homura's process-wide Philox generator (src/ops/random.rs:18-27, 53-73): a seed and the number of 128-bit
    blocks handed out since seeding; samplers reserve their blocks before they launch."""

    def __init__(self, seed: int = DEFAULT_SEED):
        self.manual_seed(seed)

    def manual_seed(self, seed: int) -> None:
        self.seed = seed & (2**64 - 1)
        self.offset = 0

    def reserve(self, blocks: int) -> tuple[int, int]:
        start = self.offset
        self.offset = (self.offset + blocks) & (2**64 - 1)
        return self.seed, start


def int_range(low: int, high: int) -> tuple[int, int]:
    """(number of values in [low, high), threshold below which a 64-bit word is rejected).
    src/ops/random.rs:201-207."""
    rng = high - low
    assert 1 <= rng <= 2**64 - 1
    return rng, (2**64 - rng) % rng


def _flat_desc(t: TensorData) -> hmc_tensor_desc:
    """A contiguous tensor as one dimension."""
    assert t.is_contiguous()
    d = hmc_tensor_desc()
    d.data, d.offset, d.dtype = t.storage.address, t.offset, t.dtype
    if t.numel == 1:
        d.ndim = 0
    else:
        d.ndim = 1
        d.sizes[0], d.strides[0] = t.numel, 1
    return d


def _round_to_compute(v: float, dtype: int) -> float:
    return float(v) if dtype == F64 else float(np.float32(v))


def _round_to_dtype(v: float, dtype: int) -> float:
    """`v` rounded to `dtype` (Sealed::from_f64) and widened back."""
    if dtype == F64:
        return float(v)
    f = np.array([v], dtype=np.float64).astype(np.float32)
    if dtype == F32:
        return float(f[0])
    return float(half_bits_to_f32(f32_to_half_bits(f, dtype), dtype)[0])


def fused_coefficient(op: int, value: float, dtype: int):
    """(coefficient exact in the computation type, small) as cpu::fused derives them
    (src/backend/cpu/mod.rs:541-566)."""
    if op == ffi.HMC_FUSED_SCALED_ADD:
        return _round_to_dtype(value, dtype), False
    if op == ffi.HMC_FUSED_LERP:
        w = _round_to_compute(value, dtype)
        small = abs(w) < 0.5
        if small:
            return w, True
        one = np.float64(1.0) if dtype == F64 else np.float32(1.0)
        wc = np.float64(w) if dtype == F64 else np.float32(w)
        return float(wc - one), False
    return _round_to_compute(value, dtype), False


def adamw_scalars(dtype: int, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
                  step: float) -> ffi.hmc_adamw_scalars:
    sc = ffi.hmc_adamw_scalars()
    sc.has_decay = int(weight_decay != 0.0)
    sc.decay = _round_to_compute(1.0 - lr * weight_decay, dtype)
    coeff, small = fused_coefficient(ffi.HMC_FUSED_LERP, 1.0 - beta1, dtype)
    sc.lerp_coeff, sc.lerp_small = coeff, int(small)
    sc.beta2 = _round_to_compute(beta2, dtype)
    sc.one_minus_beta2 = _round_to_compute(1.0 - beta2, dtype)
    bias_correction2 = 1.0 - beta2 ** step
    sc.bias2_sqrt = _round_to_compute(bias_correction2 ** 0.5, dtype)
    sc.eps = _round_to_dtype(eps, dtype)
    sc.neg_step_size = _round_to_compute(-(lr / (1.0 - beta1 ** step)), dtype)
    return sc
