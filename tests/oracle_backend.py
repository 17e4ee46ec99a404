"""The CPU checker behind the interface of homura_b200.host.CudaBackend, over host (numpy) storage.
TEST INFRASTRUCTURE: it loads oracle/_build/liboracle.so, which no product code may touch."""
from __future__ import annotations

import ctypes
import importlib.util
import math
from pathlib import Path
from typing import Optional, Sequence

import numpy as np

from homura_b200 import ffi
from homura_b200.ffi import hmc_tensor_desc
from homura_b200.host import (SIZE, STORAGE, Storage, TensorData, contiguous_strides, describe, descs, lines,
                              output_desc, scalar_bits)

ROOT = Path(__file__).resolve().parent.parent


def _load_oracle():
    spec = importlib.util.spec_from_file_location("oracle_build", ROOT / "oracle" / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    lib = ctypes.CDLL(str(mod.build()))
    D = ctypes.POINTER(hmc_tensor_desc)
    i32, i64, u64, f64, vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_uint64, ctypes.c_double, ctypes.c_void_p
    protos = {
        "orc_copy": [D, D], "orc_fill": [D, u64], "orc_unary": [i32, D, D], "orc_binary": [i32, D, D, D],
        "orc_binary_constant": [i32, D, D, u64, i32], "orc_binary_scalar": [i32, D, D, f64, i32],
        "orc_fused": [i32, D, D, D, D, f64], "orc_where": [D, D, D, D], "orc_where_constant": [D, D, D, u64, D, u64],
        "orc_reduce": [i32, D, D, D], "orc_var": [D, D, D, f64, i32], "orc_arg_reduce": [D, D, D, D, i32],
        "orc_softmax": [D, D, i64, i64, i64, i32],
        "orc_adamw_step": [i32, i64, vp, vp, vp, vp, f64, f64, f64, f64, f64, f64],
        "orc_random_uniform": [i32, vp, i64, u64, u64, f64, f64], "orc_random_normal": [i32, vp, i64, u64, u64, f64, f64],
        "orc_random_int": [vp, i64, u64, u64, i64, i64, ctypes.POINTER(u64)],
        "orc_triangle": [D, D, i64, i32], "orc_flip": [D, D],
        "orc_index_check": [D, i64, i64, i32, i64, ctypes.POINTER(u64)], "orc_index_select": [D, D, D, i32, i32],
        "orc_gather": [D, D, D, i32], "orc_index_overwrite": [D, D, D, i32], "orc_index_add": [D, D, D, i32],
        "orc_scatter_add": [D, D, D, i32], "orc_index_positions": [D, D, i64, i64, i32], "orc_mask_coordinates": [D, vp, i64],
        "orc_addr": [D, D, D, D, f64, f64, i64, i64], "orc_exclusive_cumprod": [D, D, i64, i64, i64, i32],
    }
    for name, args in protos.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = i32, args
    lib.orc_f32_to_f16.restype, lib.orc_f32_to_f16.argtypes = ctypes.c_uint16, [ctypes.c_float]
    lib.orc_f32_to_bf16.restype, lib.orc_f32_to_bf16.argtypes = ctypes.c_uint16, [ctypes.c_float]
    lib.orc_f16_to_f32.restype, lib.orc_f16_to_f32.argtypes = ctypes.c_float, [ctypes.c_uint16]
    lib.orc_bf16_to_f32.restype, lib.orc_bf16_to_f32.argtypes = ctypes.c_float, [ctypes.c_uint16]
    lib.orc_erf.restype, lib.orc_erf.argtypes = f64, [f64]
    lib.orc_mask_count.restype, lib.orc_mask_count.argtypes = i64, [D]
    lib.orc_philox.restype, lib.orc_philox.argtypes = None, [ctypes.POINTER(ctypes.c_uint32)] * 3
    lib.orc_random_int_batch.restype, lib.orc_random_int_batch.argtypes = i64, [vp, i64, u64, u64, u64, i64, u64, u64]
    return lib


class OraclePanic(RuntimeError):
    """The CPU kernel would panic (unsupported dtype / op, empty max, ...)."""


class OracleBackend:
    name = "oracle"

    def __init__(self):
        self.lib = _load_oracle()

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise OraclePanic(f"oracle status {rc}")

    def synchronize(self) -> None:
        pass

    def empty(self, shape, dtype: int) -> TensorData:
        shape = tuple(shape)
        n = math.prod(shape)
        arr = np.zeros(max(n, 1), dtype=STORAGE[dtype])
        return TensorData(Storage(n * SIZE[dtype], array=arr), dtype, shape, tuple(contiguous_strides(shape)))

    def upload(self, array: np.ndarray, dtype: int, shape=None) -> TensorData:
        array = np.ascontiguousarray(array, dtype=STORAGE[dtype])
        shape = tuple(array.shape if shape is None else shape)
        flat = array.reshape(-1).copy()
        if flat.size == 0:
            flat = np.zeros(1, dtype=STORAGE[dtype])
        return TensorData(Storage(array.nbytes, array=flat), dtype, shape, tuple(contiguous_strides(shape)))

    def download_storage(self, t: TensorData) -> np.ndarray:
        return t.storage.array

    def download(self, t: TensorData) -> np.ndarray:
        if t.numel == 0:
            return np.empty(t.shape, dtype=STORAGE[t.dtype])
        es = SIZE[t.dtype]
        view = np.lib.stride_tricks.as_strided(t.storage.array[t.offset:], shape=t.shape,
                                               strides=[s * es for s in t.strides], writeable=False)
        return np.ascontiguousarray(view).reshape(t.shape)

    # ---- backend functions (names and argument meaning of src/backend/cpu) ----
    def copy(self, dst, src):
        d = descs("copy", [dst, src.expand(dst.shape)])
        if d is not None:
            self._check(self.lib.orc_copy(d[0], d[1]))

    def fill(self, dst, value):
        d = descs("fill", [dst])
        if d is not None:
            self._check(self.lib.orc_fill(d[0], scalar_bits(value, dst.dtype)))

    def unary(self, op, out, src):
        d = descs("unary", [out, src])
        if d is not None:
            self._check(self.lib.orc_unary(op, d[0], d[1]))

    def binary(self, op, out, a, b):
        d = descs("binary", [out, a, b])
        if d is not None:
            self._check(self.lib.orc_binary(op, d[0], d[1], d[2]))

    def binary_promoted(self, op, out, a, b):
        """homura's route for operands of different dtypes: cast both, then the binary kernel
        (src/ops/binary.rs:55-60)."""
        ac, bc = self.empty(a.shape, out.dtype), self.empty(b.shape, out.dtype)
        self.copy(ac, a)
        self.copy(bc, b)
        self.binary(op, out, ac, bc)

    def binary_constant(self, op, out, a, value, constant_first):
        d = descs("binary_constant", [out, a])
        if d is not None:
            self._check(self.lib.orc_binary_constant(op, d[0], d[1], scalar_bits(value, a.dtype), int(constant_first)))

    def binary_scalar(self, op, out, a, s, scalar_first):
        d = descs("binary_scalar", [out, a])
        if d is not None:
            self._check(self.lib.orc_binary_scalar(op, d[0], d[1], float(s), int(scalar_first)))

    def fused(self, op, value, out, a, b, c=None):
        ops = [out, a, b] + ([c] if c is not None else [])
        d = descs("fused", ops)
        if d is not None:
            self._check(self.lib.orc_fused(op, d[0], d[1], d[2], d[3] if c is not None else None, float(value)))

    def where_(self, out, cond, x, y):
        d = descs("where_", [out, cond, x, y])
        if d is not None:
            self._check(self.lib.orc_where(d[0], d[1], d[2], d[3]))

    def where_constant(self, out, cond, x, y):
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
        self._check(self.lib.orc_where_constant(d[0], d[1], xd, xb, yd, yb))

    def reduce(self, op, out, src, mask):
        r = describe("reduce", src, mask)
        if r is not None:
            self._check(self.lib.orc_reduce(op, output_desc("reduce", r, out), r.kept, r.red))

    def var(self, out, src, mask, correction, take_sqrt):
        r = describe("var", src, mask)
        if r is not None:
            self._check(self.lib.orc_var(output_desc("var", r, out), r.kept, r.red, float(correction), int(take_sqrt)))

    def arg_reduce(self, values, indices, src, dim, is_max):
        nd = len(src.shape)
        r = describe("arg_reduce", src, [d == dim for d in range(nd)])
        if r is None:
            return
        v = output_desc("arg_reduce", r, values) if values is not None else None
        self._check(self.lib.orc_arg_reduce(v, output_desc("arg_reduce", r, indices), r.kept, r.red, int(is_max)))

    def softmax(self, out, src, dim, log):
        ln = lines("softmax", out, src, dim, out.strides)
        if ln is None:
            return
        (o, s), n, so, si = ln
        self._check(self.lib.orc_softmax(o, s, n, so, si, int(log)))

    # ---- samplers, the mask builder, flip ----
    def _data(self, t: TensorData) -> int:
        assert t.is_contiguous()
        return t.storage.array.ctypes.data + t.offset * SIZE[t.dtype]

    def random_uniform(self, out, gen, low, high):
        per_block = 2 if out.dtype == ffi.HMC_F64 else 4
        seed, start = gen.reserve(-(-out.numel // per_block))
        self._check(self.lib.orc_random_uniform(out.dtype, self._data(out), out.numel, seed, start, float(low), float(high)))

    def random_normal(self, out, gen, mean, std):
        seed, start = gen.reserve(-(-out.numel // 2))
        self._check(self.lib.orc_random_normal(out.dtype, self._data(out), out.numel, seed, start, float(mean), float(std)))

    def random_int(self, out, gen, low, high):
        used = ctypes.c_uint64()
        self._check(self.lib.orc_random_int(self._data(out), out.numel, gen.seed, gen.offset, low, high, ctypes.byref(used)))
        gen.reserve(used.value)

    def triangle(self, out, src, diagonal, upper):
        from homura_b200.host import descs_with_dims, merge_dims
        if src.numel == 0:
            return
        batch = merge_dims(src.shape[:-2], [out.strides[:-2], src.strides[:-2]])
        dims = list(batch) + [(src.shape[-2], [out.strides[-2], src.strides[-2]]), (src.shape[-1], [out.strides[-1], src.strides[-1]])]
        o, i = descs_with_dims("triangle", [out, src], [out.offset, src.offset], dims)
        self._check(self.lib.orc_triangle(o, i, int(diagonal), int(bool(upper))))

    def flip(self, out, src, dims):
        if src.numel == 0:
            return
        strides, offset = list(src.strides), src.offset
        for d in dims:
            offset += (src.shape[d] - 1) * strides[d]
            strides[d] = -strides[d]
        flipped = TensorData(src.storage, src.dtype, tuple(src.shape), tuple(strides), offset)
        o, i = descs("flip", [out, flipped])
        self._check(self.lib.orc_flip(o, i))

    def index_check(self, index, low, high, exempt=None):
        if index.numel == 0:
            return None
        d, = descs("index_check", [index])
        slot = (ctypes.c_uint64 * 2)()
        self._check(self.lib.orc_index_check(d, low, high, int(exempt is not None), exempt or 0, slot))
        return None if slot[0] == 2**64 - 1 else (int(slot[0]), int(np.array([slot[1]], dtype=np.uint64).view(np.int64)[0]))

    def index_select(self, out, src, dim, index, wrap_negative=False):
        from homura_b200.host import index_select_descs
        if out.numel == 0:
            return
        o, s, i, at = index_select_descs("index_select", out, src, dim, index)
        self._check(self.lib.orc_index_select(o, s, i, at, int(wrap_negative)))

    def gather(self, out, src, dim, index):
        from homura_b200.host import around
        if out.numel == 0:
            return
        (o, s, i), at = around("gather", [out, src, index], tuple(out.shape), dim)
        s.sizes[at] = src.shape[dim]
        self._check(self.lib.orc_gather(o, s, i, at))

    def index_overwrite(self, out, dim, positions, src):
        from homura_b200.host import around
        if src.numel == 0:
            return
        (s, o), at = around("index_overwrite", [src, out], tuple(src.shape), dim)
        o.sizes[at] = out.shape[dim]
        p = hmc_tensor_desc()
        p.data, p.offset, p.dtype, p.ndim = positions.storage.address, positions.offset, ffi.HMC_I64, 1
        p.sizes[0], p.strides[0] = positions.numel, 1
        self._check(self.lib.orc_index_overwrite(o, s, p, at))

    def index_add(self, out, dim, index, src):
        from homura_b200.host import around
        if src.numel == 0:
            return
        (o, s), at = around("index_add", [out, src], tuple(out.shape), dim)
        s.sizes[at] = index.numel
        i = hmc_tensor_desc()
        i.data, i.offset, i.dtype, i.ndim = index.storage.address, index.offset, index.dtype, 1
        i.sizes[0], i.strides[0] = index.numel, index.strides[0] if index.shape else 1
        self._check(self.lib.orc_index_add(o, s, i, at))

    def scatter_add(self, out, dim, index, src):
        from homura_b200.host import around
        if index.numel == 0:
            return
        (i, o, s), at = around("scatter_add", [index, out, src], tuple(index.shape), dim)
        o.sizes[at] = out.shape[dim]
        self._check(self.lib.orc_scatter_add(o, s, i, at))

    def index_positions(self, out, coords, sizes):
        from homura_b200.host import contiguous_strides, descs
        if out.numel == 0:
            return
        strides = contiguous_strides(sizes)
        for k, c in enumerate(coords):
            d = descs("index_positions", [out, c.expand(out.shape)])
            self._check(self.lib.orc_index_positions(d[0], d[1], sizes[k], strides[k], int(k == 0)))

    def mask_coordinates(self, mask):
        rank = len(mask.shape)
        d = hmc_tensor_desc()
        d.data, d.offset, d.dtype, d.ndim = mask.storage.address, mask.offset, ffi.HMC_BOOL, rank
        for k in range(rank):
            d.sizes[k], d.strides[k] = mask.shape[k], mask.strides[k]
        count = int(self.lib.orc_mask_count(d))
        out = self.empty((rank, count), ffi.HMC_I64)
        if count:
            self._check(self.lib.orc_mask_coordinates(d, out.storage.array.ctypes.data, count))
        return [out.select(0, k) for k in range(rank)]

    def addr(self, out, v1, v2, input, alpha, beta):
        from homura_b200.host import addr_operands
        d, a, b, ai, bi = addr_operands("addr", out, v1, v2, input, alpha, beta)
        if d is None:
            return
        self._check(self.lib.orc_addr(d[0], d[1], d[2], d[3] if len(d) > 3 else None, a, b, ai, bi))

    def exclusive_cumprod(self, out, src, dim, reverse):
        ln = lines("exclusive_cumprod", out, src, dim, out.strides)
        if ln is None:
            return
        (o, s), n, so, si = ln
        self._check(self.lib.orc_exclusive_cumprod(o, s, n, so, si, int(bool(reverse))))

    # ---- the sharded reductions' local and combine steps, restated on the host for the CPU tests ----
    def storage(self, nbytes: int) -> Storage:
        return Storage(nbytes, array=np.zeros(max(nbytes, 1), dtype=np.uint8))

    def reduce_partial(self, op, partial: Storage, src, mask):
        """f64 partial sums / products in the CPU's fold order: the fold of the exactly widened elements."""
        from homura_b200.host import F64
        wide = self.empty(src.shape, F64)
        self.copy(wide, src)
        kept = [n for n, m in zip(src.shape, mask) if not m]
        out = self.empty(kept, F64)
        self.reduce(ffi.HMC_REDUCE_SUM if op == ffi.HMC_REDUCE_MEAN else op, out, wide, mask)
        partial.array[:8 * out.numel] = self.download(out).reshape(-1).view(np.uint8)

    def shard_combine_float(self, op, out, gathered: Storage, ranks, nout, count):
        from homura_b200.host import F64
        g = gathered.array[:8 * ranks * nout].view(np.float64).reshape(ranks, nout)
        acc = np.ones(nout) if op == ffi.HMC_REDUCE_PROD else np.zeros(nout)
        with np.errstate(all="ignore"):
            for r in range(ranks):
                acc = acc * g[r] if op == ffi.HMC_REDUCE_PROD else acc + g[r]
            if op == ffi.HMC_REDUCE_MEAN:
                acc = acc / float(count)
        self.copy(out, self.upload(acc, F64, out.shape))

    def shard_combine_means(self, means: Storage, gathered: Storage, ranks, nout, count):
        g = gathered.array[:8 * ranks * nout].view(np.float64).reshape(ranks, nout)
        acc = np.zeros(nout)
        with np.errstate(all="ignore"):
            for r in range(ranks):
                acc = acc + g[r]
            acc = acc / float(count)
        means.array[:8 * nout] = acc.view(np.uint8)

    def var_partial(self, partial: Storage, src, mask, means: Storage):
        """f64 sums of (x - mean)^2 in the CPU's fold order."""
        from homura_b200.host import F64
        wide = self.empty(src.shape, F64)
        self.copy(wide, src)
        kept = [n for n, m in zip(src.shape, mask) if not m]
        m = means.array[:8 * math.prod(kept)].view(np.float64).reshape([n if not r else 1 for n, r in zip(src.shape, mask)])
        with np.errstate(all="ignore"):
            d = self.download(wide) - m
            sq = self.upload(d * d, F64, src.shape)
        out = self.empty(kept, F64)
        self.reduce(ffi.HMC_REDUCE_SUM, out, sq, mask)
        partial.array[:8 * out.numel] = self.download(out).reshape(-1).view(np.uint8)

    def shard_combine_var(self, out, gathered: Storage, ranks, nout, count, correction, take_sqrt):
        from homura_b200.host import F64
        g = gathered.array[:8 * ranks * nout].view(np.float64).reshape(ranks, nout)
        acc = np.zeros(nout)
        with np.errstate(all="ignore"):
            for r in range(ranks):
                acc = acc + g[r]
            divisor = float(count) - correction
            divisor = divisor if divisor > 0.0 else 0.0
            v = np.full(nout, np.nan) if count == 0 else acc / divisor
            if take_sqrt:
                v = np.sqrt(v)
        self.copy(out, self.upload(v, F64, out.shape))

    def shard_combine_int(self, op, out, gathered: Storage, ranks, nout):
        g = gathered.array[:8 * ranks * nout].view(np.uint64).reshape(ranks, nout)
        acc = np.ones(nout, dtype=np.uint64) if op == ffi.HMC_REDUCE_PROD else np.zeros(nout, dtype=np.uint64)
        with np.errstate(over="ignore"):
            for r in range(ranks):
                acc = acc * g[r] if op == ffi.HMC_REDUCE_PROD else acc + g[r]
        out.storage.array[out.offset:out.offset + nout] = acc.view(np.int64)

    def shard_combine_extreme(self, is_max, values, indices, gathered_values: Storage, dtype, gathered_indices, offsets,
                              ranks, nout):
        """First NaN, then first of equals, in rank order (src/backend/cpu/reduce.rs:75-86)."""
        from values import is_nan_raw, storage_to_f64
        gv = gathered_values.array[:SIZE[dtype] * ranks * nout].view(STORAGE[dtype]).reshape(ranks, nout)
        gi = None if gathered_indices is None else gathered_indices.array[:8 * ranks * nout].view(np.int64).reshape(ranks, nout)
        best, best_i = gv[0].copy(), (gi[0] + offsets[0] if gi is not None else np.zeros(nout, dtype=np.int64))
        for r in range(1, ranks):
            x = gv[r]
            kx, kb = storage_to_f64(x, dtype), storage_to_f64(best, dtype)
            if dtype == 5:  # I64: compare exactly
                kx, kb = x, best
            better = (kx > kb) if is_max else (kx < kb)
            take = ~is_nan_raw(best, dtype) & (is_nan_raw(x, dtype) | better)
            best = np.where(take, x, best)
            if gi is not None:
                best_i = np.where(take, gi[r] + offsets[r], best_i)
        if values is not None:
            values.storage.array[values.offset:values.offset + nout] = best
        if indices is not None:
            indices.storage.array[indices.offset:indices.offset + nout] = best_i

    def adamw_step(self, param, grad, exp_avg, exp_avg_sq, *, lr, beta1, beta2, eps, weight_decay, step):
        """The op-by-op sequence of homura's optimizer on contiguous copies, written back in place."""
        def flat(t):
            c = self.empty(t.shape, t.dtype)
            self.copy(c, t)
            return c
        p, g, m, v = flat(param), flat(grad), flat(exp_avg), flat(exp_avg_sq)
        self._check(self.lib.orc_adamw_step(param.dtype, param.numel, p.storage.address, g.storage.address,
                                            m.storage.address, v.storage.address, lr, beta1, beta2, eps,
                                            weight_decay, float(step)))
        self.copy(param, p)
        self.copy(exp_avg, m)
        self.copy(exp_avg_sq, v)
