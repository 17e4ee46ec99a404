"""A small restatement of the part of homura's operator front-end (src/ops/{unary,binary,reduce,composite}.rs,
src/dtype.rs promotion) that sits between its public Tensor API and the backend functions, so that the golden
cases, which are written against the Tensor API, can be run on either backend (the CPU checker or the CUDA
library). TEST INFRASTRUCTURE; homura's own front-end is unchanged by the CUDA backend."""
from __future__ import annotations

import math
from typing import Optional, Sequence, Union

import numpy as np

from homura_b200 import ffi
from homura_b200.host import (BF16, BOOL, F16, F32, F64, I8, I16, I32, I64, U8, TensorData, contiguous_strides, is_float,
                              is_int)

DEFAULT_DTYPE = F32
Scalar = Union[bool, int, float]

UNARY = {n: getattr(ffi, "HMC_UNARY_" + n.upper()) for n in
         ["neg", "abs", "sign", "relu", "exp", "log", "sqrt", "rsqrt", "reciprocal", "sin", "cos", "erf", "tanh", "sigmoid",
          "log_sigmoid", "silu", "gelu", "gelu_tanh", "logical_not"]}
BINARY = {n: getattr(ffi, "HMC_BINARY_" + n.upper()) for n in
          ["add", "sub", "mul", "div", "pow", "maximum", "minimum", "greater", "greater_equal", "less", "less_equal",
           "equal", "not_equal", "logical_and", "logical_or"]}
REDUCE = {n: getattr(ffi, "HMC_REDUCE_" + n.upper()) for n in ["sum", "prod", "mean", "max", "min", "all", "any"]}


class Panic(Exception):
    """homura's front-end panics here."""


def kind(dt: int) -> int:
    return 0 if dt == BOOL else (1 if is_int(dt) else 2)


def promote_types(a: int, b: int) -> int:
    """src/dtype.rs:429-470."""
    if a == b:
        return a
    ka, kb = kind(a), kind(b)
    if ka == 0:
        return b
    if kb == 0:
        return a
    if ka == 2 and kb == 2:
        return F64 if F64 in (a, b) else F32
    if ka == 2:
        return a
    if kb == 2:
        return b
    rank = {I8: 1, I16: 2, I32: 3, I64: 4}
    if {a, b} == {U8, I8}:
        return I16
    if a == U8:
        return b
    if b == U8:
        return a
    return a if rank[a] >= rank[b] else b


def scalar_dtype(s: Scalar) -> int:
    if isinstance(s, bool):
        return BOOL
    if isinstance(s, int):
        return I64
    return DEFAULT_DTYPE


def result_type(operands) -> int:
    """src/dtype.rs:480-535: tensors with dimensions > 0-dim tensors > scalars, unless a lower priority
    operand is of a higher category."""
    slots = [None, None, None]
    for o in operands:
        if isinstance(o, TensorData):
            i, dt = (1 if len(o.shape) == 0 else 0), o.dtype
        else:
            i, dt = 2, scalar_dtype(o)
        slots[i] = dt if slots[i] is None else promote_types(slots[i], dt)

    def combine(h, l):
        if h is None:
            return l
        if l is None:
            return h
        if is_float(h):
            return h
        if h == BOOL or is_float(l):
            return promote_types(h, l)
        return h

    return combine(slots[0], combine(slots[1], slots[2]))


def broadcast_shapes(a: Sequence[int], b: Sequence[int]) -> tuple:
    n = max(len(a), len(b))
    a = (1,) * (n - len(a)) + tuple(a)
    b = (1,) * (n - len(b)) + tuple(b)
    out = []
    for x, y in zip(a, b):
        if x == y or y == 1:
            out.append(x)
        elif x == 1:
            out.append(y)
        else:
            raise Panic(f"shapes {a} and {b} do not broadcast")
    return tuple(out)


def cast_data(be, t: TensorData, dtype: int) -> TensorData:
    """src/ops/mod.rs:186-195."""
    if t.dtype == dtype:
        return t
    out = be.empty(t.shape, dtype)
    be.copy(out, t)
    return out


def contiguous(be, t: TensorData) -> TensorData:
    out = be.empty(t.shape, t.dtype)
    be.copy(out, t)
    return out


def to(be, t: TensorData, dtype: int) -> TensorData:
    return cast_data(be, t, dtype)


def unary_op(be, name: str, x: TensorData) -> TensorData:
    """src/ops/unary.rs:18-57."""
    op = UNARY[name]
    dt = x.dtype
    if name == "logical_not":
        compute = dt
    elif name in ("neg", "abs", "relu"):
        if dt == BOOL:
            raise Panic(f"{name} is not supported for bool tensors")
        compute = dt
    elif name == "sign":
        compute = dt
    elif name in ("silu", "gelu", "gelu_tanh", "log_sigmoid"):
        if not is_float(dt):
            raise Panic(f"{name} is not implemented for this dtype")
        compute = dt
    else:
        compute = dt if is_float(dt) else DEFAULT_DTYPE
    out = be.empty(x.shape, BOOL if name == "logical_not" else compute)
    be.unary(op, out, cast_data(be, x, compute))
    return out


def fill_value(s: Scalar, dtype: int) -> Scalar:
    """Scalar::checked_to (src/dtype.rs:322-372) for the cases the goldens use: the value, in range."""
    return s


def scalar_data(be, s: Scalar, dtype: int) -> TensorData:
    t = be.empty((), dtype)
    be.fill(t, s)
    return t


def binary_op(be, name: str, lhs, rhs) -> TensorData:
    """src/ops/binary.rs:68-143."""
    op = BINARY[name]
    common = result_type([lhs, rhs])
    if name == "div" and not is_float(common):
        compute = DEFAULT_DTYPE
    elif name in ("logical_and", "logical_or"):
        compute = BOOL
    else:
        compute = common
    is_bool = lambda o: (o.dtype == BOOL) if isinstance(o, TensorData) else isinstance(o, bool)
    if name == "sub" and (is_bool(lhs) or is_bool(rhs)):
        raise Panic("subtraction with a bool tensor is not supported")
    if compute == BOOL and name == "pow":
        raise Panic("pow is not supported for bool tensors")
    if is_int(compute) and name == "pow" and not isinstance(rhs, TensorData) and int(rhs) < 0:
        raise Panic("Integers to negative integer powers are not allowed.")
    out_dtype = BOOL if name in ("greater", "greater_equal", "less", "less_equal", "equal", "not_equal", "logical_and",
                                 "logical_or") else compute
    shape_of = lambda o: tuple(o.shape) if isinstance(o, TensorData) else ()
    shape = broadcast_shapes(shape_of(lhs), shape_of(rhs))
    out = be.empty(shape, out_dtype)
    keeps_scalar = name in ("mul", "div") and compute in (F16, BF16)
    lt, rt = isinstance(lhs, TensorData), isinstance(rhs, TensorData)
    if lt != rt:
        scalar_first = not lt
        t, s = (rhs, lhs) if scalar_first else (lhs, rhs)
        td = cast_data(be, t, compute).expand(shape)
        if keeps_scalar:
            be.binary_scalar(op, out, td, float(s), scalar_first)
        else:
            be.binary_constant(op, out, td, s, scalar_first)
    else:
        mat = lambda o: (cast_data(be, o, compute) if isinstance(o, TensorData) else scalar_data(be, o, compute)).expand(shape)
        be.binary(op, out, mat(lhs), mat(rhs))
    return out


def select(be, cond: TensorData, x, y, dtype: int) -> TensorData:
    """src/ops/binary.rs:183-216."""
    if cond.dtype != BOOL:
        raise Panic("where expected condition to be a boolean tensor")
    shape_of = lambda o: tuple(o.shape) if isinstance(o, TensorData) else ()
    shape = broadcast_shapes(broadcast_shapes(cond.shape, shape_of(x)), shape_of(y))
    out = be.empty(shape, dtype)
    c = cond.expand(shape)
    mat = lambda o: cast_data(be, o, dtype).expand(shape) if isinstance(o, TensorData) else o
    be.where_constant(out, c, mat(x), mat(y))
    return out


def where_(be, cond: TensorData, x, y) -> TensorData:
    return select(be, cond, x, y, result_type([x, y]))


def masked_fill(be, x: TensorData, mask: TensorData, value: Scalar) -> TensorData:
    return select(be, mask, fill_value(value, x.dtype), x, x.dtype)


def dims_mask(dims: Sequence[int], nd: int) -> list:
    if len(dims) == 0:
        return [True] * nd
    mask = [False] * nd
    for d in dims:
        mask[d % nd if nd else 0] = True
    return mask


def reduced_shape(shape, mask, keepdim):
    out = []
    for n, m in zip(shape, mask):
        if not m:
            out.append(n)
        elif keepdim:
            out.append(1)
    return tuple(out)


def reduce_op(be, name: str, x: TensorData, dims: Sequence[int] = (), keepdim: bool = False) -> TensorData:
    """src/ops/reduce.rs:56-90."""
    op = REDUCE[name]
    dt = x.dtype
    mask = dims_mask(list(dims), len(x.shape))
    if name in ("sum", "prod") and not is_float(dt):
        out_dtype = I64
    elif name == "mean" and not is_float(dt):
        raise Panic("mean(): could not infer output dtype")
    elif name in ("all", "any") and dt != U8:
        out_dtype = BOOL
    else:
        out_dtype = dt
    if name in ("max", "min") and any(m and n == 0 for n, m in zip(x.shape, mask)):
        raise Panic(f"{name}(): Expected reduction dim to be specified for input.numel() == 0")
    out = be.empty(reduced_shape(x.shape, mask, keepdim), out_dtype)
    be.reduce(op, out, x, mask)
    return out


def arg_op(be, x: TensorData, dim: Optional[int], keepdim: bool, is_max: bool, values: bool):
    """src/ops/reduce.rs:92-135."""
    src = x
    if dim is None:
        src = (x if x.is_contiguous() else contiguous(be, x)).reshape(x.numel)
        dim, keepdim = 0, False
    nd = len(src.shape)
    dim = dim % nd if nd else 0
    size = 1 if nd == 0 else src.shape[dim]
    if size == 0:
        raise Panic("Expected reduction dim to have non-zero size.")
    mask = [d == dim for d in range(nd)]
    shape = reduced_shape(src.shape, mask, keepdim)
    vals = be.empty(shape, src.dtype) if values else None
    idx = be.empty(shape, I64)
    be.arg_reduce(vals, idx, src, dim, is_max)
    return vals, idx


def var_op(be, x: TensorData, dims: Sequence[int], correction: int, keepdim: bool, take_sqrt: bool) -> TensorData:
    if not is_float(x.dtype):
        raise Panic("std and var only support floating point dtypes")
    mask = dims_mask(list(dims), len(x.shape))
    out = be.empty(reduced_shape(x.shape, mask, keepdim), x.dtype)
    be.var(out, x, mask, float(correction), take_sqrt)
    return out


def softmax_op(be, x: TensorData, dim: int, log: bool) -> TensorData:
    """src/ops/composite.rs:11-27: integers go to the default float dtype first."""
    src = x if is_float(x.dtype) else cast_data(be, x, DEFAULT_DTYPE)
    nd = len(src.shape)
    out = be.empty(src.shape, src.dtype)
    be.softmax(out, src, dim % nd if nd else 0, log)
    return out


def sum_to_size(be, x: TensorData, size: Sequence[int]) -> TensorData:
    shape = x.shape
    lead = len(shape) - len(size)
    dims = [d for d in range(len(shape)) if d < lead or (size[d - lead] == 1 and shape[d] != 1)]
    if not dims:
        return x
    summed = reduce_op(be, "sum", x, dims, True)
    return summed.reshape(tuple(size))


class T:
    """A tensor bound to a backend, with the slice of homura's Tensor API the tests use."""

    def __init__(self, be, data: TensorData):
        self.be, self.data = be, data

    @property
    def dtype(self):
        return self.data.dtype

    @property
    def shape(self):
        return tuple(self.data.shape)

    def raw(self) -> np.ndarray:
        return self.be.download(self.data)

    def _w(self, d):
        return T(self.be, d)

    def _o(self, other):
        return other.data if isinstance(other, T) else other

    def view(self, f):
        return self._w(f(self.data))

    # unary
    def __getattr__(self, name):
        if name in UNARY:
            return lambda: self._w(unary_op(self.be, name, self.data))
        raise AttributeError(name)

    def gelu(self, approximate="none"):
        return self._w(unary_op(self.be, "gelu_tanh" if approximate == "tanh" else "gelu", self.data))

    # binary
    def _bin(self, name, other, reverse=False):
        a, b = (self._o(other), self.data) if reverse else (self.data, self._o(other))
        return self._w(binary_op(self.be, name, a, b))

    def add(self, o): return self._bin("add", o)
    def sub(self, o): return self._bin("sub", o)
    def rsub(self, o): return self._bin("sub", o, True)
    def mul(self, o): return self._bin("mul", o)
    def div(self, o): return self._bin("div", o)
    def rdiv(self, o): return self._bin("div", o, True)
    def pow(self, o): return self._bin("pow", o)
    def maximum(self, o): return self._bin("maximum", o)
    def minimum(self, o): return self._bin("minimum", o)
    def greater(self, o): return self._bin("greater", o)
    def greater_equal(self, o): return self._bin("greater_equal", o)
    def less(self, o): return self._bin("less", o)
    def less_equal(self, o): return self._bin("less_equal", o)
    def equal(self, o): return self._bin("equal", o)
    def not_equal(self, o): return self._bin("not_equal", o)
    def logical_and(self, o): return self._bin("logical_and", o)
    def logical_or(self, o): return self._bin("logical_or", o)

    def clamp(self, lo, hi): return self.maximum(lo).minimum(hi)
    def clamp_min(self, lo): return self.maximum(lo)
    def clamp_max(self, hi): return self.minimum(hi)

    def masked_fill(self, mask, value): return self._w(masked_fill(self.be, self.data, mask.data, value))
    def to(self, dtype): return self._w(to(self.be, self.data, dtype))
    def contiguous(self): return self._w(contiguous(self.be, self.data))

    # composites (src/ops/composite.rs:450-508)
    def addcmul(self, t1, t2, value): return self.add(t1.mul(value).mul(t2))
    def addcdiv(self, t1, t2, value): return self.add(t1.mul(value).div(t2))

    def lerp(self, end, weight):
        diff = end.sub(self)
        if not isinstance(weight, T):
            wf = float(weight)
            return self.add(diff.mul(weight)) if abs(wf) < 0.5 else end.sub(diff.mul(1.0 - wf))
        low = self.add(weight.mul(diff))
        high = end.sub(diff.mul(weight.neg().add(1.0)))
        return self._w(where_(self.be, weight.abs().less(0.5).data, low.data, high.data))

    # reductions
    def _red(self, name, dims=(), keepdim=False):
        dims = [dims] if isinstance(dims, int) else list(dims)
        return self._w(reduce_op(self.be, name, self.data, dims, keepdim))

    def sum(self): return self._red("sum")
    def sum_dim(self, dims, keepdim=False): return self._red("sum", dims, keepdim)
    def mean(self): return self._red("mean")
    def mean_dim(self, dims, keepdim=False): return self._red("mean", dims, keepdim)
    def prod(self): return self._red("prod")
    def prod_dim(self, dim, keepdim=False): return self._red("prod", dim, keepdim)
    def max(self): return self._red("max")
    def min(self): return self._red("min")
    def all(self): return self._red("all")
    def any(self): return self._red("any")
    def all_dim(self, dim, keepdim=False): return self._red("all", dim, keepdim)
    def any_dim(self, dim, keepdim=False): return self._red("any", dim, keepdim)

    def max_dim(self, dim, keepdim=False):
        v, i = arg_op(self.be, self.data, dim, keepdim, True, True)
        return self._w(v), self._w(i)

    def min_dim(self, dim, keepdim=False):
        v, i = arg_op(self.be, self.data, dim, keepdim, False, True)
        return self._w(v), self._w(i)

    def argmax(self): return self._w(arg_op(self.be, self.data, None, False, True, False)[1])
    def argmin(self): return self._w(arg_op(self.be, self.data, None, False, False, False)[1])
    def argmax_dim(self, dim, keepdim=False): return self._w(arg_op(self.be, self.data, dim, keepdim, True, False)[1])
    def argmin_dim(self, dim, keepdim=False): return self._w(arg_op(self.be, self.data, dim, keepdim, False, False)[1])

    def var(self, correction): return self._w(var_op(self.be, self.data, [], correction, False, False))
    def var_dim(self, dims, correction, keepdim=False):
        return self._w(var_op(self.be, self.data, [dims] if isinstance(dims, int) else dims, correction, keepdim, False))
    def std_dim(self, dims, correction, keepdim=False):
        return self._w(var_op(self.be, self.data, [dims] if isinstance(dims, int) else dims, correction, keepdim, True))

    def softmax(self, dim): return self._w(softmax_op(self.be, self.data, dim, False))
    def log_softmax(self, dim): return self._w(softmax_op(self.be, self.data, dim, True))
    def sum_to_size(self, size): return self._w(sum_to_size(self.be, self.data, size))


def where(cond: T, x, y) -> T:
    o = lambda v: v.data if isinstance(v, T) else v
    return T(cond.be, where_(cond.be, cond.data, o(x), o(y)))
