"""Reductions against the CPU checker, after homura's tests/rocm_reduce.rs. Integer / bool sums, max, min,
all, any and the arg reductions: bit for bit. Float sums, products, means and variances are accumulated in
f64 on both sides, in different orders: the GPU result must lie within 2 ulp of the CPU's for F16/BF16/F32
and within 1e-12 relative (plus homura's condition-number bounds, tests/rocm_reduce.rs:150-289) for F64."""
import ctypes
import itertools

import numpy as np
import pytest

from frontend import T
from gpu_common import both, pairs, same
from homura_b200 import ffi
from homura_b200.host import (ALL_DTYPES, BF16, BOOL, DTYPE_NAMES, F16, F32, F64, FLOATS, I32, I64, INTS, U8, describe)
from values import assert_bitwise, assert_ulp, check_within, f64_to_storage, storage_to_f64, values, words

pytestmark = pytest.mark.gpu
EPS64 = 2.0 ** -53

# shapes chosen to reach every plan: lanes per output 1 / 32 / 256, columns, splits, several reduced dims
SHAPES = [
    ((37, 1000), [1]), ((37, 1000), [0]), ((37, 1000), []), ((5, 7, 9), [1]), ((5, 7, 9), [0, 2]), ((5, 7, 9), [2]),
    ((1031,), []), ((3, 70000), [1]), ((70000, 3), [0]), ((70000, 3), [1]), ((300, 40), [0]), ((2, 3, 4, 5), [1, 3]),
    ((64, 2048), [1]), ((2048, 64), [0]), ((1 << 20,), []), ((4, 5), [0, 1]), ((1, 1), [0]), ((6, 0), [1]), ((0, 6), [1]),
    # long rows folded by one warp each (many outputs): whole vectors, and a ragged row length
    ((4800, 1028), [1]), ((4740, 1026), [1]),
    # a tall strip of columns: hundreds of chunks, folded by a second kernel instead of the last block
    ((400000, 40), [0]),
]


def plan_of(cuda, t, mask):
    r = describe("test", t, mask)
    kind, splits, chunk = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    assert cuda.lib.hmc_test_reduce_plan(r.kept, r.red, ctypes.byref(kind), ctypes.byref(splits), ctypes.byref(chunk)) == 0
    return kind.value, splits.value


def normal(n, seed, scale=1.0):
    w = words(seed, 2 * n)
    u1 = ((w[:n] >> np.uint64(11)).astype(np.float64) + 0.5) / float(1 << 53)
    u2 = (w[n:] >> np.uint64(11)).astype(np.float64) / float(1 << 53)
    return scale * np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def check_sum(got, want, dtype, xs_abs_sum, n, what):
    """|gpu - cpu| <= 2 n eps64 sum|x| + ulp_out, and the north-star bar on top."""
    check_within(got, want, dtype, 2.0 * n * EPS64 * xs_abs_sum, what)
    if dtype != F64:
        assert_ulp(got, want, dtype, 2, what)


def test_every_plan_is_reached(cuda):
    seen = set()
    for shape, dims in SHAPES:
        if 0 in shape:
            continue
        t = cuda.empty(shape, F32)
        mask = [d in dims or not dims for d in range(len(shape))]
        kind, splits = plan_of(cuda, t, mask)
        seen.add((kind, splits > 1))
    for want in [(1001, False), (1032, False), (1256, False), (1256, True), (1, False), (1, True)]:
        assert want in seen, f"no shape reaches plan {want}: {sorted(seen)}"
    assert plan_of(cuda, cuda.empty((400000, 40), F32), [True, False])[1] > 64, "the tall strip is not cut into many chunks"


@pytest.mark.parametrize("dtype", ALL_DTYPES, ids=DTYPE_NAMES)
def test_exact_reductions_on_every_shape(oracle, cuda, dtype):
    """max, min, all, any for every dtype; sum and prod of integers and bools: same bits."""
    for shape, dims in SHAPES:
        n = int(np.prod(shape))
        if dtype not in (F32, I32, BOOL, BF16) and n > 100000:
            continue
        o, g = both(oracle, cuda, values(dtype, n, 101), dtype, shape)
        ops = ["all", "any"]
        reduces_empty = any(shape[d] == 0 for d in (dims or range(len(shape))))
        if not reduces_empty:
            ops += ["max", "min"]
        if dtype not in FLOATS:
            ops += ["sum", "prod"]
        for op in ops:
            same(lambda t: t._red(op, dims), o, g, f"{op} {shape} over {dims}")
        # strided source: the same reduction of the transposed view
        if len(shape) == 2 and n > 0:
            same(lambda t: t.view(lambda d: d.t())._red("max", dims), o, g, f"max of transposed {shape} over {dims}")


@pytest.mark.parametrize("dtype", ALL_DTYPES, ids=DTYPE_NAMES)
def test_arg_reductions_are_exact(oracle, cuda, dtype):
    for shape, dims in SHAPES:
        n = int(np.prod(shape))
        if n == 0 or (dtype not in (F32, I32) and n > 100000):
            continue
        o, g = both(oracle, cuda, values(dtype, n, 103), dtype, shape)
        for dim in range(len(shape)):
            for is_max in (True, False):
                f = (lambda t: t.max_dim(dim)) if is_max else (lambda t: t.min_dim(dim, True))
                (ov, oi), (gv, gi) = f(o), f(g)
                assert_bitwise(gi.raw(), oi.raw(), I64, f"arg indices {shape} dim {dim}")
                assert_bitwise(gv.raw(), ov.raw(), dtype, f"arg values {shape} dim {dim}")
        same(lambda t: t.argmax(), o, g, f"argmax {shape}")
        same(lambda t: t.view(lambda d: d.permute(*reversed(range(len(shape))))).argmin_dim(0), o, g, f"argmin permuted {shape}")


def test_ties_and_nans_pick_the_first(oracle, cuda):
    x = np.zeros((64, 5000), dtype=np.float32)
    x[:, 100] = x[:, 4000] = 7.0
    x[3, 2000] = x[3, 10] = np.nan
    x[5, :] = -0.0
    x[5, 77] = 0.0
    o, g = both(oracle, cuda, x, F32)
    for f in (lambda t: t.max_dim(1), lambda t: t.min_dim(1), lambda t: t.max_dim(0), lambda t: t.min_dim(0)):
        (ov, oi), (gv, gi) = f(o), f(g)
        assert_bitwise(gi.raw(), oi.raw(), I64, "tie indices")
        assert_bitwise(gv.raw(), ov.raw(), F32, "tie values")
    assert int(g.max_dim(1)[1].raw()[0]) == 100 and int(g.max_dim(1)[1].raw()[3]) == 10
    assert int(g.argmax().raw()) == 3 * 5000 + 10


@pytest.mark.parametrize("dtype", FLOATS, ids=[DTYPE_NAMES[d] for d in FLOATS])
def test_float_sums_means_products(oracle, cuda, dtype):
    for shape, dims in SHAPES:
        n = int(np.prod(shape))
        if n == 0:
            continue
        raw = f64_to_storage(normal(n, 105), dtype)
        o, g = both(oracle, cuda, raw, dtype, shape)
        xs = np.abs(storage_to_f64(raw, dtype)).reshape(shape)
        axes = tuple(dims) if dims else None
        abs_sum = xs.sum(axis=axes)
        nred = n // max(abs_sum.size, 1)
        check_sum(g._red("sum", dims).raw(), o._red("sum", dims).raw(), dtype, abs_sum, nred, f"sum {shape} {dims}")
        check_sum(g._red("mean", dims).raw(), o._red("mean", dims).raw(), dtype, abs_sum / nred, nred, f"mean {shape} {dims}")
        # products of values near 1 stay finite
        near_one = f64_to_storage(1.0 + normal(n, 106, 1e-3), dtype)
        po, pg = both(oracle, cuda, near_one, dtype, shape)
        want = po._red("prod", dims).raw()
        check_within(pg._red("prod", dims).raw(), want, dtype, 2.0 * nred * EPS64 * np.abs(storage_to_f64(want, dtype)),
                     f"prod {shape} {dims}")
    # special values and random bit patterns: infinities and NaNs must be classified alike
    for name, o, g in pairs(oracle, cuda, dtype, 107):
        want, got = o.sum().raw(), g.sum().raw()
        fw = storage_to_f64(want, dtype)
        if np.isfinite(fw).all():
            check_within(got, want, dtype, 1e-6 * np.abs(fw) + 1e-30, f"sum {name}")
        else:
            assert_bitwise(got, want, dtype, f"sum {name}")


@pytest.mark.parametrize("dtype", FLOATS, ids=[DTYPE_NAMES[d] for d in FLOATS])
def test_var_and_std(oracle, cuda, dtype):
    for shape, dims in SHAPES:
        n = int(np.prod(shape))
        if n == 0:
            continue
        raw = f64_to_storage(3.0 + normal(n, 109), dtype)
        o, g = both(oracle, cuda, raw, dtype, shape)
        nred = n // max(int(np.prod([s for d, s in enumerate(shape) if dims and d not in dims])), 1)
        for correction, take_sqrt in ((1, False), (0, False), (2, True)):
            f = (lambda t: t.std_dim(dims, correction)) if take_sqrt else (lambda t: t.var_dim(dims, correction))
            want, got = f(o).raw(), f(g).raw()
            fw = storage_to_f64(want, dtype)
            extra = np.where(np.isfinite(fw), 4.0 * nred * EPS64 * np.abs(fw) * 1e3, 0.0)
            check_within(got, want, dtype, extra, f"var {shape} {dims} c={correction}")
            if dtype != F64:
                assert_ulp(got, want, dtype, 2, f"var {shape} {dims} c={correction}")
    # exact cases: constant rows have variance 0, n = 1 with correction 1 is NaN, empty is NaN
    c = np.full((9, 700), 2.5, dtype=np.float64)
    o, g = both(oracle, cuda, f64_to_storage(c, dtype), dtype, (9, 700))
    assert_bitwise(g.var_dim(1, 1).raw(), o.var_dim(1, 1).raw(), dtype, "constant rows")
    assert (storage_to_f64(g.var_dim(1, 1).raw(), dtype) == 0).all()
    one_o, one_g = both(oracle, cuda, f64_to_storage([[1.0], [2.0]], dtype), dtype, (2, 1))
    assert_bitwise(one_g.var_dim(1, 1).raw(), one_o.var_dim(1, 1).raw(), dtype, "single element")
    e_o, e_g = both(oracle, cuda, np.zeros((3, 0), dtype=np.float64), dtype, (3, 0))
    assert_bitwise(e_g.var_dim(1, 0).raw(), e_o.var_dim(1, 0).raw(), dtype, "empty reduction")


def test_reductions_are_reproducible(cuda):
    raw = f64_to_storage(normal(1 << 22, 111), F32)
    t = T(cuda, cuda.upload(raw, F32, (1 << 11, 1 << 11)))
    for dims in ([], [0], [1]):
        first = t._red("sum", dims).raw()
        for _ in range(3):
            assert (t._red("sum", dims).raw().view(np.uint32) == first.view(np.uint32)).all()
    # reductions cut into chunks, whose partials are folded by whichever block finishes last: forty runs, one result
    tall = T(cuda, cuda.upload(f64_to_storage(normal(1 << 23, 112), F32), F32, (1 << 13, 1 << 10)))
    for f in (lambda x: x._red("sum", [0]), lambda x: x._red("sum", []), lambda x: x.var_dim([0], 1)):
        first = f(tall).raw().view(np.uint32)
        for _ in range(40):
            assert (f(tall).raw().view(np.uint32) == first).all()


def test_wrong_results_are_rejected(oracle, cuda):
    raw = f64_to_storage(normal(1 << 16, 113), F64)
    o, g = both(oracle, cuda, raw, F64)
    want = o.sum().raw()
    bad = want * (1.0 + 1e-5) + 1e-3
    with pytest.raises(AssertionError):
        check_within(bad, want, F64, 2.0 * (1 << 16) * EPS64 * np.abs(raw).sum(), "off by 1e-5")
    f32 = T(cuda, cuda.upload(raw.astype(np.float32), F32))
    narrow = np.float32(np.sum(raw.astype(np.float32), dtype=np.float32))
    # a sum accumulated in f32 (numpy pairwise) is usually more than 2 ulp away from the f64 fold at this size;
    # the f64 fold of the GPU is not
    assert_ulp(f32.sum().raw(), T(oracle, oracle.upload(raw.astype(np.float32), F32)).sum().raw(), F32, 1, "f32 sum")


def test_workspace_too_small_is_refused(cuda):
    from homura_b200.host import output_desc
    t = cuda.empty((1 << 22,), F32)
    r = describe("reduce", t, [True])
    out = cuda.empty((), F32)
    o = output_desc("reduce", r, out)
    assert cuda.lib.hmc_reduce(cuda.ctx, ffi.HMC_REDUCE_SUM, o, r.kept, r.red, None, 0) == ffi.HMC_INVALID
    assert b"workspace" in cuda.lib.hmc_last_error()
    i = cuda.upload(np.zeros(4, dtype=np.int32), I32)
    ri = describe("reduce", i, [True])
    assert cuda.lib.hmc_reduce(cuda.ctx, ffi.HMC_REDUCE_MEAN, output_desc("r", ri, cuda.empty((), I32)), ri.kept, ri.red,
                               None, 0) == ffi.HMC_INVALID
    e = cuda.empty((3, 0), F32)
    re_ = describe("reduce", e, [False, True])
    assert cuda.lib.hmc_reduce(cuda.ctx, ffi.HMC_REDUCE_MAX, output_desc("r", re_, cuda.empty((3,), F32)), re_.kept,
                               re_.red, None, 0) == ffi.HMC_INVALID
