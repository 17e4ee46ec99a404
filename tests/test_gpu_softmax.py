"""softmax / log_softmax against the CPU checker (both in f64, different summation orders and two libms'
exp), after homura's tests/rocm_reduce.rs check_softmax: |gpu - cpu| <= (2 n eps + 2 eps) |cpu| + ulp_out,
rows sum to 1, and within 2 ulp for F16/BF16/F32."""
import ctypes

import numpy as np
import pytest

from frontend import T
from gpu_common import both, pairs
from homura_b200.host import BF16, DTYPE_NAMES, F16, F32, F64, FLOATS, lines
from test_gpu_reduce import normal
from values import assert_bitwise, assert_ulp, check_within, f64_to_storage, storage_to_f64

pytestmark = pytest.mark.gpu
EPS64 = 2.0 ** -53

SHAPES = [((64, 2048), 1), ((64, 2048), 0), ((7, 100), 1), ((300, 33), 1), ((5, 17, 9), 1), ((3, 40000), 1),
          ((2, 9000), 1), ((1031,), 0), ((4, 4100), 1), ((), 0), ((5, 1), 1), ((16, 8192), 1), ((16, 8200), 1),
          ((13, 600), 1), ((600, 13), 0), ((6, 1001), 1), ((4, 4101), 1), ((3, 12288), 1), ((1000, 64), 1), ((9, 2048), 1), ((3, 70001), 1), ((2, 1 << 17), 1), ((70000, 2), 0)]


def check_softmax(got, want, dtype, n, what, log):
    fw = storage_to_f64(want, dtype)
    scale = np.where(np.isfinite(fw), np.abs(fw), 0.0)
    check_within(got, want, dtype, (2.0 * n * EPS64 + 2.0 * EPS64) * (scale + (1.0 if log else 0.0)) * 8.0, what)
    if dtype != F64:
        assert_ulp(got, want, dtype, 2, what)


@pytest.mark.parametrize("dtype", FLOATS, ids=[DTYPE_NAMES[d] for d in FLOATS])
def test_softmax_on_every_plan(oracle, cuda, dtype):
    kinds = set()
    for shape, dim in SHAPES:
        n = int(np.prod(shape)) if shape else 1
        raw = f64_to_storage(normal(n, 121, 3.0), dtype)
        o, g = both(oracle, cuda, raw, dtype, shape)
        rows = shape[dim] if shape else 1
        for log in (False, True):
            f = (lambda t: t.log_softmax(dim)) if log else (lambda t: t.softmax(dim))
            want, got = f(o).raw(), f(g).raw()
            check_softmax(got, want, dtype, rows, f"softmax {shape} dim {dim} log={log}", log)
        if not log and shape:
            s = storage_to_f64(g.softmax(dim).raw(), dtype).sum(axis=dim)
            assert np.allclose(s, 1.0, atol=1e-2 if dtype in (F16, BF16) else 1e-5)
        if shape:
            ln = lines("t", g.data, g.data, dim, g.data.strides)
            k, grp, cache = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
            assert cuda.lib.hmc_test_softmax_plan(ln[0][1], ln[1], ln[3], ctypes.byref(k), ctypes.byref(grp), ctypes.byref(cache)) == 0
            kinds.add((k.value, grp.value))
    # rows in registers (a warp, half a block, a block per row), streaming rows, and, for the narrower dtypes, whole
    # aligned rows staged in shared memory by a warp
    assert {(0, 32), (0, 128), (0, 256), (1, 256)} <= kinds, kinds
    assert dtype == F64 or (2, 32) in kinds, kinds
    assert (3, 256) in kinds, kinds  # few long rows: maxima, sums and the outputs in three launches


def test_causal_mask_rows(oracle, cuda):
    """Attention logits with an upper-triangular -inf mask: masked entries are exactly 0, a fully masked
    row is NaN, as on the CPU."""
    n = 512
    x = normal(4 * n * n, 123, 3.0).reshape(4, n, n).astype(np.float32)
    x[:, np.triu_indices(n, 1)[0], np.triu_indices(n, 1)[1]] = -np.inf
    x[1, 7, :] = -np.inf
    x[2, 9, 3] = np.nan
    o, g = both(oracle, cuda, x, F32)
    for log in (False, True):
        f = (lambda t: t.log_softmax(-1)) if log else (lambda t: t.softmax(-1))
        want, got = f(o).raw(), f(g).raw()
        check_softmax(got, want, F32, n, f"causal log={log}", log)
    sm = g.softmax(-1).raw()
    assert (sm[0][np.triu_indices(n, 1)] == 0).all() and np.isnan(sm[1, 7]).all() and np.isnan(sm[2, 9]).all()


@pytest.mark.parametrize("dtype", FLOATS, ids=[DTYPE_NAMES[d] for d in FLOATS])
def test_softmax_of_special_values_and_layouts(oracle, cuda, dtype):
    for name, o, g in pairs(oracle, cuda, dtype, 125):
        if len(o.shape) == 0 or 0 in o.shape:
            continue
        want, got = o.softmax(-1).raw(), g.softmax(-1).raw()
        fw = storage_to_f64(want, dtype)
        check_within(got, want, dtype, np.where(np.isfinite(fw), 1e-9 * np.abs(fw), 0.0), f"softmax {name}")
