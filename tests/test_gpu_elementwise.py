"""Elementwise kernels against the CPU checker on the same bits, after homura's tests/rocm_elementwise.rs:
every dtype, every layout of the generator, special values and random bit patterns.

Bars: integer, bool and comparison results and the IEEE float ops (+ - * / sqrt, min/max, neg, abs, sign,
relu, fused steps, casts) bit for bit (a NaN only has to meet a NaN); for F16/BF16/F32 the transcendental ops
bit for bit where the device restates the C library's function (exp, log, tanh, pow and the formulas on them)
and within one ulp otherwise (sin, cos, erf, gelu; the half types' fast exp / sigmoid / silu); for F64, whose
transcendentals come from two different libms, homura's own bound k * u * m + ulp(out)
(tests/rocm_elementwise.rs:168-236)."""
import math

import numpy as np
import pytest

from frontend import T, where
from gpu_common import both, pairs, same
from homura_b200 import ffi
from homura_b200.host import ALL_DTYPES, BF16, BOOL, DTYPE_NAMES, F16, F32, F64, FLOATS, I8, I16, I32, I64, INTS, U8
from values import (assert_bitwise, assert_ulp, check_within, f64_to_storage, large_layouts, storage_to_f64, values,
                    words)

pytestmark = pytest.mark.gpu


def uniform(n, r, seed):
    w = words(seed, n)
    return ((w >> np.uint64(11)).astype(np.float64) / float(1 << 53) * 2.0 - 1.0) * r


def near_zero(n, seed):
    w = words(seed, n)
    e = (w % np.uint64(300)).astype(np.int64) - 320
    m = ((w >> np.uint64(20)) % np.uint64(1000)).astype(np.float64) / 1000.0 + 1.0
    s = np.where((w >> np.uint64(63)) == 1, -1.0, 1.0)
    v = s * np.ldexp(m, e.astype(np.int32))
    return np.concatenate([v, [0.0, -0.0, 5.96e-8, 1e-40, -1e-45, 5e-324]])


@pytest.mark.parametrize("dtype", ALL_DTYPES, ids=DTYPE_NAMES)
def test_ieee_unary_ops_are_bitwise(oracle, cuda, dtype):
    ops = ["neg", "abs", "sign", "relu", "sqrt", "rsqrt", "reciprocal", "logical_not"]
    for name, o, g in pairs(oracle, cuda, dtype, 1):
        for op in ops:
            if dtype == BOOL and op in ("neg", "abs", "relu"):
                continue
            same(lambda t: getattr(t, op)(), o, g, f"{op} {name}")


def test_large_layouts_take_several_rounds_of_the_grid(oracle, cuda):
    for name, (o, g) in large_layouts([oracle, cuda], F32, 2):
        same(lambda t: t.sqrt(), T(oracle, o), T(cuda, g), name)
        same(lambda t: t.neg(), T(oracle, o), T(cuda, g), name)
    for name, (o, g) in large_layouts([oracle, cuda], BF16, 3, n=(1 << 22) + 1000):
        same(lambda t: t.abs(), T(oracle, o), T(cuda, g), name)
        same(lambda t: t.to(F32), T(oracle, o), T(cuda, g), name)


TRANSCENDENTAL = {
    # op: (f, magnitude of the largest intermediate m(x, y), k, tails)
    "exp": (lambda t: t.exp(), lambda x, y: np.abs(y), 2.0, [88.7, 88.72, 88.73, -87.3, -103.9, -104.0, 709.7, 709.8, -745.1, 11.09, -17.3]),
    "log": (lambda t: t.log(), lambda x, y: np.abs(y), 2.0, [1e-300, 1e300, 1.0 + 1e-7]),
    "sin": (lambda t: t.sin(), lambda x, y: np.abs(y), 2.0, [math.pi, 1e6, 1e20, 355.0]),
    "cos": (lambda t: t.cos(), lambda x, y: np.abs(y), 2.0, [math.pi / 2, 1e6, 1e20, 33.0]),
    "tanh": (lambda t: t.tanh(), lambda x, y: np.abs(y), 2.0, [9.0, 20.0, -20.0, 1e-5]),
    "erf": (lambda t: t.erf(), lambda x, y: np.abs(y), 2.0, [5.9, 6.0, 6.1, -7.0, 1.49999, 1.5, 1.50001, 3.0]),
    "sigmoid": (lambda t: t.sigmoid(), lambda x, y: np.abs(y), 4.0, [-30.0, -88.0, -104.0, 30.0, 40.0, -745.0]),
    "silu": (lambda t: t.silu(), lambda x, y: np.abs(x) / (1.0 + np.exp(-x)), 4.0, [-30.0, -88.0, -104.0, 30.0, 40.0, -745.0]),
    "log_sigmoid": (lambda t: t.log_sigmoid(), lambda x, y: np.abs(np.minimum(x, 0.0)) + np.log1p(np.exp(-np.abs(x))), 6.0,
                    [-30.0, -31.0, -1e4, 30.0, 31.0, 40.0, 1e4]),
    "gelu": (lambda t: t.gelu("none"), lambda x, y: 0.5 * np.abs(x) * 2.0, 4.0, [-10.0, -10.5, -12.0, -30.0, 10.0]),
    "gelu_tanh": (lambda t: t.gelu("tanh"), lambda x, y: 0.5 * np.abs(x) * 2.0, 4.0, [-10.0, -10.5, -12.0, -30.0, 10.0]),
}
ULP_REPORT = {}
# F16/BF16/F32 tensors are computed in f32. exp, log, log1p, tanh and pow restate the host C library's algorithms
# (homura_b200/csrc/libm32.cuh), so these ops and the formulas built on them have the CPU's bits; sin, cos and erf
# are evaluated in f64 and rounded once, at most one ulp from the CPU's. F16/BF16 exp, sigmoid and silu use the
# special function unit in f32 and are rounded to 11 / 8 bits: one ulp next to a rounding tie.
ULP_BAR = {"exp": 0, "log": 0, "tanh": 0, "sigmoid": 0, "silu": 0, "log_sigmoid": 0, "gelu_tanh": 0,
           "sin": 1, "cos": 1, "erf": 1, "gelu": 1}
HALF_FAST = ("exp", "sigmoid", "silu")
# F64 tensors: exp, tanh and log1p restate the C library's double-precision algorithms as well
# (homura_b200/csrc/libm64.cuh), so every op built on them alone has the CPU's bits; log, sin and cos are the CUDA
# library's against glibc's (each within an ulp of the true value).
ULP_BAR_F64 = {"exp": 0, "tanh": 0, "sigmoid": 0, "silu": 0, "log_sigmoid": 0, "gelu_tanh": 0, "erf": 0, "gelu": 0,
               "log": 1, "sin": 1, "cos": 1}


@pytest.mark.parametrize("op", list(TRANSCENDENTAL))
@pytest.mark.parametrize("dtype", FLOATS, ids=[DTYPE_NAMES[d] for d in FLOATS])
def test_transcendental_unary_ops(oracle, cuda, op, dtype):
    f, m, k, tails = TRANSCENDENTAL[op]
    inputs = [(name, o, g) for name, o, g in pairs(oracle, cuda, dtype, 11)]
    for r in (1.0, 10.0, 100.0):
        inputs.append((f"uniform +-{r}",) + both(oracle, cuda, f64_to_storage(uniform(4096, r, 12), dtype), dtype))
    inputs.append(("near zero",) + both(oracle, cuda, f64_to_storage(near_zero(2048, 13), dtype), dtype))
    inputs.append(("tails",) + both(oracle, cuda, f64_to_storage(tails, dtype), dtype))
    worst, differ, total = 0, 0, 0
    u = 2.0 ** -53 if dtype == F64 else 2.0 ** -24
    for name, o, g in inputs:
        want, got = f(o).raw(), f(g).raw()
        xs = storage_to_f64(o.contiguous().raw(), dtype)
        with np.errstate(all="ignore"):
            # F64 results come from two different f64 libms (glibc on the CPU, CUDA's on the GPU), each within
            # about 2 ulp of the true value: twice homura's factor covers their distance.
            extra = (2.0 * k if dtype == F64 else k) * u * m(xs, storage_to_f64(want, dtype))
        extra = np.where(np.isfinite(extra), extra, 0.0)
        mu, nd = check_within(got, want, dtype, extra, f"{op} {name}")
        worst, differ, total = max(worst, mu), differ + nd, total + want.size
    ULP_REPORT[(op, DTYPE_NAMES[dtype])] = (worst, differ, total)
    print(f"ulp {op:<12} {DTYPE_NAMES[dtype]:<5}: max {worst} ulp, {differ} of {total} elements differ")
    if dtype == F64:
        bar = ULP_BAR_F64[op]
    else:
        bar = 1 if (dtype in (F16, BF16) and op in HALF_FAST) else ULP_BAR[op]
    assert worst <= bar, f"{op}: {worst} ulp from the CPU result (bar {bar}), {differ} of {total} differ"


def test_the_bound_rejects_wrong_results(oracle, cuda):
    o, g = both(oracle, cuda, f64_to_storage(uniform(4096, 10.0, 21), F64), F64)
    want = o.exp().raw()
    with pytest.raises(AssertionError):
        check_within(g.to(F32).exp().to(F64).raw(), want, F64, 2.0 * 2.0 ** -53 * np.abs(want), "narrow")
    with pytest.raises(AssertionError):
        check_within(g.cos().raw(), o.sin().raw(), F64, 2.0 ** -52, "cos for sin")
    with pytest.raises(AssertionError):
        check_within((want * (1.0 + 64 * 2.0 ** -52)), want, F64, 2.0 * 2.0 ** -53 * np.abs(want), "64 ulp off")


ARITH = ["add", "sub", "mul", "div", "maximum", "minimum"]
COMPARE = ["greater", "greater_equal", "less", "less_equal", "equal", "not_equal"]


@pytest.mark.parametrize("dtype", ALL_DTYPES, ids=DTYPE_NAMES)
def test_binary_ops_are_bitwise(oracle, cuda, dtype):
    la, lb = pairs(oracle, cuda, dtype, 5), pairs(oracle, cuda, dtype, 6)
    for (name, oa, ga), (_, ob, gb) in zip(la, lb):
        for op in ARITH + COMPARE:
            if dtype == BOOL and op == "sub":
                continue
            same_b = lambda f: assert_bitwise(f(ga, gb).raw(), f(oa, ob).raw(), f(oa, ob).dtype, f"{op} {name}")
            same_b(lambda a, b: getattr(a, op)(b))
        if dtype == BOOL:
            same_b = lambda f: assert_bitwise(f(ga, gb).raw(), f(oa, ob).raw(), BOOL, f"logical {name}")
            same_b(lambda a, b: a.logical_and(b))
            same_b(lambda a, b: a.logical_or(b))
        if dtype in INTS:
            assert_bitwise(ga.pow(gb).raw(), oa.pow(ob).raw(), dtype, f"int pow {name}")


@pytest.mark.parametrize("dtype", ALL_DTYPES, ids=DTYPE_NAMES)
def test_mixed_layouts_and_in_place(oracle, cuda, dtype):
    """A transposed operand against a contiguous one, a row and a column broadcast, and out = a op a."""
    raw_a, raw_b = values(dtype, 96 * 130, 7), values(dtype, 96 * 130, 8)
    (oa, ga), (ob, gb) = both(oracle, cuda, raw_a, dtype, (96, 130)), both(oracle, cuda, raw_b, dtype, (130, 96))
    for op in ("add", "mul", "maximum", "less"):
        f = lambda a, b: getattr(a, op)(b.view(lambda d: d.t()))
        assert_bitwise(f(ga, gb).raw(), f(oa, ob).raw(), f(oa, ob).dtype, f"{op} transposed")
        row = lambda a: getattr(a, op)(a.view(lambda d: d.narrow(0, 3, 1).expand(96, 130)))
        col = lambda a: getattr(a, op)(a.view(lambda d: d.narrow(1, 5, 1).expand(96, 130)))
        assert_bitwise(row(ga).raw(), row(oa).raw(), row(oa).dtype, f"{op} row broadcast")
        assert_bitwise(col(ga).raw(), col(oa).raw(), col(oa).dtype, f"{op} column broadcast")
    # in place: the output is one of the inputs
    for be, a in ((oracle, oa), (cuda, ga)):
        be.binary(ffi.HMC_BINARY_ADD, a.data, a.data, a.data)
    assert_bitwise(ga.raw(), oa.raw(), dtype, "in place add")


@pytest.mark.parametrize("dtype", FLOATS, ids=[DTYPE_NAMES[d] for d in FLOATS])
def test_float_pow_and_scalars(oracle, cuda, dtype):
    base = f64_to_storage(np.abs(uniform(4096, 10.0, 31)) + 0.01, dtype)
    expo = f64_to_storage(uniform(4096, 4.0, 32), dtype)
    (oa, ga), (ob, gb) = both(oracle, cuda, base, dtype), both(oracle, cuda, expo, dtype)
    want, got = oa.pow(ob).raw(), ga.pow(gb).raw()
    u = 2.0 ** -53 if dtype == F64 else 2.0 ** -24
    special_o, special_g = both(oracle, cuda, values(dtype, 4096, 33), dtype)
    expo_o, expo_g = both(oracle, cuda, values(dtype, 4096, 36), dtype)
    if dtype == F64:
        check_within(got, want, dtype, 4.0 * u * np.abs(storage_to_f64(want, dtype)), "pow")
    else:
        # the f32 power is the C library's powf restated: the CPU's bits, special values and bit patterns included
        assert_bitwise(got, want, dtype, "pow")
        assert_bitwise(special_g.pow(expo_g).raw(), special_o.pow(expo_o).raw(), dtype, "pow of bit patterns")
        assert_bitwise(special_g.pow(gb).raw(), special_o.pow(ob).raw(), dtype, "pow of bit patterns, small exponents")
    for s in (2.0, 0.5, -1.5, 3):
        w, g = special_o.pow(s).raw(), special_g.pow(s).raw()
        fw = storage_to_f64(w, dtype)
        if dtype == F64:
            check_within(g, w, dtype, np.where(np.isfinite(fw), 4.0 * u * np.abs(fw), 0.0), f"pow {s}")
        elif s == 2.0:
            # the square is one multiplication on the GPU; the C library's powf(x, 2) is not always the nearest value
            assert_ulp(g, w, dtype, 1, f"pow {s}")
        else:
            assert_bitwise(g, w, dtype, f"pow {s}")
    for name, o, g in pairs(oracle, cuda, dtype, 34):
        for f in (lambda t: t.mul(2.5), lambda t: t.div(3.0), lambda t: t.rdiv(2.0), lambda t: t.add(2.5),
                  lambda t: t.rsub(1.0), lambda t: t.maximum(0.25), lambda t: t.less(0.5), lambda t: t.clamp(-1.5, 2.5)):
            same(f, o, g, f"scalar op {name}")


@pytest.mark.parametrize("dtype", INTS + [BOOL], ids=[DTYPE_NAMES[d] for d in INTS + [BOOL]])
def test_integer_constants(oracle, cuda, dtype):
    for name, o, g in pairs(oracle, cuda, dtype, 35):
        fs = [lambda t: t.add(1), lambda t: t.mul(3), lambda t: t.maximum(2), lambda t: t.greater_equal(1),
              lambda t: t.div(2), lambda t: t.mul(2.5)]
        if dtype != BOOL:
            fs += [lambda t: t.sub(1), lambda t: t.rsub(7), lambda t: t.pow(3), lambda t: t.clamp(-1, 2)]
        for f in fs:
            same(f, o, g, f"constant op {name}")


@pytest.mark.parametrize("dtype", FLOATS, ids=[DTYPE_NAMES[d] for d in FLOATS])
def test_fused_steps_are_bitwise(oracle, cuda, dtype):
    la, lb, lc = (pairs(oracle, cuda, dtype, s) for s in (41, 42, 43))
    cases = [(ffi.HMC_FUSED_SCALED_ADD, 0.1, False), (ffi.HMC_FUSED_SCALED_ADD, -3.0, False), (ffi.HMC_FUSED_LERP, 0.3, False),
             (ffi.HMC_FUSED_LERP, 0.7, False), (ffi.HMC_FUSED_LERP, 0.1, False), (ffi.HMC_FUSED_ADDCMUL, 0.001, True),
             (ffi.HMC_FUSED_ADDCDIV, -2.0, True), (ffi.HMC_FUSED_ADDCDIV, 1e-3, True)]
    for (name, oa, ga), (_, ob, gb), (_, oc, gc) in zip(la, lb, lc):
        for op, value, three in cases:
            outs = []
            for be, a, b, c in ((oracle, oa, ob, oc), (cuda, ga, gb, gc)):
                out = be.empty(a.shape, dtype)
                be.fused(op, value, out, a.data, b.data, c.data if three else None)
                outs.append(be.download(out))
            assert_bitwise(outs[1], outs[0], dtype, f"fused {op} {value} {name}")


@pytest.mark.parametrize("dtype", ALL_DTYPES, ids=DTYPE_NAMES)
def test_where_and_masked_fill(oracle, cuda, dtype):
    for (name, ox, gx), (_, oy, gy), (_, oc, gc) in zip(pairs(oracle, cuda, dtype, 51), pairs(oracle, cuda, dtype, 52),
                                                        pairs(oracle, cuda, BOOL, 53)):
        assert_bitwise(where(gc, gx, gy).raw(), where(oc, ox, oy).raw(), dtype, f"where {name}")
        v = True if dtype == BOOL else (7 if dtype in INTS else -1e9 if dtype != F16 else -6e4)
        assert_bitwise(gx.masked_fill(gc, v).raw(), ox.masked_fill(oc, v).raw(), dtype, f"masked_fill {name}")
        if dtype != BOOL:
            w = 0.5 if dtype in FLOATS else 3
            assert_bitwise(where(gc, gx, w).raw(), where(oc, ox, w).raw(), where(oc, ox, w).dtype, f"where scalar {name}")
            assert_bitwise(where(gc, w, w * 2).raw(), where(oc, w, w * 2).raw(), where(oc, w, w * 2).dtype, "where scalars")


@pytest.mark.parametrize("dtype", [F32, BF16, U8, F64], ids=["f32", "bf16", "u8", "f64"])
def test_long_rows_are_cut_into_segments(oracle, cuda, dtype):
    """Several rows, each longer than one block's reach (row groups x segments), with broadcast operands and a
    ragged tail; and a transposed operand whose tiles are not whole."""
    rows, cols = 5, 70001
    (oa, ga), (ob, gb) = both(oracle, cuda, values(dtype, rows * cols, 95), dtype, (rows, cols)), \
        both(oracle, cuda, values(dtype, rows * cols, 96), dtype, (rows, cols))
    for op in ("add", "maximum"):
        f = lambda a, b: getattr(a, op)(b)
        assert_bitwise(f(ga, gb).raw(), f(oa, ob).raw(), dtype, f"{op} [5, 70001]")
        row = lambda a: getattr(a, op)(a.view(lambda d: d.narrow(0, 2, 1).expand(rows, cols)))
        col = lambda a: getattr(a, op)(a.view(lambda d: d.narrow(1, 11, 1).expand(rows, cols)))
        assert_bitwise(row(ga).raw(), row(oa).raw(), dtype, f"{op} row broadcast, long rows")
        assert_bitwise(col(ga).raw(), col(oa).raw(), dtype, f"{op} column broadcast, long rows")
        off = lambda a, b: getattr(a.view(lambda d: d.narrow(1, 3, 60000)), op)(b.view(lambda d: d.narrow(1, 1, 60000)))
        assert_bitwise(off(ga, gb).raw(), off(oa, ob).raw(), dtype, f"{op} misaligned windows")
    (ot, gt) = both(oracle, cuda, values(dtype, 333 * 517, 97), dtype, (333, 517))
    (ou, gu) = both(oracle, cuda, values(dtype, 333 * 517, 98), dtype, (517, 333))
    t = lambda a, b: a.add(b.view(lambda d: d.t()))
    assert_bitwise(t(gt, gu).raw(), t(ot, ou).raw(), dtype, "transposed operand, ragged tiles")
    c = lambda a: a.view(lambda d: d.t()).contiguous()
    assert_bitwise(c(gt).raw(), c(ot).raw(), dtype, "contiguous() of a transposed view")


@pytest.mark.parametrize("dtype", [BF16, F32, I64, U8], ids=["bf16", "f32", "i64", "u8"])
def test_transposed_operands_through_the_tile_ring(oracle, cuda, dtype):
    """Transposed inputs large enough that every block laps its ring of shared-memory stages several times:
    whole aligned tiles (fetched by bulk copies), ragged edge tiles and windows whose rows are not 16-byte
    aligned (filled element by element) in one launch; one, two and three transposed inputs; outer dimensions."""
    n, m = 2200, 2120  # 35 x 34 tiles, the last of each ragged
    (ox, gx), (oy, gy), (oz, gz) = (both(oracle, cuda, values(dtype, n * m, 300 + i), dtype, (m, n)) for i in range(3))
    (op_, gp) = both(oracle, cuda, values(dtype, n * m, 310), dtype, (n, m))
    tr = lambda d: d.t()
    unary = (lambda t: t.view(tr).neg()) if dtype != U8 else (lambda t: t.view(tr).contiguous())
    assert_bitwise(unary(gx).raw(), unary(ox).raw(), dtype, "unary on x.t()")
    one = lambda p, x: p.add(x.view(tr))
    assert_bitwise(one(gp, gx).raw(), one(op_, ox).raw(), dtype, "p + x.t()")
    two = lambda x, y: x.view(tr).mul(y.view(tr))
    assert_bitwise(two(gx, gy).raw(), two(ox, oy).raw(), dtype, "x.t() * y.t()")
    (oc, gc) = both(oracle, cuda, values(BOOL, n * m, 311), BOOL, (m, n))
    three = lambda c, x, y: where(c.view(tr), x.view(tr), y.view(tr))
    assert_bitwise(three(gc, gx, gy).raw(), three(oc, ox, oy).raw(), dtype, "where on three transposed inputs")
    window = lambda x: x.view(lambda d: d.narrow(0, 1, m - 2).narrow(1, 3, n - 5).t()).contiguous()
    assert_bitwise(window(gz).raw(), window(oz).raw(), dtype, "misaligned window of x.t()")
    (ob, gb) = both(oracle, cuda, values(dtype, 3 * 200 * 328, 312), dtype, (3, 200, 328))
    batched = lambda x: x.view(lambda d: d.transpose(1, 2)).contiguous()
    assert_bitwise(batched(gb).raw(), batched(ob).raw(), dtype, "batched transpose")


def test_promoting_add_matches_cast_then_add(oracle, cuda):
    """bf16 + f32 -> f32 in one kernel has the bits of homura's cast kernels followed by add."""
    x = values(BF16, 700 * 300, 61).reshape(700, 300)
    bias = values(F32, 700, 62).reshape(700, 1)
    for be_pair in [both(oracle, cuda, x, BF16)]:
        (ox, gx) = be_pair
    ob, gb = both(oracle, cuda, bias, F32)
    outs = []
    for be, a, b in ((oracle, ox, ob), (cuda, gx, gb)):
        out = be.empty((700, 300), F32)
        be.binary_promoted(ffi.HMC_BINARY_ADD, out, a.data, b.data.expand(700, 300))
        outs.append(be.download(out))
    assert_bitwise(outs[1], outs[0], F32, "promoting add")
    assert_bitwise(gx.add(gb).raw(), outs[0], F32, "front-end add with promotion on the GPU")


def test_unsupported_combinations_are_refused(cuda):
    from homura_b200.host import BackendError
    x = cuda.upload(np.zeros(8, dtype=np.int32), I32)
    out = cuda.empty((8,), I32)
    with pytest.raises(BackendError) as e:
        cuda.unary(ffi.HMC_UNARY_EXP, out, x)
    assert e.value.status == ffi.HMC_INVALID
    with pytest.raises(BackendError):
        cuda.binary(ffi.HMC_BINARY_DIV, out, x, x)
    with pytest.raises(BackendError):
        cuda.unary(ffi.HMC_UNARY_NEG, cuda.empty((8,), F32), x)
    b = cuda.upload(np.zeros(8, dtype=np.uint8), BOOL)
    with pytest.raises(BackendError):
        cuda.unary(ffi.HMC_UNARY_NEG, cuda.empty((8,), BOOL), b)
    with pytest.raises(BackendError):
        cuda.binary(ffi.HMC_BINARY_SUB, cuda.empty((8,), BOOL), b, b)
    with pytest.raises(BackendError):
        cuda.binary(99, out, x, x)


@pytest.mark.parametrize("dtypes", [(BF16, F32), (F16, F32), (BF16, BF16), (F16, F16), (F32, F32)],
                         ids=["bf16+f32", "f16+f32", "bf16", "f16", "f32"])
def test_unary_binary_binary_in_one_kernel_has_the_three_kernels_bits(oracle, cuda, dtypes):
    """(unary(x) op b) op c fused: the bits of hmc_unary, hmc_binary and the promoting binary run one after the other
    on the GPU, and of the CPU checker's three steps wherever the unary step has the CPU's bits; contiguous
    operands, a row and a column broadcast, and a transposed x: with rows whose byte stride is no multiple of 16 (the
    general tiled kernel), with ragged 64 x 64 tiles (the copy engine's kernel, results stored in pairs), and with an
    odd number of columns (stored one by one)."""
    t, tc = dtypes
    for rows, cols in ((300, 520), (328, 520), (328, 521)):
        _chain_case(oracle, cuda, t, tc, rows, cols)


def _chain_case(oracle, cuda, t, tc, rows, cols):
    x_raw = f64_to_storage(uniform(rows * cols, 6.0, 71), t)
    b_raw = f64_to_storage(uniform(cols, 2.0, 72), t)
    c_raw = f64_to_storage(uniform(rows, 3.0, 73), tc)
    (ox, gx), (ob, gb), (oc, gc) = (both(oracle, cuda, x_raw, t, (rows, cols)), both(oracle, cuda, b_raw, t, (1, cols)),
                                    both(oracle, cuda, c_raw, tc, (rows, 1)))
    names = {"relu": ffi.HMC_UNARY_RELU, "exp": ffi.HMC_UNARY_EXP, "tanh": ffi.HMC_UNARY_TANH, "sigmoid": ffi.HMC_UNARY_SIGMOID,
             "silu": ffi.HMC_UNARY_SILU, "gelu": ffi.HMC_UNARY_GELU, "gelu_tanh": ffi.HMC_UNARY_GELU_TANH}
    binops = {"add": ffi.HMC_BINARY_ADD, "sub": ffi.HMC_BINARY_SUB, "mul": ffi.HMC_BINARY_MUL}
    for uname, first, second in (("silu", "mul", "add"), ("gelu_tanh", "add", "mul"), ("tanh", "sub", "sub"), ("relu", "mul", "add"),
                                 ("exp", "mul", "sub"), ("sigmoid", "add", "add"), ("gelu", "mul", "mul")):
        def steps(u, b, c):
            un = u.gelu("none") if uname == "gelu" else (u.gelu("tanh") if uname == "gelu_tanh" else getattr(u, uname)())
            return getattr(getattr(un, first)(b), second)(c)
        want_gpu = steps(gx, gb, gc)
        out = cuda.empty((rows, cols), want_gpu.dtype)
        cuda.unary_binary_binary(names[uname], binops[first], binops[second], out, gx.data, gb.data, gc.data)
        assert_bitwise(cuda.download(out), want_gpu.raw(), want_gpu.dtype, f"{uname} {first} {second}: one kernel vs three")
        # the same on x.t() (the tiled kernel with three inputs)
        gxt = T(cuda, cuda.upload(np.ascontiguousarray(x_raw.reshape(rows, cols).T), t, (cols, rows))).view(lambda d: d.t())
        cuda.unary_binary_binary(names[uname], binops[first], binops[second], out, gxt.data, gb.data, gc.data)
        assert_bitwise(cuda.download(out), want_gpu.raw(), want_gpu.dtype, f"{uname} {first} {second}: transposed x")
        if t == F32 and uname != "gelu":
            # f32 unary steps are the CPU's bits, so the whole chain is
            assert_bitwise(cuda.download(out), steps(ox, ob, oc).raw(), want_gpu.dtype, f"{uname} {first} {second}: vs the CPU's three steps")
    with pytest.raises(Exception):
        cuda.unary_binary_binary(ffi.HMC_UNARY_LOG, ffi.HMC_BINARY_ADD, ffi.HMC_BINARY_ADD, out, gx.data, gb.data, gc.data)
