"""Properties that do not depend on a CPU run, checked at the full sizes of the benchmark configurations (where the
CPU checker would take minutes): identities that must hold bit for bit between different kernels of the library
(the tiled kernel against the contiguous one, a one-pass reduction against its parts), round trips, and exact
integer totals; plus tensors of more than 2^31 elements, which take the 64-bit index paths."""
import ctypes

import numpy as np
import pytest

from homura_b200 import ffi
from homura_b200.host import BF16, BOOL, F32, F64, I16, I32, I64, U8, Generator, TensorData

pytestmark = pytest.mark.gpu


def equal_bits(cuda, a, b):
    """Every element of two same-shaped tensors has the same bits (compared on the device: NOT_EQUAL of the integer
    views of the storage, then ANY)."""
    es = {BF16: 2, F32: 4, F64: 8, I64: 8, I32: 4, U8: 1, BOOL: 1}[a.dtype]
    as_int = {1: U8, 2: I16, 4: I32, 8: I64}[es]
    ia = TensorData(a.storage, as_int, a.shape, a.strides, a.offset)
    ib = TensorData(b.storage, as_int, b.shape, b.strides, b.offset)
    ne = cuda.empty(a.shape, BOOL)
    cuda.binary(ffi.HMC_BINARY_NOT_EQUAL, ne, ia, ib)
    out = cuda.empty((), BOOL)
    cuda.reduce(ffi.HMC_REDUCE_ANY, out, ne, [True] * len(a.shape))
    return not bool(cuda.download(out))


def test_c2_step_identities_at_8192x8192(cuda):
    n = 8192
    x = cuda.empty((n * n,), BF16)
    cuda.random_normal(x, Generator(2), 0.0, 1.0)
    x = x.reshape(n, n)
    # the tiled kernel (silu of x.t()) against the contiguous kernel followed by a transposing copy
    a, b, s = cuda.empty((n, n), BF16), cuda.empty((n, n), BF16), cuda.empty((n, n), BF16)
    cuda.unary(ffi.HMC_UNARY_SILU, a, x.t())
    cuda.unary(ffi.HMC_UNARY_SILU, s, x)
    cuda.copy(b, s.t())
    assert equal_bits(cuda, a, b), "silu(x.t()) differs from silu(x).t()"
    # bf16 -> f32 -> bf16 is the identity; a transposed cast equals the cast of the transposed copy
    f, back = cuda.empty((n, n), F32), cuda.empty((n, n), BF16)
    cuda.copy(f, x)
    cuda.copy(back, f)
    assert equal_bits(cuda, back, x), "bf16 -> f32 -> bf16 changed bits"
    ft, ft2 = cuda.empty((n, n), F32), cuda.empty((n, n), F32)
    cuda.copy(ft, x.t())
    cuda.copy(ft2, f.t())
    assert equal_bits(cuda, ft, ft2), "cast of x.t() differs from the transposed cast"
    # the promoting add (bf16 + f32 [N, 1] -> f32) against cast-then-add
    bias = cuda.empty((n,), F32)
    cuda.random_normal(bias, Generator(3), 0.0, 1.0)
    col = bias.reshape(n, 1).expand(n, n)
    y, y2 = cuda.empty((n, n), F32), cuda.empty((n, n), F32)
    cuda.binary_promoted(ffi.HMC_BINARY_ADD, y, x, col)
    cuda.binary(ffi.HMC_BINARY_ADD, y2, f, col)
    assert equal_bits(cuda, y, y2), "promoting add differs from cast + add"
    # x * 1 = x, -(-x) = x
    one = cuda.empty((1, n), BF16)
    cuda.fill(one, 1.0)
    cuda.binary(ffi.HMC_BINARY_MUL, a, x, one.expand(n, n))
    assert equal_bits(cuda, a, x), "x * 1 changed bits"
    cuda.unary(ffi.HMC_UNARY_NEG, a, x)
    cuda.unary(ffi.HMC_UNARY_NEG, b, a)
    assert equal_bits(cuda, b, x), "-(-x) changed bits"


def test_c3_reduction_identities_at_16384x4096(cuda):
    r, c = 16384, 4096
    i = cuda.empty((r * c,), I64)
    cuda.random_int(i, Generator(4), -1000, 1001)
    x = cuda.empty((r, c), I32)
    cuda.copy(x, i.reshape(r, c))
    # integer sums are exact: total = sum of the row sums = sum of the column sums
    rows, cols, total, t2, t3 = cuda.empty((r,), I64), cuda.empty((c,), I64), cuda.empty((), I64), cuda.empty((), I64), cuda.empty((), I64)
    cuda.reduce(ffi.HMC_REDUCE_SUM, rows, x, [False, True])
    cuda.reduce(ffi.HMC_REDUCE_SUM, cols, x, [True, False])
    cuda.reduce(ffi.HMC_REDUCE_SUM, total, x, [True, True])
    cuda.reduce(ffi.HMC_REDUCE_SUM, t2, rows, [True])
    cuda.reduce(ffi.HMC_REDUCE_SUM, t3, cols, [True])
    assert int(cuda.download(total)) == int(cuda.download(t2)) == int(cuda.download(t3))
    # the maximum of the row maxima is the maximum; the row argmax points at a maximum (gathered on the host for a sample)
    xf = cuda.empty((r, c), F32)
    cuda.copy(xf, x)
    rmax, ridx, gmax, g2 = cuda.empty((r,), F32), cuda.empty((r,), I64), cuda.empty((), F32), cuda.empty((), F32)
    cuda.arg_reduce(rmax, ridx, xf, 1, True)
    cuda.reduce(ffi.HMC_REDUCE_MAX, gmax, xf, [True, True])
    cuda.reduce(ffi.HMC_REDUCE_MAX, g2, rmax, [True])
    assert float(cuda.download(gmax)) == float(cuda.download(g2)) == 1000.0
    idx, mx = cuda.download(ridx), cuda.download(rmax)
    for row in (0, 1, r // 2, r - 1):
        line = cuda.download(xf.narrow(0, row, 1)).reshape(-1)
        assert line[idx[row]] == mx[row] == line.max() and idx[row] == int(np.argmax(line))
    # var over rows (one pass) against its definition from two reductions, and the same over columns
    for mask, shape in (([False, True], (r,)), ([True, False], (c,))):
        v, m, sq = cuda.empty(shape, F32), cuda.empty(shape, F32), cuda.empty(shape, F32)
        cuda.var(v, xf, mask, 0, False)
        cuda.reduce(ffi.HMC_REDUCE_MEAN, m, xf, mask)
        x2 = cuda.empty((r, c), F32)
        cuda.binary(ffi.HMC_BINARY_MUL, x2, xf, xf)
        cuda.reduce(ffi.HMC_REDUCE_MEAN, sq, x2, mask)
        got = cuda.download(v).astype(np.float64)
        want = cuda.download(sq).astype(np.float64) - cuda.download(m).astype(np.float64) ** 2
        assert np.allclose(got, want, rtol=1e-4), "var differs from E[x^2] - E[x]^2"


def test_c4_softmax_properties_at_2048_rows(cuda):
    b, n = 64, 2048
    x = cuda.empty((b * n * n,), F32)
    cuda.random_normal(x, Generator(5), 0.0, 3.0)
    x = x.reshape(b, n, n)
    ones = cuda.empty((n, n), BOOL)
    cuda.fill(ones, True)
    mask = cuda.empty((n, n), BOOL)
    cuda.triangle(mask, ones, 1, True)
    cuda.where_constant(x, mask.reshape(1, n, n).expand(b, n, n), float("-inf"), x)
    s, ls, e = cuda.empty((b, n, n), F32), cuda.empty((b, n, n), F32), cuda.empty((b, n, n), F32)
    cuda.softmax(s, x, 2, False)
    cuda.softmax(ls, x, 2, True)
    # rows sum to 1, masked entries are exactly 0, exp(log_softmax) = softmax to the last places
    sums = cuda.empty((b, n), F32)
    cuda.reduce(ffi.HMC_REDUCE_SUM, sums, s, [False, False, True])
    assert np.abs(cuda.download(sums).astype(np.float64) - 1.0).max() < 1e-5
    upper = cuda.empty((b, n, n), F32)
    cuda.triangle(upper, s, 1, True)
    top = cuda.empty((), F32)
    cuda.reduce(ffi.HMC_REDUCE_MAX, top, upper, [True, True, True])
    assert float(cuda.download(top)) == 0.0, "a masked logit got a nonzero probability"
    cuda.unary(ffi.HMC_UNARY_EXP, e, ls)
    d = cuda.empty((b, n, n), F32)
    cuda.binary(ffi.HMC_BINARY_SUB, d, e, s)
    cuda.unary(ffi.HMC_UNARY_ABS, d, d)
    worst = cuda.empty((), F32)
    cuda.reduce(ffi.HMC_REDUCE_MAX, worst, d, [True, True, True])
    assert float(cuda.download(worst)) < 2e-6


def test_more_than_2_to_the_31_elements(cuda):
    n = (1 << 31) + 1000
    a, b = cuda.empty((n,), U8), cuda.empty((n,), U8)
    cuda.fill(a, 3)
    cuda.binary(ffi.HMC_BINARY_ADD, b, a, a)
    total, top = cuda.empty((), I64), cuda.empty((), U8)
    cuda.reduce(ffi.HMC_REDUCE_SUM, total, b, [True])
    cuda.reduce(ffi.HMC_REDUCE_MAX, top, b, [True])
    assert int(cuda.download(total)) == 6 * n and int(cuda.download(top)) == 6
    assert (cuda.download(b.narrow(0, n - 5000, 5000)) == 6).all()
    # a mark near the end: argmax finds it with its 64-bit index; a [2, n/2] view folds over rows longer than 2^30
    cuda.fill(b.narrow(0, n - 7, 1), 9)
    v, i = cuda.empty((), U8), cuda.empty((), I64)
    cuda.arg_reduce(v, i, b, 0, True)
    assert int(cuda.download(v)) == 9 and int(cuda.download(i)) == n - 7
    half = n // 2
    two = b.narrow(0, 0, 2 * half).reshape(2, half)
    sums = cuda.empty((2,), I64)
    cuda.reduce(ffi.HMC_REDUCE_SUM, sums, two, [False, True])
    got = cuda.download(sums)
    assert got[0] == 6 * half and got[1] == 6 * half + 3
    # a strided walk over the long tensor: every second element, copied and summed
    odd = cuda.empty((half,), U8)
    cuda.copy(odd, b.narrow(0, 0, 2 * half).reshape(half, 2).select(1, 1))
    cuda.reduce(ffi.HMC_REDUCE_SUM, total, odd, [True])
    assert int(cuda.download(total)) == 6 * half + (3 if (n - 7) % 2 == 1 and n - 7 < 2 * half else 0)
