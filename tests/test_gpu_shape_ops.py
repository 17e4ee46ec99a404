"""triangle (tril / triu) and flip against the CPU checker through the C ABI, bit for bit, on contiguous tensors and
on views (transposed, windows that break the 16-byte alignment, batches with their own strides)."""
import numpy as np
import pytest

from homura_b200.host import ALL_DTYPES, BF16, BOOL, DTYPE_NAMES, F32, F64, I64, U8
from values import assert_bitwise, values

pytestmark = pytest.mark.gpu


def both(oracle, cuda, raw, dtype, shape):
    return oracle.upload(raw, dtype, shape), cuda.upload(raw, dtype, shape)


@pytest.mark.parametrize("dtype", [BOOL, BF16, F32, I64], ids=["bool", "bf16", "f32", "i64"])
def test_triangle_on_every_layout(oracle, cuda, dtype):
    shapes = [(5, 7), (64, 64), (1, 9), (9, 1), (130, 70), (3, 2, 33, 260), (2, 257, 300), (2, 3, 40, 96), (1, 3, 1056)]
    for shape in shapes:
        n = int(np.prod(shape))
        (os_, gs) = both(oracle, cuda, values(dtype, n, 400), dtype, shape)
        for diagonal in (-300, -3, -1, 0, 1, 5, 64, 300):
            for upper in (False, True):
                oo, go = oracle.empty(shape, dtype), cuda.empty(shape, dtype)
                oracle.triangle(oo, os_, diagonal, upper)
                cuda.triangle(go, gs, diagonal, upper)
                assert_bitwise(cuda.download(go), oracle.download(oo), dtype, f"triangle {shape} k={diagonal} upper={upper}")
    # views: the matrix transposed, a misaligned window, an output with gaps between rows
    (os_, gs) = both(oracle, cuda, values(dtype, 200 * 300, 401), dtype, (200, 300))
    views = [lambda d: d.t(), lambda d: d.narrow(1, 3, 250).narrow(0, 1, 190), lambda d: d.narrow(1, 0, 128)]
    for k, view in enumerate(views):
        so, sg = view(os_), view(gs)
        oo, go = oracle.empty(so.shape, dtype), cuda.empty(sg.shape, dtype)
        oracle.triangle(oo, so, 2, True)
        cuda.triangle(go, sg, 2, True)
        assert_bitwise(cuda.download(go), oracle.download(oo), dtype, f"triu of view {k}")
        # in place on the view (out is src): tril keeps and zeroes in one pass
        oracle.triangle(so, so, -1, False)
        cuda.triangle(sg, sg, -1, False)
        assert_bitwise(cuda.download(gs), oracle.download(os_), dtype, f"tril in place on view {k}")


def test_the_causal_mask_of_c4(oracle, cuda):
    n = 2048
    ones_o, ones_g = both(oracle, cuda, np.ones(n * n, dtype=np.uint8), BOOL, (n, n))
    mo, mg = oracle.empty((n, n), BOOL), cuda.empty((n, n), BOOL)
    oracle.triangle(mo, ones_o, 1, True)
    cuda.triangle(mg, ones_g, 1, True)
    got = cuda.download(mg)
    assert (got == oracle.download(mo)).all() and (got == np.triu(np.ones((n, n), dtype=np.uint8), 1)).all()


@pytest.mark.parametrize("dtype", [U8, BF16, F32, F64], ids=["u8", "bf16", "f32", "f64"])
def test_flip_on_every_layout(oracle, cuda, dtype):
    cases = [((7,), [0]), ((5, 9), [0]), ((5, 9), [1]), ((5, 9), [0, 1]), ((3, 4, 5), [1]), ((3, 4, 5), [0, 2]),
             ((2, 300, 70), [1, 2]), ((1000, 260), [0]), ((1000, 260), [1]), ((4, 4), [])]
    for shape, dims in cases:
        n = int(np.prod(shape))
        (os_, gs) = both(oracle, cuda, values(dtype, n, 410), dtype, shape)
        oo, go = oracle.empty(shape, dtype), cuda.empty(shape, dtype)
        oracle.flip(oo, os_, dims)
        cuda.flip(go, gs, dims)
        got = cuda.download(go)
        assert_bitwise(got, oracle.download(oo), dtype, f"flip {shape} along {dims}")
        assert (got == np.flip(cuda.download(gs), axis=tuple(dims))).all() or dtype in (BF16, F32, F64)
    # a flipped transposed window
    (os_, gs) = both(oracle, cuda, values(dtype, 120 * 90, 411), dtype, (120, 90))
    view = lambda d: d.t().narrow(0, 2, 80)
    oo, go = oracle.empty((80, 120), dtype), cuda.empty((80, 120), dtype)
    oracle.flip(oo, view(os_), [0, 1])
    cuda.flip(go, view(gs), [0, 1])
    assert_bitwise(cuda.download(go), oracle.download(oo), dtype, "flip of a transposed window")


@pytest.mark.parametrize("dtype", ALL_DTYPES, ids=DTYPE_NAMES)
def test_addr_on_every_dtype(oracle, cuda, dtype):
    """out = beta * input + alpha * outer(v1, v2), every rounding where the CPU kernel has it: bit for bit."""
    floats = dtype in (BF16, F32, F64) or DTYPE_NAMES[dtype] == "f16"
    for n, m in ((1, 1), (7, 5), (130, 257), (1000, 520)):
        v1o, v1g = both(oracle, cuda, values(dtype, n, 420), dtype, (n,))
        v2o, v2g = both(oracle, cuda, values(dtype, m, 421), dtype, (m,))
        ino, ing = both(oracle, cuda, values(dtype, n * m, 422), dtype, (n, m))
        coefficients = [(1, 1), (1, 0), (0.5, 2.0), (-3, 0), (2, 1)] if floats else [(1, 1), (1, 0), (3, -2), (0, 1), (-1, 0)]
        for alpha, beta in coefficients:
            oo, go = oracle.empty((n, m), dtype), cuda.empty((n, m), dtype)
            oracle.addr(oo, v1o, v2o, ino, alpha, beta)
            cuda.addr(go, v1g, v2g, ing, alpha, beta)
            assert_bitwise(cuda.download(go), oracle.download(oo), dtype, f"addr [{n}, {m}] alpha={alpha} beta={beta}")
    # strided vectors, a broadcast input (a row [m] and a single element), and a transposed input
    n, m = 300, 260
    bigo, bigg = both(oracle, cuda, values(dtype, 2 * n + 3 * m + n * m, 423), dtype, (2 * n + 3 * m + n * m,))
    cut = lambda t: (t.narrow(0, 0, 2 * n).reshape(n, 2).select(1, 1), t.narrow(0, 2 * n, 3 * m).reshape(m, 3).select(1, 0),
                     t.narrow(0, 2 * n + 3 * m, n * m).reshape(m, n).t())
    for inp in (lambda v1, v2, c: c, lambda v1, v2, c: v2, lambda v1, v2, c: v1.narrow(0, 2, 1)):
        oo, go = oracle.empty((n, m), dtype), cuda.empty((n, m), dtype)
        a1, a2, ac = cut(bigo)
        b1, b2, bc = cut(bigg)
        oracle.addr(oo, a1, a2, inp(a1, a2, ac), 1, 1)
        cuda.addr(go, b1, b2, inp(b1, b2, bc), 1, 1)
        assert_bitwise(cuda.download(go), oracle.download(oo), dtype, "addr on strided vectors and a broadcast input")


@pytest.mark.parametrize("dtype", [BF16, F32, F64], ids=["bf16", "f32", "f64"])
def test_exclusive_cumprod(oracle, cuda, dtype):
    """The sequential product in the accumulation type (f32 for the half dtypes, f64 otherwise): bit for bit."""
    from values import f64_to_storage, words
    for shape in ((1,), (9,), (5, 300), (300, 5), (3, 40, 7), (2, 1025)):
        n = int(np.prod(shape))
        w = words(430, n)
        near_one = 0.5 + (w >> np.uint64(11)).astype(np.float64) / float(1 << 53) * 1.5   # products neither vanish nor overflow
        raw = f64_to_storage(np.where(w % np.uint64(97) == 0, -near_one, near_one), dtype)
        so, sg = both(oracle, cuda, raw, dtype, shape)
        for dim in range(len(shape)):
            for reverse in (False, True):
                oo, go = oracle.empty(shape, dtype), cuda.empty(shape, dtype)
                oracle.exclusive_cumprod(oo, so, dim, reverse)
                cuda.exclusive_cumprod(go, sg, dim, reverse)
                assert_bitwise(cuda.download(go), oracle.download(oo), dtype, f"exclusive_cumprod {shape} dim {dim} reverse {reverse}")
    # special values and a transposed source
    so, sg = both(oracle, cuda, values(dtype, 64 * 33, 431), dtype, (64, 33))
    oo, go = oracle.empty((33, 64), dtype), cuda.empty((33, 64), dtype)
    oracle.exclusive_cumprod(oo, so.t(), 1, False)
    cuda.exclusive_cumprod(go, sg.t(), 1, False)
    assert_bitwise(cuda.download(go), oracle.download(oo), dtype, "exclusive_cumprod of special values, transposed")
