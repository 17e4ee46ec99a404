"""index_check, index_select (embedding lookups) and gather against the CPU checker through the C ABI: bit for bit,
for every element size, I32 and I64 indices, negative positions, repeated positions, views and every dimension."""
import numpy as np
import pytest

from homura_b200.host import BF16, BOOL, DTYPE_NAMES, F16, F32, F64, I32, I64, U8, f32_to_half_bits
from values import assert_bitwise, values, words

pytestmark = pytest.mark.gpu


def both(oracle, cuda, raw, dtype, shape):
    return oracle.upload(raw, dtype, shape), cuda.upload(raw, dtype, shape)


def positions(n, size, seed, negative=False):
    w = words(seed, n)
    p = (w % np.uint64(size)).astype(np.int64)
    if negative:
        p = np.where((w >> np.uint64(40)) % np.uint64(3) == 0, p - size, p)
    return p


@pytest.mark.parametrize("dtype", [U8, BF16, F32, F64], ids=["u8", "bf16", "f32", "f64"])
def test_index_select_on_every_dimension(oracle, cuda, dtype):
    for shape in ((50, 64), (7, 33, 40), (1000, 136), (5, 3, 2, 16), (9,)):
        n = int(np.prod(shape))
        so, sg = both(oracle, cuda, values(dtype, n, 500), dtype, shape)
        for dim in range(len(shape)):
            for idt, m, neg in ((I64, 77, False), (I32, 5, True), (I64, 1, False)):
                p = positions(m, shape[dim], 501 + dim, neg)
                io, ig = both(oracle, cuda, p.astype(np.int32) if idt == I32 else p, idt, (m,))
                oshape = tuple(m if d == dim else s for d, s in enumerate(shape))
                oo, go = oracle.empty(oshape, dtype), cuda.empty(oshape, dtype)
                oracle.index_select(oo, so, dim, io, neg)
                cuda.index_select(go, sg, dim, ig, neg)
                assert_bitwise(cuda.download(go), oracle.download(oo), dtype, f"index_select {shape} dim {dim} m {m}")
    # an embedding table read through views: a transposed table, a strided index, an output window
    v, d_ = 300, 128
    to, tg = both(oracle, cuda, values(dtype, v * d_, 510), dtype, (d_, v))
    p = positions(64, v, 511)
    io, ig = both(oracle, cuda, np.stack([p, p[::-1]], axis=1), I64, (64, 2))
    bo, bg = oracle.empty((70, d_), dtype), cuda.empty((70, d_), dtype)
    oracle.fill(bo, 0)
    cuda.fill(bg, 0)
    oracle.index_select(bo.narrow(0, 3, 64), to.t(), 0, io.select(1, 1))
    cuda.index_select(bg.narrow(0, 3, 64), tg.t(), 0, ig.select(1, 1))
    assert_bitwise(cuda.download(bg), oracle.download(bo), dtype, "index_select through views")


@pytest.mark.parametrize("dtype", [BOOL, BF16, F32, I64], ids=["bool", "bf16", "f32", "i64"])
def test_gather_on_every_dimension(oracle, cuda, dtype):
    for shape, ishape in (((40, 50), (40, 50)), ((40, 50), (13, 7)), ((6, 9, 20), (6, 4, 20)), ((6, 9, 20), (2, 9, 3)), ((31,), (100,))):
        n = int(np.prod(shape))
        so, sg = both(oracle, cuda, values(dtype, n, 520), dtype, shape)
        for dim in range(len(shape)):
            # along `dim` the index may be longer or shorter than src; elsewhere it must not reach beyond it
            ish = tuple(ishape[d] if d == dim else min(ishape[d], shape[d]) for d in range(len(shape)))
            m = int(np.prod(ish))
            for idt in (I64, I32):
                p = positions(m, shape[dim], 521 + dim)
                io, ig = both(oracle, cuda, p.astype(np.int32) if idt == I32 else p, idt, ish)
                oo, go = oracle.empty(ish, dtype), cuda.empty(ish, dtype)
                oracle.gather(oo, so, dim, io)
                cuda.gather(go, sg, dim, ig)
                got = cuda.download(go)
                assert_bitwise(got, oracle.download(oo), dtype, f"gather {shape} index {ish} dim {dim}")
    # numpy's take_along_axis agrees where the shapes allow it
    so, sg = both(oracle, cuda, np.arange(12 * 9, dtype=np.int64), I64, (12, 9))
    p = positions(12 * 9, 9, 530).reshape(12, 9)
    _, ig = both(oracle, cuda, p, I64, (12, 9))
    go = cuda.empty((12, 9), I64)
    cuda.gather(go, sg, 1, ig)
    assert (cuda.download(go) == np.take_along_axis(np.arange(108).reshape(12, 9), p, axis=1)).all()
    # a transposed source and index
    oo, go = oracle.empty((9, 12), I64), cuda.empty((9, 12), I64)
    io, ig = both(oracle, cuda, p % 12, I64, (12, 9))
    oracle.gather(oo, so.t(), 1, io.t())
    cuda.gather(go, sg.t(), 1, ig.t())
    assert_bitwise(cuda.download(go), oracle.download(oo), I64, "gather on transposed views")


def test_index_check_reports_the_first_offender(oracle, cuda):
    n = 100003
    p = positions(n, 1000, 540)
    for idt in (I64, I32):
        raw = p.astype(np.int32) if idt == I32 else p.copy()
        io, ig = both(oracle, cuda, raw, idt, (n,))
        assert oracle.index_check(io, 0, 1000) is None and cuda.index_check(ig, 0, 1000) is None
        bad = raw.copy()
        bad[[77777, 500, 99999]] = [1000, -1001, 5000]
        io, ig = both(oracle, cuda, bad, idt, (n,))
        assert cuda.index_check(ig, 0, 1000) == oracle.index_check(io, 0, 1000) == (500, -1001)
        assert cuda.index_check(ig, -2000, 1000) == oracle.index_check(io, -2000, 1000) == (77777, 1000)
        # an exempt value (nll_loss's ignore_index) is not an offender
        assert cuda.index_check(ig, 0, 1000, exempt=-1001) == oracle.index_check(io, 0, 1000, exempt=-1001) == (77777, 1000)
    # row-major order of the logical positions of a view
    grid = np.zeros((50, 60), dtype=np.int64)
    grid[3, 59] = grid[40, 2] = 99
    io, ig = both(oracle, cuda, grid, I64, (50, 60))
    assert cuda.index_check(ig.t(), 0, 10) == oracle.index_check(io.t(), 0, 10) == (2 * 50 + 40, 99)
    assert cuda.index_check(ig, 0, 10) == oracle.index_check(io, 0, 10) == (3 * 60 + 59, 99)


@pytest.mark.parametrize("dtype", [U8, BF16, F32, F64], ids=["u8", "bf16", "f32", "f64"])
def test_index_overwrite_last_position_wins(oracle, cuda, dtype):
    for shape, dim, size in (((300, 40), 0, 100), ((7, 300, 5), 1, 64), ((5, 9), 1, 9), ((2000,), 0, 50), ((3, 4), 0, 10)):
        m = shape[dim]
        n = int(np.prod(shape))
        so, sg = both(oracle, cuda, values(dtype, n, 550), dtype, shape)
        p = positions(m, size, 551)  # m > size in most cases: many repeated positions
        po, pg = both(oracle, cuda, p, I64, (m,))
        oshape = tuple(size if d == dim else s for d, s in enumerate(shape))
        base = values(dtype, int(np.prod(oshape)), 552)
        oo, go = both(oracle, cuda, base, dtype, oshape)
        oracle.index_overwrite(oo, dim, po, so)
        cuda.index_overwrite(go, dim, pg, sg)
        assert_bitwise(cuda.download(go), oracle.download(oo), dtype, f"index_overwrite {shape} dim {dim} into {size}")
    # numpy agrees: assignment with repeated indices keeps the last
    src = np.arange(20 * 3, dtype=np.int64).reshape(20, 3)
    p = positions(20, 6, 553)
    want = np.full((6, 3), -1, dtype=np.int64)
    want[p] = src
    out = cuda.upload(np.full((6, 3), -1, dtype=np.int64), I64)
    cuda.index_overwrite(out, 0, cuda.upload(p, I64), cuda.upload(src, I64))
    assert (cuda.download(out) == want).all()


def test_mask_coordinates_are_nonzero_transposed(oracle, cuda):
    for shape in ((1000,), (37, 53), (5, 6, 70), (2, 3, 4, 5), (70000,)):
        n = int(np.prod(shape))
        for density in (0, 1, 3, 50):
            w = words(560 + density, n)
            raw = np.ones(n, dtype=np.uint8) if density == 0 else ((w % np.uint64(density)) == 0).astype(np.uint8)
            if density == 50:
                raw[:] = 0 if n > 5000 else raw  # an empty result for the long shapes
            mo, mg = both(oracle, cuda, raw, BOOL, shape)
            want, got = oracle.mask_coordinates(mo), cuda.mask_coordinates(mg)
            assert len(want) == len(got) == len(shape)
            nz = np.nonzero(raw.reshape(shape))
            for d in range(len(shape)):
                g = cuda.download(got[d])
                assert (g == oracle.download(want[d])).all() and (g == nz[d]).all(), f"coordinates {shape} density {density} dim {d}"
    # a transposed mask: coordinates follow the view's own row-major order
    raw = ((words(570, 40 * 90) % np.uint64(4)) == 0).astype(np.uint8)
    mo, mg = both(oracle, cuda, raw, BOOL, (40, 90))
    want, got = oracle.mask_coordinates(mo.t()), cuda.mask_coordinates(mg.t())
    nz = np.nonzero(raw.reshape(40, 90).T)
    for d in range(2):
        assert (cuda.download(got[d]) == oracle.download(want[d])).all() and (cuda.download(got[d]) == nz[d]).all()


ADD_DTYPES = [BOOL, U8, I32, I64, F16, BF16, F32, F64]


def small_values(dtype, n, seed):
    """Values whose sums stay finite in every dtype (floats of mixed magnitude, so that the order of an f64 sum shows)."""
    w = words(seed, n)
    if dtype in (F16, BF16, F32, F64):
        f = ((w % np.uint64(2001)).astype(np.float64) - 1000.0) / 8.0 * (10.0 ** ((w >> np.uint64(20)) % np.uint64(7)).astype(np.float64)) / 1000.0
        if dtype == F64:
            return f
        f32 = f.astype(np.float32)
        return f32 if dtype == F32 else f32_to_half_bits(f32, dtype)
    return values(dtype, n, seed)


@pytest.mark.parametrize("dtype", ADD_DTYPES, ids=lambda d: f"dt{d}")
def test_index_add_sums_in_the_order_of_the_positions(oracle, cuda, dtype):
    for shape, dim, size in (((500, 33), 0, 40), ((6, 700, 5), 1, 90), ((9, 300), 1, 7), ((5000,), 0, 300), ((3, 4), 0, 10),
                             ((2100, 8), 0, 1)):
        m = shape[dim]
        so, sg = both(oracle, cuda, small_values(dtype, int(np.prod(shape)), 600), dtype, shape)
        p = positions(m, size, 601)
        p[::7] -= size  # negative positions count from the end
        po, pg = both(oracle, cuda, p, I64, (m,))
        oshape = tuple(size if d == dim else s for d, s in enumerate(shape))
        base = small_values(dtype, int(np.prod(oshape)), 602)
        oo, go = both(oracle, cuda, base, dtype, oshape)
        oracle.index_add(oo, dim, po, so)
        cuda.index_add(go, dim, pg, sg)
        assert_bitwise(cuda.download(go), oracle.download(oo), dtype, f"index_add {shape} dim {dim} into {size}")


def test_index_add_of_a_view_and_against_numpy(oracle, cuda):
    src = (words(610, 64 * 48) % np.uint64(1000)).astype(np.int64).reshape(64, 48)
    p = positions(48, 20, 611)
    so, sg = both(oracle, cuda, src, I64, (64, 48))
    po, pg = both(oracle, cuda, p, I64, (48,))
    oo, go = both(oracle, cuda, np.zeros((20, 64), dtype=np.int64), I64, (20, 64))
    oracle.index_add(oo, 0, po, so.t())
    cuda.index_add(go, 0, pg, sg.t())
    want = np.zeros((20, 64), dtype=np.int64)
    np.add.at(want, p, src.T)
    assert (cuda.download(go) == want).all() and (oracle.download(oo) == want).all()


@pytest.mark.parametrize("dtype", ADD_DTYPES, ids=lambda d: f"dt{d}")
def test_scatter_add_sums_in_row_major_order(oracle, cuda, dtype):
    for ishape, sshape, oshape, dim in (((300, 40), (300, 40), (9, 40), 0), ((50, 600), (64, 700), (50, 13), 1),
                                        ((4, 90, 6), (4, 90, 6), (5, 3, 7), 1), ((7000,), (7000,), (100,), 0),
                                        ((3, 4), (3, 4), (8, 4), 0)):
        so, sg = both(oracle, cuda, small_values(dtype, int(np.prod(sshape)), 620), dtype, sshape)
        idx = positions(int(np.prod(ishape)), oshape[dim], 621)
        io, ig = both(oracle, cuda, idx, I64, ishape)
        base = small_values(dtype, int(np.prod(oshape)), 622)
        oo, go = both(oracle, cuda, base, dtype, oshape)
        oracle.scatter_add(oo, dim, io, so)
        cuda.scatter_add(go, dim, ig, sg)
        assert_bitwise(cuda.download(go), oracle.download(oo), dtype, f"scatter_add {ishape} of {sshape} into {oshape} dim {dim}")
    # numpy agrees for integers
    src = (words(630, 30 * 20) % np.uint64(100)).astype(np.int64).reshape(30, 20)
    idx = positions(30 * 20, 11, 631).reshape(30, 20)
    out = cuda.upload(np.zeros((11, 20), dtype=np.int64), I64)
    cuda.scatter_add(out, 0, cuda.upload(idx, I64), cuda.upload(src, I64))
    want = np.zeros((11, 20), dtype=np.int64)
    np.add.at(want, (idx, np.arange(20)[None, :].repeat(30, 0)), src)
    assert (cuda.download(out) == want).all()


def test_index_positions_of_broadcast_indices(oracle, cuda):
    sizes = (7, 11, 5)
    rows = positions(6, 7, 640).reshape(6, 1) - 7 * (np.arange(6).reshape(6, 1) % 2)  # some negative
    cols = positions(9, 11, 641).reshape(1, 9)
    deep = positions(54, 5, 642).reshape(6, 9)
    got, want = [], []
    for be, sink in ((oracle, want), (cuda, got)):
        out = be.empty((6, 9), I64)
        be.index_positions(out, [be.upload(rows, I64), be.upload(cols, I64), be.upload(deep, I64)], sizes)
        sink.append(be.download(out))
    expect = np.ravel_multi_index((np.broadcast_to(rows % 7, (6, 9)), np.broadcast_to(cols, (6, 9)), deep), sizes)
    assert (got[0] == want[0]).all() and (got[0] == expect).all()


def test_index_add_with_many_tiles_and_three_sort_passes(oracle, cuda):
    m, size = 300_000, 100_000  # 17 bits of position: three passes of eight bits; 293 tiles of 1024 keys
    so, sg = both(oracle, cuda, small_values(F32, m * 2, 650), F32, (m, 2))
    p = positions(m, size, 651)
    p[: m // 3] = 77  # one long run
    po, pg = both(oracle, cuda, p, I64, (m,))
    base = small_values(F32, size * 2, 652)
    oo, go = both(oracle, cuda, base, F32, (size, 2))
    oracle.index_add(oo, 0, po, so)
    cuda.index_add(go, 0, pg, sg)
    assert_bitwise(cuda.download(go), oracle.download(oo), F32, "index_add of 300000 slices into 100000")


def test_add_family_with_targets_beyond_32_bits(cuda):
    """An output of more than 2^32 elements: the sort runs on 64-bit keys (five passes for index_add's 33 bits)."""
    size = (1 << 32) + 4096
    out = cuda.empty((size,), U8)
    cuda.fill(out, 7)
    w = words(660, 3000)
    p = (w % np.uint64(size)).astype(np.int64)
    p[:500] = p[500:1000]            # repeated targets
    p[1000:1010] = size - 1           # the last element, ten times
    src = (words(661, 3000) % np.uint64(200)).astype(np.uint8)
    want = {}
    for j, v in zip(p.tolist(), src.tolist()):
        want[j] = want.get(j, 7) + v
    targets = np.array(sorted(want), dtype=np.int64)
    expect = np.array([want[j] & 255 for j in targets.tolist()], dtype=np.uint8)
    pg, sg, tg = cuda.upload(p, I64), cuda.upload(src, U8), cuda.upload(targets, I64)
    got = cuda.empty((len(targets),), U8)

    cuda.index_add(out, 0, pg, sg)
    cuda.gather(got, out, 0, tg)
    assert (cuda.download(got) == expect).all(), "index_add into 2^32 + 4096 elements"
    neighbours = cuda.upload(np.array([0, 1, size - 2], dtype=np.int64)[~np.isin([0, 1, size - 2], targets)], I64)
    seen = cuda.empty((neighbours.numel,), U8)
    if neighbours.numel:
        cuda.gather(seen, out, 0, neighbours)
        assert (cuda.download(seen) == 7).all(), "elements no position names keep their value"

    cuda.fill(out, 7)
    cuda.scatter_add(out, 0, pg, sg)
    cuda.gather(got, out, 0, tg)
    assert (cuda.download(got) == expect).all(), "scatter_add into 2^32 + 4096 elements"


def test_index_value_at_a_position_beyond_any_testable_check(cuda):
    """The second step of index_check alone: the value at logical position 2^60 + 5 of a view with a zero stride."""
    import ctypes
    from homura_b200.ffi import hmc_tensor_desc
    base = cuda.upload(np.arange(100, 164, dtype=np.int64), I64)
    d = hmc_tensor_desc()
    d.data, d.offset, d.dtype, d.ndim = base.storage.ptr, 0, I64, 2
    d.sizes[0], d.strides[0] = 1 << 56, 0
    d.sizes[1], d.strides[1] = 64, 1
    slot = cuda.upload(np.array([(1 << 60) + 5, 0], dtype=np.uint64).view(np.int64), I64)
    cuda._check(cuda.lib.hmc_test_index_value(cuda.ctx, d, ctypes.cast(slot.storage.ptr, ctypes.POINTER(ctypes.c_uint64))))
    assert cuda.download(slot).tolist() == [(1 << 60) + 5, 105]
    # UINT64_MAX: nothing was found, nothing is written
    slot = cuda.upload(np.array([-1, 42], dtype=np.int64), I64)
    cuda._check(cuda.lib.hmc_test_index_value(cuda.ctx, d, ctypes.cast(slot.storage.ptr, ctypes.POINTER(ctypes.c_uint64))))
    assert cuda.download(slot).tolist() == [-1, 42]
