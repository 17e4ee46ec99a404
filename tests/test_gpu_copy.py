"""Casts, strided copies and fills against the CPU checker, after homura's tests/rocm_copy.rs: all 100 dtype
pairs on every layout with special values (NaN payloads, values next to rounding ties, out-of-range floats)
and random bit patterns, bit for bit; the half-type roundings on millions of patterns."""
import numpy as np
import pytest

from frontend import T
from gpu_common import both, pairs, same
from homura_b200.host import ALL_DTYPES, BF16, BOOL, DTYPE_NAMES, F16, F32, F64, I64, STORAGE
from values import assert_bitwise, assert_same, special_f64, values, words

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("src", ALL_DTYPES, ids=DTYPE_NAMES)
def test_every_cast_on_every_layout(oracle, cuda, src):
    for name, o, g in pairs(oracle, cuda, src, 71):
        for dst in ALL_DTYPES:
            same(lambda t: t.to(dst) if dst != src else t.contiguous(), o, g, f"{DTYPE_NAMES[src]}->{DTYPE_NAMES[dst]} {name}")


def test_nan_payloads_convert_like_the_cpu(oracle, cuda):
    bits = np.array([0x7FF0000000000001, 0xFFF4000000001234, 0x7FF8000020000000, 0x7FF8000000000000, 0xFFF8000000000000,
                     0x7FF7FFFFFFFFFFFF], dtype=np.uint64).view(np.float64)
    o, g = both(oracle, cuda, bits, F64)
    for dst in (F32, F16, BF16):
        assert_same(g.to(dst).raw(), o.to(dst).raw(), dst, f"f64 NaN -> {DTYPE_NAMES[dst]}")
    f32 = np.array([0x7F800001, 0xFFC01234, 0x7FFFFFFF, 0x7FA00000], dtype=np.uint32).view(np.float32)
    o, g = both(oracle, cuda, f32, F32)
    for dst in (F64, F16, BF16):
        assert_same(g.to(dst).raw(), o.to(dst).raw(), dst, f"f32 NaN -> {DTYPE_NAMES[dst]}")


def test_half_roundings_on_many_patterns(oracle, cuda):
    pats = words(81, 1 << 22).astype(np.uint32).view(np.float32)
    o, g = both(oracle, cuda, pats, F32)
    for dst in (F16, BF16):
        assert_same(g.to(dst).raw(), o.to(dst).raw(), dst, f"f32 -> {DTYPE_NAMES[dst]} on 2^22 patterns")
    every = np.arange(1 << 16, dtype=np.uint16)
    for src in (F16, BF16):
        o, g = both(oracle, cuda, every, src)
        for dst in (F32, F64, F16 if src == BF16 else BF16, I64, BOOL):
            assert_same(g.to(dst).raw(), o.to(dst).raw(), dst, f"every {DTYPE_NAMES[src]} -> {DTYPE_NAMES[dst]}")
    d = words(82, 1 << 20).view(np.float64)
    o, g = both(oracle, cuda, d, F64)
    for dst in (F32, F16, BF16, I64):
        assert_same(g.to(dst).raw(), o.to(dst).raw(), dst, f"f64 patterns -> {DTYPE_NAMES[dst]}")


@pytest.mark.parametrize("dtype", ALL_DTYPES, ids=DTYPE_NAMES)
def test_fill_and_copy_into_views(oracle, cuda, dtype):
    raw = values(dtype, 40 * 50, 91)
    value = True if dtype == BOOL else 3
    outs = []
    for be in (oracle, cuda):
        base = be.upload(raw, dtype, (40, 50))
        be.fill(base.narrow(0, 3, 10).narrow(1, 7, 20), value)       # a window
        be.fill(base.t().narrow(0, 40, 5), value)                    # columns of the transposed view
        src = be.upload(values(dtype, 50, 92), dtype)
        be.copy(base.narrow(0, 30, 4), src)                          # broadcast rows into a view
        be.copy(base.t().narrow(0, 0, 3), base.t().narrow(0, 10, 3))  # strided to strided
        outs.append(be.download(base))
    assert_bitwise(outs[1], outs[0], dtype, "fill / copy into views")
