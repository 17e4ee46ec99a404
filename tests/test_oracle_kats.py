"""Known-answer tests that live in homura's sources, replayed on the CPU checker: the cast table and the
half-type rounding rules (src/dtype.rs:606-665), erf and integer powers (src/backend/cpu/num.rs:225-257), the
order of strided visits (src/backend/cpu/iter.rs:106-123) and the promotion tables (src/dtype.rs:543-604)."""
import math

import numpy as np
import pytest

from frontend import T, promote_types, result_type
from homura_b200.host import (ALL_DTYPES, BF16, BOOL, F16, F32, F64, I8, I16, I32, I64, STORAGE, U8, TensorData,
                              half_bits_to_f32)
from values import f64_to_storage, storage_to_f64


def cast(oracle, value, src, dst):
    raw = np.array([value], dtype=STORAGE[src]) if src not in (F16, BF16) else f64_to_storage([value], src)
    out = T(oracle, oracle.upload(raw, src)).to(dst).raw()
    return out[0]


def test_element_cast(oracle):
    assert cast(oracle, -1.7, F32, I32) == -1
    assert cast(oracle, 300, I64, U8) == 44
    assert cast(oracle, 300.0, F32, U8) == 44
    assert cast(oracle, -1.0, F64, U8) == 255
    assert cast(oracle, -129.9, F32, I8) == 127
    assert cast(oracle, -2.5, F16, U8) == 254
    assert cast(oracle, math.nan, F64, I32) == 0
    assert cast(oracle, math.inf, F64, I64) == 2**63 - 1
    assert cast(oracle, math.inf, F64, I32) == -1
    assert cast(oracle, 1e30, F32, I16) == -1
    assert cast(oracle, 0.1, F64, BOOL) == 1
    assert cast(oracle, 1, BOOL, F16) == 0x3C00
    assert cast(oracle, 2.5, F16, F32) == 2.5


def test_half_casts_round_through_f32(oracle):
    p = lambda e: 2.0 ** e
    assert cast(oracle, np.float32(1.0 + p(-8) + p(-21)), F32, BF16) == 0x3F81
    assert cast(oracle, 1.0 + p(-8) + p(-21), F64, BF16) == 0x3F81
    assert cast(oracle, 1.0 + p(-8) + p(-40), F64, BF16) == 0x3F80
    assert cast(oracle, 1.0 + p(-11) + p(-40), F64, F16) == 0x3C00
    back = lambda bits, dt: float(half_bits_to_f32(np.array([bits], dtype=np.uint16), dt)[0])
    assert back(cast(oracle, (1 << 24) + 1, I64, BF16), BF16) == p(24)
    assert back(cast(oracle, (1 << 24) + (1 << 16) + 1, I64, BF16), BF16) == p(24)
    assert back(cast(oracle, 2**63 - 1, I64, BF16), BF16) == p(63)
    assert cast(oracle, 70000, I64, F16) == 0x7C00
    nan16 = cast(oracle, math.nan, F64, F16)
    assert (nan16 & 0x7C00) == 0x7C00 and (nan16 & 0x3FF) != 0
    neg = cast(oracle, -math.nan, F64, BF16)
    assert neg & 0x8000


def test_erf_values(oracle):
    cases = [(0.0, 0.0), (1e-10, 1.1283791670955126e-10), (0.5, 0.5204998778130465), (1.0, 0.8427007929497149),
             (2.0, 0.9953222650189527), (2.4999, 0.9995928300996666), (2.5, 0.999593047982555), (3.0, 0.9999779095030014),
             (4.0, 0.9999999845827421), (-1.5, -0.9661051464753108)]
    for x, want in cases:
        got = oracle.lib.orc_erf(x)
        assert abs(got - want) <= 3.0 * np.finfo(np.float64).eps * abs(want), f"erf({x}) = {got}"
    assert oracle.lib.orc_erf(math.inf) == 1.0
    assert math.isnan(oracle.lib.orc_erf(math.nan))


def test_integer_power(oracle):
    def ipow(dt, base, exp):
        a = T(oracle, oracle.upload(np.array([base], dtype=STORAGE[dt]), dt))
        b = T(oracle, oracle.upload(np.array([exp], dtype=STORAGE[dt]), dt))
        return int(a.pow(b).raw()[0])
    assert ipow(I64, 3, 4) == 81
    assert ipow(I32, -2, 3) == -8
    assert ipow(I8, 2, 7) == -128
    assert ipow(I64, -1, -3) == -1
    assert ipow(I64, 5, -1) == 0


def test_strided_visits_are_row_major(oracle):
    # copy of a transposed view visits the output in row-major order (iter.rs `contiguous_and_transposed`)
    base = oracle.upload(np.arange(6, dtype=np.int32), I32)
    view = TensorData(base.storage, I32, (2, 3), (1, 2), 0)
    got = T(oracle, view).contiguous().raw()
    assert got.tolist() == [[0, 2, 4], [1, 3, 5]]
    bcast = TensorData(base.storage, I32, (3,), (0,), 4)
    assert T(oracle, bcast).contiguous().raw().tolist() == [4, 4, 4]
    empty = TensorData(base.storage, I32, (2, 0), (1, 1), 0)
    assert T(oracle, empty).contiguous().raw().shape == (2, 0)
    zero_dim = TensorData(base.storage, I32, (), (), 5)
    assert T(oracle, zero_dim).contiguous().raw().tolist() == 5


def test_promotion_table():
    assert promote_types(U8, I8) == I16
    assert promote_types(U8, I32) == I32
    assert promote_types(I16, I32) == I32
    assert promote_types(F16, BF16) == F32
    assert promote_types(BF16, F64) == F64
    assert promote_types(I64, F16) == F16
    assert promote_types(BOOL, U8) == U8
    for d in ALL_DTYPES:
        assert promote_types(d, d) == d and promote_types(BOOL, d) == d


def test_result_type_priorities(oracle):
    t = lambda dt, nd: oracle.empty((2,) * nd, dt)
    assert result_type([t(F16, 1), 2.0]) == F16
    assert result_type([t(I32, 1), 2.5]) == F32
    assert result_type([t(I64, 2), t(F64, 0)]) == F64
    assert result_type([t(F32, 2), t(F64, 0)]) == F32
    assert result_type([t(U8, 1), -1]) == U8
    assert result_type([t(BOOL, 1), 1]) == I64


def test_exhaustive_half_conversions_agree_with_numpy(oracle):
    """Every f16 pattern widens exactly; every widened value rounds back to itself (NaNs quietened)."""
    bits = np.arange(1 << 16, dtype=np.uint16)
    lib = oracle.lib
    f16 = np.array([lib.orc_f16_to_f32(int(b)) for b in bits[::7]], dtype=np.float32)
    want = bits[::7].view(np.float16).astype(np.float32)
    ok = (f16.view(np.uint32) == want.view(np.uint32)) | (np.isnan(f16) & np.isnan(want))
    assert ok.all()
    for b in bits[::97]:
        f = lib.orc_f16_to_f32(int(b))
        back = lib.orc_f32_to_f16(f)
        assert back == (b | 0x0200 if (b & 0x7FFF) > 0x7C00 else b)
        g = lib.orc_bf16_to_f32(int(b))
        back = lib.orc_f32_to_bf16(g)
        assert back == (b | 0x0040 if (b & 0x7FFF) > 0x7F80 else b)


def test_addr_and_exclusive_cumprod_by_hand(oracle):
    """The checker's addr and exclusive_cumprod on cases worked by hand (homura's tests/linalg.rs and tests/reduce.rs hold
    the same identities: addr with beta 0 ignores the input, integers wrap, the first product of a line is 1)."""
    from homura_b200.host import F32, I8
    v1 = oracle.upload(np.array([1.0, 2.0, 3.0], dtype=np.float32), F32)
    v2 = oracle.upload(np.array([10.0, 20.0], dtype=np.float32), F32)
    inp = oracle.upload(np.full((3, 2), np.nan, dtype=np.float32), F32)
    out = oracle.empty((3, 2), F32)
    oracle.addr(out, v1, v2, inp, 2.0, 0.0)   # beta 0: the NaNs of the input are not read
    assert (oracle.download(out) == np.array([[20, 40], [40, 80], [60, 120]], dtype=np.float32)).all()
    oracle.addr(out, v1, v2, oracle.upload(np.ones((3, 2), dtype=np.float32), F32), 1.0, 0.5)
    assert (oracle.download(out) == np.array([[10.5, 20.5], [20.5, 40.5], [30.5, 60.5]], dtype=np.float32)).all()
    a = oracle.upload(np.array([100, -7], dtype=np.int8), I8)
    b = oracle.upload(np.array([3], dtype=np.int8), I8)
    c = oracle.upload(np.array([[5], [6]], dtype=np.int8), I8)
    o8 = oracle.empty((2, 1), I8)
    oracle.addr(o8, a, b, c, 2, -1)            # 2 * 300 - 5 = 595 -> 83 (mod 256); 2 * -21 - 6 = -48
    assert oracle.download(o8).reshape(-1).tolist() == [83, -48]
    x = oracle.upload(np.array([[2.0, 3.0, 4.0], [0.5, 0.0, 7.0]], dtype=np.float32), F32)
    y = oracle.empty((2, 3), F32)
    oracle.exclusive_cumprod(y, x, 1, False)
    assert (oracle.download(y) == np.array([[1, 2, 6], [1, 0.5, 0]], dtype=np.float32)).all()
    oracle.exclusive_cumprod(y, x, 1, True)
    assert (oracle.download(y) == np.array([[12, 4, 1], [0, 7, 1]], dtype=np.float32)).all()


def test_index_add_and_scatter_add_by_hand(oracle):
    """cpu::index_add / scatter_add: f64 sums from the element's own value in the order of the contributions, one
    rounding (src/backend/cpu/misc.rs:219-317)."""
    import numpy as np
    from homura_b200.host import F32, I64, U8
    # 2^24 + 1 + 1 in f32: added one at a time in f32 the ones are lost; in f64 they are kept and the sum rounds to 2^24 + 2
    out = oracle.upload(np.array([16777216.0, 5.0], dtype=np.float32), F32)
    src = oracle.upload(np.array([1.0, 1.0, 2.5], dtype=np.float32), F32)
    oracle.index_add(out, 0, oracle.upload(np.array([0, -2, 1], dtype=np.int64), I64), src)
    assert oracle.download(out).tolist() == [16777218.0, 7.5]
    # integers wrap once, at the end
    out = oracle.upload(np.array([250, 0], dtype=np.uint8), U8)
    oracle.index_add(out, 0, oracle.upload(np.array([0, 0, 1], dtype=np.int64), I64), oracle.upload(np.array([3, 4, 9], dtype=np.uint8), U8))
    assert oracle.download(out).tolist() == [1, 9]
    out = oracle.upload(np.zeros((2, 3), dtype=np.int64), I64)
    idx = oracle.upload(np.array([[0, 1, 0], [0, 0, 1]], dtype=np.int64), I64)
    oracle.scatter_add(out, 0, idx, oracle.upload(np.array([[1, 2, 3], [10, 20, 30]], dtype=np.int64), I64))
    assert oracle.download(out).tolist() == [[11, 20, 3], [0, 2, 30]]
