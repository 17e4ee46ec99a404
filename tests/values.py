"""Inputs and comparisons of the differential tests, after homura's tests/common/rocm.rs: deterministic words
(SplitMix64), special values of every dtype followed by random *bit patterns* (every float pattern can
occur, NaN payloads and subnormals included), the eleven layouts every kernel is run on, and the comparison
classes (same bits with NaN ~ NaN; distance in ulps; bounded absolute error)."""
from __future__ import annotations

import math

import numpy as np

from homura_b200.host import (ALL_DTYPES, BF16, BOOL, DTYPE_NAMES, F16, F32, F64, FLOATS, I8, I16, I32, I64, SIZE,
                              STORAGE, U8, TensorData, f32_to_half_bits, half_bits_to_f32, is_float)

MASK64 = (1 << 64) - 1


class Words:
    """SplitMix64 (tests/common/rocm.rs:28-42)."""

    def __init__(self, seed: int):
        self.s = seed & MASK64

    def next(self) -> int:
        self.s = (self.s + 0x9E3779B97F4A7C15) & MASK64
        z = self.s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        return z ^ (z >> 31)

    def array(self, n: int) -> np.ndarray:
        return np.array([self.next() for _ in range(n)], dtype=np.uint64)


def words(seed: int, n: int) -> np.ndarray:
    """n SplitMix64 words, vectorised (state k = seed + k * gamma)."""
    k = np.arange(1, n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(seed & MASK64) + k * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def p2(e: int) -> float:
    return math.ldexp(1.0, e)


def special_f64() -> list:
    bits = lambda b: float(np.array([b], dtype=np.uint64).view(np.float64)[0])
    f32min = float(np.float32(2.0 ** -126))
    f32sub = p2(-149)
    v = [0.0, -0.0, 1.0, -1.0, 0.5, -2.5, 2.5, 255.9, -0.5, 300.0, -129.9, 1e30, -1e30, 65504.0, 65520.0, -65536.0,
         math.inf, -math.inf, math.nan, -math.nan, bits(0x7FF0000000000001), bits(0xFFF4000000001234),
         bits(0x7FF8000020000000), 2.2250738585072014e-308, -2.2250738585072014e-308 / 3.0, bits(1),
         1.7976931348623157e308, -1.7976931348623157e308, 3.4028234663852886e38, f32min, f32sub, f32sub / 2.0,
         f32sub * 0.75, 6.0e-8, p2(-24) * 1.5, p2(-133), 9.2e18, -9.3e18, p2(63), -p2(63), p2(63) - 1024.0, p2(31),
         -p2(31) - 1.0, p2(53) + 1.0, 1.0 + p2(-8) + p2(-21), 1.0 + p2(-8) + p2(-40), 1.0 + p2(-11) + p2(-40),
         1.0 + p2(-11), 1.0 + p2(-8), 1.0 + p2(-24), 1.0 + p2(-24) + p2(-52), -(1.0 + p2(-8) + p2(-21))]
    v += [(i - 20.0) * 0.37 for i in range(40)]
    return v


def special_i64() -> list:
    v = [0, 1, -1, 2, 127, 128, -128, -129, 255, 256, -255, 300, 32767, 32768, -32769, 65535, 65536, 2**31 - 1, -2**31,
         2**31, 2**63 - 1, -2**63, 2**63 - 2, (1 << 24) + 1, (1 << 24) + (1 << 16) + 1, (1 << 53) + 1,
         (1 << 53) + (1 << 30) + 1, 65504, 65520, 70000]
    v += [i * 7 - 140 for i in range(40)]
    return v


def f64_to_storage(values, dtype: int) -> np.ndarray:
    """float64 values as raw elements of a float dtype (rounded through f32 for the half types)."""
    a = np.asarray(values, dtype=np.float64)
    if dtype == F64:
        return a.copy()
    with np.errstate(over="ignore", invalid="ignore"):
        f = a.astype(np.float32)
    if dtype == F32:
        return f
    return f32_to_half_bits(f, dtype)


def storage_to_f64(raw: np.ndarray, dtype: int) -> np.ndarray:
    if dtype in (F16, BF16):
        return half_bits_to_f32(raw, dtype).astype(np.float64)
    if dtype == BOOL:
        return (raw != 0).astype(np.float64)
    return raw.astype(np.float64)


def values(dtype: int, n: int, seed: int) -> np.ndarray:
    """n raw elements: the special values first, then random bit patterns (tests/common/rocm.rs:165-211)."""
    r = words(seed, n)
    if dtype == BOOL:
        special = np.array([0, 1], dtype=np.uint8)
        rnd = (r & np.uint64(1)).astype(np.uint8)
    elif dtype in (U8, I8, I16, I32, I64):
        special = np.array([v & MASK64 for v in special_i64()], dtype=np.uint64).astype(STORAGE[dtype])
        rnd = r.astype(STORAGE[dtype])
    elif dtype == F64:
        special = np.array(special_f64(), dtype=np.float64)
        rnd = r.view(np.float64)
    elif dtype == F32:
        with np.errstate(over="ignore", invalid="ignore"):
            special = np.array(special_f64(), dtype=np.float64).astype(np.float32)
        rnd = r.astype(np.uint32).view(np.float32)
    else:
        special = f64_to_storage(special_f64(), dtype)
        rnd = r.astype(np.uint16)
    out = rnd.copy()
    k = min(n, len(special))
    out[:k] = special[:k]
    return out


# name, elements of the base, view of the base (tests/common/rocm.rs:284-308)
VIEWS = [
    ("contiguous [3, 5]", 15, lambda t: t.reshape(3, 5)),
    ("contiguous with an offset [7]", 10, lambda t: t.narrow(0, 2, 7)),
    ("transposed [5, 3]", 15, lambda t: t.reshape(3, 5).transpose(0, 1)),
    ("broadcast [4, 3, 5] (stride 0)", 15, lambda t: t.reshape(1, 3, 5).expand(4, 3, 5)),
    ("narrow with an offset [2, 3]", 20, lambda t: t.reshape(4, 5).narrow(0, 1, 2).narrow(1, 1, 3)),
    ("0-dim", 1, lambda t: t.reshape(())),
    ("empty [0, 3]", 0, lambda t: t.reshape(0, 3)),
    ("odd [1031]", 1031, lambda t: t),
    ("permuted [5, 4, 3, 2]", 120, lambda t: t.reshape(2, 3, 4, 5).permute(3, 2, 1, 0)),
    ("every other [600]", 1200, lambda t: t.reshape(600, 2).select(1, 1)),
    ("past one block [3, 257]", 771, lambda t: t.reshape(3, 257).transpose(0, 1)),
    # beyond homura's list: rows long enough for the vector path, with a misaligned start
    ("rows [37, 1000] of [37, 1003]", 37 * 1003, lambda t: t.reshape(37, 1003).narrow(1, 3, 1000)),
    ("column broadcast [64, 300]", 64, lambda t: t.reshape(64, 1).expand(64, 300)),
]


def layouts(backends, dtype: int, seed: int):
    """[(name, [view on each backend])]: the same raw values in the same layout on every backend."""
    out = []
    for name, n, view in VIEWS:
        raw = values(dtype, n, seed)
        out.append((name, [view(b.upload(raw, dtype)) for b in backends]))
    return out


def large_layouts(backends, dtype: int, seed: int, n: int = (1 << 24) + 1000):
    raw = values(dtype, 2 * n, seed)
    bases = [b.upload(raw, dtype) for b in backends]
    return [("large contiguous", [t.narrow(0, 0, n) for t in bases]),
            ("large strided", [t.reshape(n, 2).select(1, 1) for t in bases])]


def is_nan_raw(raw: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == F16:
        return (raw & 0x7FFF) > 0x7C00
    if dtype == BF16:
        return (raw & 0x7FFF) > 0x7F80
    if dtype in (F32, F64):
        return np.isnan(raw)
    return np.zeros(raw.shape, dtype=bool)


def as_bits(raw: np.ndarray) -> np.ndarray:
    return raw.view({1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[raw.dtype.itemsize])


def assert_bitwise(got: np.ndarray, want: np.ndarray, dtype: int, what: str) -> None:
    """Same shape and bytes, except that a NaN only has to meet a NaN (tests/common/rocm.rs:361-377)."""
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    g, w = as_bits(got), as_bits(want)
    same = (g == w) | (is_nan_raw(got, dtype) & is_nan_raw(want, dtype))
    if not same.all():
        i = int(np.argmin(same.reshape(-1)))
        raise AssertionError(f"{what} [{DTYPE_NAMES[dtype]}]: element {i} differs: got {int(g.reshape(-1)[i]):#x}, "
                             f"want {int(w.reshape(-1)[i]):#x} ({int((~same).sum())} of {same.size} differ)")


def assert_same(got: np.ndarray, want: np.ndarray, dtype: int, what: str) -> None:
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    g, w = as_bits(got), as_bits(want)
    if not (g == w).all():
        i = int(np.argmin((g == w).reshape(-1)))
        raise AssertionError(f"{what} [{DTYPE_NAMES[dtype]}]: element {i} differs: got {int(g.reshape(-1)[i]):#x}, "
                             f"want {int(w.reshape(-1)[i]):#x} ({int((g != w).sum())} of {g.size} differ)")


def ordered(raw: np.ndarray, dtype: int) -> np.ndarray:
    """Raw float elements as integers whose difference counts representable values."""
    b = as_bits(raw).astype(np.int64) if raw.dtype.itemsize < 8 else as_bits(raw).view(np.int64)
    sign = np.int64(1) << np.int64(8 * raw.dtype.itemsize - 1)
    if raw.dtype.itemsize == 8:
        mag = b & np.int64(0x7FFFFFFFFFFFFFFF)
        return np.where(b < 0, -mag, mag)
    mag = b & (sign - 1)
    return np.where((b & sign) != 0, -mag, mag)


def ulp_stats(got: np.ndarray, want: np.ndarray, dtype: int, what: str):
    """(max ulp distance, number of differing elements). NaN must meet NaN, infinities must agree."""
    assert got.shape == want.shape, f"{what}: shape"
    gn, wn = is_nan_raw(got, dtype), is_nan_raw(want, dtype)
    assert (gn == wn).all(), f"{what} [{DTYPE_NAMES[dtype]}]: NaN classification differs at {int(np.argmax(gn != wn))}"
    gf, wf = storage_to_f64(got, dtype), storage_to_f64(want, dtype)
    inf = np.isinf(gf) | np.isinf(wf)
    assert (gf[inf] == wf[inf]).all(), f"{what} [{DTYPE_NAMES[dtype]}]: infinities differ"
    ok = ~(gn | inf)
    og, ow = ordered(got, dtype)[ok], ordered(want, dtype)[ok]
    # exact integer distances (an f64 difference of 63-bit integers would be rounded to multiples of 512); values of
    # opposite sign, whose distance could overflow, are apart by their magnitudes' sum, computed in f64 when it is huge
    same_sign = (og >= 0) == (ow >= 0)
    with np.errstate(over="ignore"):
        d = np.where(same_sign, np.abs(og - ow), 0).astype(np.float64)
    d = np.where(same_sign, d, np.abs(og.astype(np.float64)) + np.abs(ow.astype(np.float64)))
    # +0 and -0 are the same value
    zero = (gf[ok] == 0) & (wf[ok] == 0)
    d = np.where(zero, 0, d)
    return (int(d.max()) if d.size else 0), int((d > 0).sum())


def assert_ulp(got, want, dtype, max_ulp, what):
    m, n = ulp_stats(got, want, dtype, what)
    assert m <= max_ulp, f"{what} [{DTYPE_NAMES[dtype]}]: {m} ulp apart (limit {max_ulp}), {n} elements differ"
    return m, n


def ulp_of(dtype: int, v: np.ndarray) -> np.ndarray:
    """Spacing of `dtype` at |v| (tests/common/rocm.rs:399-413)."""
    man, min_exp = {F16: (10, -14), BF16: (7, -126), F32: (23, -126), F64: (52, -1022)}[dtype]
    a = np.abs(np.asarray(v, dtype=np.float64))
    biased = (a.view(np.uint64) >> np.uint64(52)).astype(np.int64)
    e = np.where(biased == 0, -1023, biased - 1023)
    return np.ldexp(1.0, (np.maximum(e, min_exp) - man).astype(np.int64))


def check_within(got, want, dtype, extra, what):
    """|got - want| <= extra + ulp_out(max(|got|, |want|)); NaN meets NaN, infinity the same infinity
    (tests/common/rocm.rs:490-537). Returns (max ulp distance, differing elements)."""
    gn, wn = is_nan_raw(got, dtype), is_nan_raw(want, dtype)
    assert (gn == wn).all(), f"{what} [{DTYPE_NAMES[dtype]}]: NaN classification differs at {int(np.argmax(gn != wn))}"
    gf, wf = storage_to_f64(got, dtype), storage_to_f64(want, dtype)
    inf = np.isinf(gf) | np.isinf(wf)
    assert (gf[inf] == wf[inf]).all(), f"{what} [{DTYPE_NAMES[dtype]}]: infinities differ"
    ok = ~(gn | inf)
    diff = np.abs(gf[ok] - wf[ok])
    bound = np.broadcast_to(np.asarray(extra, dtype=np.float64), gf.shape)[ok] + ulp_of(dtype, np.maximum(np.abs(gf[ok]), np.abs(wf[ok])))
    bad = ~(diff <= bound)
    if bad.any():
        i = int(np.argmax(bad))
        raise AssertionError(f"{what} [{DTYPE_NAMES[dtype]}]: got {gf[ok][i]!r}, want {wf[ok][i]!r}: |diff| {diff[i]:e} > "
                             f"bound {bound[i]:e} ({int(bad.sum())} of {bad.size})")
    return ulp_stats(got, want, dtype, what)
