"""Shared pieces of the GPU-vs-oracle differential tests."""
from __future__ import annotations

import numpy as np

from frontend import T
from homura_b200.host import DTYPE_NAMES
from values import assert_bitwise, layouts


def pairs(oracle, cuda, dtype, seed):
    """[(layout name, T on the oracle, T on the GPU)] over the generator's layouts."""
    return [(name, T(oracle, o), T(cuda, g)) for name, (o, g) in layouts([oracle, cuda], dtype, seed)]


def both(oracle, cuda, raw: np.ndarray, dtype: int, shape=None):
    return T(oracle, oracle.upload(raw, dtype, shape)), T(cuda, cuda.upload(raw, dtype, shape))


def same(f, o: T, g: T, what: str):
    """f applied on both sides gives the same bits (NaN ~ NaN)."""
    want, got = f(o), f(g)
    assert got.dtype == want.dtype, f"{what}: dtype"
    assert_bitwise(got.raw(), want.raw(), want.dtype, what)
