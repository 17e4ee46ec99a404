"""The oracle's casts against homura's own C++ restatement of them (csrc/elem.hpp compiled for the host into
oracle/_ref by oracle/build.py, where homura's sources are present): all 100 dtype pairs on the special values
and on random bit patterns, bit for bit. Skipped where oracle/_ref has not been built."""
import ctypes
import importlib.util
from pathlib import Path

import numpy as np
import pytest

from frontend import T
from homura_b200.host import ALL_DTYPES, DTYPE_NAMES, STORAGE
from values import assert_same, values

ROOT = Path(__file__).resolve().parent.parent


def _ref():
    spec = importlib.util.spec_from_file_location("oracle_build", ROOT / "oracle" / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    path = mod.build_ref()
    if path is None or not Path(path).exists():
        pytest.skip("oracle/_ref is not built (homura's sources are not mounted here)")
    lib = ctypes.CDLL(str(path))
    lib.ref_convert.restype = ctypes.c_int
    lib.ref_convert.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
    return lib


@pytest.mark.parametrize("src", ALL_DTYPES, ids=DTYPE_NAMES)
def test_every_cast_agrees_with_the_reference_header(oracle, src):
    lib = _ref()
    raw = values(src, 20000, 401)
    t = T(oracle, oracle.upload(raw, src))
    for dst in ALL_DTYPES:
        want = np.zeros(raw.size, dtype=STORAGE[dst])
        assert lib.ref_convert(dst, src, raw.ctypes.data, want.ctypes.data, raw.size) == 0
        got = t.to(dst).raw() if dst != src else t.contiguous().raw()
        assert_same(got, want, dst, f"{DTYPE_NAMES[src]} -> {DTYPE_NAMES[dst]}")
