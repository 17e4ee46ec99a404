"""Device samplers against the CPU checker through the C ABI: uniform samples and integers bit for bit (they share
homura's Philox blocks, word order and conversions), normal samples within an ulp or two (log, cos and sin are the
device library's; homura's tests/rocm_random.rs makes the same allowance), and the same number of blocks reserved."""
import ctypes

import numpy as np
import pytest

from homura_b200 import ffi
from homura_b200.host import BF16, F16, F32, F64, FLOATS, I32, I64, DTYPE_NAMES, BackendError, Generator, _flat_desc
from values import assert_bitwise, check_within

pytestmark = pytest.mark.gpu

FLOAT_IDS = [DTYPE_NAMES[d] for d in FLOATS]


@pytest.mark.parametrize("dtype", FLOATS, ids=FLOAT_IDS)
def test_uniform_samples_are_the_cpu_bits(oracle, cuda, dtype):
    for n in (1, 3, 4, 5, 1000, 4001, (1 << 20) + 3):
        for low, high in ((0.0, 1.0), (2.0, 3.0), (-1000.0, 1000.0), (0.25, 0.25), (-60000.0, 60000.0)):
            go, gg = Generator(42), Generator(42)
            go.reserve(7), gg.reserve(7)
            o, g = oracle.empty((n,), dtype), cuda.empty((n,), dtype)
            oracle.random_uniform(o, go, low, high)
            cuda.random_uniform(g, gg, low, high)
            assert_bitwise(cuda.download(g), oracle.download(o), dtype, f"uniform [{low}, {high}) n={n}")
            assert go.offset == gg.offset
    # an output that does not start on a vector boundary, in the middle of a larger buffer
    big_o, big_g = oracle.empty((1030,), dtype), cuda.empty((1030,), dtype)
    cuda.fill(big_g, 0.0)
    oracle.random_uniform(big_o.narrow(0, 1, 1001), Generator(9), 0.0, 1.0)
    cuda.random_uniform(big_g.narrow(0, 1, 1001), Generator(9), 0.0, 1.0)
    assert_bitwise(cuda.download(big_g), oracle.download(big_o), dtype, "uniform into an unaligned window")
    # the widest interval of the dtype: a sample that rounds up to `to` becomes `from`
    top = {F16: 65504.0, BF16: 3.3895313892515355e38, F32: 3.4028234663852886e38, F64: 8.98846567431158e307}[dtype]
    o, g = oracle.empty((50001,), dtype), cuda.empty((50001,), dtype)
    oracle.random_uniform(o, Generator(3), 0.0, top)
    cuda.random_uniform(g, Generator(3), 0.0, top)
    assert_bitwise(cuda.download(g), oracle.download(o), dtype, "uniform over [0, max)")


@pytest.mark.parametrize("dtype", FLOATS, ids=FLOAT_IDS)
def test_normal_samples_match_within_the_last_place(oracle, cuda, dtype):
    for n in (1, 2, 7, 10001, (1 << 18) + 1):
        go, gg = Generator(42), Generator(42)
        o, g = oracle.empty((n,), dtype), cuda.empty((n,), dtype)
        oracle.random_normal(o, go, 0.5, 2.0)
        cuda.random_normal(g, gg, 0.5, 2.0)
        # two libms: log, cos and sin may each differ in the last place of f64, which r * cos(theta) carries at the
        # scale of std * r <= 2 * 8.6; on top of it one ulp of the output dtype (the bound of homura's device tests)
        check_within(cuda.download(g), oracle.download(o), dtype, 8 * 2.3e-16 * 2.0 * 8.6, f"normal n={n}")
        assert go.offset == gg.offset == -(-n // 2)


def test_integers_are_the_cpu_bits(oracle, cuda):
    cases = [(0, 2**32), (-3, 4), (0, 2**63 + 1), (-2**63, 2**63 - 1), (2**63 - 2, 2**63 - 1), (-7, 1000003), (5, 6),
             (0, 2**21), (0, 2**21 - 1), (-2, 2**21 + 3), (0, 50257), (0, 3 * 2**40), (0, 2**16)]
    for low, high in cases:
        for n in (1, 2, 301, 100001):
            go, gg = Generator(11), Generator(11)
            go.reserve(3), gg.reserve(3)
            o, g = oracle.empty((n,), I64), cuda.empty((n,), I64)
            oracle.random_int(o, go, low, high)
            cuda.random_int(g, gg, low, high)
            assert (cuda.download(g) == oracle.download(o)).all(), f"randint [{low}, {high}) n={n}"
            assert go.offset == gg.offset, f"blocks reserved for [{low}, {high}) n={n}"
    # many tiles, with rejections: several rounds of the position kernel
    n = (1 << 21) + 17
    o, g = oracle.empty((n,), I64), cuda.empty((n,), I64)
    go, gg = Generator(1), Generator(1)
    oracle.random_int(o, go, 0, 2**63 + 2**62)
    cuda.random_int(g, gg, 0, 2**63 + 2**62)
    assert (cuda.download(g) == oracle.download(o)).all() and go.offset == gg.offset


def test_samplers_refuse_what_they_cannot_fill(cuda):
    t = cuda.empty((8,), I32)
    with pytest.raises(BackendError):
        cuda._check(cuda.lib.hmc_random_uniform(cuda.ctx, _flat_desc(t), 1, 0, 0.0, 1.0))
    f = cuda.empty((4, 4), F32)
    d = ffi.hmc_tensor_desc()
    d.data, d.dtype, d.ndim = f.storage.address, F32, 2
    d.sizes[0], d.sizes[1], d.strides[0], d.strides[1] = 4, 4, 4, 1
    assert cuda.lib.hmc_random_normal(cuda.ctx, ctypes.byref(d), 1, 0, 0.0, 1.0) == ffi.HMC_INVALID
    i = cuda.empty((8,), I64)
    assert cuda.lib.hmc_random_int(cuda.ctx, _flat_desc(i), 1, 0, 4, 0, 7, 2, None) == ffi.HMC_INVALID  # no workspace
    assert cuda.lib.hmc_random_int(cuda.ctx, _flat_desc(i), 1, 0, 4, 0, 0, 0, None) == ffi.HMC_INVALID  # empty range
