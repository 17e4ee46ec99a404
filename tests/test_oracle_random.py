"""The CPU checker's samplers against what homura's own tests pin (src/ops/random.rs:468-527, tests/random.rs): the
Random123 known-answer vectors of Philox4x32-10, the unit-interval conversions, the extreme integer ranges, and the
seeded-sampling properties; plus the generator's block accounting, which the device path must share."""
import ctypes

import numpy as np

from homura_b200.host import BF16, F16, F32, F64, I64, Generator, int_range
from values import storage_to_f64


def philox(oracle, counter, key):
    c = (ctypes.c_uint32 * 4)(*counter)
    k = (ctypes.c_uint32 * 2)(*key)
    out = (ctypes.c_uint32 * 4)()
    oracle.lib.orc_philox(c, k, out)
    return list(out)


def test_philox_known_answers(oracle):
    # src/ops/random.rs:476-497 (kat_vectors of the Random123 distribution)
    assert philox(oracle, [0] * 4, [0] * 2) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert philox(oracle, [0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert philox(oracle, [0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_uniform_samples_stay_below_one_and_use_the_dtype_bits(oracle):
    # src/ops/random.rs:499-514: a sample of a narrow dtype is exactly representable and never rounds up to 1
    for dtype, bits in ((F16, 11), (BF16, 8), (F32, 24), (F64, 53)):
        gen = Generator(42)
        t = oracle.empty((4001,), dtype)
        oracle.random_uniform(t, gen, 0.0, 1.0)
        v = storage_to_f64(oracle.download(t), dtype)
        assert (v >= 0).all() and (v < 1).all()
        assert (v * 2.0**bits == np.floor(v * 2.0**bits)).all(), "more bits than the dtype's significand"
        assert gen.offset == -(-4001 // (2 if dtype == F64 else 4))
    # tests/random.rs:9-27: a thousand default samples span the unit interval; the same seed gives the same numbers
    a, b = oracle.empty((1000,), F32), oracle.empty((1000,), F32)
    oracle.random_uniform(a, Generator(42), 0.0, 1.0)
    oracle.random_uniform(b, Generator(42), 0.0, 1.0)
    va = oracle.download(a)
    assert (va == oracle.download(b)).all() and va.min() < 0.01 and 0.99 < va.max() < 1.0
    # an interval: [2, 3)
    oracle.random_uniform(a, Generator(7), 2.0, 3.0)
    va = oracle.download(a)
    assert (va >= 2.0).all() and (va < 3.0).all()


def test_normal_samples_have_the_moments(oracle):
    # tests/random.rs:13, 24-30
    gen = Generator(42)
    gen.reserve(250)  # after rand([1000])
    n = oracle.empty((10001,), F32)
    oracle.random_normal(n, gen, 0.0, 1.0)
    v = oracle.download(n).astype(np.float64)
    assert abs(v.mean()) < 0.05 and abs(v.std(ddof=1) - 1.0) < 0.05
    assert gen.offset == 250 + 5001


def test_integer_sampling_covers_extreme_ranges(oracle):
    # src/ops/random.rs:516-527
    def sample(n, low, high, seed=1):
        t = oracle.empty((n,), I64)
        oracle.random_int(t, Generator(seed), low, high)
        return oracle.download(t)
    v = sample(64, -2**63, 2**63 - 1)
    assert (v < 2**63 - 1).all()
    assert (sample(4, 2**63 - 2, 2**63 - 1) == 2**63 - 2).all()
    v = sample(1000, -2, 1)
    assert set(v.tolist()) == {-2, -1, 0}
    # tests/random.rs:32-34
    v = sample(2000, -3, 4, seed=42)
    assert v.min() == -3 and v.max() == 3
    assert int_range(-3, 4) == (7, 2**64 % 7)


def test_rejections_reserve_further_batches(oracle):
    # a range that rejects almost half of the words: later batches must be reserved, block by block as the CPU does
    low, high = 0, 2**63 + 1
    rng, threshold = int_range(low, high)
    assert threshold == 2**63 - 1
    gen = Generator(5)
    t = oracle.empty((301,), I64)
    oracle.random_int(t, gen, low, high)
    assert gen.offset > 151, "no word was rejected"
    # the batches by hand
    out = np.zeros(301, dtype=np.int64)
    done, offset = 0, 0
    while done < 301:
        needed = 301 - done
        blocks = -(-needed // 2)
        got = oracle.lib.orc_random_int_batch(out[done:].ctypes.data, needed, 5, offset, blocks, low, rng, threshold)
        offset += blocks
        done += min(got, needed)
    assert offset == gen.offset and (out == oracle.download(t)).all()
