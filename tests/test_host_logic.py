"""The host glue: dimension merging (src/backend/rocm/copy.rs:34-57 and its CPU twin's tests,
src/backend/cpu/iter.rs:106-123), reduction descriptions, scalar bits, the limit of 25 dimensions."""
import numpy as np
import pytest

from homura_b200 import ffi
from homura_b200.host import (BF16, F16, F32, F64, I8, I32, I64, U8, BOOL, BackendError, MAX_DIMS, Storage, TensorData,
                              adamw_scalars, contiguous_strides, describe, descs, fused_coefficient, merge_dims,
                              scalar_bits)


def fake(shape, strides=None, dtype=F32, offset=0):
    arr = np.zeros(4, dtype=np.float32)
    return TensorData(Storage(16, array=arr), dtype, tuple(shape), tuple(strides or contiguous_strides(shape)), offset)


def test_contiguous_operands_merge_into_one_dimension():
    assert merge_dims([2, 3, 4], [[12, 4, 1]]) == [(24, [1])]
    assert merge_dims([2, 3], [[3, 1], [1, 2]]) == [(2, [3, 1]), (3, [1, 2])]
    assert merge_dims([2, 0], [[1, 1]]) is None
    assert merge_dims([], [[]]) == []
    assert merge_dims([3], [[0]]) == [(3, [0])]
    assert merge_dims([1, 5, 1], [[7, 1, 9]]) == [(5, [1])]


def test_broadcast_rows_and_columns_stay_two_dimensional():
    # a[1024,1024] * b[1024] expanded: strides [0, 1]
    assert merge_dims([1024, 1024], [[1024, 1], [1024, 1], [0, 1]]) == [(1024, [1024, 1024, 0]), (1024, [1, 1, 1])]
    # fully broadcast single element merges to one dimension of stride 0
    assert merge_dims([4, 5], [[5, 1], [0, 0]]) == [(20, [1, 0])]


def test_extreme_strides_do_not_merge_by_overflow():
    half = 2**63
    assert len(merge_dims([2, 2], [[0, half]])) == 2


def test_more_than_25_unmergeable_dimensions_are_refused():
    shape = [2] * 26
    strides = [3 ** (26 - i) for i in range(26)]
    with pytest.raises(BackendError) as e:
        descs("unary", [fake(shape, strides), fake(shape, strides)])
    assert e.value.status == ffi.HMC_INVALID
    assert "at most 25 dimensions" in str(e.value) and "unary" in str(e.value)
    assert MAX_DIMS == 25


def test_describe_splits_kept_and_reduced_dimensions():
    src = fake([4, 5, 6])
    r = describe("reduce", src, [False, True, False])
    assert (r.kept.ndim, r.red.ndim) == (2, 1)
    assert list(r.kept.sizes[:2]) == [4, 6] and list(r.kept.strides[:2]) == [30, 1]
    assert (r.red.sizes[0], r.red.strides[0]) == (5, 6)
    r = describe("reduce", src, [True, True, True])
    assert r.kept.ndim == 0 and (r.red.sizes[0], r.red.strides[0]) == (120, 1)
    r = describe("reduce", fake([3, 0]), [False, True])
    assert r.red.ndim == 1 and r.red.sizes[0] == 0
    assert describe("reduce", fake([0, 3]), [False, True]) is None


def test_scalar_bits():
    assert scalar_bits(1.0, F32) == 0x3F800000
    assert scalar_bits(-2.0, F64) == 0xC000000000000000
    assert scalar_bits(1.0, BF16) == 0x3F80 and scalar_bits(1.0, F16) == 0x3C00
    assert scalar_bits(-1, U8) == 255 and scalar_bits(-1, I64) == 2**64 - 1
    assert scalar_bits(2.9, I32) == 2 and scalar_bits(-2.9, I8) == 0xFE
    assert scalar_bits(0.5, BOOL) == 1 and scalar_bits(0, BOOL) == 0
    assert scalar_bits(1e-8, F16) == 0
    assert scalar_bits(float("inf"), BF16) == 0x7F80


def test_fused_coefficients_follow_the_cpu_kernel():
    assert fused_coefficient(ffi.HMC_FUSED_LERP, 0.3, F32) == (float(np.float32(0.3)), True)
    c, small = fused_coefficient(ffi.HMC_FUSED_LERP, 0.7, F32)
    assert not small and c == float(np.float32(0.7) - np.float32(1.0))
    assert fused_coefficient(ffi.HMC_FUSED_SCALED_ADD, 0.1, BF16)[0] == 0.10009765625
    assert fused_coefficient(ffi.HMC_FUSED_ADDCMUL, 0.1, F64)[0] == 0.1


def test_adamw_scalars():
    sc = adamw_scalars(F32, 1e-4, 0.9, 0.999, 1e-8, 0.01, 1.0)
    assert sc.has_decay == 1 and sc.lerp_small == 1
    assert sc.decay == float(np.float32(1.0 - 1e-4 * 0.01))
    assert sc.eps == float(np.float32(1e-8))
    assert adamw_scalars(F16, 1e-3, 0.9, 0.999, 1e-8, 0.0, 2.0).eps == 0.0


def test_debug_runs_refuse_descriptions_that_reach_beyond_their_storage(monkeypatch):
    """HOMURA_CUDA_DEBUG=1: the farthest element a description can reach is checked against the storage on the host,
    for same-shaped operands and for the two halves of a reduction."""
    from homura_b200 import host
    from homura_b200.host import F32, BackendError, Storage, TensorData

    monkeypatch.setattr(host, "CHECK_REACH", True)
    st = Storage(16 * 4, ptr=4096, device=0)
    good = TensorData(st, F32, (4, 4), (4, 1))
    assert len(host.descs("fits", [good, good])) == 2
    assert host.describe("fits", good, [False, True]) is not None
    assert host.descs("window", [TensorData(st, F32, (2, 2), (4, 1), 10)]) is not None   # reaches element 15
    with pytest.raises(BackendError, match="reaches element 16 of a storage of 16"):
        host.descs("wide", [TensorData(st, F32, (4, 5), (4, 1))])
    with pytest.raises(BackendError, match="reaches element 18"):
        host.describe("strided rows", TensorData(st, F32, (4, 4), (4, 2)), [False, True])
    with pytest.raises(BackendError, match="reaches element 16"):
        host.descs("offset", [TensorData(st, F32, (2, 2), (4, 1), 11)])
    # empty operands reach nothing
    assert host.descs("empty", [TensorData(st, F32, (0, 9), (9, 1))]) is None
    monkeypatch.setattr(host, "CHECK_REACH", False)
    assert host.descs("unchecked", [TensorData(st, F32, (4, 5), (4, 1))]) is not None
