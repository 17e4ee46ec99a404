"""Reductions of a tensor split along its outermost dimension over the GPUs of one machine, one process per
GPU (``include/homura_cuda_shard.h``). homura has no multi-GPU layer; this is the exchange step its reductions
need once a tensor is sharded, and nothing else: elementwise work, reductions over inner dimensions and softmax
over the last dimension run on each shard with the ordinary backend functions.

A reduction that folds the sharded dimension = local partials (accumulator precision) -> all-gather of a few
bytes per output into every rank's own memory -> fold in rank order on every rank. The result is bit-identical
on all ranks and from run to run, and follows homura's rules across shards as within one (f64 accumulation,
wrapping integers, first NaN then first of equals, global indices).

The communicator is anything with ``ranks``, ``rank`` and ``allgather(send, recv, nbytes)`` over backend
storages: :class:`NcclComm` on GPUs; the CPU tests pair the orchestration below with a gloo communicator.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Sequence

from . import ffi
from .host import I64, SIZE, BackendError, Storage, TensorData, is_float


def split_rows(n: int, ranks: int) -> list:
    """(start, length) of each rank's block of a dimension of n: ceil-sized blocks, the last ones may be
    short or empty."""
    per = -(-n // ranks) if ranks else 0
    out = []
    for r in range(ranks):
        start = min(r * per, n)
        out.append((start, min(per, n - start)))
    return out


class NcclComm:
    """An NCCL communicator bound to a CudaBackend's context (its device and stream)."""

    def __init__(self, backend, ranks: int, rank: int, unique_id: bytes):
        from . import load_shard
        self.lib = load_shard()
        self.backend, self.ranks, self.rank = backend, ranks, rank
        handle = ctypes.c_void_p()
        buf = (ctypes.c_uint8 * ffi.HMC_COMM_ID_BYTES).from_buffer_copy(unique_id)
        self._check(self.lib.hmc_comm_create(backend.ctx, ranks, rank, buf, ctypes.byref(handle)))
        self.handle = handle

    @staticmethod
    def unique_id() -> bytes:
        from . import load_shard
        lib = load_shard()
        buf = (ctypes.c_uint8 * ffi.HMC_COMM_ID_BYTES)()
        if lib.hmc_comm_unique_id(buf) != ffi.HMC_OK:
            raise BackendError(ffi.HMC_CUDA_ERROR, lib.hmc_last_error().decode())
        return bytes(buf)

    def _check(self, status: int) -> None:
        if status != ffi.HMC_OK:
            raise BackendError(status, self.lib.hmc_last_error().decode())

    def allgather(self, send: Storage, recv: Storage, nbytes: int) -> None:
        self._check(self.lib.hmc_comm_allgather(self.handle, send.ptr, recv.ptr, nbytes))

    def close(self) -> None:
        if self.handle is not None:
            handle, self.handle = self.handle, None
            self._check(self.lib.hmc_comm_destroy(handle))


class ShardedReducer:
    """Reductions over the sharded (outermost) dimension. `shard` is this rank's block of the global tensor;
    `offsets[r]` is the first global index of rank r's block along that dimension; `global_rows` its size."""

    def __init__(self, backend, comm, offsets: Sequence[int], global_rows: int):
        self.be, self.comm = backend, comm
        self.offsets, self.global_rows = list(offsets), global_rows

    def _gather(self, local: Storage, bytes_per_rank: int) -> Storage:
        gathered = self.be.storage(bytes_per_rank * self.comm.ranks)
        self.comm.allgather(local, gathered, bytes_per_rank)
        return gathered

    def reduce(self, op: int, out: TensorData, shard: TensorData, mask: Sequence[bool]) -> None:
        """SUM, PROD, MEAN, MAX or MIN of the global tensor over the dimensions in `mask` (which include
        dimension 0) into the contiguous `out`, on every rank. Every rank holds at least one row."""
        assert len(mask) == len(shard.shape) and mask[0], "the sharded (first) dimension must be reduced"
        be, nout = self.be, out.numel
        if op in (ffi.HMC_REDUCE_SUM, ffi.HMC_REDUCE_PROD, ffi.HMC_REDUCE_MEAN) and is_float(shard.dtype):
            local = be.storage(8 * nout)
            be.reduce_partial(op, local, shard, mask)
            gathered = self._gather(local, 8 * nout)
            reduced_per_row = math.prod(n for n, m in zip(shard.shape[1:], mask[1:]) if m)
            be.shard_combine_float(op, out, gathered, self.comm.ranks, nout, self.global_rows * reduced_per_row)
        elif op in (ffi.HMC_REDUCE_SUM, ffi.HMC_REDUCE_PROD):
            local = be.empty(out.shape, I64)
            be.reduce(op, local, shard, mask)
            gathered = self._gather(local.storage, 8 * nout)
            be.shard_combine_int(op, out, gathered, self.comm.ranks, nout)
        elif op in (ffi.HMC_REDUCE_MAX, ffi.HMC_REDUCE_MIN):
            local = be.empty(out.shape, shard.dtype)
            be.reduce(op, local, shard, mask)
            gathered = self._gather(local.storage, SIZE[shard.dtype] * nout)
            be.shard_combine_extreme(op == ffi.HMC_REDUCE_MAX, out, None, gathered, shard.dtype, None, None,
                                     self.comm.ranks, nout)
        elif op in (ffi.HMC_REDUCE_ALL, ffi.HMC_REDUCE_ANY):
            # every rank's result is 0 or 1 in out's dtype (Bool, or U8 for U8 tensors): all = the minimum over
            # the ranks, any = the maximum
            local = be.empty(out.shape, out.dtype)
            be.reduce(op, local, shard, mask)
            gathered = self._gather(local.storage, SIZE[out.dtype] * nout)
            be.shard_combine_extreme(op == ffi.HMC_REDUCE_ANY, out, None, gathered, out.dtype, None, None,
                                     self.comm.ranks, nout)
        else:
            raise BackendError(ffi.HMC_INVALID, "this reduction is not available across shards")

    def var(self, out: TensorData, shard: TensorData, mask: Sequence[bool], correction: float, take_sqrt: bool) -> None:
        """Variance (standard deviation with take_sqrt) of the global tensor over the dimensions in `mask` (which
        include dimension 0), in two rounds as on one GPU: the f64 means of the whole tensor, then the squared
        deviations from them."""
        assert len(mask) == len(shard.shape) and mask[0], "the sharded (first) dimension must be reduced"
        assert is_float(shard.dtype)
        be, nout = self.be, out.numel
        count = self.global_rows * math.prod(n for n, m in zip(shard.shape[1:], mask[1:]) if m)
        sums = be.storage(8 * nout)
        be.reduce_partial(ffi.HMC_REDUCE_SUM, sums, shard, mask)
        means = be.storage(8 * nout)
        be.shard_combine_means(means, self._gather(sums, 8 * nout), self.comm.ranks, nout, count)
        squares = be.storage(8 * nout)
        be.var_partial(squares, shard, mask, means)
        be.shard_combine_var(out, self._gather(squares, 8 * nout), self.comm.ranks, nout, count, correction, take_sqrt)

    def arg_reduce(self, values: Optional[TensorData], indices: TensorData, shard: TensorData, is_max: bool) -> None:
        """Index (global, along the sharded dimension 0) and optionally value of the maximum or minimum."""
        be, nout = self.be, indices.numel
        lv = be.empty(indices.shape, shard.dtype)
        li = be.empty(indices.shape, I64)
        be.arg_reduce(lv, li, shard, 0, is_max)
        gv = self._gather(lv.storage, SIZE[shard.dtype] * nout)
        gi = self._gather(li.storage, 8 * nout)
        be.shard_combine_extreme(is_max, values, indices, gv, shard.dtype, gi, self.offsets, self.comm.ranks, nout)
