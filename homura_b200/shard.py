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
from .host import F64, I64, SIZE, BackendError, Storage, TensorData, contiguous_strides, is_float


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

    def set_timeout(self, seconds: float) -> None:
        """How long a call may wait for progress before the communicator is aborted (60 s by default)."""
        self._check(self.lib.hmc_comm_set_timeout(self.handle, max(1, int(seconds * 1000))))

    def wait(self) -> None:
        """Waits until the stream has run everything queued so far, collectives included, for at most the timeout;
        raises (and the communicator is aborted) when a peer never joined."""
        self._check(self.lib.hmc_comm_wait(self.handle))

    def abort(self) -> None:
        """Tears the communicator down without its peers (after one of them is known to be gone)."""
        self._check(self.lib.hmc_comm_abort(self.handle))

    def close(self) -> None:
        if self.handle is not None:
            handle, self.handle = self.handle, None
            self._check(self.lib.hmc_comm_destroy(handle))


class RankWatch:
    """Who is still there, kept in a key-value store all ranks reach (a torch.distributed store, or anything with
    ``set(key, value)`` and ``check([keys])``): a rank that stops between steps says so first, and its peers look
    before they queue the next collective, so nobody launches a kernel that would wait for a rank that is gone.
    Failure detection on the host: no kernel waits, nothing has to time out."""

    def __init__(self, store, rank: int, ranks: int, job: str = "hmc"):
        self.store, self.rank, self.ranks, self.job = store, rank, ranks, job

    def _key(self, r: int) -> str:
        return f"{self.job}/left/{r}"

    def leave(self, reason: str = "") -> None:
        """Announces that this rank takes part in no further collective."""
        self.store.set(self._key(self.rank), reason or "left")

    def check(self) -> None:
        """Raises when a peer has announced that it left."""
        for r in range(self.ranks):
            if r != self.rank and self.store.check([self._key(r)]):
                raise BackendError(ffi.HMC_CUDA_ERROR, f"rank {r} has left the job: no collective is queued")


class ShardedReducer:
    """Reductions over the sharded (outermost) dimension. `shard` is this rank's block of the global tensor;
    `offsets[r]` is the first global index of rank r's block along that dimension; `global_rows` its size.

    A rank may hold an empty block (more ranks than rows): it contributes the identity of sums and products.
    Maxima, minima and their indices need a value from every rank, so they are refused on every rank alike,
    before any local work or collective, when some block is empty: the block lengths follow from `offsets` and
    `global_rows`, which all ranks share, so no rank is left waiting in the all-gather.

    With a `watch` (RankWatch) every collective first looks whether a peer has announced that it left, and raises
    instead of queuing a kernel that would wait for it.

    The partial and gathered buffers are kept and reused from call to call (all work is ordered on the backend's
    one stream, so a buffer is free again when the next call's kernels run)."""

    def __init__(self, backend, comm, offsets: Sequence[int], global_rows: int, watch: Optional[RankWatch] = None):
        self.be, self.comm, self.watch = backend, comm, watch
        self.offsets, self.global_rows = list(offsets), global_rows
        assert len(self.offsets) == comm.ranks, "one offset per rank"
        ends = self.offsets[1:] + [global_rows]
        self.lengths = [e - o for o, e in zip(self.offsets, ends)]
        assert all(n >= 0 for n in self.lengths), "offsets must not decrease and must end within global_rows"
        self._buffers = {}

    def _buffer(self, tag: str, nbytes: int) -> Storage:
        key = (tag, nbytes)
        if key not in self._buffers:
            self._buffers[key] = self.be.storage(nbytes)
        return self._buffers[key]

    def _gather(self, local: Storage, bytes_per_rank: int, tag: str = "gathered") -> Storage:
        if self.watch is not None:
            self.watch.check()  # before the collective is queued: a peer that is gone would never answer it
        gathered = self._buffer(tag, bytes_per_rank * self.comm.ranks)
        self.comm.allgather(local, gathered, bytes_per_rank)
        return gathered

    def _need_every_block(self, what: str) -> None:
        empty = [r for r, n in enumerate(self.lengths) if n == 0]
        if empty:
            raise BackendError(ffi.HMC_INVALID, f"{what} across shards needs a nonempty block on every rank "
                                                f"(rank {empty[0]} holds none of the {self.global_rows} rows)")

    def _fill(self, storage: Storage, dtype: int, n: int, value) -> None:
        self.be.fill(TensorData(storage, dtype, (n,), (1,)), value)

    def reduce(self, op: int, out: TensorData, shard: TensorData, mask: Sequence[bool]) -> None:
        """SUM, PROD, MEAN, MAX, MIN, ALL or ANY of the global tensor over the dimensions in `mask` (which
        include dimension 0) into the contiguous `out`, on every rank."""
        assert len(mask) == len(shard.shape) and mask[0], "the sharded (first) dimension must be reduced"
        be, nout = self.be, out.numel
        empty = shard.numel == 0
        if op in (ffi.HMC_REDUCE_MAX, ffi.HMC_REDUCE_MIN):
            self._need_every_block("max and min")
        if nout == 0:
            return
        if op in (ffi.HMC_REDUCE_SUM, ffi.HMC_REDUCE_PROD, ffi.HMC_REDUCE_MEAN) and is_float(shard.dtype):
            local = self._buffer("f64", 8 * nout)
            if empty:
                self._fill(local, F64, nout, 1.0 if op == ffi.HMC_REDUCE_PROD else 0.0)
            else:
                be.reduce_partial(op, local, shard, mask)
            gathered = self._gather(local, 8 * nout)
            reduced_per_row = math.prod(n for n, m in zip(shard.shape[1:], mask[1:]) if m)
            be.shard_combine_float(op, out, gathered, self.comm.ranks, nout, self.global_rows * reduced_per_row)
        elif op in (ffi.HMC_REDUCE_SUM, ffi.HMC_REDUCE_PROD):
            store = self._buffer("i64", 8 * nout)
            local = TensorData(store, I64, tuple(out.shape), tuple(contiguous_strides(out.shape)))
            if empty:
                self._fill(store, I64, nout, 1 if op == ffi.HMC_REDUCE_PROD else 0)
            else:
                be.reduce(op, local, shard, mask)
            gathered = self._gather(store, 8 * nout)
            be.shard_combine_int(op, out, gathered, self.comm.ranks, nout)
        elif op in (ffi.HMC_REDUCE_MAX, ffi.HMC_REDUCE_MIN):
            store = self._buffer("extreme", SIZE[shard.dtype] * nout)
            local = TensorData(store, shard.dtype, tuple(out.shape), tuple(contiguous_strides(out.shape)))
            be.reduce(op, local, shard, mask)
            gathered = self._gather(store, SIZE[shard.dtype] * nout)
            be.shard_combine_extreme(op == ffi.HMC_REDUCE_MAX, out, None, gathered, shard.dtype, None, None,
                                     self.comm.ranks, nout)
        elif op in (ffi.HMC_REDUCE_ALL, ffi.HMC_REDUCE_ANY):
            # every rank's result is 0 or 1 in out's dtype (Bool, or U8 for U8 tensors): all = the minimum over
            # the ranks, any = the maximum; an empty block is all-true and any-false
            store = self._buffer("flags", SIZE[out.dtype] * nout)
            local = TensorData(store, out.dtype, tuple(out.shape), tuple(contiguous_strides(out.shape)))
            if empty:
                self._fill(store, out.dtype, nout, 1 if op == ffi.HMC_REDUCE_ALL else 0)
            else:
                be.reduce(op, local, shard, mask)
            gathered = self._gather(store, SIZE[out.dtype] * nout)
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
        if nout == 0:
            return
        empty = shard.numel == 0
        count = self.global_rows * math.prod(n for n, m in zip(shard.shape[1:], mask[1:]) if m)
        sums = self._buffer("f64", 8 * nout)
        if empty:
            self._fill(sums, F64, nout, 0.0)
        else:
            be.reduce_partial(ffi.HMC_REDUCE_SUM, sums, shard, mask)
        means = self._buffer("means", 8 * nout)
        be.shard_combine_means(means, self._gather(sums, 8 * nout), self.comm.ranks, nout, count)
        squares = self._buffer("squares", 8 * nout)
        if empty:
            self._fill(squares, F64, nout, 0.0)
        else:
            be.var_partial(squares, shard, mask, means)
        be.shard_combine_var(out, self._gather(squares, 8 * nout), self.comm.ranks, nout, count, correction, take_sqrt)

    def arg_reduce(self, values: Optional[TensorData], indices: TensorData, shard: TensorData, is_max: bool) -> None:
        """Index (global, along the sharded dimension 0) and optionally value of the maximum or minimum."""
        self._need_every_block("argmax and argmin")
        be, nout = self.be, indices.numel
        if nout == 0:
            return
        vs, is_ = self._buffer("extreme", SIZE[shard.dtype] * nout), self._buffer("i64", 8 * nout)
        lv = TensorData(vs, shard.dtype, tuple(indices.shape), tuple(contiguous_strides(indices.shape)))
        li = TensorData(is_, I64, tuple(indices.shape), tuple(contiguous_strides(indices.shape)))
        be.arg_reduce(lv, li, shard, 0, is_max)
        gv = self._gather(vs, SIZE[shard.dtype] * nout, "gathered values")
        gi = self._gather(is_, 8 * nout, "gathered indices")
        be.shard_combine_extreme(is_max, values, indices, gv, shard.dtype, gi, self.offsets, self.comm.ranks, nout)

    def sum_f64(self, out: TensorData, partials: Storage, n: int) -> None:
        """out (a contiguous F64 scalar) = the sum over all ranks of this rank's `n` f64 `partials`: the partials
        are folded in their order on each rank, the ranks' sums in rank order. What a gradient norm over sharded
        parameters needs (hmc_adamw_step_many leaves one partial per tensor): one all-gather of 8 bytes per rank."""
        assert out.dtype == F64 and out.numel == 1
        be = self.be
        local = self._buffer("f64", 8)
        if n == 0:
            self._fill(local, F64, 1, 0.0)
        else:
            be.reduce_partial(ffi.HMC_REDUCE_SUM, local, TensorData(partials, F64, (n,), (1,)), [True])
        be.shard_combine_float(ffi.HMC_REDUCE_SUM, out, self._gather(local, 8), self.comm.ranks, 1, n * self.comm.ranks)
