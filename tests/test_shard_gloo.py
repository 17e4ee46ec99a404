"""The multi-rank path on the CPU: two gloo ranks run the sharded-reduction orchestration
(homura_b200/shard.py: split, local partials, all-gather, rank-ordered combine) with host stand-ins for the
device steps, and every rank must reproduce the single-rank result: bit for bit for integers, extremes and
indices, within 2 ulp for f64-accumulated float sums."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


class GlooComm:
    def __init__(self, ranks, rank):
        self.ranks, self.rank = ranks, rank

    def allgather(self, send, recv, nbytes):
        mine = torch.from_numpy(send.array.reshape(-1).view(np.uint8)[:nbytes].copy())
        parts = [torch.empty(nbytes, dtype=torch.uint8) for _ in range(self.ranks)]
        dist.all_gather(parts, mine)
        for r, p in enumerate(parts):
            recv.array.reshape(-1).view(np.uint8)[r * nbytes:(r + 1) * nbytes] = p.numpy()


def _worker(rank, world, port, results):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from frontend import T
        from homura_b200 import ffi
        from homura_b200.host import BOOL, F32, BF16, I32, I64
        from homura_b200.shard import ShardedReducer, split_rows
        from oracle_backend import OracleBackend
        from values import assert_bitwise, assert_ulp, f64_to_storage, values

        be = OracleBackend()
        rows, cols = 37, 53  # 37 rows over 2 ranks: 19 + 18
        blocks = split_rows(rows, world)
        start, length = blocks[rank]
        red = ShardedReducer(be, GlooComm(world, rank), [b[0] for b in blocks], rows)
        rng = np.random.default_rng(7)
        data = {F32: rng.standard_normal((rows, cols)).astype(np.float32),
                BF16: f64_to_storage(rng.standard_normal((rows, cols)), BF16),
                I32: rng.integers(-1000, 1001, size=(rows, cols), dtype=np.int32)}
        data[F32][20, 5] = np.nan          # a NaN in the second shard only
        data[F32][3, 7] = data[F32][30, 7] = 9.0  # equal maxima in both shards
        for dt, full in data.items():
            whole = T(be, be.upload(full, dt))
            shard = be.upload(full[start:start + length], dt)
            is_f = dt != I32
            for mask, shape in (([True, False], (cols,)), ([True, True], ())):
                dims = [d for d, m in enumerate(mask) if m]
                ops = [("sum", ffi.HMC_REDUCE_SUM), ("max", ffi.HMC_REDUCE_MAX), ("min", ffi.HMC_REDUCE_MIN)]
                if is_f:
                    ops.append(("mean", ffi.HMC_REDUCE_MEAN))
                for name, op in ops:
                    out_dt = dt if (is_f or name in ("max", "min")) else I64
                    out = be.empty(shape, out_dt)
                    red.reduce(op, out, shard, mask)
                    want = whole._red(name, dims).raw()
                    got = be.download(out)
                    if is_f and name in ("sum", "mean"):
                        assert_ulp(got, want, dt, 2, f"{name} {mask}")
                    else:
                        assert_bitwise(got, want, out_dt, f"{name} {mask}")
                # all / any (0/1 results combine as minimum / maximum); variance and standard deviation in two rounds
                for name, op in (("all", ffi.HMC_REDUCE_ALL), ("any", ffi.HMC_REDUCE_ANY)):
                    out = be.empty(shape, BOOL)
                    red.reduce(op, out, shard, mask)
                    assert_bitwise(be.download(out), whole._red(name, dims).raw(), BOOL, f"{name} {mask}")
                if is_f:
                    for correction, take_sqrt in ((1, False), (0, True)):
                        out = be.empty(shape, dt)
                        red.var(out, shard, mask, correction, take_sqrt)
                        w = whole.std_dim(dims, correction) if take_sqrt else whole.var_dim(dims, correction)
                        got = be.download(out)
                        assert_ulp(got, w.raw(), dt, 2, f"var/std {mask} correction {correction}")
            for is_max in (True, False):
                v, i = be.empty((cols,), dt), be.empty((cols,), I64)
                red.arg_reduce(v, i, shard, is_max)
                wv, wi = whole.max_dim(0) if is_max else whole.min_dim(0)
                assert_bitwise(be.download(i), wi.raw(), I64, "global indices")
                assert_bitwise(be.download(v), wv.raw(), dt, "values")
        # more ranks than rows: rank 1 holds an empty block. Sums, products, means, variances, all / any take the
        # identity from it; max / min / argmax are refused on every rank before anything is exchanged.
        from homura_b200.host import BackendError, F64, TensorData
        one_row = rng.standard_normal((1, cols)).astype(np.float32)
        blocks = split_rows(1, world)
        assert blocks[1] == (1, 0)
        start, length = blocks[rank]
        red = ShardedReducer(be, GlooComm(world, rank), [b[0] for b in blocks], 1)
        whole, shard = T(be, be.upload(one_row, F32)), be.upload(one_row[start:start + length], F32)
        for name, op in (("sum", ffi.HMC_REDUCE_SUM), ("prod", ffi.HMC_REDUCE_PROD), ("mean", ffi.HMC_REDUCE_MEAN)):
            out = be.empty((cols,), F32)
            red.reduce(op, out, shard, [True, False])
            assert_bitwise(be.download(out), whole._red(name, [0]).raw(), F32, f"{name} with an empty block")
        for name, op in (("all", ffi.HMC_REDUCE_ALL), ("any", ffi.HMC_REDUCE_ANY)):
            out = be.empty((cols,), BOOL)
            red.reduce(op, out, shard, [True, False])
            assert_bitwise(be.download(out), whole._red(name, [0]).raw(), BOOL, f"{name} with an empty block")
        ishard = be.upload(np.arange(cols, dtype=np.int32).reshape(1, cols)[start:start + length], I32)
        out = be.empty((), I64)
        red.reduce(ffi.HMC_REDUCE_SUM, out, ishard, [True, True])
        assert int(be.download(out)) == cols * (cols - 1) // 2
        out = be.empty((cols,), F32)
        red.var(out, shard, [True, False], 0, False)
        assert (be.download(out) == 0).all()
        for refused in (lambda: red.reduce(ffi.HMC_REDUCE_MAX, be.empty((cols,), F32), shard, [True, False]),
                        lambda: red.reduce(ffi.HMC_REDUCE_MIN, be.empty((), F32), shard, [True, True]),
                        lambda: red.arg_reduce(be.empty((cols,), F32), be.empty((cols,), I64), shard, True)):
            try:
                refused()
                raise AssertionError("an empty block was accepted")
            except BackendError as e:
                assert e.status == ffi.HMC_INVALID and "nonempty block on every rank" in str(e)
        # the ranks' f64 partials (one per tensor of an optimizer step) folded in order, then in rank order
        parts = np.array([0.5, 1e-30, 3.0, -1.25][: 4 - rank], dtype=np.float64)  # 4 partials on rank 0, 3 on rank 1
        store = be.upload(parts, F64).storage
        total = be.empty((), F64)
        red.sum_f64(total, store, parts.size)
        want = (0.5 + 1e-30 + 3.0 - 1.25) + (0.5 + 1e-30 + 3.0)
        assert float(be.download(total)) == want
        results[rank] = "ok"
    except BaseException as e:  # report to the parent instead of dying silently
        import traceback
        results[rank] = "".join(traceback.format_exception(e))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_single_rank_results():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}, "\n".join(str(v) for v in results.values())


def _leaving_worker(rank, world, port, store_path, results):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import time
        from homura_b200 import ffi
        from homura_b200.host import BackendError, F32
        from homura_b200.shard import RankWatch, ShardedReducer, split_rows
        from oracle_backend import OracleBackend

        be = OracleBackend()
        rows, cols = 10, 7
        blocks = split_rows(rows, world)
        start, length = blocks[rank]
        watch = RankWatch(dist.FileStore(store_path, world), rank, world)
        red = ShardedReducer(be, GlooComm(world, rank), [b[0] for b in blocks], rows, watch=watch)
        full = np.arange(rows * cols, dtype=np.float32).reshape(rows, cols)
        shard = be.upload(full[start:start + length], F32)
        out = be.empty((cols,), F32)
        red.reduce(ffi.HMC_REDUCE_SUM, out, shard, [True, False])       # a step with everybody there
        assert (be.download(out) == full.sum(axis=0)).all()
        dist.barrier()
        if rank == 1:
            watch.leave("finished early")                                # between steps, nothing in flight
            results[rank] = "left"
            return
        deadline = time.time() + 20
        while True:                                                      # the peers learn of it on the host ...
            try:
                watch.check()
            except BackendError:
                break
            assert time.time() < deadline, "the departure never showed in the store"
            time.sleep(0.05)
        try:                                                             # ... and queue no collective that would wait for it
            red.reduce(ffi.HMC_REDUCE_SUM, out, shard, [True, False])
            results[rank] = "the collective was queued although a rank had left"
        except BackendError as e:
            assert e.status == ffi.HMC_CUDA_ERROR and "rank 1 has left" in str(e)
            results[rank] = "ok"
    except BaseException as e:
        import traceback
        results[rank] = "".join(traceback.format_exception(e))
    finally:
        dist.destroy_process_group()


def test_a_rank_that_leaves_between_steps_is_noticed_before_the_next_collective(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_leaving_worker, args=(2, port, str(tmp_path / "ranks"), results), nprocs=2, join=True)
    assert dict(results) == {0: "ok", 1: "left"}, "\n".join(str(v) for v in results.values())


def test_split_rows():
    from homura_b200.shard import split_rows
    assert split_rows(10, 4) == [(0, 3), (3, 3), (6, 3), (9, 1)]
    assert split_rows(8, 8) == [(i, 1) for i in range(8)]
    assert split_rows(3, 4) == [(0, 1), (1, 1), (2, 1), (3, 0)]
    assert split_rows(1 << 32, 8)[7] == (7 << 29, 1 << 29)
