"""The sharded reductions on real GPUs: one process per GPU, NCCL all-gather of the partials, rank-ordered
combine. Needs at least two GPUs (skipped otherwise); every rank must hold the same bits, which must match the
CPU checker's result on the whole tensor (bit for bit for integers, extremes and indices; within 2 ulp for the
f64-accumulated float sums)."""
import ctypes
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _device_count():
    import homura_b200
    n = ctypes.c_int32()
    homura_b200.load().hmc_device_count(ctypes.byref(n))
    return n.value


def _worker(rank, world, unique_id, results):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        from frontend import T
        from homura_b200 import ffi
        from homura_b200.host import BF16, BOOL, F32, I32, I64, CudaBackend
        from homura_b200.shard import NcclComm, ShardedReducer, split_rows
        from oracle_backend import OracleBackend
        from values import assert_bitwise, assert_ulp, f64_to_storage

        be = CudaBackend(rank)
        comm = NcclComm(be, world, rank, unique_id)
        oracle = OracleBackend()
        rows, cols = 4099, 1030
        blocks = split_rows(rows, world)
        start, length = blocks[rank]
        red = ShardedReducer(be, comm, [b[0] for b in blocks], rows)
        rng = np.random.default_rng(11)
        data = {F32: rng.standard_normal((rows, cols)).astype(np.float32),
                BF16: f64_to_storage(rng.standard_normal((rows, cols)), BF16),
                I32: rng.integers(-1000, 1001, size=(rows, cols), dtype=np.int32)}
        data[F32][rows - 5, 5] = np.nan
        data[F32][3, 7] = data[F32][rows - 3, 7] = 9.0
        digest = []
        for dt, full in data.items():
            whole = T(oracle, oracle.upload(full, dt))
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
                    want, got = whole._red(name, dims).raw(), be.download(out)
                    if is_f and name in ("sum", "mean"):
                        assert_ulp(got, want, dt, 2, f"{name} {mask}")
                    else:
                        assert_bitwise(got, want, out_dt, f"{name} {mask}")
                    digest.append(got.tobytes())
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
                        digest.append(got.tobytes())
            for is_max in (True, False):
                v, i = be.empty((cols,), dt), be.empty((cols,), I64)
                red.arg_reduce(v, i, shard, is_max)
                wv, wi = whole.max_dim(0) if is_max else whole.min_dim(0)
                assert_bitwise(be.download(i), wi.raw(), I64, "global indices")
                assert_bitwise(be.download(v), wv.raw(), dt, "values")
        be.synchronize()
        comm.close()
        be.close()
        import hashlib
        results[rank] = "ok " + hashlib.sha256(b"".join(digest)).hexdigest()
    except BaseException as e:
        import traceback
        results[rank] = "".join(traceback.format_exception(e))


def test_sharded_reductions_over_nccl():
    n = _device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = min(n, 4)
    import multiprocessing as mp
    from homura_b200.shard import NcclComm
    uid = NcclComm.unique_id()
    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    results = manager.dict()
    procs = [ctx.Process(target=_worker, args=(r, world, uid, results)) for r in range(world)]
    [p.start() for p in procs]
    [p.join(timeout=300) for p in procs]
    for p in procs:
        if p.is_alive():
            p.kill()
    got = dict(results)
    assert len(got) == world and all(v.startswith("ok ") for v in got.values()), "\n".join(str(v) for v in got.values())
    assert len(set(got.values())) == 1, "ranks disagree on the bits of the results"


def _failure_worker(rank, world, unique_id, store_path, results):
    """Rank 1 first stalls (stays alive but skips a collective), then leaves between steps after saying so; rank 0
    must come back from both with an error status and a usable context, never waiting for ever."""
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        import time
        import torch.distributed as dist
        from homura_b200 import ffi
        from homura_b200.host import F32, BackendError, CudaBackend
        from homura_b200.shard import NcclComm, RankWatch, ShardedReducer, split_rows

        be = CudaBackend(rank)
        store = dist.FileStore(store_path, world)
        watch = RankWatch(store, rank, world)
        rows, cols = 64, 128
        blocks = split_rows(rows, world)
        start, length = blocks[rank]
        full = np.arange(rows * cols, dtype=np.float32).reshape(rows, cols) % 97
        shard = be.upload(full[start:start + length], F32)
        out = be.empty((cols,), F32)

        # 1. a peer that is alive but never joins a collective: the bounded wait gives up, the communicator is
        #    aborted, the context keeps working
        comm = NcclComm(be, world, rank, unique_id[0])
        comm.set_timeout(20.0)
        red = ShardedReducer(be, comm, [b[0] for b in blocks], rows)
        red.reduce(ffi.HMC_REDUCE_SUM, out, shard, [True, False])
        comm.wait()
        assert (be.download(out) == full.sum(axis=0)).all()
        store.set(f"first/{rank}", "done")
        if rank == 0:
            while not store.check(["first/1"]):
                time.sleep(0.01)
            comm.set_timeout(1.5)
            t0 = time.time()
            red.reduce(ffi.HMC_REDUCE_SUM, out, shard, [True, False])     # rank 1 does not take part
            try:
                comm.wait()
                outcome = "the wait came back although the peer never joined"
            except BackendError as e:
                took = time.time() - t0
                assert e.status == ffi.HMC_CUDA_ERROR and "aborted" in str(e), str(e)
                assert took < 15.0, f"gave up only after {took:.1f} s"
                outcome = "ok"
            try:
                red.reduce(ffi.HMC_REDUCE_SUM, out, shard, [True, False])
                outcome = "an aborted communicator accepted a collective"
            except BackendError as e:
                assert e.status == ffi.HMC_INVALID
            # the context still works: an ordinary reduction of the shard
            local = be.empty((cols,), F32)
            be.reduce(ffi.HMC_REDUCE_SUM, local, shard, [True, False])
            assert (be.download(local) == full[start:start + length].sum(axis=0)).all()
            store.set("stall/over", "1")
            comm.close()
            if outcome != "ok":
                results[rank] = outcome
                return
        else:
            while not store.check(["stall/over"]):                         # alive, but absent from the collective
                time.sleep(0.01)
            comm.abort()                                                   # its peer is gone from this communicator
            comm.close()

        # 2. a fresh communicator; rank 1 leaves between steps and says so; rank 0 sees it before queuing anything
        comm = NcclComm(be, world, rank, unique_id[1])
        comm.set_timeout(20.0)
        red = ShardedReducer(be, comm, [b[0] for b in blocks], rows, watch=watch)
        red.reduce(ffi.HMC_REDUCE_MAX, out, shard, [True, False])
        comm.wait()
        assert (be.download(out) == full.max(axis=0)).all()
        store.set(f"second/{rank}", "done")
        if rank == 1:
            while not store.check(["second/0"]):
                time.sleep(0.01)
            watch.leave("finished early")
            comm.abort()
            comm.close()
            be.close()
            results[rank] = "left"
            return
        deadline = time.time() + 30
        while True:
            try:
                watch.check()
            except BackendError:
                break
            assert time.time() < deadline, "the departure never showed in the store"
            time.sleep(0.02)
        try:
            red.reduce(ffi.HMC_REDUCE_MAX, out, shard, [True, False])
            results[rank] = "the collective was queued although a rank had left"
            return
        except BackendError as e:
            assert "rank 1 has left" in str(e)
        comm.abort()
        comm.close()
        be.synchronize()
        be.close()
        results[rank] = "ok"
    except BaseException as e:
        import traceback
        results[rank] = "".join(traceback.format_exception(e))


def test_a_stalled_or_departed_rank_does_not_hang_its_peer(tmp_path):
    """Two ranks on two GPUs, NVLS off, plain NCCL point-to-point: the failures are made on the host (a rank that
    sits out a collective; a rank that announces that it leaves between steps, nothing in flight)."""
    if _device_count() < 2:
        pytest.skip("needs at least two GPUs")
    import multiprocessing as mp
    from homura_b200.shard import NcclComm
    uids = [NcclComm.unique_id(), NcclComm.unique_id()]
    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    results = manager.dict()
    procs = [ctx.Process(target=_failure_worker, args=(r, 2, uids, str(tmp_path / "ranks"), results)) for r in range(2)]
    [p.start() for p in procs]
    [p.join(timeout=240) for p in procs]
    for p in procs:
        if p.is_alive():
            p.kill()
    assert dict(results) == {0: "ok", 1: "left"}, "\n".join(str(v) for v in dict(results).values())
