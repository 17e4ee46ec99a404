"""Benchmark of the elementwise / reduction hot path on B200: achieved HBM GB/s by algorithmic bytes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2|c3|c4|c5|inputs|all]

The headline (top-level `value`, `e2e`, `roofline`) is the elementwise / broadcast configuration, one step =
    x bf16 [8192, 8192] ~ N(0, 1), bias f32 [8192, 1], scale bf16 [1, 8192]
    y  = silu(x)     * scale + bias   (bf16 + f32 -> f32)          3 kernels
    yt = silu(x.t()) * scale + bias   (transposed, non-contiguous)  3 kernels
    c  = x.to(f32)                    (contiguous cast copy)        1 kernel
through the C ABI of include/homura_cuda.h, outputs preallocated from the caching allocator.
Algorithmic bytes per step (distinct input elements + output elements, temporaries count zero):
silu 4N, mul 4N, promoting add 6N (twice), cast 6N, with N = 8192^2: 34 N = 2281.7 MB.

The same run adds, under `workloads`, one record per other configuration, each kernel timed alone with L2 flushed
before it (a "whole step" of reductions over one input would be served from L2 and is not reported). The flush
writes a 512 MB buffer and reads it back, so that the L2 holds unmodified lines when the timed kernel starts (after
a write-only flush a read-only kernel is charged the write-back of the flush buffer; each record's `flush` entry
shows the difference on its first kernel):
    c3  reductions of f32 / i32 [16384, 4096] (sum, mean, var over rows and columns, max + argmax, full sums)
    c4  softmax / log_softmax of causally masked f32 [8, 32, 2048, 2048], row mean of squares of bf16 [32768, 4096]
    fused  the headline expression silu(x) * scale + bias, contiguous and on x.t(), as one kernel each (6 bytes per
        element instead of 14, the three kernels' bits)
    c5  one GPU's eighth of the sharded configuration: a * b + c on flat f32 2^29, its sum and maximum, and an
        AdamW step (lr 1e-4, wd 0.01) over the 291 Llama-3-8B-shaped f32 tensors (1/8 of the rows of each,
        1 003 782 656 parameters, one launch) with the gradient norm
and, with N > 1 ranks (torchrun), a `sharded` record: the c5 step with its tensors being shards of global ones,
so that the global sum, maximum and gradient norm gather the ranks' partials over NCCL (all-gather) and fold them
in rank order inside the timed region, next to the same rank's unsharded timings.

`value` is the whole job's GB/s with inputs resident in HBM: the timed region of K steps is repeated and the
median repeat is reported (minimum alongside); `e2e` is the same metric with the inputs coming from pinned host
memory and the results going back to it inside the timed region, every step, by the blocking copy calls of the C
ABI; two threads with a context each take the steps in turn, so that one step's results and the next step's
inputs cross PCIe at the same time. With N > 1 ranks every rank runs the headline workload on its own GPU:
independent replicas, weak scaling, no data-path collective; the time is the maximum over ranks. `--impl
reference` times the CPU restatement of homura's single-threaded CPU backend on a bounded sample of the same
workload on the host cores.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS = COLS = 8192
N2 = ROWS * COLS
STEP_BYTES = 34 * N2
METRIC = "hbm_gbs_algorithmic"
UNIT = "GB/s"
WORKLOAD = "c2_elementwise_broadcast_bf16_8192x8192"
REPEATS = 7
# dram__bytes_read.sum + dram__bytes_write.sum per launch of each kernel of the headline step, from one ncu
# capture on B200 (summarised under profiles/). Writes are below the algorithmic output where the
# tail of the output still sits in L2 when the capture ends.
NCU_TRAFFIC_BYTES = {"silu": 216.6e6, "mul_scale": 213.2e6, "add_bias": 342.4e6, "silu_t": 215.0e6, "mul_scale_t": 213.4e6,
                     "add_bias_t": 343.6e6, "cast": 343.6e6}


def philox_normal(n: int, seed: int) -> np.ndarray:
    """Seeded N(0, 1) values (numpy's Philox bit generator), float32."""
    return np.random.Generator(np.random.Philox(seed)).standard_normal(n, dtype=np.float32)


def f32_to_bf16_bits(f: np.ndarray) -> np.ndarray:
    x = f.astype(np.float32).view(np.uint32).astype(np.uint64)
    return ((x + 0x7FFF + ((x >> 16) & 1)) >> 16).astype(np.uint16)


def peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 50 ms while running."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, period_ms: int = 50):
        self.index, self.period_ms, self.proc, self.lines = index, period_ms, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
            deadline = time.time() + 3.0   # the first sample takes a moment: have one before the timed work starts
            while not self.lines and time.time() < deadline:
                time.sleep(0.01)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(2 * self.period_ms / 1e3)
            self.proc.terminate()
            self.proc.wait()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "period_ms": self.period_ms}


class Workload:
    """The headline step on one backend (device tensors and preallocated outputs)."""

    name = WORKLOAD
    dtype = "bf16"

    def __init__(self, be, rows: int = ROWS, cols: int = COLS, seed: int = 0):
        from homura_b200.host import BF16, F32
        self.be, self.rows, self.cols = be, rows, cols
        self.host_x = f32_to_bf16_bits(philox_normal(rows * cols, 11 + seed)).reshape(rows, cols)
        self.host_bias = philox_normal(rows, 12 + seed).reshape(rows, 1)
        self.host_scale = f32_to_bf16_bits(philox_normal(cols, 13 + seed)).reshape(1, cols)
        self.x = be.upload(self.host_x, BF16)
        self.bias = be.upload(self.host_bias, F32)
        self.scale = be.upload(self.host_scale, BF16)
        self.s = be.empty((rows, cols), BF16)      # silu(x), then silu(x) * scale
        self.st = be.empty((cols, rows), BF16)     # the same for x.t()
        self.y = be.empty((rows, cols), F32)
        self.yt = be.empty((cols, rows), F32)
        self.c = be.empty((rows, cols), F32)
        self.launches_per_step = 7
        n = rows * cols
        self.op_bytes = {"silu": 4 * n, "mul_scale": 4 * n + 2 * cols, "add_bias": 6 * n + 4 * rows,
                         "silu_t": 4 * n, "mul_scale_t": 4 * n + 2 * rows, "add_bias_t": 6 * n + 4 * cols, "cast": 6 * n}

    def ops(self):
        from homura_b200 import ffi
        be, r, c = self.be, self.rows, self.cols
        xt = self.x.t()
        # for the transposed product the roles of the broadcast operands swap: scale spans the rows of x.t()
        scale_t = self.scale.reshape(c, 1).expand(c, r)
        bias_t = self.bias.reshape(1, r).expand(c, r)
        return [
            ("silu", lambda: be.unary(ffi.HMC_UNARY_SILU, self.s, self.x)),
            ("mul_scale", lambda: be.binary(ffi.HMC_BINARY_MUL, self.s, self.s, self.scale.expand(r, c))),
            ("add_bias", lambda: be.binary_promoted(ffi.HMC_BINARY_ADD, self.y, self.s, self.bias.expand(r, c))),
            ("silu_t", lambda: be.unary(ffi.HMC_UNARY_SILU, self.st, xt)),
            ("mul_scale_t", lambda: be.binary(ffi.HMC_BINARY_MUL, self.st, self.st, scale_t)),
            ("add_bias_t", lambda: be.binary_promoted(ffi.HMC_BINARY_ADD, self.yt, self.st, bias_t)),
            ("cast", lambda: be.copy(self.c, self.x)),
        ]

    def step(self):
        for _, f in self.ops():
            f()


class FusedWorkload:
    """The headline expression y = silu(x) * scale + bias, and the same on x.t(), each as ONE kernel that keeps the two
    intermediates in registers and rounds them where the three kernels would (same bits): 6 bytes per element (read x,
    write the f32 result) instead of the 14 the three-kernel form moves."""

    name = "c2_fused_expression_bf16_8192x8192"
    dtype = "bf16"

    def __init__(self, be, rows: int = ROWS, cols: int = COLS, seed: int = 0):
        w = Workload(be, rows, cols, seed)
        self.w, self.be = w, be
        n = rows * cols
        self.op_bytes = {"silu_mul_add": 6 * n + 2 * cols + 4 * rows, "silu_mul_add_t": 6 * n + 2 * rows + 4 * cols}
        self.launches_per_step = 2
        # dram read + write bytes per launch from an ncu capture of this workload at this size
        self.ncu_traffic = {"silu_mul_add": 345.6e6, "silu_mul_add_t": 350.0e6} if (rows, cols) == (ROWS, COLS) else {}

    def ops(self):
        from homura_b200 import ffi
        be, w = self.be, self.w
        r, c = w.rows, w.cols
        args = (ffi.HMC_UNARY_SILU, ffi.HMC_BINARY_MUL, ffi.HMC_BINARY_ADD)
        return [
            ("silu_mul_add", lambda: be.unary_binary_binary(*args, w.y, w.x, w.scale, w.bias)),
            ("silu_mul_add_t", lambda: be.unary_binary_binary(*args, w.yt, w.x.t(), w.scale.reshape(c, 1), w.bias.reshape(1, r))),
        ]

    def step(self):
        for _, f in self.ops():
            f()


def _tile_fill(be, big, small):
    """Fills the contiguous `big` with repetitions of the contiguous `small` (a device-side broadcast copy)."""
    n = small.numel
    flat = big.reshape(big.numel)
    reps = flat.numel // n
    if reps:
        be.copy(flat.narrow(0, 0, reps * n).reshape(reps, n), small.reshape(1, n).expand(reps, n))
    rest = flat.numel - reps * n
    if rest:
        be.copy(flat.narrow(0, reps * n, rest), small.reshape(n).narrow(0, 0, rest))


class C3Workload:
    """Reductions of f32 / i32 [16384, 4096]."""

    name = "c3_reductions_16384x4096"
    dtype = "f32 / i32, accumulated in f64 / i64"

    def __init__(self, be, seed: int = 0):
        from homura_b200.host import F32, I32, I64
        self.be = be
        r, c = 16384, 4096
        n = r * c
        self.x = be.upload(philox_normal(n, 21 + seed).reshape(r, c), F32)
        rng = np.random.Generator(np.random.Philox(22 + seed))
        self.i = be.upload(rng.integers(-1000, 1001, size=(r, c), dtype=np.int32), I32)
        e = be.empty
        self.out = {"rows_f": e((r,), F32), "cols_f": e((c,), F32), "full_f": e((), F32), "rows_idx": e((r,), I64),
                    "rows_i": e((r,), I64), "cols_i": e((c,), I64), "full_i": e((), I64), "rows_iv": e((r,), I32)}
        b4 = 4 * n
        self.op_bytes = {k: b4 for k in ["sum_rows", "mean_rows", "var_rows", "sum_cols", "mean_cols", "var_cols", "max_rows",
                                         "sum_full", "isum_rows", "isum_cols", "imax_rows", "isum_full"]}
        self.launches_per_step = 12
        # dram read + write bytes per launch from an ncu capture of this workload (every input is read once)
        self.ncu_traffic = {"sum_rows": 273.0e6, "mean_rows": 270.0e6, "var_rows": 268.9e6, "sum_cols": 269.5e6, "mean_cols": 269.7e6,
                            "var_cols": 271.6e6, "max_rows": 270.7e6, "sum_full": 272.2e6, "isum_rows": 268.7e6, "isum_cols": 269.6e6,
                            "imax_rows": 269.0e6, "isum_full": 268.6e6}

    def ops(self):
        from homura_b200 import ffi
        be, x, i, o = self.be, self.x, self.i, self.out
        R, C, A = [False, True], [True, False], [True, True]
        return [
            ("sum_rows", lambda: be.reduce(ffi.HMC_REDUCE_SUM, o["rows_f"], x, R)),
            ("mean_rows", lambda: be.reduce(ffi.HMC_REDUCE_MEAN, o["rows_f"], x, R)),
            ("var_rows", lambda: be.var(o["rows_f"], x, R, 1.0, False)),
            ("sum_cols", lambda: be.reduce(ffi.HMC_REDUCE_SUM, o["cols_f"], x, C)),
            ("mean_cols", lambda: be.reduce(ffi.HMC_REDUCE_MEAN, o["cols_f"], x, C)),
            ("var_cols", lambda: be.var(o["cols_f"], x, C, 1.0, False)),
            ("max_rows", lambda: be.arg_reduce(o["rows_f"], o["rows_idx"], x, 1, True)),
            ("sum_full", lambda: be.reduce(ffi.HMC_REDUCE_SUM, o["full_f"], x, A)),
            ("isum_rows", lambda: be.reduce(ffi.HMC_REDUCE_SUM, o["rows_i"], i, R)),
            ("isum_cols", lambda: be.reduce(ffi.HMC_REDUCE_SUM, o["cols_i"], i, C)),
            ("imax_rows", lambda: be.arg_reduce(o["rows_iv"], o["rows_idx"], i, 1, True)),
            ("isum_full", lambda: be.reduce(ffi.HMC_REDUCE_SUM, o["full_i"], i, A)),
        ]

    def step(self):
        for _, f in self.ops():
            f()

    def size_sweep(self, runner) -> dict:
        """The row, column and full sums and the row variance on 1, 4 and 8 copies of the input (268 MB, 1 GB, 2 GB), each
        kernel alone with L2 flushed: what a launch costs at the start and the end shrinks with the size, what the kernel
        sustains does not."""
        from homura_b200 import ffi
        from homura_b200.host import F32
        be = self.be
        r, c = self.x.shape
        out = {}
        for copies in (1, 4, 8):
            x = self.x if copies == 1 else be.empty((copies * r, c), F32)
            if copies > 1:
                _tile_fill(be, x, self.x)
            rows_f, full_f = be.empty((copies * r,), F32), be.empty((), F32)
            ops = [("sum_rows", lambda: be.reduce(ffi.HMC_REDUCE_SUM, rows_f, x, [False, True])),
                   ("var_rows", lambda: be.var(rows_f, x, [False, True], 1.0, False)),
                   ("sum_cols", lambda: be.reduce(ffi.HMC_REDUCE_SUM, self.out["cols_f"], x, [True, False])),
                   ("var_cols", lambda: be.var(self.out["cols_f"], x, [True, False], 1.0, False)),
                   ("sum_full", lambda: be.reduce(ffi.HMC_REDUCE_SUM, full_f, x, [True, True]))]
            per_op = runner.flushed_per_op(ops, reps=7)
            nbytes = 4 * copies * r * c
            out[f"{nbytes / 1e6:.0f} MB"] = {k: {"gbs": nbytes / (v * 1e-3) / 1e9, "ms": v} for k, v in per_op.items()}
            del x, rows_f, full_f
        return out


class C4Workload:
    """softmax / log_softmax of causally masked f32 logits [8, 32, 2048, 2048] and the row mean of squares of
    bf16 [32768, 4096] as homura's rms_norm composes it (to f32, pow 2, mean)."""

    name = "c4_softmax_8x32x2048x2048"
    dtype = "f32 / bf16, row maths in f64"

    def __init__(self, be, seed: int = 0, batch: int = 256):
        from homura_b200.host import BF16, BOOL, F32
        self.be = be
        n = 2048
        logits = (3.0 * philox_normal(n * n, 31 + seed)).reshape(n, n)
        one = be.upload(logits, F32)
        self.logits = be.empty((batch, n, n), F32)
        _tile_fill(be, self.logits, one)
        self.mask = be.upload(np.triu(np.ones((n, n), dtype=np.uint8), 1), BOOL)
        self.masked = be.empty((batch, n, n), F32)
        self.soft = be.empty((batch, n, n), F32)
        k_rows, k_cols = 32768, 4096
        self.h = be.upload(f32_to_bf16_bits(philox_normal(k_rows * k_cols, 32 + seed)).reshape(k_rows, k_cols), BF16)
        self.h32 = be.empty((k_rows, k_cols), F32)
        self.ms = be.empty((k_rows, 1), F32)
        m = batch * n * n
        k = k_rows * k_cols
        self.op_bytes = {"masked_fill": 8 * m + n * n, "softmax": 8 * m, "log_softmax": 8 * m, "to_f32": 6 * k, "pow2": 8 * k,
                         "mean_rows": 4 * k + 4 * k_rows}
        self.launches_per_step = 6
        # dram read + write bytes per launch: an ncu capture of a 16-matrix slice (488.4 and 485.2 MB per 16 matrices of
        # 2048 x 2048), scaled to this batch: rows are independent, so traffic grows in proportion
        self.ncu_traffic = {"softmax": 488.4e6 * batch / 16, "log_softmax": 485.2e6 * batch / 16}

    def ops(self):
        from homura_b200 import ffi
        be = self.be
        b, n = self.logits.shape[0], 2048
        mask = self.mask.reshape(1, n, n).expand(b, n, n)
        return [
            ("masked_fill", lambda: be.where_constant(self.masked, mask, float("-inf"), self.logits)),
            ("softmax", lambda: be.softmax(self.soft, self.masked, 2, False)),
            ("log_softmax", lambda: be.softmax(self.soft, self.masked, 2, True)),
            ("to_f32", lambda: be.copy(self.h32, self.h)),
            ("pow2", lambda: be.binary_constant(ffi.HMC_BINARY_POW, self.h32, self.h32, 2.0, False)),
            ("mean_rows", lambda: be.reduce(ffi.HMC_REDUCE_MEAN, self.ms, self.h32, [False, True])),
        ]

    def step(self):
        for _, f in self.ops():
            f()


def llama3_8b_shapes() -> list:
    """The 291 parameter tensors of Llama-3-8B (8 030 261 248 elements): embedding, 32 layers of (q, k, v, o, gate,
    up, down, two norm weights), the final norm and the output head."""
    shapes = [(128256, 4096)]
    for _ in range(32):
        shapes += [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (14336, 4096), (14336, 4096), (4096, 14336),
                   (4096,), (4096,)]
    shapes += [(4096,), (128256, 4096)]
    return shapes


class C5Workload:
    """One GPU's eighth of the configuration sharded over 8 GPUs: a * b + c on flat f32 tensors of 2^29 elements
    (2^32 / 8), their sum and maximum, and an AdamW step (lr 1e-4, wd 0.01) over the Llama-3-8B-shaped f32
    parameters with the gradient norm. Every parameter tensor is split by rows, so a rank holds rows / 8 of each
    of the 291 tensors. With a `reducer` the tensors are shards of global ones and the reductions that fold the
    sharded dimension exchange their partials over the communicator."""

    name = "c5_flat_elementwise_adamw_llama3_8b_shard"
    dtype = "f32, sums in f64"
    SHARDS = 8

    def __init__(self, be, seed: int = 0, log2n: int = 29, reducer=None, param_scale: int = 1):
        from homura_b200.host import F32, F64
        self.be, self.reducer = be, reducer
        n = 1 << log2n
        base = [be.upload(philox_normal(1 << 22, 41 + seed + j), F32) for j in range(3)]
        self.a, self.b, self.c = (be.empty((n,), F32) for _ in range(3))
        for t, s0 in zip((self.a, self.b, self.c), base):
            _tile_fill(be, t, s0)
        self.t = be.empty((n,), F32)
        self.s = be.empty((), F32)
        # AdamW: params N(0, 0.02), grads N(0, 1e-3), moments start at 0; `param_scale` > 1 shrinks every tensor's
        # rows further (for short profiler captures)
        p0 = be.upload(0.02 * philox_normal(1 << 22, 51 + seed), F32)
        g0 = be.upload(1e-3 * philox_normal(1 << 22, 52 + seed), F32)
        self.tensors = []
        for shape in llama3_8b_shapes():
            local = (max(1, shape[0] // (self.SHARDS * param_scale)),) + tuple(shape[1:])
            p, g, m, v = (be.empty(local, F32) for _ in range(4))
            _tile_fill(be, p, p0)
            _tile_fill(be, g, g0)
            be.fill(m, 0.0)
            be.fill(v, 0.0)
            self.tensors.append((p, g, m, v))
        self.params = sum(t[0].numel for t in self.tensors)
        self.group = be.adamw_group(self.tensors, with_grad_sq=True)
        self.norm_sq = be.empty((), F64)
        self.norm = be.empty((), F64)
        self.step_no = 0
        self.op_bytes = {"mul": 12 * n, "add": 12 * n, "sum": 4 * n, "max": 4 * n,
                         "adamw_291_tensors": 28 * self.params, "grad_norm": 8 * len(self.tensors)}
        self.launches_per_step = 4 + 2 + 2 + (3 if reducer is not None else 0) * 2
        # dram read + write bytes per launch of the AdamW kernel: an ncu capture at 1/64 of the model's rows (3.457 GB for
        # 125.5 M parameters: 27.5 bytes a parameter), scaled by the parameters of this launch
        self.ncu_traffic = {"adamw_291_tensors": 27.55 * self.params}

    def ops(self):
        from homura_b200 import ffi
        from homura_b200.host import F64, TensorData
        be = self.be

        def adamw():
            self.step_no += 1
            self.group.step(lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=float(self.step_no))

        # with several ranks the tensors are shards of a global one: the reductions fold the sharded dimension, so
        # they gather the ranks' partials over NCCL and combine them in rank order
        if self.reducer is not None:
            reduce = lambda op: self.reducer.reduce(op, self.s, self.t, [True])
            norm_sq = lambda: self.reducer.sum_f64(self.norm_sq, self.group.grad_sq, len(self.tensors))
        else:
            reduce = lambda op: be.reduce(op, self.s, self.t, [True])
            partials = TensorData(self.group.grad_sq, F64, (len(self.tensors),), (1,))
            norm_sq = lambda: be.reduce(ffi.HMC_REDUCE_SUM, self.norm_sq, partials, [True])

        def grad_norm():
            # the per-tensor sums of squares come out of the AdamW launch; fold them (across ranks too) and root
            norm_sq()
            be.unary(ffi.HMC_UNARY_SQRT, self.norm, self.norm_sq)
        return [
            ("mul", lambda: be.binary(ffi.HMC_BINARY_MUL, self.t, self.a, self.b)),
            ("add", lambda: be.binary(ffi.HMC_BINARY_ADD, self.t, self.t, self.c)),
            ("sum", lambda: reduce(ffi.HMC_REDUCE_SUM)),
            ("max", lambda: reduce(ffi.HMC_REDUCE_MAX)),
            ("adamw_291_tensors", adamw),
            ("grad_norm", grad_norm),
        ]

    def step(self):
        for _, f in self.ops():
            f()


class InputsWorkload:
    """The step before the path in every config: the samplers that make the inputs (rand bf16 [8192, 8192],
    randn f32 [16384, 4096], randint over a range that rejects words and one that does not) and the causal mask
    in front of the softmax (triu on f32 [64, 2048, 2048], and the Bool mask itself). Bytes are those written,
    plus the triangle's reads of the kept half."""

    name = "inputs_samplers_and_mask"
    dtype = "bf16 / f32 / i64"

    def __init__(self, be, seed: int = 0):
        from homura_b200.host import BF16, BOOL, F32, I64, Generator
        self.be = be
        self.gen = Generator(1234 + seed)
        self.u = be.empty((8192 * 8192,), BF16)
        self.n = be.empty((16384 * 4096,), F32)
        self.i = be.empty((1 << 26,), I64)
        b, m = 64, 2048
        self.logits = be.empty((b, m, m), F32)
        be.fill(self.logits, 1.0)
        self.masked = be.empty((b, m, m), F32)
        self.ones = be.empty((m, m), BOOL)
        be.fill(self.ones, True)
        self.mask = be.empty((m, m), BOOL)
        # an embedding lookup: 32768 rows of a bf16 [128256, 4096] table (Llama-3 vocabulary and width)
        vocab, width, tokens = 128256, 4096, 32768
        self.table = be.empty((vocab, width), BF16)
        be.fill(self.table, 0.5)
        self.tokens = be.empty((tokens,), I64)
        be.random_int(self.tokens, self.gen, 0, vocab)
        self.embedded = be.empty((tokens, width), BF16)
        # and its backward pass: the rows' gradients added into a table-shaped gradient in token order (index_add:
        # keys, three sort passes of four launches, the adding kernel); about vocab * (1 - exp(-tokens / vocab))
        # distinct rows are read and written
        self.table_grad = be.empty((vocab, width), BF16)
        be.fill(self.table_grad, 0.0)
        touched = int(vocab * (1.0 - math.exp(-tokens / vocab)))
        e = b * m * m
        self.op_bytes = {"embedding_bf16": 4 * tokens * width + 8 * tokens,
                         "embedding_grad_bf16": 2 * tokens * width + 4 * touched * width + 8 * tokens, "rand_bf16": 2 * self.u.numel, "randn_f32": 4 * self.n.numel, "randint_pow2": 8 * self.i.numel,
                         "randint_reject": 8 * self.i.numel, "triu_f32": 4 * e + 2 * e, "mask_bool": m * m + m * m // 2}
        self.launches_per_step = 24

    def ops(self):
        be = self.be
        return [
            ("embedding_bf16", lambda: be.index_select(self.embedded, self.table, 0, self.tokens)),
            ("embedding_grad_bf16", lambda: be.index_add(self.table_grad, 0, self.tokens, self.embedded)),
            ("rand_bf16", lambda: be.random_uniform(self.u, self.gen, 0.0, 1.0)),
            ("randn_f32", lambda: be.random_normal(self.n, self.gen, 0.0, 1.0)),
            ("randint_pow2", lambda: be.random_int(self.i, self.gen, 0, 1 << 16)),
            ("randint_reject", lambda: be.random_int(self.i, self.gen, -3, 50257)),
            ("triu_f32", lambda: be.triangle(self.masked, self.logits, 1, True)),
            ("mask_bool", lambda: be.triangle(self.mask, self.ones, 1, True)),
        ]

    def step(self):
        for _, f in self.ops():
            f()


class Events:
    def __init__(self, be):
        self.be = be

    def new(self):
        ev = ctypes.c_void_p()
        self.be._check(self.be.lib.hmc_event_create(self.be.ctx, ctypes.byref(ev)))
        return ev

    def record(self, ev):
        self.be._check(self.be.lib.hmc_event_record(self.be.ctx, ev))

    def elapsed(self, a, b) -> float:
        ms = ctypes.c_float()
        self.be._check(self.be.lib.hmc_event_elapsed_ms(a, b, ctypes.byref(ms)))
        return ms.value

    def destroy(self, ev):
        self.be.lib.hmc_event_destroy(ev)


class Runner:
    """Timing of one backend's work with events on its stream; with several ranks every region starts at a
    barrier and its time is the maximum over ranks."""

    def __init__(self, be, dist, local: int, world: int):
        self.be, self.dist, self.local, self.world = be, dist, local, world
        self.ev = Events(be)
        self.scratch = None
        self.scratch_sum = None

    def barrier(self):
        self.be.synchronize()
        if self.dist is not None:
            import torch
            self.dist.barrier(device_ids=[self.local])
            torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.dist is None:
            return list(values)
        import torch
        t = torch.tensor(list(values), device="cuda", dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def timed_steps(self, w, steps: int, warmup: int, repeats: int) -> list:
        """`repeats` regions of exactly `steps` steps each after `warmup` steps; ms per region, max over ranks."""
        for _ in range(warmup):
            w.step()
        out = []
        self.host_ms_per_region = []  # how long the host took to queue a region (well below the region: not host-bound)
        start, stop = self.ev.new(), self.ev.new()
        for _ in range(repeats):
            self.barrier()
            t0 = time.perf_counter()
            self.ev.record(start)
            for _ in range(steps):
                w.step()
            self.ev.record(stop)
            self.host_ms_per_region.append((time.perf_counter() - t0) * 1e3)
            self.be.synchronize()
            out.append(self.ev.elapsed(start, stop))
        self.barrier()
        self.ev.destroy(start)
        self.ev.destroy(stop)
        return self.max_over_ranks(out)

    def flush(self, i: int = 0, read_back: bool = True) -> None:
        """Empties the L2 of anything the next kernel could hit: 512 MB (four times the L2) are written, then read
        back. The read matters for what is timed next: after a write alone the L2 is full of modified lines, and a
        kernel that only reads then pays, in its own time, for writing up to 126 MB of the flush buffer back to HBM
        (measured here: +13 us on a 268 MB read, which caps it near 4.8 TB/s). After the read the L2 holds the same
        lines unmodified, and evicting them costs nothing."""
        from homura_b200 import ffi
        from homura_b200.host import I64, U8, TensorData
        be = self.be
        if self.scratch is None:
            self.scratch = be.storage(512 << 20)
            self.scratch_sum = be.empty((), I64)
        be._check(be.lib.hmc_memset(be.ctx, self.scratch.ptr, i & 0xFF, self.scratch.nbytes))
        if read_back:
            be.reduce(ffi.HMC_REDUCE_SUM, self.scratch_sum, TensorData(self.scratch, U8, (self.scratch.nbytes,), (1,)), [True])

    def flushed_per_op(self, ops, reps: int = 10, warm: int = 3, read_back: bool = True) -> dict:
        """Mean ms of each op alone, the L2 emptied before every launch (see flush).

        The host must not be what is timed: an op whose launch reaches the stream after the flush before it has
        finished shows the host's delay as device time between its two events (seen here as a constant 8 us on the ops
        whose Python glue also asks for a workspace). So all iterations of an op are queued without waiting in between,
        each behind a flush that is longer on the device (the buffer is written twice) than an iteration takes to
        queue; the warm-up iterations absorb the start. The record carries both rates so that this can be checked."""
        ev = self.ev
        per_op = {}
        pairs = [(ev.new(), ev.new()) for _ in range(warm + reps)]
        self.host_ms_per_iteration, self.device_ms_per_iteration = 0.0, float("inf")
        self.queue_rates = {}
        for name, f in ops:
            self.be.synchronize()
            t0 = time.perf_counter()
            for i, (a, b) in enumerate(pairs):
                self.flush(i + 1, read_back=False)
                self.flush(i, read_back)
                ev.record(a)
                f()
                ev.record(b)
            host_ms = (time.perf_counter() - t0) * 1e3 / len(pairs)
            self.be.synchronize()
            device_ms = ev.elapsed(pairs[0][0], pairs[-1][1]) / (len(pairs) - 1)
            self.queue_rates[name] = (host_ms, device_ms)
            self.host_ms_per_iteration = max(self.host_ms_per_iteration, host_ms)
            self.device_ms_per_iteration = min(self.device_ms_per_iteration, device_ms)
            per_op[name] = float(np.mean([ev.elapsed(a, b) for a, b in pairs[warm:]]))
        for a, b in pairs:
            ev.destroy(a)
            ev.destroy(b)
        return per_op


def roofline_of(w, per_op: dict, traffic: dict | None = None) -> dict:
    """The roofline entry of a workload: its kernel furthest below the HBM peak that carries real traffic (ops
    of a few KB, such as folding 291 partial sums, are launch-bound and not measured against bandwidth)."""
    peak, peak_kind = peaks()
    gbs = {k: w.op_bytes[k] / (v * 1e-3) / 1e9 for k, v in per_op.items()}
    streaming = [k for k in per_op if w.op_bytes[k] >= (64 << 20)] or list(per_op)
    dominant = max(per_op, key=per_op.get)
    worst = min(streaming, key=lambda k: gbs[k])
    total_ms = sum(per_op.values())
    def entry(k):
        return {"bound": "hbm", "kernel": k, "achieved": gbs[k], "peak": peak, "peak_kind": peak_kind, "unit": UNIT,
                "frac": gbs[k] / peak, "traffic": (traffic or {}).get(k), "algorithmic_bytes": w.op_bytes[k],
                "share_of_step": per_op[k] / total_ms}
    return {"dominant": entry(dominant), "worst": entry(worst), "per_kernel_gbs": gbs, "per_kernel_ms": per_op}


def workload_record(runner: Runner, w, steps: int, warmup: int) -> dict:
    """One `workloads` entry: every kernel alone with L2 flushed (the honest per-kernel figures, and their sum as
    the step), plus the same step back to back."""
    per_op = runner.flushed_per_op(w.ops())
    rates = (runner.host_ms_per_iteration, runner.device_ms_per_iteration)
    queue_rates = dict(runner.queue_rates)
    per_op = dict(zip(per_op.keys(), runner.max_over_ranks(per_op.values())))
    regions = runner.timed_steps(w, steps, warmup, 3)
    step_bytes = sum(w.op_bytes.values())
    flushed_ms = sum(per_op.values())
    r = roofline_of(w, per_op, getattr(w, "ncu_traffic", None))
    back_ms = float(np.median(regions)) / steps
    # what the flush's read-back is worth: the first op again after a flush that only writes
    first = w.ops()[:1]
    write_only = runner.max_over_ranks(runner.flushed_per_op(first, read_back=False).values())[0]
    flush_note = {"op": first[0][0], "ms_after_write_then_read_flush": per_op[first[0][0]], "ms_after_write_only_flush": write_only,
                  "note": "a flush that only writes leaves the L2 full of modified lines whose write-back is then charged to the "
                          "timed kernel; the figures of this record are taken after a flush that writes and reads back"}
    flush_note["host_ms_to_queue_an_iteration"], flush_note["device_ms_per_iteration"] = rates
    flush_note["host_and_device_ms_per_iteration_by_op"] = queue_rates
    extra = {"size_sweep": w.size_sweep(runner)} if hasattr(w, "size_sweep") and runner.world == 1 else {}
    return {"workload": w.name, "dtype": w.dtype, "metric": METRIC, "unit": UNIT, "flush": flush_note,
            "value": step_bytes / (flushed_ms * 1e-3) / 1e9, "ms_per_step": flushed_ms,
            "value_basis": "sum of the kernels' times, each alone with L2 flushed before it",
            "back_to_back": {"value": step_bytes / (back_ms * 1e-3) / 1e9, "ms_per_step": back_ms,
                             "note": "consecutive kernels over one input are partly served from the 126 MB L2"},
            "algorithmic_bytes_per_step": step_bytes, "kernels_per_step": w.launches_per_step,
            "roofline": dict(r["worst"], per_kernel_gbs=r["per_kernel_gbs"], per_kernel_ms=r["per_kernel_ms"]),
            "frac_of_measured_copy": {k: v / r["worst"]["peak"] for k, v in r["per_kernel_gbs"].items()}, **extra}


def cpu_sample(seconds_budget: float = 20.0) -> dict:
    """The CPU restatement of homura's CPU backend (single-threaded, as the original is by construction:
    every kernel runs inside one global lock, src/backend/cpu/mod.rs:40-64) on rows of the same workload."""
    sys.path.insert(0, str(ROOT / "tests"))
    from oracle_backend import OracleBackend
    be = OracleBackend()
    rows = 256
    w = Workload(be, rows=rows, cols=COLS)
    w.step()  # warm the pages
    t0 = time.perf_counter()
    reps = 0
    while True:
        w.step()
        reps += 1
        if time.perf_counter() - t0 > seconds_budget or reps >= 64:
            break
    dt = time.perf_counter() - t0
    nbytes = 34 * rows * COLS * reps
    return {"value": nbytes / dt / 1e9, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": f"{reps} passes of the 7-kernel step on x bf16 [{rows}, {COLS}] ({rows * COLS} of {N2} elements per pass)",
            "seconds": dt}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, str(ROOT / "tests"))
    from oracle_backend import OracleBackend
    be = OracleBackend()
    rows = 1024
    w = Workload(be, rows=rows, cols=COLS)
    for _ in range(args.warmup):
        w.step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        w.step()
    dt = time.perf_counter() - t0
    value = 34 * rows * COLS * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": f"each step covers x bf16 [{rows}, {COLS}] of [{ROWS}, {COLS}]"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 1, "kind": "port",
                         "sample": f"{args.steps} steps of the 7-kernel pass on {rows} of {ROWS} rows; homura's CPU "
                                   "backend is single-threaded by construction"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def end_to_end(be, w, runner: Runner, rank: int, steps: int) -> dict:
    """The headline step with its inputs coming from pinned host memory and its three results going back to it
    inside the timed region, every step, through the blocking copies of the C ABI."""
    from homura_b200.host import CudaBackend

    def pinned(nbytes):
        p = ctypes.c_void_p()
        be._check(be.lib.hmc_host_alloc(nbytes, ctypes.byref(p)))
        return p
    hx, hb, hs = pinned(w.host_x.nbytes), pinned(w.host_bias.nbytes), pinned(w.host_scale.nbytes)
    ctypes.memmove(hx, w.host_x.ctypes.data, w.host_x.nbytes)
    ctypes.memmove(hb, w.host_bias.ctypes.data, w.host_bias.nbytes)
    ctypes.memmove(hs, w.host_scale.ctypes.data, w.host_scale.nbytes)
    out_bytes = 4 * N2
    hy, hyt, hc = pinned(out_bytes), pinned(out_bytes), pinned(out_bytes)
    h2d = w.host_x.nbytes + w.host_bias.nbytes + w.host_scale.nbytes
    d2h = 3 * out_bytes

    # Two lanes, as two threads of a homura program would run them: each has its own context (stream), its own device
    # tensors and result buffers, and makes the same blocking calls; while one lane's results travel to the host the
    # other lane's inputs travel to the device (PCIe carries both directions at once) and its kernels run.
    be2 = CudaBackend(be.device)
    w2 = Workload(be2, seed=rank)
    hy2, hyt2, hc2 = pinned(out_bytes), pinned(out_bytes), pinned(out_bytes)
    lanes = [(be, w, (hy, hyt, hc)), (be2, w2, (hy2, hyt2, hc2))]

    def e2e_step(lane):
        b, wl, (y, yt, c) = lane
        lib, ctx = b.lib, b.ctx
        b._check(lib.hmc_copy_from_host(ctx, wl.x.storage.ptr, hx, w.host_x.nbytes))
        b._check(lib.hmc_copy_from_host(ctx, wl.bias.storage.ptr, hb, w.host_bias.nbytes))
        b._check(lib.hmc_copy_from_host(ctx, wl.scale.storage.ptr, hs, w.host_scale.nbytes))
        wl.step()
        b._check(lib.hmc_copy_to_host(ctx, y, wl.y.storage.ptr, out_bytes))
        b._check(lib.hmc_copy_to_host(ctx, yt, wl.yt.storage.ptr, out_bytes))
        b._check(lib.hmc_copy_to_host(ctx, c, wl.c.storage.ptr, out_bytes))

    def run_lanes(counts):
        failures = []

        def body(lane, count):
            try:
                for _ in range(count):
                    e2e_step(lane)
            except BaseException as e:  # reported by the main thread
                failures.append(e)
        other = threading.Thread(target=body, args=(lanes[1], counts[1]))
        other.start()
        body(lanes[0], counts[0])
        other.join()
        be2.synchronize()
        if failures:
            raise failures[0]

    e2e_steps = max(4, min(steps, 10))
    run_lanes((2, 2))
    runner.barrier()
    start, stop = runner.ev.new(), runner.ev.new()
    runner.ev.record(start)
    run_lanes((e2e_steps - e2e_steps // 2, e2e_steps // 2))
    runner.ev.record(stop)  # after the other lane's work has completed: the region covers both
    be.synchronize()
    e2e_ms = runner.max_over_ranks([runner.ev.elapsed(start, stop)])[0]
    for p in (hx, hb, hs, hy, hyt, hc, hy2, hyt2, hc2):
        be.lib.hmc_host_free(p)
    be2.close()
    return {"value": STEP_BYTES * e2e_steps * runner.world / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / e2e_steps, "lanes": 2, "steps": e2e_steps}


def sharded_record(be, runner: Runner, rank: int, world: int, steps: int, warmup: int) -> dict:
    """The c5 step on `world` ranks whose tensors are the shards of global ones: per rank the same work as one GPU's
    share, plus, inside the timed region, the exchange the global sum, maximum and gradient norm need (an NCCL
    all-gather of 8 bytes per rank and a rank-ordered combine kernel each)."""
    from homura_b200 import ffi
    from homura_b200.shard import NcclComm, ShardedReducer
    box = [NcclComm.unique_id() if rank == 0 else None]
    runner.dist.broadcast_object_list(box, src=0)
    comm = NcclComm(be, world, rank, box[0])
    n_local = 1 << 29
    reducer = ShardedReducer(be, comm, [r * n_local for r in range(world)], world * n_local)
    w = C5Workload(be, seed=rank, log2n=29, reducer=reducer)
    alone = C5Workload.__new__(C5Workload)      # the same tensors without the exchange, for the per-op comparison
    alone.__dict__.update(w.__dict__)
    alone.reducer = None
    step_bytes = sum(w.op_bytes.values())
    regions = runner.timed_steps(w, steps, warmup, REPEATS)
    regions_alone = runner.timed_steps(alone, steps, warmup, 3)
    per_op = runner.flushed_per_op(w.ops())
    per_op = dict(zip(per_op.keys(), runner.max_over_ranks(per_op.values())))
    per_op_alone = runner.flushed_per_op(alone.ops())
    per_op_alone = dict(zip(per_op_alone.keys(), runner.max_over_ranks(per_op_alone.values())))
    # the exchange by itself: all-gather of one f64 per rank and the combine kernel, on an 8-byte partial
    from homura_b200.host import F64, TensorData
    part = be.storage(8)
    be.fill(TensorData(part, F64, (1,), (1,)), 1.0)
    exchange = runner.flushed_per_op([("allgather_8_bytes_per_rank_and_combine",
                                       lambda: be.shard_combine_float(ffi.HMC_REDUCE_SUM, w.s, reducer._gather(part, 8), world, 1, world))])
    exchange_ms = runner.max_over_ranks(exchange.values())[0]
    med = float(np.median(regions))
    med_alone = float(np.median(regions_alone))
    rec = {"workload": w.name + "_sharded", "dtype": w.dtype, "metric": METRIC, "unit": UNIT, "ranks": world,
           "collective": "ncclAllGather of the ranks' 8-byte partials + rank-ordered combine kernel, three per step "
                         "(global sum, global maximum, gradient norm), on the compute stream",
           "value": step_bytes * steps * world / (med * 1e-3) / 1e9, "ms_per_step": med / steps,
           "value_min_time": step_bytes * steps * world / (min(regions) * 1e-3) / 1e9,
           "repeats": len(regions), "steps_per_repeat": steps,
           "unsharded_same_ranks": {"value": step_bytes * steps * world / (med_alone * 1e-3) / 1e9, "ms_per_step": med_alone / steps},
           "algorithmic_bytes_per_step_per_rank": step_bytes,
           "per_op_ms_sharded": per_op, "per_op_ms_unsharded": per_op_alone,
           "exchange_ms": exchange_ms, "exchange_share_of_step": 3 * exchange_ms / sum(per_op.values()),
           "params_per_rank": w.params}
    comm.close()
    return rec


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="all", choices=["all", "c2", "c3", "c4", "c5", "fused", "inputs"],
                    help="all (default): the headline with the c3 / c4 / c5 records (and the sharded record with several "
                         "ranks); c2: the headline alone; another name: that workload's record alone")
    ap.add_argument("--c4-batch", type=int, default=256,
                    help="matrices of [2048, 2048] logits in the c4 workload (256 = [8, 32, 2048, 2048]); a smaller "
                         "number keeps a profiler capture short")
    ap.add_argument("--c5-log2n", type=int, default=29,
                    help="log2 of the elements of the flat c5 tensors (29 = one GPU's eighth of 2^32); smaller for short "
                         "profiler captures")
    ap.add_argument("--c5-param-scale", type=int, default=1,
                    help="shrinks the rows of every AdamW tensor by this factor (for short profiler captures)")
    ap.add_argument("--profile", action="store_true",
                    help="only the warm-up and the timed steps of the chosen workload (no per-kernel loop, end-to-end "
                         "pass or CPU sample): the short command to run under ncu")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from homura_b200.host import CudaBackend
    be = CudaBackend(local)
    runner = Runner(be, dist, local, world)

    def make(name):
        if name == "c2":
            return Workload(be, seed=rank)
        if name == "c3":
            return C3Workload(be, seed=rank)
        if name == "c4":
            return C4Workload(be, seed=rank, batch=args.c4_batch)
        if name == "fused":
            return FusedWorkload(be, seed=rank)
        if name == "c5":
            return C5Workload(be, seed=rank, log2n=args.c5_log2n, param_scale=args.c5_param_scale)
        return InputsWorkload(be, seed=rank)

    def finish():
        be.close()
        if dist is not None:
            dist.destroy_process_group()

    if args.profile:
        w = make("c2" if args.workload == "all" else args.workload)
        regions = runner.timed_steps(w, args.steps, args.warmup, 1)
        if rank == 0:
            print(json.dumps({"metric": METRIC, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                              "value": sum(w.op_bytes.values()) * args.steps * world / (regions[0] * 1e-3) / 1e9,
                              "ms_per_step": regions[0] / args.steps, "profile_run": True, "workload": w.name,
                              "gpu_launches": w.launches_per_step * args.steps}))
        return finish()

    if args.workload not in ("all", "c2"):
        # one workload's record alone
        with ClockSampler(local) as clocks:
            rec = workload_record(runner, make(args.workload), args.steps, args.warmup)
        if rank == 0:
            rec.update({"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
                        "vs_baseline": None, "data": "synthetic", "config": {"workload": rec["workload"]},
                        "clocks": clocks.summary(), "gpu_launches": rec["kernels_per_step"] * (13 + 3 * args.steps + args.warmup)})
            print(json.dumps(rec))
        return finish()

    # ---- the headline: device-resident throughput, W warm-up steps, then REPEATS regions of exactly K steps ----
    w = make("c2")
    launches = 0
    with ClockSampler(local) as clocks:
        regions = runner.timed_steps(w, args.steps, args.warmup, REPEATS)
        launches += w.launches_per_step * (args.warmup + REPEATS * args.steps)
        per_op = runner.flushed_per_op(w.ops())
        per_op = dict(zip(per_op.keys(), runner.max_over_ranks(per_op.values())))
        launches += w.launches_per_step * 13
    ms = float(np.median(regions))
    host_ms_per_region = float(np.median(runner.host_ms_per_region))
    value = STEP_BYTES * args.steps * world / (ms * 1e-3) / 1e9
    peak, peak_kind = peaks()
    r = roofline_of(w, per_op, NCU_TRAFFIC_BYTES)
    roofline = dict(r["dominant"], per_kernel_gbs=r["per_kernel_gbs"], per_kernel_ms=r["per_kernel_ms"],
                    worst_kernel=r["worst"]["kernel"], worst_frac=r["worst"]["frac"])
    e2e = end_to_end(be, w, runner, rank, args.steps)
    launches += w.launches_per_step * (e2e["steps"] + 4)
    del w

    workloads, sharded = {}, None
    if args.workload == "all":
        with ClockSampler(local) as clocks2:
            names = ["fused", "c3", "c4", "c5"] if world == 1 else ["c5"]   # the others do not shard: one GPU only
            for name in names:
                wl = make(name)
                workloads[name] = workload_record(runner, wl, max(3, args.steps // 4), args.warmup)
                launches += wl.launches_per_step * (13 + 3 * max(3, args.steps // 4) + args.warmup)
                del wl
                be.synchronize()
                be.allocator.empty_cache()
            if world > 1:
                sharded = sharded_record(be, runner, rank, world, max(3, args.steps // 4), args.warmup)
        workloads_clocks = clocks2.summary()
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_sample()
    runner.barrier()
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows": ROWS, "cols": COLS, "kernels_per_step": 7,
                       "algorithmic_bytes_per_step": STEP_BYTES, "l2": "inputs_larger_than_l2 (x is 134 MB, outputs 268 MB)",
                       "ranks": "independent replicas of the step, one per GPU, no data-path collective" if world > 1 else "one GPU",
                       "elements_per_s": 7 * N2 * args.steps * world / (ms * 1e-3),
                       "frac_of_nominal_8tbs": value / world / 8000.0, "frac_of_measured_copy": value / world / peak},
            "repeats": {"n": len(regions), "steps_each": args.steps, "value_is": "median",
                        "gbs_median": value, "gbs_best": STEP_BYTES * args.steps * world / (min(regions) * 1e-3) / 1e9,
                        "gbs_worst": STEP_BYTES * args.steps * world / (max(regions) * 1e-3) / 1e9,
                        "ms_per_step_all": [t / args.steps for t in regions],
                        "host_ms_to_queue_a_region": host_ms_per_region, "device_ms_per_region": ms},
            "clocks": clocks.summary(),
            "e2e": e2e,
            "gpu_launches": 7 * args.steps * len(regions),
            "gpu_launches_whole_run": launches,
            "roofline": roofline,
            "cpu_baseline": cpu,
        }
        if workloads:
            line["workloads"] = workloads
            line["workloads_clocks"] = workloads_clocks
        if sharded is not None:
            line["sharded"] = sharded
        print(json.dumps(line))
    finish()


if __name__ == "__main__":
    main()
