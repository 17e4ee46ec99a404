"""homura's bitwise Adam / AdamW fixtures (tests/optim.rs:159-244) on the CUDA library: op by op, and
through the single fused kernel, which must leave the same bits; and fused vs op-by-op on larger tensors in
mixed layouts (homura requires the update not to depend on layout, tests/optim.rs:430-480)."""
import numpy as np
import pytest

import optim_cases
from homura_b200.host import BF16, DTYPE_NAMES, F16, F32, F64, FLOATS
from optim_protocol import Adam
from test_gpu_reduce import normal
from values import assert_bitwise, f64_to_storage

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", optim_cases.cases("adam_steps.safetensors"))
def test_adam_multi_step_bitwise(cuda, case):
    optim_cases.multi_step(cuda, case)


@pytest.mark.parametrize("case", optim_cases.cases("adam_edges.safetensors"))
def test_adam_edge_values_bitwise(cuda, case):
    optim_cases.edge_values(cuda, case)


@pytest.mark.parametrize("case", [c for c in optim_cases.cases("adam_steps.safetensors")
                                  if optim_cases.fusable("adam_steps.safetensors", c)])
def test_fused_adamw_kernel_matches_the_fixtures(cuda, case):
    optim_cases.multi_step(cuda, case, fused_kernel=True)


@pytest.mark.parametrize("case", [c for c in optim_cases.cases("adam_edges.safetensors")
                                  if optim_cases.fusable("adam_edges.safetensors", c)])
def test_fused_adamw_kernel_matches_the_edge_fixtures(cuda, case):
    optim_cases.edge_values(cuda, case, fused_kernel=True)


@pytest.mark.parametrize("dtype", FLOATS, ids=[DTYPE_NAMES[d] for d in FLOATS])
def test_fused_kernel_equals_op_by_op_in_any_layout(oracle, cuda, dtype):
    rows, cols = 257, 1030
    p0 = f64_to_storage(normal(rows * cols, 131, 0.02), dtype)
    grads = [f64_to_storage(normal(rows * cols, 132 + t, 1e-3), dtype) for t in range(3)]
    results = []
    for be, fused, transposed in ((oracle, False, False), (cuda, False, False), (cuda, True, False), (cuda, True, True)):
        if transposed:
            # parameter and gradient are transposed views of [cols, rows] storage; the state is contiguous
            to_t = lambda raw: be.upload(np.ascontiguousarray(raw.reshape(rows, cols).T), dtype, (cols, rows)).t()
        else:
            to_t = lambda raw: be.upload(raw, dtype, (rows, cols))
        p = to_t(p0)
        opt = Adam(be, [(1e-3, [p])], betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, amsgrad=False, maximize=False,
                   decoupled=True)
        for t in range(3):
            opt.step({id(p): to_t(grads[t])}, fused_kernel=fused)
        st = opt.state[id(p)]
        results.append([be.download(x) for x in (p, st.exp_avg, st.exp_avg_sq)])
    for other in results[1:]:
        for got, want, what in zip(other, results[0], ("param", "exp_avg", "exp_avg_sq")):
            # f16 moments underflow to 0 here, so 0/0 appears: a NaN only has to meet a NaN
            assert_bitwise(got, want, dtype, what)


@pytest.mark.parametrize("dtype", FLOATS, ids=[DTYPE_NAMES[d] for d in FLOATS])
def test_many_tensors_in_one_launch_equal_the_per_tensor_kernel(oracle, cuda, dtype):
    """hmc_adamw_step_many over a group of tensors of very different sizes (empty, a few elements, just below and
    above a chunk, several chunks, a view that does not start on a 32-byte boundary, a transposed view that goes
    through the per-tensor kernel) leaves the bits of hmc_adamw_step on each, three steps in a row; the sums of
    squared gradients are those of `g.mul(g).sum()` before its last rounding (f64, within 1e-12 relative of the
    CPU checker's sequential sum) and identical from run to run."""
    from homura_b200 import ffi
    sizes = [0, 1, 7, 512, 4095, 4096, 4097, 8192 * 3 + 5, 100_000, 1 << 20]
    steps = 3
    hyper = dict(lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)

    def tensors(be, offset_views):
        out = []
        for i, n in enumerate(sizes):
            raw_p = f64_to_storage(normal(n + 3, 500 + i, 0.02), dtype)
            raw_g = f64_to_storage(normal(n + 3, 600 + i, 1e-3), dtype)
            p, g = be.upload(raw_p, dtype), be.upload(raw_g, dtype)
            m, v = be.empty((n + 3,), dtype), be.empty((n + 3,), dtype)
            be.fill(m, 0.0)
            be.fill(v, 0.0)
            start = 3 if (offset_views and i % 2) else 0  # odd tensors start 3 elements into their storage
            out.append(tuple(t.narrow(0, start, n) for t in (p, g, m, v)))
        return out

    single, many = tensors(cuda, True), tensors(cuda, True)
    rows, cols = 70, 130
    raw = f64_to_storage(normal(rows * cols, 700, 0.02), dtype)
    rawg = f64_to_storage(normal(rows * cols, 701, 1e-3), dtype)
    def transposed(be):
        p, g = be.upload(raw, dtype, (cols, rows)).t(), be.upload(rawg, dtype, (cols, rows)).t()
        m, v = be.empty((rows, cols), dtype), be.empty((rows, cols), dtype)
        be.fill(m, 0.0)
        be.fill(v, 0.0)
        return (p, g, m, v)
    single_t, many_t = transposed(cuda), transposed(cuda)
    group = cuda.adamw_group(many, with_grad_sq=True)
    mixed = cuda.adamw_group([many_t], with_grad_sq=False)
    assert len(mixed.strided) == 1 and len(group.flat) == len(sizes)
    squares = []
    for t in range(1, steps + 1):
        for p, g, m, v in single + [single_t]:
            cuda.adamw_step(p, g, m, v, step=float(t), **hyper)
        group.step(step=float(t), **hyper)
        mixed.step(step=float(t), **hyper)
        squares.append(group.grad_squares())
    for i, (a, b) in enumerate(zip(single + [single_t], many + [many_t])):
        for x, y, what in zip(a, b, ("param", "grad", "exp_avg", "exp_avg_sq")):
            assert_bitwise(cuda.download(y), cuda.download(x), dtype, f"tensor {i} {what}")
    assert all((s == squares[0]).all() for s in squares[1:]), "the sums of squares changed between identical steps"
    # against the CPU checker: g * g rounded to the dtype, summed in f64
    for i, (_, g, _, _) in enumerate(many):
        og = oracle.upload(cuda.download(g), dtype)
        sq = oracle.empty(og.shape, dtype)
        oracle.binary(ffi.HMC_BINARY_MUL, sq, og, og)
        from values import storage_to_f64
        want = float(np.sum(storage_to_f64(oracle.download(sq), dtype), dtype=np.float64)) if sizes[i] else 0.0
        assert abs(squares[0][i] - want) <= 1e-12 * abs(want), f"sum of squares of tensor {i}: {squares[0][i]} vs {want}"


def test_many_tensor_step_refuses_a_small_workspace(cuda):
    import ctypes
    from homura_b200 import ffi
    from homura_b200.host import adamw_scalars
    t = [cuda.empty((5000,), F32) for _ in range(4)]
    group = cuda.adamw_group([t])
    sc = adamw_scalars(F32, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1.0)
    status = cuda.lib.hmc_adamw_step_many(cuda.ctx, F32, group.table, 1, ctypes.byref(sc), None, group.workspace.ptr, 16)
    assert status == ffi.HMC_INVALID and b"too small" in cuda.lib.hmc_last_error()
    status = cuda.lib.hmc_adamw_step_many(cuda.ctx, ffi.HMC_I32, group.table, 1, ctypes.byref(sc), None, group.workspace.ptr,
                                          group.workspace.nbytes)
    assert status == ffi.HMC_INVALID
