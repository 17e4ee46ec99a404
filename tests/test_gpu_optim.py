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
