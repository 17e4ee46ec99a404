"""Pins the CPU checker: homura's golden cases for the hot path (PyTorch results at homura's tolerances) and
its Adam / AdamW fixtures bit for bit."""
import pytest

import golden_cases
import optim_cases


def test_every_hot_path_golden_case_passes_on_the_oracle(oracle):
    assert golden_cases.run_all(oracle) >= 180


@pytest.mark.parametrize("case", optim_cases.cases("adam_steps.safetensors"))
def test_adam_multi_step_bitwise(oracle, case):
    optim_cases.multi_step(oracle, case)


@pytest.mark.parametrize("case", optim_cases.cases("adam_edges.safetensors"))
def test_adam_edge_values_bitwise(oracle, case):
    optim_cases.edge_values(oracle, case)


@pytest.mark.parametrize("case", [c for c in optim_cases.cases("adam_steps.safetensors")
                                  if optim_cases.fusable("adam_steps.safetensors", c)])
def test_one_call_adamw_step_of_the_oracle_matches_the_fixtures(oracle, case):
    optim_cases.multi_step(oracle, case, fused_kernel=True)
