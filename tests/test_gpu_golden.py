"""homura's golden cases for the hot path (PyTorch results) on the CUDA library, at homura's tolerances."""
import pytest

import golden_cases

pytestmark = pytest.mark.gpu


def test_every_hot_path_golden_case_passes_on_the_gpu(cuda):
    assert golden_cases.run_all(cuda) >= 180
