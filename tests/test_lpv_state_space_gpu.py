"""lpv.state_space on the kernels: every case of the reference-made golden file (state dimensions
2 and 3, all accepted shapes of B, C and D, with and without zi, out_idx)."""
import pytest

import philtorch_b200 as ptb
from state_space_common import load_cases, run_case

pytestmark = pytest.mark.gpu
CASES = load_cases()


@pytest.mark.parametrize("case", sorted(CASES))
def test_state_space_golden(case):
    run_case(CASES[case], "cuda", ptb.lpv.state_space)
    ptb.check_errors()
