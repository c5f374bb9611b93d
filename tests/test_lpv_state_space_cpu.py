"""lpv.state_space: the input / output / feed-through maps for every accepted shape of B, C and D,
against golden vectors made by running the reference's philtorch.lpv.state_space.  The recurrence
itself is replaced by a plain differentiable loop here, so the shape logic is checked without a
GPU (tests/test_lpv_state_space_gpu.py runs the same cases on the kernels)."""
import pytest
import torch

from state_space_common import load_cases, run_case

CASES = load_cases()


def _loop_recurrence(A, zi, x, *, out_idx=None, **_):
    M = A.size(-1)
    if x.dim() == 2:
        x = torch.cat([x.unsqueeze(-1), x.new_zeros(x.shape + (M - 1,))], dim=-1)
    h, out = zi, []
    for t in range(x.shape[1]):
        At = A[:, t] if A.dim() == 4 else A[t]
        h = (At @ h.unsqueeze(-1)).squeeze(-1) + x[:, t]
        out.append(h)
    y = torch.stack(out, 1)
    return y if out_idx is None else y[:, :, out_idx]


@pytest.mark.parametrize("case", sorted(CASES))
def test_state_space_maps(case, monkeypatch):
    from philtorch_b200.lpv import ssm

    monkeypatch.setattr(ssm, "_ext_ss_recur", _loop_recurrence)
    run_case(CASES[case], "cpu", ssm.state_space)


def test_rejected_shapes(monkeypatch):
    from philtorch_b200.lpv import ssm

    monkeypatch.setattr(ssm, "_ext_ss_recur", _loop_recurrence)
    A, x = torch.zeros(5, 2, 2), torch.zeros(3, 5)
    with pytest.raises(ValueError):
        ssm.state_space(A, x, B=torch.zeros(7, 9))
    with pytest.raises(ValueError):
        ssm.state_space(A, x, C=torch.zeros(2), out_idx=0)
    with pytest.raises(AssertionError):   # a per-state input vector needs a scalar sequence
        ssm.state_space(A, torch.zeros(3, 5, 4), B=torch.zeros(2))
