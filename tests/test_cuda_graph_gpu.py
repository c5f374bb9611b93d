"""The ops can be captured in a CUDA graph (no allocation outside torch's allocator, no
synchronisation, launches on the current stream): a forward+backward pair is captured once and
replayed on new inputs."""
import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200 import workloads
from conftest import rel_err
from oracle import cport

pytestmark = pytest.mark.gpu


def test_lti_forward_backward_replays_in_a_graph():
    w = workloads.lti_first_order(B=16, T=20000)
    a, zi, x, gy = (w[k].cuda() for k in ("a", "zi", "x", "gy"))
    ops = torch.ops.philtorch_b200

    def step():
        y = ops.lti_recur(a, zi, x)
        ga, gzi, gx = ops.lti_recur_bwd(a, zi, y, gy, None, True, True)
        return y, ga, gx

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):   # first launches set kernel attributes: outside the capture
            step()
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y, ga, gx = step()
    # new inputs in the captured buffers
    g = torch.Generator().manual_seed(7)
    x2 = torch.randn(x.shape, generator=g)
    x.copy_(x2)
    graph.replay()
    torch.cuda.synchronize()
    y_ref = cport.lti_recur(w["a"], w["zi"], x2)
    ga_ref, _, gx_ref = cport.lti_recur_bwd(w["a"], w["zi"], y_ref, w["gy"])
    assert rel_err(y, y_ref) <= 1e-4 and rel_err(gx, gx_ref) <= 1e-4 and rel_err(ga, ga_ref) <= 1e-4
    ptb.check_errors()


def test_spline_prefilter_replays_in_a_graph():
    """The public call with its autograd graph: few long rows (cut into pieces), forward + backward
    captured once and replayed on a new signal; no host-to-device copy and no synchronisation on the way."""
    from oracle import callers
    from philtorch_b200.lti.interp import cspline
    g = torch.Generator().manual_seed(5)
    x0 = torch.randn(2, 1 << 16, generator=g)
    x = x0.cuda().requires_grad_()
    gy = torch.randn(2, 1 << 16, generator=g).cuda()

    def step():
        c = cspline(x)
        return c, torch.autograd.grad(c, x, gy)[0]

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        c, gx = step()
    x2 = torch.randn(x0.shape, generator=g)
    with torch.no_grad():
        x.copy_(x2)
    graph.replay()
    torch.cuda.synchronize()
    assert rel_err(c.detach(), torch.from_numpy(callers.cspline(x2.double().numpy(), False))) <= 1e-4
    xe = x2.cuda().requires_grad_()
    ce = cspline(xe, parallel_form=False)           # whole rows, other kernels, eager
    assert rel_err(gx, torch.autograd.grad(ce, xe, gy)[0]) <= 1e-4
    ptb.check_errors()
