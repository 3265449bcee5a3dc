"""Backward of dense min / max reductions: the winner of every segment (arg-reduction rule: NaN beats
numbers, lowest index among equals) receives the segment's gradient, every other element is exactly
zero (reference: AutoDiff.cpp:5036-5050, ReduceMinMaxBackwardKernel.cu:151-192)."""
import numpy as np
import pytest
import torch

from thor_b200 import DataType
from thor_b200.expression import Expression as ex
from thor_b200.reductions import ReduceMinMaxBackward

pytestmark = pytest.mark.gpu


def _want(x: np.ndarray, g: np.ndarray, is_max: bool) -> np.ndarray:
    """x [outer, red, inner] float64 (NaN allowed), g [outer, inner]."""
    key = np.where(np.isnan(x), np.inf if is_max else -np.inf, x)
    # NaN wins: give it the extreme key; among several NaNs / equal values the first index wins, which argmax / argmin do
    has_nan = np.isnan(x).any(axis=1, keepdims=True)
    key = np.where(has_nan & ~np.isnan(x), -np.inf if is_max else np.inf, key)
    win = key.argmax(axis=1) if is_max else key.argmin(axis=1)
    out = np.zeros_like(x)
    o, i = np.meshgrid(np.arange(x.shape[0]), np.arange(x.shape[2]), indexing="ij")
    out[o, win, i] = g
    return out


@pytest.mark.parametrize("is_max", [True, False])
@pytest.mark.parametrize("outer,red,inner", [(64, 4096, 1), (1, 100000, 1), (33, 1000, 1), (7, 37, 1), (1, 4096, 512), (16, 300, 24), (5, 9, 3), (3, 1, 40)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_route_matches_the_definition(is_max, outer, red, inner, dtype):
    g = torch.Generator(device="cuda").manual_seed(outer * 31 + red)
    x = torch.randn(outer, red, inner, device="cuda", generator=g).to(dtype)
    grad = torch.randn(outer, inner, device="cuda", generator=g)
    op = ReduceMinMaxBackward(is_max, x, grad, outer, red, inner)
    got = op.run()
    torch.cuda.synchronize()
    assert got.dtype == dtype
    want = _want(x.double().cpu().numpy(), grad.double().cpu().numpy(), is_max)
    want_t = torch.from_numpy(want).to(dtype)  # one rounding of the routed gradient to the storage dtype
    assert torch.equal(got.cpu().float(), want_t.float())
    assert int((got != 0).sum()) <= outer * inner


def test_ties_go_to_the_first_index_and_nan_wins():
    x = torch.tensor([[1.0, 5.0, 5.0, 2.0], [3.0, float("nan"), 9.0, float("nan")], [-1.0, -1.0, -1.0, -1.0]], device="cuda").reshape(3, 4, 1)
    grad = torch.tensor([[10.0], [20.0], [30.0]], device="cuda")
    got = ReduceMinMaxBackward(True, x, grad, 3, 4, 1).run().reshape(3, 4).cpu().numpy()
    assert np.array_equal(got, np.array([[0, 10, 0, 0], [0, 20, 0, 0], [30, 0, 0, 0]], dtype=np.float32))
    got = ReduceMinMaxBackward(False, x, grad, 3, 4, 1).run().reshape(3, 4).cpu().numpy()
    assert np.array_equal(got, np.array([[10, 0, 0, 0], [0, 20, 0, 0], [30, 0, 0, 0]], dtype=np.float32))


@pytest.mark.parametrize("axes,gshape", [([1], (96, 1)), ([0], (1, 640)), ([], (1,))])
def test_autodiff_of_reduce_max_uses_the_route_stage(axes, gshape):
    x = torch.randn(96, 640, device="cuda")
    g = torch.randn(*gshape, device="cuda")
    eq = ex.compile({"m": (ex.input("x") * 2.0).reduce_max(axes)})
    plan = eq.compile_backward(["x"]).stamp({"x": x, "__grad_output": g})
    plan.run()
    torch.cuda.synchronize()
    assert "ReduceMinMaxBackward" in plan.stage_kind_names() and "minmax_backward" in plan.physical_stage_names()
    xt = x.clone().requires_grad_(True)
    y = xt * 2.0
    m = y.amax(dim=axes[0], keepdim=True) if axes else y.max().reshape(1)
    m.backward(g)  # continuous random data: no ties, so torch's rule and the arg rule agree
    assert torch.allclose(plan.output("x_grad"), xt.grad, rtol=1e-6, atol=0)


def test_min_backward_in_bf16_keeps_the_input_dtype():
    x = torch.randn(128, 256, device="cuda").bfloat16()
    g = torch.randn(128, 1, device="cuda").bfloat16()
    plan = ex.compile({"m": ex.input("x").reduce_min([1])}).compile_backward(["x"]).stamp({"x": x, "__grad_output": g})
    plan.run()
    torch.cuda.synchronize()
    dx = plan.output("x_grad")
    assert dx.dtype == torch.bfloat16
    idx = x.float().argmin(dim=1)
    want = torch.zeros_like(x)
    want[torch.arange(128, device="cuda"), idx] = g[:, 0]
    assert torch.equal(dx, want)
