"""The first-class softmax / log-softmax op (reference: Expression.cpp:3724-3748, executed by cuDNN in
StampedEquation.cpp:1677-1688) routed to the row program.

cuDNN's arithmetic is not part of the reference's sources, so the oracle here is the mathematical
definition evaluated in float64 (parity unpinned beyond the tolerances the reference's own softmax
tests use): fp32 outputs <= 1e-5 relative, 16-bit outputs <= 1 output ulp."""
import numpy as np
import pytest
import torch

import oracle as o
from oracle import expr_oracle as eo
from thor_b200 import DataType
from thor_b200.expression import Expression as ex

pytestmark = pytest.mark.gpu

_TORCH = {DataType.fp32: torch.float32, DataType.fp16: torch.float16, DataType.bf16: torch.bfloat16}


def _ref(x64: np.ndarray, axes, algorithm: int) -> np.ndarray:
    m = x64.max(axis=axes, keepdims=True) if algorithm != 0 else 0.0
    d = x64 - m
    e = np.exp(d)
    s = e.sum(axis=axes, keepdims=True)
    return d - np.log(s) if algorithm == 2 else e / s


def _check(got: torch.Tensor, want64: np.ndarray, dtype: DataType):
    g = got.float().cpu().numpy().astype(np.float64)
    if dtype == DataType.fp32:
        np.testing.assert_allclose(g, want64, rtol=1e-5, atol=1e-7)
    else:
        d = eo.ulp_distance(g, want64, int(dtype))
        assert float(d.max()) <= 1.0, float(d.max())


@pytest.mark.parametrize("dtype", [DataType.fp32, DataType.bf16, DataType.fp16])
@pytest.mark.parametrize("rows,cols", [(64, 4096), (33, 1000), (1000, 40)])
def test_softmax_accurate_is_one_row_program(dtype, rows, cols):
    x = (torch.randn(rows, cols, device="cuda") * 3.0).to(_TORCH[dtype])
    plan = ex.compile(ex.input("x").softmax()).stamp({"x": x})
    plan.run()
    torch.cuda.synchronize()
    assert plan.physical_stage_names() == ["row_program"] and plan.kernel_launches_per_run() == 1
    out = plan.output()
    assert out.dtype == _TORCH[dtype] and tuple(out.shape) == (rows, cols)
    _check(out, _ref(x.double().cpu().numpy(), 1, 1), dtype)


@pytest.mark.parametrize("algorithm", [0, 2])
def test_fast_and_log_variants(algorithm):
    x = torch.randn(128, 512, device="cuda")
    e = ex.input("x").softmax(algorithm, 1) if algorithm == 0 else ex.input("x").log_softmax(1)
    plan = ex.compile(e).stamp({"x": x})
    plan.run()
    torch.cuda.synchronize()
    assert plan.physical_stage_names() == ["row_program"]
    np.testing.assert_allclose(plan.output().cpu().numpy().astype(np.float64), _ref(x.double().cpu().numpy(), 1, algorithm), rtol=1e-5, atol=2e-6)


def test_softmax_rejects_the_log_algorithm_like_the_reference():
    with pytest.raises(Exception, match="logSoftmax"):
        ex.input("x").softmax(2, 1)


def test_instance_mode_reduces_every_axis_but_the_first_in_one_row_program():
    x = torch.randn(64, 8, 16, 4, device="cuda")
    plan = ex.compile(ex.input("x").softmax(1, 0)).stamp({"x": x})
    plan.run()
    torch.cuda.synchronize()
    assert plan.physical_stage_names() == ["row_program"]
    np.testing.assert_allclose(plan.output().cpu().numpy().astype(np.float64), _ref(x.double().cpu().numpy(), (1, 2, 3), 1), rtol=1e-5, atol=1e-9)


def test_channel_mode_on_rank_four_runs_staged():
    x = torch.randn(16, 24, 8, 32, device="cuda")
    plan = ex.compile(ex.input("x").softmax(1, 1)).stamp({"x": x})
    plan.run()
    torch.cuda.synchronize()
    assert "row_program" not in plan.physical_stage_names()
    np.testing.assert_allclose(plan.output().cpu().numpy().astype(np.float64), _ref(x.double().cpu().numpy(), 1, 1), rtol=1e-5, atol=1e-9)


@pytest.mark.parametrize("log", [False, True])
def test_softmax_backward_matches_the_closed_form(log):
    """dx = y * (g - sum(g * y)) for softmax, g - softmax(x) * sum(g) for log-softmax (AutoDiff.cpp:4695-4722)."""
    rows, cols = 256, 1024
    x = torch.randn(rows, cols, device="cuda")
    g = torch.randn(rows, cols, device="cuda")
    fwd = ex.compile(ex.input("x").log_softmax() if log else ex.input("x").softmax())
    plan = fwd.compile_backward(["x"]).stamp({"x": x, "__grad_output": g})
    plan.run()
    torch.cuda.synchronize()
    assert plan.physical_stage_names() == ["row_program"], plan.physical_stage_names()
    x64, g64 = x.double().cpu().numpy(), g.double().cpu().numpy()
    y = _ref(x64, 1, 1)
    want = g64 - y * g64.sum(axis=1, keepdims=True) if log else y * (g64 - (g64 * y).sum(axis=1, keepdims=True))
    got = plan.output("x_grad").cpu().numpy().astype(np.float64)
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=2e-6 * float(np.abs(want).max()))
