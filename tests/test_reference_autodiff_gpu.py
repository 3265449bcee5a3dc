"""LayerNorm backward on the GPU against the REFERENCE's own backward graph.

The oracle here is the graph that the reference's buildBackwardOutputs builds for these shapes (golden file written by
tests/golden/make_autodiff_golden.py from oracle/ref_autodiff.cpp), evaluated node by node in numpy with the reference's
per-node dtype rule (oracle/graph_eval.py).  The GPU runs the host layer's own backward graph as one row program.
Tolerances: dx within 1 bf16 ulp; dgamma / dbeta are fp32-accumulated column sums rounded once to bf16, within 1 bf16 ulp."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle as o
from oracle import graph_eval as ge
from oracle.expr_oracle import ulp_distance
from thor_b200 import DataType
from thor_b200.expression import Expression as ex

pytestmark = pytest.mark.gpu
GOLDEN = json.loads((Path(__file__).parent / "golden" / "autodiff_reference_graphs.json").read_text())


def _layernorm():
    x, gamma, beta = ex.input("x"), ex.input("gamma"), ex.input("beta")
    xc = x - x.reduce_mean([1])
    rstd = 1.0 / ((xc * xc).reduce_mean([1]) + 1e-5).sqrt()
    return {"output": (xc * rstd * gamma + beta).cast(DataType.bf16)}


@pytest.mark.parametrize("case,copy_warpgroup", [("layernorm_bf16_64x256", 0), ("layernorm_bf16_512x8192", 0), ("layernorm_bf16_512x8192", -1)])
def test_layernorm_backward_matches_the_reference_graph(case, copy_warpgroup):
    rows, cols = GOLDEN[case]["inputs"]["x"][0]
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    gamma = (torch.rand(cols, device="cuda", generator=g) * 0.2 + 0.9).bfloat16()
    beta = (torch.randn(cols, device="cuda", generator=g) * 0.02).bfloat16()
    dy = (torch.randn(rows, cols, device="cuda", generator=g) * 1e-2).bfloat16()
    plan = ex.compile(_layernorm(), row_program={"copy_warpgroup": copy_warpgroup}).compile_backward(["x", "gamma", "beta"]).stamp(
        {"x": x, "gamma": gamma, "beta": beta, "__grad_output": dy})
    plan.run()
    torch.cuda.synchronize()
    assert plan.physical_stage_names() == ["row_program"] and plan.waits_expired() == 0
    host = {"x": x, "gamma": gamma, "beta": beta, "__grad_output": dy}
    want = ge.evaluate(GOLDEN[case]["graph"], {k: v.float().cpu().numpy().astype(np.float64) for k, v in host.items()})
    for name in ("x_grad", "gamma_grad", "beta_grad"):
        got = plan.output(name).float().cpu().numpy().astype(np.float64).reshape(want[name].shape)
        d = ulp_distance(got, want[name], o.BF16)
        # dx is a sum of terms of size ~1e-2 that cancel; the row program adds them in another order (hoisted row sums,
        # fused multiply-adds), fp32 noise of 2e-8 absolute that shows as more than one ulp only where dx itself is tiny
        slack = 2e-8 if name == "x_grad" else 2e-7 * rows * 1e-2
        d = np.where(np.abs(got - want[name]) <= slack, 0.0, d)
        assert float(d.max()) <= 1.0, f"{name}: {float(d.max())} bf16 ulp from the reference graph's value"
        assert float((d == 0).mean()) >= 0.98, f"{name}: {(d == 0).mean():.4f} identical"


def test_unrounded_column_sums_round_to_the_gradient_outputs():
    """A caller that holds one shard of the rows asks for the column sums before their rounding: the fp32 rows of
    "__column_sums" are the values the bf16 gradient outputs were rounded from, and two half-row shards added in fp32
    and rounded once give the whole problem's gradients to the last bit of most columns (fp32 re-association only)."""
    rows, cols = 1024, 8192
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    gamma = (torch.rand(cols, device="cuda", generator=g) * 0.2 + 0.9).bfloat16()
    beta = torch.zeros(cols, device="cuda").bfloat16()
    dy = (torch.randn(rows, cols, device="cuda", generator=g) * 1e-2).bfloat16()
    bwd = ex.compile(_layernorm(), unrounded_column_sums=True).compile_backward(["x", "gamma", "beta"])

    def run(r0, r1):
        plan = bwd.stamp({"x": x[r0:r1], "gamma": gamma, "beta": beta, "__grad_output": dy[r0:r1]})
        plan.run()
        torch.cuda.synchronize()
        return plan

    whole = run(0, rows)
    names = whole.column_sum_names()
    assert sorted(names) == ["beta_grad", "gamma_grad"]
    sums = whole.output("__column_sums")
    assert sums.dtype == torch.float32 and tuple(sums.shape) == (2, cols)
    for i, name in enumerate(names):
        assert torch.equal(sums[i].bfloat16().view(torch.int16), whole.output(name).reshape(-1).view(torch.int16))
    halves = [run(0, rows // 2), run(rows // 2, rows)]
    combined = halves[0].output("__column_sums") + halves[1].output("__column_sums")
    rel = ((combined - sums).abs().max() / sums.abs().max()).item()
    assert rel <= 1e-6
    same = (combined.bfloat16().view(torch.int16) == sums.bfloat16().view(torch.int16)).float().mean().item()
    assert same >= 0.99
    plain = ex.compile(_layernorm()).compile_backward(["x", "gamma", "beta"]).stamp({"x": x, "gamma": gamma, "beta": beta, "__grad_output": dy})
    assert plain.column_sum_names() == [] and "__column_sums" not in plain.output_names()
