"""Row programs (softmax / LayerNorm class) against the staged execution and the CPU oracle.

Tolerances: fp32-accumulated row statistics 1e-5 relative; fp32 elementwise results <= 2 ulp given
identical row statistics (so the end-to-end bound on softmax values is 1e-5 relative); bf16 outputs
<= 1 bf16 ulp plus the fp32 rounding noise of the terms that cancel (stated per test)."""
import numpy as np
import pytest
import torch

import oracle as o
from oracle import expr_oracle as eo
from thor_b200 import DataType
from thor_b200.expression import Expression as ex

pytestmark = pytest.mark.gpu


def _softmax_expr():
    x = ex.input("x")
    e = (x - x.reduce_max([1])).exp()
    return e / e.reduce_sum([1])


@pytest.mark.parametrize("rows,cols", [(64, 4096), (33, 1000), (257, 128), (5, 32768), (1000, 36)])
def test_softmax_row_program_matches_staged_and_oracle(rows, cols):
    x = (torch.randn(rows, cols, device="cuda") * 3.0).contiguous()
    fused = ex.compile(_softmax_expr(), fuse_row_reductions=True).stamp({"x": x})
    staged = ex.compile(_softmax_expr(), fuse_row_reductions=False).stamp({"x": x})
    fused.run()
    staged.run()
    torch.cuda.synchronize()
    assert fused.physical_stage_names() == ["row_program"], fused.physical_stage_names()
    assert staged.physical_stage_names()[0].startswith("rows_")
    # the logical stage list is what the reference's planner reports (Reduction, Fused, Reduction, Fused)
    assert fused.stage_kind_names() == staged.stage_kind_names() == ["Reduction", "FusedKernel", "Reduction", "FusedKernel"]
    want, _ = o.softmax_rows(x.cpu().numpy(), want_argmax=False)
    for plan in (fused, staged):
        got = plan.output().cpu().numpy()
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-12)
    assert fused.kernel_launches_per_run() == 1 and staged.kernel_launches_per_run() >= 4
    assert fused.intermediate_bytes() <= 1 and staged.intermediate_bytes() >= rows * cols * 4


def test_softmax_rows_with_nan_and_inf_follow_the_staged_semantics():
    x = torch.randn(8, 256, device="cuda")
    x[1, 5] = float("inf")
    x[2, 7] = float("nan")
    x[3, :] = -float("inf")
    fused = ex.compile(_softmax_expr()).stamp({"x": x})
    staged = ex.compile(_softmax_expr(), fuse_row_reductions=False).stamp({"x": x})
    fused.run()
    staged.run()
    torch.cuda.synchronize()
    a, b = fused.output().cpu().numpy(), staged.output().cpu().numpy()
    assert np.array_equal(np.isnan(a), np.isnan(b))
    np.testing.assert_allclose(a[~np.isnan(a)], b[~np.isnan(b)], rtol=1e-5)


def _layernorm(dtype_out=DataType.bf16, eps=1e-5):
    x, gamma, beta = ex.input("x"), ex.input("gamma"), ex.input("beta")
    mean = x.reduce_mean([1])
    xc = x - mean
    var = (xc * xc).reduce_mean([1])
    rstd = 1.0 / (var + eps).sqrt()
    return (xc * rstd * gamma + beta).cast(dtype_out)


def _bf16(t):
    return t.view(torch.uint16).cpu().numpy()


def _ln_inputs(rows, cols, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    gamma = (torch.rand(cols, device="cuda", generator=g) * 0.2 + 0.9).bfloat16()
    beta = (torch.randn(cols, device="cuda", generator=g) * 0.02).bfloat16()
    dy = (torch.randn(rows, cols, device="cuda", generator=g) * 1e-2).bfloat16()
    return x, gamma, beta, dy


@pytest.mark.parametrize("rows,cols", [(64, 8192), (300, 1024), (17, 256), (1024, 64)])
def test_layernorm_forward_row_program(rows, cols):
    x, gamma, beta, _ = _ln_inputs(rows, cols)
    fused = ex.compile(_layernorm()).stamp({"x": x, "gamma": gamma, "beta": beta})
    staged = ex.compile(_layernorm(), fuse_row_reductions=False).stamp({"x": x, "gamma": gamma, "beta": beta})
    fused.run()
    staged.run()
    torch.cuda.synchronize()
    assert fused.physical_stage_names() == ["row_program"]
    assert len(staged.physical_stage_names()) >= 4
    want, _, _ = o.layernorm_fwd(_bf16(x), _bf16(gamma), _bf16(beta), 1e-5)
    wantf = o.to_float64(want.reshape(-1), o.BF16).reshape(rows, cols)
    for plan in (fused, staged):
        got = o.to_float64(_bf16(plan.output()).reshape(-1), o.BF16).reshape(rows, cols)
        d = eo.ulp_distance(got, wantf, o.BF16)
        assert d.max() <= 1.0, d.max()
        assert (d == 0).mean() > 0.99


@pytest.mark.parametrize("rows,cols", [(64, 8192), (300, 1024), (48, 256)])
def test_layernorm_backward_from_autodiff(rows, cols):
    """dx, dgamma, dbeta of the LayerNorm DAG produced by compile_backward, as a row program with column
    reductions, against the staged plan and the fp64 oracle."""
    x, gamma, beta, dy = _ln_inputs(rows, cols, seed=3)
    fwd = ex.compile({"y": _layernorm()})
    bwd = fwd.compile_backward(["x", "gamma", "beta"])
    binds = {"x": x, "gamma": gamma, "beta": beta, "__grad_output": dy}
    fused = bwd.stamp(binds)
    fused.run()
    torch.cuda.synchronize()
    assert fused.physical_stage_names() == ["row_program"], fused.physical_stage_names()
    dx_w, dg_w, db_w = o.layernorm_bwd(_bf16(x), _bf16(gamma), _bf16(dy), 1e-5)
    dxw = o.to_float64(dx_w.reshape(-1), o.BF16).reshape(rows, cols)
    dx = fused.output("x_grad")
    assert dx.dtype == torch.bfloat16
    got = o.to_float64(_bf16(dx).reshape(-1), o.BF16).reshape(rows, cols)
    # dx = rstd * (g - mean(g) - xhat * mean(g * xhat)): the three terms are O(|dy|) and cancel partly, so the
    # fp32 noise of the terms (a few 1e-7 of |dy| ~ 1e-2) adds to the 1-ulp bf16 rounding of the result
    d = eo.ulp_distance(got, dxw, o.BF16)
    d = np.where(np.abs(got - dxw) <= 2e-8, 0.0, d)
    assert d.max() <= 1.0, d.max()
    # gradients are written in the dtype of their input (bf16 here): fp32 column sums within 1e-5, then one bf16 rounding
    assert fused.output("gamma_grad").dtype == torch.bfloat16 and fused.output("beta_grad").dtype == torch.bfloat16
    dg = o.to_float64(_bf16(fused.output("gamma_grad")).reshape(-1), o.BF16)
    db = o.to_float64(_bf16(fused.output("beta_grad")).reshape(-1), o.BF16)
    for got_c, want_c in ((dg, dg_w), (db, db_w)):
        dd = eo.ulp_distance(got_c, eo.round_to(want_c, o.BF16), o.BF16)
        dd = np.where(np.abs(got_c - want_c) <= 1e-5 * np.abs(want_c) + 2e-7 * rows * 1e-2 + 2.0 ** -9 * np.abs(want_c), 0.0, dd)
        assert dd.max() <= 1.0, dd.max()


def test_layernorm_backward_staged_plan_agrees():
    rows, cols = 96, 512
    x, gamma, beta, dy = _ln_inputs(rows, cols, seed=5)
    fwd_f = ex.compile({"y": _layernorm()}, fuse_row_reductions=True)
    fwd_s = ex.compile({"y": _layernorm()}, fuse_row_reductions=False)
    binds = {"x": x, "gamma": gamma, "beta": beta, "__grad_output": dy}
    pf = fwd_f.compile_backward(["x", "gamma", "beta"]).stamp(binds)
    ps = fwd_s.compile_backward(["x", "gamma", "beta"]).stamp(binds)
    pf.run()
    ps.run()
    torch.cuda.synchronize()
    assert len(ps.physical_stage_names()) > 4 and "row_program" not in ps.physical_stage_names()
    for name in ("x_grad", "gamma_grad", "beta_grad"):
        a, b = pf.output(name).float(), ps.output(name).float()
        assert torch.allclose(a.reshape(-1), b.reshape(-1), rtol=2e-2 if name == "x_grad" else 1e-4, atol=1e-6), name


def test_autodiff_elementwise_chain():
    """d/dx sum(tanh(x) * y) = (1 - tanh(x)^2) * y, d/dy = tanh(x)."""
    x = torch.randn(4, 256, device="cuda")
    y = torch.randn(4, 256, device="cuda")
    g = torch.ones(4, 256, device="cuda")
    eq = ex.compile({"out": ex.input("x").tanh() * ex.input("y")})
    plan = eq.compile_backward(["x", "y"]).stamp({"x": x, "y": y, "__grad_output": g})
    plan.run()
    torch.cuda.synchronize()
    assert torch.allclose(plan.output("x_grad"), (1 - torch.tanh(x) ** 2) * y, rtol=1e-5, atol=1e-6)
    assert torch.allclose(plan.output("y_grad"), torch.tanh(x), rtol=1e-5, atol=1e-6)


def test_autodiff_unbroadcasts_with_reduce_sum():
    x = torch.randn(32, 128, device="cuda")
    w = torch.randn(128, device="cuda")
    g = torch.randn(32, 128, device="cuda")
    eq = ex.compile({"out": ex.input("x") * ex.input("w")})
    plan = eq.compile_backward(["w"]).stamp({"x": x, "w": w, "__grad_output": g})
    plan.run()
    torch.cuda.synchronize()
    assert plan.output("w_grad").shape == (128,)
    assert torch.allclose(plan.output("w_grad"), (g * x).sum(0), rtol=1e-5, atol=1e-5)


def test_full_reductions_of_one_tensor_share_one_pass():
    """sum, (x*x).reduce_sum() and max of a bf16 vector (configuration 4 at a small size): one flat reduce
    program instead of an elementwise stage and three DeviceTransformReduce passes.  The x*x node is a bf16
    node, so the product is rounded to bf16 before the fp32 accumulation (cf. Lamb.cpp:106)."""
    n = (1 << 22) + 13
    x = (torch.randn(n, device="cuda") + 0.01).bfloat16()

    def build():
        xi = ex.input("x")
        return {"sum": xi.reduce_sum(), "sumsq": (xi * xi).reduce_sum(), "max": xi.reduce_max()}

    fused = ex.compile(build()).stamp({"x": x})
    staged = ex.compile(build(), fuse_row_reductions=False).stamp({"x": x})
    fused.run()
    staged.run()
    torch.cuda.synchronize()
    assert fused.physical_stage_names() == ["row_program"]
    assert staged.stage_kind_names() == ["FusedKernel", "Reduction", "Reduction", "Reduction"]
    s, q, m = o.c4_stats(_bf16(x))
    for plan in (fused, staged):
        assert abs(float(plan.output("sum")) - s) <= 1e-5 * abs(s) + 2e-7 * n
        assert abs(float(plan.output("sumsq")) - q) <= 1e-5 * abs(q)
        assert float(plan.output("max")) == m
    assert fused.intermediate_bytes() < (1 << 20) and staged.intermediate_bytes() >= 2 * n


def test_softmax_and_argmax_of_one_tensor_share_one_pass():
    """{"y": softmax(x), "idx": argmax(x)}: one row program reads x once for both (the arg reduction joins the
    first round); the index follows the arg rule (NaN wins, lowest index among equals)."""
    rows, cols = 513, 4096
    x = torch.randint(-8, 8, (rows, cols), device="cuda").float()  # many ties
    x[7, 100] = float("nan")
    x[7, 50] = float("nan")
    x[9, :] = -1.0  # signed zeros tie: the first of them wins whatever its sign
    x[9, 20] = -0.0
    x[9, 30] = 0.0
    xi = ex.input("x")
    e = (xi - xi.reduce_max([1])).exp()
    both = ex.compile({"y": e / e.reduce_sum([1]), "idx": xi.argmax([1], squeeze_axes=[1])}).stamp({"x": x})
    alone = ex.compile(xi.argmax([1], squeeze_axes=[1])).stamp({"x": x})
    both.run()
    alone.run()
    torch.cuda.synchronize()
    assert both.physical_stage_names() == ["row_program"] and both.kernel_launches_per_run() == 1
    assert alone.physical_stage_names() == ["arg_reduce"]
    idx = both.output("idx").cpu().numpy()
    assert idx.dtype == np.uint32
    assert np.array_equal(idx, alone.output().cpu().numpy())
    assert np.array_equal(idx, eo.arg_reduce_rows(x.cpu().numpy(), True).astype(np.uint32))
    assert idx[7] == 50 and idx[9] == 20
    y = both.output("y").cpu().numpy()
    want, _ = o.softmax_rows(np.delete(x.cpu().numpy(), 7, axis=0), want_argmax=False)
    np.testing.assert_allclose(np.delete(y, 7, axis=0), want, rtol=1e-5, atol=1e-12)


def test_argmin_inside_a_bf16_row_program_with_short_rows():
    rows, cols = 300, 96
    x = torch.randn(rows, cols, device="cuda").bfloat16()
    xi = ex.input("x")
    plan = ex.compile({"m": xi.reduce_mean([1]), "idx": (xi * xi).argmin([1], squeeze_axes=[1])}).stamp({"x": x})
    plan.run()
    torch.cuda.synchronize()
    assert plan.physical_stage_names() == ["row_program"]
    sq = (x * x).float().cpu().numpy()  # the bf16-rounded product is what the arg reduction sees
    assert np.array_equal(plan.output("idx").cpu().numpy(), eo.arg_reduce_rows(sq, False).astype(np.uint32))
    np.testing.assert_allclose(plan.output("m").cpu().numpy().reshape(-1), x.float().mean(dim=1).cpu().numpy(), rtol=1e-5, atol=1e-6)


def test_values_kept_across_element_loops_do_not_change_the_result():
    """exp(x - max) is kept in registers from the sum round to the output loop; the arithmetic is the one of the
    recomputing form, so the outputs are bit-identical.  Under the fast-math option the division by the row sum becomes a
    multiplication by its reciprocal: one rounding more, within 2 ulp of the division (checked with the reciprocal alone)."""
    x = (torch.randn(777, 4096, device="cuda") * 3.0).contiguous()

    def run(tuning, fast=False):
        plan = ex.compile(_softmax_expr(), use_fast_math=fast, row_program=tuning).stamp({"x": x})
        plan.run()
        torch.cuda.synchronize()
        return plan.stage_sources()[0], plan.output().clone()

    src_keep, kept = run({})
    src_re, recomputed = run({"keep_values": -1})
    assert "kept from the first element loop" in src_keep and "kept from the first element loop" not in src_re
    assert src_keep.count("expf(") < src_re.count("expf(")
    assert torch.equal(kept, recomputed)
    src_rcp, rcp = run({"reciprocal_division": 1})  # what the fast-math option switches on, without its approximate expf
    assert "__frcp_rn" in src_rcp and "__frcp_rn" not in src_keep
    d = eo.ulp_distance(rcp.double().cpu().numpy(), kept.double().cpu().numpy(), o.FP32)
    assert float(d.max()) <= 2.0
    src_fast, _ = run({}, fast=True)
    assert "__frcp_rn" in src_fast
