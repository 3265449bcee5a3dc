"""Persistent row programs whose rows arrive by bulk copies in a ring of shared-memory buffers.

The ring changes how operands reach the registers, not the arithmetic: per-thread partial sums, the
exchange and the element expressions are the ones of the register double buffer, so the two modes
must agree bit for bit (with and without round 1 of the next row riding on the last round of the
current one).  Every device-side wait is bounded in time; a healthy run reports no expired wait."""
import numpy as np
import pytest
import torch

from thor_b200 import DataType
from thor_b200.expression import Expression as ex

pytestmark = pytest.mark.gpu


def _layernorm():
    x, gamma, beta = ex.input("x"), ex.input("gamma"), ex.input("beta")
    xc = x - x.reduce_mean([1])
    rstd = 1.0 / ((xc * xc).reduce_mean([1]) + 1e-5).sqrt()
    return {"y": (xc * rstd * gamma + beta).cast(DataType.bf16)}


def _inputs(rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(rows, cols, device="cuda", generator=g) * 2.0 + 0.5).bfloat16()
    gamma = (torch.rand(cols, device="cuda", generator=g) + 0.5).bfloat16()
    beta = (torch.randn(cols, device="cuda", generator=g) * 0.1).bfloat16()
    dy = (torch.randn(rows, cols, device="cuda", generator=g) * 1e-2).bfloat16()
    return x, gamma, beta, dy


def _run(rows, cols, tuning, backward):
    def go():
        x, gamma, beta, dy = _inputs(rows, cols, 7)
        eq = ex.compile(_layernorm(), row_program=tuning)
        if backward:
            plan = eq.compile_backward(["x", "gamma", "beta"]).stamp({"x": x, "gamma": gamma, "beta": beta, "__grad_output": dy})
            names = ["x_grad", "gamma_grad", "beta_grad"]
        else:
            plan = eq.stamp({"x": x, "gamma": gamma, "beta": beta})
            names = ["y"]
        for _ in range(3):  # several launches: the ring's barriers start from scratch in each
            plan.run()
        torch.cuda.synchronize()
        assert plan.physical_stage_names() == ["row_program"]
        return plan, [plan.output(n).view(torch.uint16).cpu().numpy().copy() for n in names]

    return go()


# rows that do not fill the last iteration of the persistent CTAs, rows shorter than a warp's span (several
# teams per CTA, so a bulk copy covers several rows and the last one is cut short), and one long row shape
SHAPES = [(4096, 8192), (1000, 1024), (333, 256), (77, 64), (5000, 40)]


RING_OFF = {"ring_buffers": -1}


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("backward", [False, True])
def test_ring_modes_agree_bit_for_bit_with_the_register_double_buffer(rows, cols, backward):
    _, want = _run(rows, cols, RING_OFF, backward)
    for tuning in ({"ring_buffers": 3, "pipeline_round_one": 1, "copy_warpgroup": -1},
                   {"ring_buffers": 4, "pipeline_round_one": -1, "copy_warpgroup": -1},
                   {"ring_buffers": -2, "pipeline_round_one": 1, "copy_warpgroup": -1},
                   {"ring_buffers": 4, "pipeline_round_one": -1, "copy_warpgroup": 1},
                   {"ring_buffers": 3, "pipeline_round_one": 1, "copy_warpgroup": 1}):
        plan, got = _run(rows, cols, tuning, backward)
        source = plan.stage_sources()[0]
        assert "tb_bulk_load" in source and "tb_mbar_wait" in source, "the ring was not used"
        assert ("ran with the previous row" in source) == (tuning["pipeline_round_one"] == 1)
        # a copy warpgroup exists only beside the teams of a program with per-column accumulators (the backward program)
        assert ("tb_release_registers();" in source) == (tuning["copy_warpgroup"] == 1 and backward)
        for g, w in zip(got, want):
            assert np.array_equal(g, w)
        assert plan.waits_expired() == 0


def test_the_default_is_the_ring_for_layernorm_and_no_wait_expires():
    plan, _ = _run(2048, 8192, {}, False)
    assert "tb_bulk_load" in plan.stage_sources()[0] and "ran with the previous row" in plan.stage_sources()[0]
    assert plan.waits_expired() == 0
    plan, _ = _run(2048, 8192, {}, True)
    # programs with per-column accumulators run one CTA per SM and give the copies a warpgroup of their own
    assert "tb_bulk_load" in plan.stage_sources()[0] and "tb_release_registers();" in plan.stage_sources()[0]
    assert plan.waits_expired() == 0


def test_programs_without_waits_report_zero():
    x = torch.randn(64, 512, device="cuda")
    xi = ex.input("x")
    e = (xi - xi.reduce_max([1])).exp()
    plan = ex.compile(e / e.reduce_sum([1])).stamp({"x": x})
    plan.run()
    assert plan.waits_expired() == 0


@pytest.mark.parametrize("backward", [False, True])
def test_a_wait_that_runs_out_is_counted_and_the_device_stays_usable(backward):
    """Failure on the host side of the ring: one CTA's generated code lacks the request for one iteration's rows, so the
    wait on that buffer's barrier can never be satisfied.  The wait gives up after its limit (20 ms here), the kernel
    runs to its end, the host reads the count, and the next launches on the same context are healthy.  The fault is asked
    for through the program's tuning options of this one equation; nothing in the process environment can trigger it."""
    plan, _ = _run(4096, 8192, {"wait_limit_ms": 20, "test_skip_fill": 6}, backward)
    assert "blockIdx.x == 0 && " in plan.stage_sources()[0]
    assert plan.waits_expired() >= 1
    with pytest.raises(Exception, match="expired device-side waits"):
        plan.run()  # a program that reported an expired wait refuses further launches
    # the same shapes without the injected fault: correct results, nothing counted
    healthy, got = _run(4096, 8192, {}, backward)
    _, want = _run(4096, 8192, RING_OFF, backward)
    for g, w in zip(got, want):
        assert np.array_equal(g, w)
    assert healthy.waits_expired() == 0
