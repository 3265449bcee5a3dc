"""Stamped plans whose independent stages run on helper streams (the reference's lane schedule,
Utilities/Expression/StampedEquation.cpp: StampedExecutionPlan::run with helper streams joined by events) give exactly
the results of the same plan run on one stream: the same kernels over the same buffers, only their order in time
differs, so the comparison is bit for bit.  Repeated runs without a host synchronisation in between check the joins
(every helper lane waits for the caller's stream before it starts and the caller's stream waits for every helper lane
before run() returns)."""
import numpy as np
import pytest
import torch

import oracle as o
from thor_b200 import DataType
from thor_b200.expression import Expression as ex

pytestmark = pytest.mark.gpu


def _statistics():
    x = ex.input("x")
    return {"sum": x.reduce_sum(), "sumsq": (x * x).reduce_sum(), "max": x.reduce_max()}


def _softmax_argmax():
    x = ex.input("x")
    e = (x - x.reduce_max([1])).exp()
    return {"y": e / e.reduce_sum([1]), "idx": x.argmax([1], squeeze_axes=[1])}


@pytest.mark.parametrize("builder,shape,dtype", [(_statistics, (1 << 22,), torch.bfloat16), (_softmax_argmax, (2048, 1024), torch.float32)])
def test_helper_lanes_give_the_single_stream_results_bit_for_bit(builder, shape, dtype):
    x = torch.randn(shape, device="cuda").to(dtype)
    lanes = ex.compile(builder(), fuse_row_reductions=False, branch_streams="always").stamp({"x": x})
    single = ex.compile(builder(), fuse_row_reductions=False, branch_streams=False).stamp({"x": x})
    assert max(lanes.stage_lanes()) >= 1 and lanes.stage_lanes() == single.stage_lanes()  # the schedule is the same; only its use differs
    lanes.run()
    single.run()
    torch.cuda.synchronize()
    for name in lanes.output_names():
        a, b = lanes.output(name), single.output(name)
        assert a.dtype == b.dtype and a.shape == b.shape
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), name


def test_statistics_on_helper_lanes_match_the_fp64_oracle():
    x = (torch.randn(1 << 22, device="cuda") * 2.0).to(torch.bfloat16)
    plan = ex.compile(_statistics(), fuse_row_reductions=False, branch_streams="always").stamp({"x": x})
    plan.run()
    torch.cuda.synchronize()
    v = x.float().cpu().numpy().astype(np.float64)
    want = {"sum": v.sum(), "sumsq": (v * v).sum(), "max": v.max()}
    for name, w in want.items():
        got = float(plan.output(name).float().cpu().reshape(-1)[0])
        # bf16 result of an fp32 accumulation: one bf16 rounding of the exact value plus the fp32 accumulation error
        assert abs(got - w) <= 2.0 ** -8 * abs(w) + 1e-3 * np.sqrt(v.size) * 2.0 ** -8, (name, got, w)


def test_repeated_runs_with_new_input_values_never_read_a_stale_or_half_written_buffer():
    """128 runs back to back on the caller's stream, the input overwritten between runs by a kernel on that stream: each
    run's results must belong to that run's input (the helper lanes start after the overwrite and finish before the next)."""
    rows, cols = 512, 1024
    x = torch.empty(rows, cols, device="cuda")
    plan = ex.compile(_softmax_argmax(), fuse_row_reductions=False, branch_streams="always").stamp({"x": x})
    assert max(plan.stage_lanes()) >= 1
    stream = torch.cuda.Stream()
    gen = torch.Generator(device="cuda").manual_seed(11)
    data = torch.randn(128, rows, cols, device="cuda", generator=gen)
    ys, idxs = [], []
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for i in range(128):
            x.copy_(data[i])
            plan.run(stream)
            ys.append(plan.output("y").clone())
            idxs.append(plan.output("idx").clone())
    stream.synchronize()
    for i in (0, 1, 63, 126, 127):
        want, arg = o.softmax_rows(data[i].cpu().numpy(), want_argmax=True)
        np.testing.assert_allclose(ys[i].cpu().numpy(), want, rtol=1e-5, atol=1e-12)
        assert np.array_equal(idxs[i].cpu().numpy().astype(np.int64).reshape(-1), np.asarray(arg).astype(np.int64).reshape(-1))
    for i in range(128):  # every run's argmax belongs to its own input
        assert torch.equal(idxs[i].reshape(-1).long(), data[i].argmax(dim=1)), i
