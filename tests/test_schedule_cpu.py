"""Lane assignment of stamped plans: the reference's pure scheduler test
(test/Utilities/Expression/StampedExecutionPlanSchedulerTest.cpp:18-109) restated as data, and the lanes of real plans
(plan-only stamps, no GPU)."""
import pytest

from thor_b200.dtypes import DataType as DT
from thor_b200.expression import Expression as ex
from thor_b200.expression import build_execution_schedule as schedule


def test_a_linear_chain_stays_on_the_callers_lane():
    lanes, events, n_lanes, ready = schedule([[], [0], [1], [2]])
    assert lanes == [0, 0, 0, 0] and n_lanes == 1 and not ready and events == [False] * 4


def test_a_fork_creates_one_helper_lane_and_the_join_returns_to_the_callers_lane():
    lanes, events, n_lanes, ready = schedule([[], [0], [0], [1, 2], [3]])
    assert lanes == [0, 0, 1, 0, 0] and n_lanes == 2 and not ready
    assert events == [True, False, True, False, False]


def test_independent_roots_use_one_caller_ready_event_and_one_join_event():
    lanes, events, n_lanes, ready = schedule([[], [], [0, 1], [2]])
    assert lanes == [0, 1, 0, 0] and n_lanes == 2 and ready
    assert events == [False, True, False, False]


def test_nested_forks_only_create_lanes_for_parallel_branches():
    lanes, _, n_lanes, _ = schedule([[], [0], [0], [1], [1], [2], [3, 4], [5, 6]])
    assert lanes == [0, 0, 1, 0, 2, 1, 0, 0] and n_lanes == 3


def test_dependencies_that_do_not_precede_their_stage_are_rejected():
    with pytest.raises(Exception, match="does not precede"):
        schedule([[1], []])


def test_three_unfused_statistics_of_one_tensor_occupy_three_lanes():
    """sum, sum of squares (x * x materialised, then reduced) and max of one vector with row fusion off: the reference's
    stage list, whose three branches share nothing but the input."""
    x = ex.input("x")
    eq = ex.compile({"sum": x.reduce_sum(), "sumsq": (x * x).reduce_sum(), "max": x.reduce_max()}, fuse_row_reductions=False)
    plan = eq.plan({"x": ((1 << 20,), DT.bf16)})
    names, lanes = plan.physical_stage_names(), plan.stage_lanes()
    assert len(names) == len(lanes) == 4
    assert sorted(set(lanes)) == [0, 1, 2]
    sq = next(i for i, n in enumerate(names) if n.startswith("flat"))
    # the reduction of x * x continues its producer's lane; the other two reductions have lanes of their own
    assert sum(1 for i, n in enumerate(names) if n == "full" and lanes[i] == lanes[sq]) == 1
    fused = ex.compile({"sum": x.reduce_sum(), "sumsq": (x * x).reduce_sum(), "max": x.reduce_max()}).plan({"x": ((1 << 20,), DT.bf16)})
    assert fused.stage_lanes() == [0]  # one flat reduce program: nothing to schedule


def test_softmax_stage_list_with_a_separate_argmax_puts_the_argmax_on_a_helper_lane():
    x = ex.input("x")
    e = (x - x.reduce_max([1])).exp()
    eq = ex.compile({"y": e / e.reduce_sum([1]), "idx": x.argmax([1], squeeze_axes=[1])}, fuse_row_reductions=False)
    plan = eq.plan({"x": ((4096, 1024), DT.fp32)})
    names, lanes = plan.physical_stage_names(), plan.stage_lanes()
    arg = names.index("arg_reduce")
    chain = [l for i, l in enumerate(lanes) if i != arg and names[i] != "view"]
    assert len(set(chain)) == 1 and lanes[arg] != chain[0]
