"""Host planner, dtype resolution and kernel generation without a GPU.

`FusedEquation.plan` stamps against shapes and dtypes only: stages are planned, every kernel is
generated and compiled for sm_100a (NVRTC needs no device), nothing is loaded or launched.  The
stage lists asserted here are the ones the reference's planner reports for the same expressions
(EquationCompiler::splitAtReductionBoundaries, EquationCompiler.cpp:7881; stage kinds in
EquationCompiler.h:27)."""
import pytest

from thor_b200 import DataType as DT
from thor_b200 import _native
from thor_b200.expression import Expression as ex


def _c2():
    a, x, b, z = ex.input("a"), ex.input("x"), ex.input("b"), ex.input("z")
    return (a * x + b).relu() * z.sigmoid()


def _softmax():
    x = ex.input("x")
    e = (x - x.reduce_max([1])).exp()
    return e / e.reduce_sum([1])


def _layernorm(eps=1e-5):
    x, gamma, beta = ex.input("x"), ex.input("gamma"), ex.input("beta")
    xc = x - x.reduce_mean([1])
    rstd = 1.0 / ((xc * xc).reduce_mean([1]) + eps).sqrt()
    return (xc * rstd * gamma + beta).cast(DT.bf16)


def test_broadcast_fused_expression_is_one_tiled_half2_stage():
    plan = ex.compile(_c2()).plan({"a": ((8192,), DT.fp16), "x": ((8192, 8192), DT.fp16), "b": ((8192,), DT.fp16), "z": ((8192, 8192), DT.fp16)})
    assert plan.stage_kind_names() == ["FusedKernel"]
    assert plan.physical_stage_names() == ["bcast_tiled_v2"]
    assert plan.kernel_launches_per_run() == 1 and plan.intermediate_bytes() == 0
    assert plan.output_spec() == ([8192, 8192], DT.fp16)
    src = plan.stage_sources()[0]
    assert "__half2" in src and "griddepcontrol" not in src and "tb_grid_wait();" in src


def test_flat_expression_without_broadcast_is_a_flat_stage():
    x, y = ex.input("x"), ex.input("y")
    plan = ex.compile((x * y + 1.0).tanh()).plan({"x": ((1 << 20,), DT.fp32), "y": ((1 << 20,), DT.fp32)})
    assert plan.physical_stage_names() == ["flat_scalar"]
    assert plan.output_spec() == ([1 << 20], DT.fp32)


def test_mixed_fp16_bf16_promotes_to_fp32_and_scalars_do_not_promote():
    x, y = ex.input("x"), ex.input("y")
    plan = ex.compile({"sum": x + y, "scaled": x * 3.0}).plan({"x": ((64, 64), DT.fp16), "y": ((64, 64), DT.bf16)})
    assert plan.output_spec("sum")[1] == DT.fp32
    assert plan.output_spec("scaled")[1] == DT.fp16


# the promotion table of the reference's own dtype tests (test_expression_dynamic_dtypes.py:180-191)
@pytest.mark.parametrize("lhs,rhs,want", [(DT.fp8_e4m3, DT.fp8_e4m3, DT.fp8_e4m3), (DT.fp8_e4m3, DT.fp8_e5m2, DT.fp16), (DT.fp8_e4m3, DT.fp16, DT.fp16),
                                           (DT.fp8_e5m2, DT.bf16, DT.bf16), (DT.fp16, DT.bf16, DT.fp32), (DT.fp16, DT.fp32, DT.fp32),
                                           (DT.bf16, DT.fp32, DT.fp32)])
def test_pairwise_tensor_promotion(lhs, rhs, want):
    plan = ex.compile(ex.input("x") + ex.input("y")).plan({"x": ((3, 5), lhs), "y": ((3, 5), rhs)})
    assert plan.output_spec() == ([3, 5], want)


@pytest.mark.parametrize("dtype", [DT.fp32, DT.fp16, DT.bf16, DT.fp8_e4m3, DT.fp8_e5m2])
def test_single_input_keeps_its_storage_dtype_and_constants_never_promote(dtype):
    x = ex.input("x")
    for expr in (((x + 1.0) * (x - 0.5)) + 2.0, (x + 1.0) * 2.0 - 0.25):
        plan = ex.compile(expr).plan({"x": ((17,), dtype)})
        assert plan.output_spec() == ([17], dtype)
        assert plan.stage_kind_names() == ["FusedKernel"]


def test_mixed_dtype_outputs_of_one_stage_keep_distinct_dtypes():
    x, y, z = ex.input("x"), ex.input("y"), ex.input("z")
    plan = ex.compile({"sum16": x + y, "mix32": x + z, "shift16": x + 1.0}).plan({"x": ((17,), DT.fp16), "y": ((17,), DT.fp16), "z": ((17,), DT.fp32)})
    assert plan.output_spec("sum16")[1] == DT.fp16 and plan.output_spec("mix32")[1] == DT.fp32 and plan.output_spec("shift16")[1] == DT.fp16
    assert plan.stage_kind_names() == ["FusedKernel"] and plan.kernel_launches_per_run() == 1


def test_softmax_is_one_row_program_or_four_stages():
    shapes = {"x": ((65536, 4096), DT.fp32)}
    fused = ex.compile(_softmax()).plan(shapes)
    staged = ex.compile(_softmax(), fuse_row_reductions=False).plan(shapes)
    assert fused.stage_kind_names() == staged.stage_kind_names() == ["Reduction", "FusedKernel", "Reduction", "FusedKernel"]
    assert fused.physical_stage_names() == ["row_program"] and fused.kernel_launches_per_run() == 1
    assert fused.intermediate_bytes() <= 1
    assert len(staged.physical_stage_names()) == 4 and staged.physical_stage_names()[0].startswith("rows_")
    assert staged.intermediate_bytes() >= 65536 * 4096 * 4
    assert fused.output_spec() == staged.output_spec() == ([65536, 4096], DT.fp32)


def test_softmax_op_keeps_the_operand_dtype_and_is_one_row_program():
    for dt in (DT.fp32, DT.bf16, DT.fp16):
        plan = ex.compile(ex.input("x").softmax()).plan({"x": ((4096, 4096), dt)})
        assert plan.physical_stage_names() == ["row_program"] and plan.kernel_launches_per_run() == 1
        assert plan.output_spec() == ([4096, 4096], dt)
    # instance mode: every axis but the first, whatever the rank
    plan = ex.compile(ex.input("x").log_softmax(0)).plan({"x": ((64, 8, 16, 4), DT.fp32)})
    assert plan.physical_stage_names() == ["row_program"]
    # backward of the op: the row maximum carries no gradient, so no min/max-backward stage appears
    bwd = ex.compile(ex.input("x").softmax()).compile_backward(["x"]).plan({"x": ((512, 1024), DT.bf16), "__grad_output": ((512, 1024), DT.bf16)})
    assert bwd.physical_stage_names() == ["row_program"] and bwd.output_spec("x_grad") == ([512, 1024], DT.bf16)


def test_row_programs_cover_reductions_over_a_trailing_block_of_axes():
    x = ex.input("x")
    xc = x - x.reduce_mean([1, 2])
    plan = ex.compile(xc / ((xc * xc).reduce_mean([1, 2]) + 1e-5).sqrt()).plan({"x": ((128, 32, 64), DT.bf16)})
    assert plan.physical_stage_names() == ["row_program"]
    assert plan.output_spec() == ([128, 32, 64], DT.fp32)


def test_backward_of_reduce_max_plans_a_route_stage():
    eq = ex.compile({"m": (ex.input("x") * 2.0).reduce_max([1])})
    bwd = eq.compile_backward(["x"]).plan({"x": ((512, 1024), DT.bf16), "__grad_output": ((512, 1), DT.fp32)})
    assert bwd.stage_kind_names() == ["FusedKernel", "ReduceMinMaxBackward", "FusedKernel"]
    assert bwd.physical_stage_names()[1] == "minmax_backward"
    assert bwd.output_spec("x_grad") == ([512, 1024], DT.bf16)


def test_argmax_stage_yields_uint32_indices():
    plan = ex.compile(ex.input("x").argmax([1], squeeze_axes=[1])).plan({"x": ((1024, 4096), DT.fp32)})
    assert plan.stage_kind_names() == ["ArgMinMax"]
    assert plan.output_spec() == ([1024], DT.uint32)


def test_layernorm_forward_and_backward_plans():
    shapes = {"x": ((32768, 8192), DT.bf16), "gamma": ((8192,), DT.bf16), "beta": ((8192,), DT.bf16)}
    fwd_eq = ex.compile({"y": _layernorm()})
    fwd = fwd_eq.plan(shapes)
    assert fwd.physical_stage_names() == ["row_program"] and fwd.kernel_launches_per_run() == 1
    assert fwd.output_spec("y") == ([32768, 8192], DT.bf16)
    bwd = fwd_eq.compile_backward(["x", "gamma", "beta"]).plan({**shapes, "__grad_output": ((32768, 8192), DT.bf16)})
    assert sorted(bwd.output_names()) == ["beta_grad", "gamma_grad", "x_grad"]
    # one row kernel plus one fold per column reduction; gradients come back in the dtype of their input
    assert bwd.physical_stage_names() == ["row_program"] and bwd.kernel_launches_per_run() == 2  # the row kernel + one fold of both column sums
    assert bwd.output_spec("x_grad") == ([32768, 8192], DT.bf16)
    assert bwd.output_spec("gamma_grad") == ([8192], DT.bf16)
    src = bwd.stage_sources()[0]
    assert "__ffma2_rn" in src, "fp32 element math of row programs uses the packed f32x2 instructions"
    # partial column sums: one fp32 row of [cols] per CTA and column reduction
    assert bwd.intermediate_bytes() == 2 * 148 * 8192 * 4


def test_three_full_reductions_share_one_pass():
    x = ex.input("x")
    plan = ex.compile({"sum": x.reduce_sum(), "sumsq": (x * x).reduce_sum(), "max": x.reduce_max()}).plan({"x": ((1 << 24,), DT.bf16)})
    assert plan.physical_stage_names() == ["row_program"]
    assert plan.kernel_launches_per_run() == 2  # one streaming pass + one fold launch (a CTA per statistic)
    for name in ("sum", "sumsq", "max"):
        assert plan.output_spec(name)[1] == DT.fp32


def test_plan_only_plans_refuse_to_run_and_own_no_memory():
    plan = ex.compile(_softmax()).plan({"x": ((64, 128), DT.fp32)})
    with pytest.raises((_native.ThorB200Error, _native.ThorB200InvalidArgument)):
        plan.run()
    with pytest.raises((_native.ThorB200Error, _native.ThorB200InvalidArgument)):
        plan.output()


def test_shape_errors_surface_at_plan_time():
    x, y = ex.input("x"), ex.input("y")
    with pytest.raises((_native.ThorB200Error, _native.ThorB200InvalidArgument)):
        ex.compile(x + y).plan({"x": ((64, 3), DT.fp32), "y": ((64, 4), DT.fp32)})
    with pytest.raises((_native.ThorB200Error, _native.ThorB200InvalidArgument)):
        ex.compile(x + y).plan({"x": ((64, 3), DT.fp32)})


def test_stable_sigmoid_costs_one_exponential_per_element():
    """exp(-max(-z, 0)) of the overflow-safe sigmoid is emitted as a select of exp(-|z|) (equal arguments where z < 0,
    exactly 1 elsewhere): half2, bfloat162 and fp32 scalar bodies."""
    plan = ex.compile(_c2()).plan({"a": ((8192,), DT.fp16), "x": ((8192, 8192), DT.fp16), "b": ((8192,), DT.fp16), "z": ((8192, 8192), DT.fp16)})
    body = plan.stage_sources()[0].split("extern \"C\"")[0]
    assert body.count("tb_h2exp") == 1 and "tb_h2sel_neg(" in body
    x = ex.input("x")
    for dtype, exp_name, select in ((DT.bf16, "h2exp(", "tb_h2sel_neg("), (DT.fp32, "expf(", "< 0.0f) ?")):
        body = ex.compile(x * x.sigmoid()).plan({"x": ((1 << 20,), dtype)}).stage_sources()[0].split("extern \"C\"")[0]
        assert body.count(exp_name) == 1 and select in body, body


def test_layernorm_programs_take_rows_through_the_bulk_copy_ring_and_softmax_keeps_its_exponential():
    shapes = {"x": ((32768, 8192), DT.bf16), "gamma": ((8192,), DT.bf16), "beta": ((8192,), DT.bf16)}
    fwd_eq = ex.compile({"y": _layernorm()})
    fwd = fwd_eq.plan(shapes).stage_sources()[0]
    assert "cp.async.bulk" not in fwd  # the instruction lives in the prelude; the program calls the wrappers
    assert "tb_bulk_load(" in fwd and "tb_mbar_wait(" in fwd and "constexpr int STAGES = 3;" in fwd and "ran with the previous row" in fwd
    assert "tb_release_registers" not in fwd  # two CTAs per SM: thread 0 requests the copies
    bwd_eq = fwd_eq.compile_backward(["x", "gamma", "beta"])
    bwd_shapes = {**shapes, "__grad_output": ((32768, 8192), DT.bf16)}
    bwd = bwd_eq.plan(bwd_shapes).stage_sources()[0]
    assert "tb_bulk_load(" in bwd and "constexpr int STAGES = 4;" in bwd and "ran with the previous row" not in bwd
    # the backward program (per-column accumulators, one CTA per SM) gives the copies a warpgroup of their own: 256 team
    # threads + 128, registers handed over, buffers released through "empty" barriers, team-only barriers in the rounds
    for needle in ("__launch_bounds__(384, 1)", "tb_release_registers();", "tb_claim_registers();", "tb_mbar_arrive(&tb_empty[stage]);", "tb_named_barrier<1, CONSUMERS>();"):
        assert needle in bwd, needle
    assert bwd.count("__syncthreads()") == 1  # the set-up barrier before the warpgroups part
    plain = ex.compile({"y": _layernorm()}, row_program={"copy_warpgroup": -1}).compile_backward(["x", "gamma", "beta"]).plan(bwd_shapes).stage_sources()[0]
    assert "__launch_bounds__(256)" in plain and "tb_release_registers" not in plain and "if (threadIdx.x == 0) {\n            const tb_u64 r0 = row0 + STAGES * row_stride;" in plain
    xi = ex.input("x")
    e = (xi - xi.reduce_max([1])).exp()
    sm = ex.compile(e / e.reduce_sum([1])).plan({"x": ((65536, 4096), DT.fp32)}).stage_sources()[0]
    assert sm.count("expf(") == 2 and "kept from the first element loop" in sm  # two lanes of one pair, once


def test_constant_subtrees_become_one_literal_and_identities_compute_nothing():
    """The reference's emitter folds literal subtrees in double and emits one float literal, and x + 0, x * 1, x / 1 alias
    their operand (CudaSourceEmitter.cpp:1965-2076, 3745-3782); the fused stage and the row program do the same."""
    x, z = ex.input("x"), ex.input("z")
    e = x * (ex.scalar(0.1) * ex.scalar(3.0)) + (ex.scalar(1.0) / ex.scalar(3.0)) + (z + 0.0) * 1.0 / (ex.scalar(2.0) - ex.scalar(1.0))
    body = ex.compile(e).plan({"x": ((1 << 16,), DT.fp16), "z": ((1 << 16,), DT.fp16)}).stage_sources()[0].split('extern "C"')[0]
    assert "0.300000012f" in body and "0.333333343f" in body  # (float)(0.1 * 3.0) and (float)(1.0 / 3.0), not fp16 products
    assert "0.100000001f" not in body and "3.0f" not in body and "2.0f" not in body and "1.0f" not in body
    # one multiplication (x by the folded literal) and two additions are all the arithmetic that is left
    assert body.count(" * ") == 1 and body.count(" + ") == 2 and " / " not in body and " - " not in body
    row = ex.compile({"y": (x * 1.0 + 0.0) / x.reduce_sum([1])}).plan({"x": ((64, 512), DT.fp32)}).stage_sources()[0]
    assert "1.0f" not in row.split("row_kernel")[1] and "0.0f)" not in row.split("// outputs")[1]


def test_the_compile_cache_is_bounded_and_evicts_the_least_recently_used():
    """Compiled modules live in a process-wide LRU cache (10 000 entries like the reference's, EquationCompiler.cpp:123-157):
    with the bound lowered, distinct stages push the oldest out and the count never exceeds the bound."""
    import ctypes

    from thor_b200 import _native

    lib = _native.lib
    lib.thor_b200_jit_cache_capacity.argtypes = [ctypes.c_size_t]
    lib.thor_b200_jit_cache_capacity.restype = ctypes.c_size_t
    lib.thor_b200_jit_cache_size.restype = ctypes.c_size_t
    previous = lib.thor_b200_jit_cache_capacity(3)
    try:
        assert previous == 10000 and lib.thor_b200_jit_cache_size() <= 3
        x = ex.input("x")
        for k in range(6):  # six different stages
            ex.compile(x * float(k + 2) + 0.5).plan({"x": ((4096,), DT.fp32)})
            assert lib.thor_b200_jit_cache_size() <= 3
        assert lib.thor_b200_jit_cache_size() == 3
    finally:
        lib.thor_b200_jit_cache_capacity(previous)
