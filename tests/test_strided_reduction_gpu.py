"""Reductions over non-adjacent axes (the reference's StridedFixedSegment path, CubReductionOperation.cuh:2946-2958,
index map CubReductionIndexing.cuh:33-53): same numeric rules as the planned reductions -- fp32 accumulation
(<= 1e-5 relative against a float64 sum of the same operands, plus the conditioning term), NaN-propagating
min / max, arg: NaN wins, lowest row-major index over the reduced axes among equals (bit-exact)."""
import numpy as np
import pytest
import torch

from thor_b200 import DataType
from thor_b200.expression import Expression as ex
from thor_b200.reductions import CubArgReduction, CubArgReductionOp, CubReduction, CubReductionOp as Op

pytestmark = pytest.mark.gpu

CASES = [((2, 3, 2), (0, 2)), ((17, 5, 33), (0, 2)), ((8, 64, 4, 128), (1, 3)), ((8, 64, 4, 128), (0, 2)), ((6, 7, 8, 9, 10), (0, 2, 4)),
         ((4, 3000, 2, 2500), (1, 3)), ((3, 1, 50, 1, 70), (0, 4))]


def _np_reduce(x64, axes, op):
    if op == Op.Sum: return x64.sum(axis=axes, keepdims=True)
    if op == Op.Mean: return x64.mean(axis=axes, keepdims=True)
    if op == Op.Max: return x64.max(axis=axes, keepdims=True)
    if op == Op.Min: return x64.min(axis=axes, keepdims=True)
    if op == Op.Product: return x64.prod(axis=axes, keepdims=True)
    if op == Op.L1Norm: return np.abs(x64).sum(axis=axes, keepdims=True)
    return np.sqrt((x64 * x64).sum(axis=axes, keepdims=True))


@pytest.mark.parametrize("shape,axes", CASES)
@pytest.mark.parametrize("op", [Op.Sum, Op.Mean, Op.Max, Op.Min, Op.L1Norm, Op.L2Norm])
def test_value_reductions_over_non_adjacent_axes(shape, axes, op):
    g = torch.Generator(device="cuda").manual_seed(len(shape) * 7 + int(op))
    x = torch.randn(*shape, device="cuda", generator=g)
    s = CubReduction(op, list(axes)).stamp(x)
    assert s.kernel_kind() == "strided"
    s.run()
    torch.cuda.synchronize()
    got = s.output.double().cpu().numpy()
    x64 = x.double().cpu().numpy()
    want = _np_reduce(x64, axes, op)
    assert got.shape == want.shape
    if op in (Op.Max, Op.Min):
        assert np.array_equal(got, want)
    else:
        scale = np.abs(x64).sum(axis=axes, keepdims=True) if op != Op.L2Norm else want
        assert np.all(np.abs(got - want) <= 1e-5 * np.abs(want) + 2e-7 * scale)


def test_product_and_bf16_input_with_scale():
    x = (torch.rand(5, 6, 7, device="cuda") * 0.5 + 0.75).bfloat16()
    s = CubReduction(Op.Product, [0, 2], output_dtype=DataType.fp32, output_scale=2.0).stamp(x)
    s.run()
    torch.cuda.synchronize()
    want = 2.0 * x.double().cpu().numpy().prod(axis=(0, 2), keepdims=True)
    np.testing.assert_allclose(s.output.double().cpu().numpy(), want, rtol=1e-5)


def test_nan_propagates_through_min_and_max():
    x = torch.randn(4, 5, 6, device="cuda")
    x[1, 2, 3] = float("nan")
    for op in (Op.Max, Op.Min):
        s = CubReduction(op, [0, 2]).stamp(x)
        s.run()
        torch.cuda.synchronize()
        out = s.output.cpu().numpy().reshape(-1)
        assert np.isnan(out[2]) and not np.isnan(np.delete(out, 2)).any()


@pytest.mark.parametrize("shape,axes", CASES)
@pytest.mark.parametrize("op", [CubArgReductionOp.ArgMax, CubArgReductionOp.ArgMin])
def test_arg_reductions_over_non_adjacent_axes(shape, axes, op):
    g = torch.Generator(device="cuda").manual_seed(sum(shape))
    x = torch.randint(-50, 50, shape, device="cuda", generator=g).float()  # many ties: the lowest flattened index must win
    s = CubArgReduction(op, list(axes)).stamp(x)
    s.run()
    torch.cuda.synchronize()
    xn = x.cpu().numpy()
    kept = [i for i in range(len(shape)) if i not in axes]
    moved = np.transpose(xn, kept + list(axes)).reshape([shape[i] for i in kept] + [-1])
    want_idx = moved.argmax(axis=-1) if op == CubArgReductionOp.ArgMax else moved.argmin(axis=-1)
    want_val = moved.max(axis=-1) if op == CubArgReductionOp.ArgMax else moved.min(axis=-1)
    assert np.array_equal(s.index.cpu().numpy().reshape(want_idx.shape), want_idx.astype(np.uint32))
    assert np.array_equal(s.value.cpu().numpy().reshape(want_val.shape), want_val)


def test_arg_reduction_nan_wins_with_the_lowest_index():
    x = torch.zeros(3, 4, 5, device="cuda")
    x[2, 1, 4] = float("nan")
    x[1, 1, 0] = float("nan")
    s = CubArgReduction(CubArgReductionOp.ArgMax, [0, 2], produce_value=False).stamp(x)
    s.run()
    torch.cuda.synchronize()
    idx = s.index.cpu().numpy().reshape(-1)
    assert idx[1] == 1 * 5 + 0 and idx[0] == 0 and idx[2] == 0


def test_expression_reduction_over_non_adjacent_axes_runs_the_strided_stage():
    x = torch.randn(6, 40, 5, 64, device="cuda")
    plan = ex.compile({"s": (ex.input("x") * 2.0).reduce_sum([1, 3]), "a": ex.input("x").argmax([0, 2])}).stamp({"x": x})
    plan.run()
    torch.cuda.synchronize()
    assert "strided" in plan.physical_stage_names() and "arg_strided" in plan.physical_stage_names()
    want = (x.double() * 2.0).sum(dim=(1, 3), keepdim=True).cpu().numpy()
    np.testing.assert_allclose(plan.output("s").double().cpu().numpy(), want, rtol=1e-5, atol=1e-4)
    moved = x.cpu().numpy().transpose(1, 3, 0, 2).reshape(40, 64, -1)
    assert np.array_equal(plan.output("a").cpu().numpy().reshape(40, 64), moved.argmax(axis=-1).astype(np.uint32))


CubReductionOp = Op


# ---- views of storage: stamped as they are, nothing is materialised (CubReduction.cpp:868-907) ------------------------
def _view_cases():
    g = torch.Generator(device="cuda").manual_seed(21)
    dense = torch.randn(7, 5, 32, device="cuda", generator=g)               # physical [I, J, K]
    big = torch.randn(40, 48, 64, device="cuda", generator=g)
    return [
        ("permuted_inner_outer", dense.permute(2, 0, 1), [2], "cols"),       # logical [K, I, J], reduce J: output [K, I] written rotated
        ("permuted_natural", dense.permute(1, 0, 2), [0], "cols"),           # logical [J, I, K], reduce J: output [I, K] in physical order
        ("permuted_large", big.permute(2, 0, 1), [2], "cols"),
        ("one_physical_block", torch.randn(2, 3, 5, 7, device="cuda", generator=g).permute(1, 0, 2, 3), [0, 2], "cols"),
        ("gapped", big[:, ::2, ::3], [1], None),
        ("broadcast", torch.randn(1, 48, 64, device="cuda", generator=g).expand(40, 48, 64), [2], None),
        ("split_block", torch.randn(2, 3, 5, 7, device="cuda", generator=g).permute(1, 2, 0, 3), [1, 2], None),
        ("diagonal", torch.randn(33, 33, device="cuda", generator=g).diagonal(), [0], None),
        ("offset_view", big[3:, 1:, :].permute(2, 0, 1), [2], None),
    ]


@pytest.mark.parametrize("op,torch_fn", [(CubReductionOp.Sum, torch.sum), (CubReductionOp.Max, torch.amax), (CubReductionOp.Mean, torch.mean)])
def test_views_reduce_without_a_copy_and_match_torch(op, torch_fn):
    for name, view, axes, kind in _view_cases():
        assert not view.is_contiguous() or view.dim() == 1
        plan = CubReduction(op, axes, DataType.fp32).stamp(view)
        plan.run()
        torch.cuda.synchronize()
        want = torch_fn(view.double(), dim=axes, keepdim=True).float()
        assert plan.output.shape == want.shape, name
        if op == CubReductionOp.Max:
            assert torch.equal(plan.output, want), name
        else:
            assert torch.allclose(plan.output, want, rtol=1e-5, atol=1e-5), (name, float((plan.output - want).abs().max()))
        if kind is not None:  # dense permutations whose reduced axes are one physical block keep the dense tiled kernels
            assert plan.kernel_kind().startswith(kind), (name, plan.kernel_kind())
        else:
            assert plan.kernel_kind() == "strided", (name, plan.kernel_kind())


def test_a_bf16_permuted_view_writes_its_rotated_output_in_the_requested_dtype():
    x = torch.randn(64, 96, 256, device="cuda").bfloat16()
    view = x.permute(2, 0, 1)  # [256, 64, 96] over dense [64, 96, 256]
    plan = CubReduction(CubReductionOp.Sum, [2], DataType.bf16).stamp(view)
    plan.run()
    torch.cuda.synchronize()
    want = view.float().sum(dim=2, keepdim=True)
    assert plan.output.dtype == torch.bfloat16 and plan.kernel_kind().startswith("cols")
    assert torch.allclose(plan.output.float(), want, rtol=2 ** -7, atol=1e-2)
