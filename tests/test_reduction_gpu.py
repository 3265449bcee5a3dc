"""GPU parity of the reduction seam.  Golden vectors are the hand-computed cases of the reference's own
tests (test/Utilities/TensorOperations/CubReductionValueOperationsTest.cpp:23-100, 442-507 and
CubArgReductionTest.cpp:94-188), restated here as data; larger cases compare with the fp64 oracle.
Tolerance for fp32-accumulated reductions: 1e-5 relative (min / max / arg results: exact)."""
import numpy as np
import pytest
import torch

import oracle as o
from oracle import expr_oracle as eo
from thor_b200 import DataType
from thor_b200.reductions import CubArgReduction, CubArgReductionOp, CubReduction, CubReductionOp, CubReductionPath, analyze_geometry

pytestmark = pytest.mark.gpu
Op = CubReductionOp
NAN, INF = float("nan"), float("inf")


def _run(values, shape, op, axis, out_dtype=DataType.fp32, scale=1.0):
    t = torch.tensor(values, dtype=torch.float32, device="cuda").reshape(shape)
    s = CubReduction(op, axis, out_dtype, scale).stamp(t)
    s.run()
    torch.cuda.synchronize()
    return s.output.float().cpu().numpy().reshape(-1), s


GOLDEN = [
    # (values, shape, axis, {op: (expected, abs tolerance)})
    ([-2.0, 3.0, -4.0], (3,), 0, {Op.Sum: ([-3.0], 0), Op.Product: ([24.0], 0), Op.Mean: ([-1.0], 0), Op.Min: ([-4.0], 0), Op.Max: ([3.0], 0),
                                   Op.L1Norm: ([9.0], 0), Op.L2Norm: ([29.0 ** 0.5], 1e-5)}),
    ([-1.0, 2.0, -3.0, 4.0, -5.0, 6.0], (2, 3), 1, {Op.Sum: ([-2.0, 5.0], 0), Op.Product: ([6.0, -120.0], 0), Op.Mean: ([-2.0 / 3, 5.0 / 3], 1e-6),
                                                     Op.Min: ([-3.0, -5.0], 0), Op.Max: ([2.0, 6.0], 0), Op.L1Norm: ([6.0, 15.0], 0),
                                                     Op.L2Norm: ([14.0 ** 0.5, 77.0 ** 0.5], 1e-5)}),
    ([-1.0, 2.0, -3.0, 4.0, -5.0, 6.0, -7.0, 8.0, -9.0, 10.0, -11.0, 12.0], (2, 3, 2), 1,
     {Op.Sum: ([-9.0, 12.0, -27.0, 30.0], 0), Op.Product: ([-15.0, 48.0, -693.0, 960.0], 0), Op.Mean: ([-3.0, 4.0, -9.0, 10.0], 0),
      Op.Min: ([-5.0, 2.0, -11.0, 8.0], 0), Op.Max: ([-1.0, 6.0, -7.0, 12.0], 0), Op.L1Norm: ([9.0, 12.0, 27.0, 30.0], 0),
      Op.L2Norm: ([35.0 ** 0.5, 56.0 ** 0.5, 251.0 ** 0.5, 308.0 ** 0.5], 1e-5)}),
]


@pytest.mark.parametrize("case", range(len(GOLDEN)))
def test_reference_golden_vectors_every_operation(case):
    values, shape, axis, expected = GOLDEN[case]
    for op, (want, tol) in expected.items():
        got, _ = _run(values, shape, op, axis)
        np.testing.assert_allclose(got, np.array(want, np.float32), rtol=0, atol=tol, err_msg=str(op))


def test_geometry_classification_matches_the_reference_paths():
    assert analyze_geometry([3], [0])[3] == CubReductionPath.DeviceTransformReduce
    assert analyze_geometry([2, 3], [1]) == (2, 3, 1, CubReductionPath.ContiguousFixedSegment)
    assert analyze_geometry([2, 3, 2], [1]) == (2, 3, 2, CubReductionPath.TiledFixedSegment)
    assert analyze_geometry([2, 3, 2], [0, 2])[3] == CubReductionPath.StridedFixedSegment
    assert analyze_geometry([32768, 8192], [0]) == (1, 32768, 8192, CubReductionPath.TiledFixedSegment)


def test_mean_and_l2_finalize_in_fp32_before_fp16_store():
    got, _ = _run([40000.0, 40000.0, -40000.0, -40000.0], (2, 2), Op.Mean, 1, DataType.fp16)
    assert list(got) == [40000.0, -40000.0]
    got, _ = _run([300.0, 400.0, 500.0, 1200.0], (2, 2), Op.L2Norm, 1, DataType.fp16)
    assert list(got) == [500.0, 1300.0]


def test_min_max_propagate_nan_on_every_path():
    for op in (Op.Min, Op.Max):
        assert np.isnan(_run([1.0, NAN, -2.0], (3,), op, 0)[0]).all()
        assert np.isnan(_run([NAN, 1.0, 2.0, 3.0, NAN, 4.0], (2, 3), op, 1)[0]).all()
        assert np.isnan(_run([1.0, 2.0, NAN, NAN, 5.0, 6.0, 7.0, 8.0, NAN, NAN, 11.0, 12.0], (2, 3, 2), op, 1)[0]).all()
    for op in (Op.Sum, Op.Product, Op.Mean, Op.L1Norm, Op.L2Norm):
        assert np.isnan(_run([1.0, NAN, 3.0], (3,), op, 0)[0]).all()


def test_infinities():
    vals = [-INF, 1.0, INF]
    assert _run(vals, (3,), Op.Min, 0)[0][0] == -INF
    assert _run(vals, (3,), Op.Max, 0)[0][0] == INF
    assert _run(vals, (3,), Op.L1Norm, 0)[0][0] == INF
    assert _run(vals, (3,), Op.L2Norm, 0)[0][0] == INF


def test_runtime_output_scale_is_applied_before_the_store_conversion():
    got, _ = _run([1.0, 2.0, 3.0, 4.0], (2, 2), Op.Sum, 1, DataType.fp32, scale=0.5)
    assert list(got) == [1.5, 3.5]


@pytest.mark.parametrize("dtype", [o.FP32, o.FP16, o.BF16, o.FP8_E4M3, o.FP8_E5M2], ids=lambda d: o.NAMES[d])
@pytest.mark.parametrize("shape,axes", [((1 << 20,), [0]), ((1000003,), [0]), ((513, 4096), [1]), ((4096, 37), [1]), ((64, 100000), [1]),
                                        ((3, 70001), [1]), ((2048, 1024), [0]), ((33, 257, 40), [1]), ((7, 300, 129), [1]), ((5, 4, 6, 64), [1, 2])])
def test_random_shapes_against_the_fp64_oracle(dtype, shape, axes):
    from _exprutil import from_device, to_device

    rng = np.random.default_rng(hash((dtype, shape)) % (1 << 31))
    storage = o.from_float32((rng.standard_normal(int(np.prod(shape))) * 0.5 + 0.01).astype(np.float32), dtype).reshape(shape)
    dev = to_device(storage, dtype)
    src = eo.OTensor.input(o.to_float64(storage.reshape(-1), dtype).reshape(shape), dtype)
    for op, kind in [(Op.Sum, "sum"), (Op.Mean, "mean"), (Op.Max, "max"), (Op.Min, "min"), (Op.L1Norm, "norm1"), (Op.L2Norm, "norm2")]:
        s = CubReduction(op, axes, DataType.fp32).stamp(dev, input_dtype=DataType(dtype))
        s.run()
        torch.cuda.synchronize()
        got = s.output.float().cpu().numpy().reshape(-1).astype(np.float64)
        want = src._reduce(kind, axes, ()).v.reshape(-1)
        if kind in ("max", "min"):
            assert np.array_equal(got, want), (kind, s.kernel_kind())
        else:
            # 1e-5 relative, plus the conditioning term of a sum that cancels: 2e-7 of the sum of magnitudes
            l1 = src._reduce("norm1", axes, ()).v.reshape(-1)
            l1 = l1 / np.prod([shape[a] for a in axes]) if kind == "mean" else l1
            l1 = np.sqrt(l1) if kind == "norm2" else l1
            assert (np.abs(got - want) <= 1e-5 * np.abs(want) + 2e-7 * l1).all(), (kind, s.kernel_kind(), float(np.abs(got - want).max()))


def test_kernel_family_selection():
    assert CubReduction(Op.Sum, [0]).stamp(torch.zeros(1 << 22, device="cuda")).kernel_kind() == "full"
    assert CubReduction(Op.Sum, [1]).stamp(torch.zeros(4096, 4096, device="cuda")).kernel_kind() == "rows_cta"
    assert CubReduction(Op.Sum, [1]).stamp(torch.zeros(4096, 256, device="cuda")).kernel_kind() == "rows_warp"
    assert CubReduction(Op.Sum, [1]).stamp(torch.zeros(4096, 16, device="cuda")).kernel_kind() == "rows_subwarp"
    assert CubReduction(Op.Sum, [1]).stamp(torch.zeros(8, 1 << 20, device="cuda")).kernel_kind() == "rows_split"
    s = CubReduction(Op.Sum, [0]).stamp(torch.zeros(32768, 1024, device="cuda"))
    assert s.kernel_kind() == "cols_split" and s.workspace_bytes() > 1


def test_unaligned_row_starts_need_no_padding():
    """Rows of odd length start at unaligned addresses; the kernel peels to a 16-byte boundary itself."""
    x = torch.randn(257, 1001, device="cuda", dtype=torch.float16)
    s = CubReduction(Op.Sum, [1], DataType.fp32).stamp(x)
    s.run()
    torch.cuda.synchronize()
    want = x.double().sum(dim=1, keepdim=True)
    assert torch.allclose(s.output.double(), want, rtol=1e-5, atol=1e-4)


def test_results_are_bitwise_reproducible():
    x = torch.randn(1 << 24, device="cuda")
    s = CubReduction(Op.Sum, [0]).stamp(x)
    s.run()
    torch.cuda.synchronize()
    first = s.output.clone()
    for _ in range(3):
        s.run()
    torch.cuda.synchronize()
    assert torch.equal(first, s.output)


# ---- arg reductions -------------------------------------------------------------------------------------

def _arg(values, shape, op, axes):
    t = torch.tensor(values, dtype=torch.float32, device="cuda").reshape(shape)
    s = CubArgReduction(op, axes).stamp(t)
    s.run()
    torch.cuda.synchronize()
    return s.value.cpu().numpy().reshape(-1), s.index.cpu().numpy().reshape(-1).astype(np.int64)


def test_arg_reference_golden_vectors():
    v, i = _arg([5.0, -2.0, 7.0, -2.0, 4.0, 7.0], (2, 3), CubArgReductionOp.ArgMin, [0, 1])
    assert list(v) == [-2.0] and list(i) == [1]
    v, i = _arg([5.0, -2.0, 7.0, -2.0, 4.0, 7.0], (2, 3), CubArgReductionOp.ArgMax, [0, 1])
    assert list(v) == [7.0] and list(i) == [2]
    vals = [3.0, 1.0, 1.0, 2.0, -5.0, -1.0, -5.0, -2.0]
    v, i = _arg(vals, (2, 4), CubArgReductionOp.ArgMin, [1])
    assert list(v) == [1.0, -5.0] and list(i) == [1, 0]
    v, i = _arg(vals, (2, 4), CubArgReductionOp.ArgMax, [1])
    assert list(v) == [3.0, -1.0] and list(i) == [0, 1]
    mid = [9.0, 1.0, 5.0, 8.0, -1.0, 4.0, 0.0, 7.0, 6.0, 2.0, 3.0, -2.0]
    v, i = _arg(mid, (2, 3, 2), CubArgReductionOp.ArgMin, [1])
    assert list(v) == [-1.0, 1.0, 0.0, -2.0] and list(i) == [2, 0, 0, 2]
    v, i = _arg(mid, (2, 3, 2), CubArgReductionOp.ArgMax, [1])
    assert list(v) == [9.0, 8.0, 6.0, 7.0] and list(i) == [0, 1, 1, 0]


def test_arg_nan_wins_and_lowest_index_wins_ties():
    vals = [3.0, NAN, 2.0, NAN, 5.0, 5.0, 1.0, 1.0]
    v, i = _arg(vals, (2, 4), CubArgReductionOp.ArgMin, [1])
    assert np.isnan(v[0]) and v[1] == 1.0 and list(i) == [1, 2]
    v, i = _arg(vals, (2, 4), CubArgReductionOp.ArgMax, [1])
    assert np.isnan(v[0]) and v[1] == 5.0 and list(i) == [1, 0]
    v, i = _arg([INF, INF, -INF, -INF], (2, 2), CubArgReductionOp.ArgMin, [1])
    assert list(v) == [INF, -INF] and list(i) == [0, 0]
    v, i = _arg([INF, INF, -INF, -INF], (2, 2), CubArgReductionOp.ArgMax, [1])
    assert list(v) == [INF, -INF] and list(i) == [0, 0]


@pytest.mark.parametrize("shape,axes", [((4096, 4096), [1]), ((300, 1001), [1]), ((1 << 22,), [0]), ((9, 70000), [1]), ((17, 300, 64), [1]), ((5, 999, 3), [1])])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_arg_random_with_many_ties(shape, axes, dtype):
    rng = np.random.default_rng(11)
    vals = rng.integers(-4, 5, size=shape).astype(np.float32)  # few distinct values: many ties
    vals.reshape(-1)[rng.integers(0, vals.size, 5)] = np.nan
    x = torch.from_numpy(vals).to(dtype).cuda()
    for op, is_max in ((CubArgReductionOp.ArgMax, True), (CubArgReductionOp.ArgMin, False)):
        s = CubArgReduction(op, axes).stamp(x)
        s.run()
        torch.cuda.synchronize()
        src = eo.OTensor.input(vals.astype(np.float64), o.FP32)
        want = src._arg(is_max, axes, ()).v.reshape(-1)
        assert np.array_equal(s.index.cpu().numpy().reshape(-1).astype(np.float64), want)
