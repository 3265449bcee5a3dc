"""Value reductions against the REFERENCE's own device code: its fp32 operators, finalise-and-store output iterator,
CUB calls and tiled [outer, reduction, inner] kernels (Utilities/TensorOperations/Cub/CubReductionOperation.cuh),
compiled from the reference checkout into oracle/_ref and launched on the same device buffers.

min / max are exact (the result is one of the inputs; NaN propagates); sums and means accumulate in fp32 in a
different order on the two sides, so they agree to 1e-5 relative with an absolute floor for cancelling sums
(1e-6 x the sum of magnitudes), and 16-bit outputs to one output ulp."""
import numpy as np
import pytest
import torch

import oracle as o
from thor_b200 import DataType
from thor_b200.reductions import CubReduction, CubReductionOp

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(o.reference_cub_reduce_lib() is None, reason="oracle/_ref holds no build of the reference's reductions")]

_TORCH = {DataType.fp32: torch.float32, DataType.fp16: torch.float16, DataType.bf16: torch.bfloat16}
_OPS = {"sum": CubReductionOp.Sum, "mean": CubReductionOp.Mean, "max": CubReductionOp.Max, "min": CubReductionOp.Min}


def _reference(op, x3, out_dtype):
    outer, red, inner = x3.shape
    in_dtype = {torch.float32: DataType.fp32, torch.float16: DataType.fp16, torch.bfloat16: DataType.bf16}[x3.dtype]
    path, ws_bytes = o.reference_cub_reduce_workspace(op, int(in_dtype), int(out_dtype), outer, red, inner)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    out = torch.full((outer * inner,), float("nan"), dtype=_TORCH[out_dtype], device="cuda")
    o.reference_cub_reduce(op, path, x3.data_ptr(), int(in_dtype), out.data_ptr(), int(out_dtype), outer, red, inner, ws.data_ptr(), ws_bytes,
                           torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return out, path


def _ours(op, x3, out_dtype):
    s = CubReduction(_OPS[op], 1, out_dtype).stamp(x3)
    s.run()
    torch.cuda.synchronize()
    return s.output.reshape(-1)


def _compare(op, x3, out_dtype, got, want):
    g, w = got.double().cpu().numpy(), want.double().cpu().numpy()
    assert np.array_equal(np.isnan(g), np.isnan(w))
    if op in ("max", "min"):
        assert np.array_equal(g, w, equal_nan=True)
        return
    mag = x3.double().abs().sum(dim=1).reshape(-1).cpu().numpy()
    if op == "mean":
        mag = mag / x3.shape[1]
    tol = 1e-5 * np.abs(w) + 1e-6 * mag
    if out_dtype != DataType.fp32:
        tol = tol + np.abs(w) * (2.0 ** -10 if out_dtype == DataType.fp16 else 2.0 ** -7)
    same_inf = np.isinf(g) & np.isinf(w) & (np.sign(g) == np.sign(w))  # a sum that overflows the 16-bit output on both sides
    with np.errstate(invalid="ignore"):
        bad = (np.abs(g - w) > tol) & ~same_inf
    assert not bad.any(), (float(np.abs(g - w).max()), int(bad.sum()))


SHAPES = [
    # [outer, reduction, inner]: full reductions, contiguous rows, column / middle-axis reductions
    (1, 1 << 20, 1), (1, 100003, 1), (1, 7, 1),
    (4096, 4096, 1), (333, 1000, 1), (10000, 36, 1), (3, 70001, 1),
    (1, 4096, 8192), (1, 2048, 1000), (8, 100, 64), (5, 333, 7), (2, 50, 4096), (1, 1000, 33),
]


@pytest.mark.parametrize("outer,red,inner", SHAPES)
@pytest.mark.parametrize("op", ["sum", "mean", "max", "min"])
def test_fp32_reductions_match_the_reference_device_code(op, outer, red, inner):
    g = torch.Generator(device="cuda").manual_seed(outer * 31 + red * 7 + inner)
    x = torch.randn(outer, red, inner, device="cuda", generator=g) * 3.0 + 0.25
    want, _ = _reference(op, x, DataType.fp32)
    _compare(op, x, DataType.fp32, _ours(op, x, DataType.fp32), want)


@pytest.mark.parametrize("in_dtype,out_dtype", [(DataType.bf16, DataType.fp32), (DataType.fp16, DataType.fp32), (DataType.bf16, DataType.bf16), (DataType.fp32, DataType.fp16)])
@pytest.mark.parametrize("outer,red,inner", [(1, 1 << 18, 1), (512, 2048, 1), (1, 1024, 2048), (4, 300, 48)])
@pytest.mark.parametrize("op", ["sum", "mean", "max"])
def test_16_bit_inputs_and_outputs_match_the_reference_device_code(op, outer, red, inner, in_dtype, out_dtype):
    g = torch.Generator(device="cuda").manual_seed(red + inner)
    x = (torch.randn(outer, red, inner, device="cuda", generator=g) * 2.0 + 0.5).to(_TORCH[in_dtype])
    want, _ = _reference(op, x, out_dtype)
    _compare(op, x, out_dtype, _ours(op, x, out_dtype), want)


@pytest.mark.parametrize("outer,red,inner", [(1, 5000, 1), (64, 257, 1), (1, 300, 96)])
def test_nan_and_infinities_propagate_like_the_reference(outer, red, inner):
    x = torch.randn(outer, red, inner, device="cuda")
    x[0, red // 2, 0] = float("nan")
    x[-1, 1, -1] = float("inf")
    x[-1, red - 1, -1] = float("-inf") if outer * inner > 1 else x[-1, red - 1, -1]
    for op in ("sum", "max", "min"):
        want, _ = _reference(op, x, DataType.fp32)
        got = _ours(op, x, DataType.fp32)
        g, w = got.cpu().numpy(), want.cpu().numpy()
        assert np.array_equal(np.isnan(g), np.isnan(w)), op
        if op != "sum":
            assert np.array_equal(g, w, equal_nan=True), op
        else:
            assert np.array_equal(np.isinf(g), np.isinf(w))


def test_paths_follow_the_reference_geometry_rule():
    x = torch.randn(1, 4096, 1, device="cuda")
    assert _reference("sum", x, DataType.fp32)[1] == 0
    assert _reference("sum", torch.randn(16, 64, 1, device="cuda"), DataType.fp32)[1] == 1
    assert _reference("sum", torch.randn(2, 64, 8, device="cuda"), DataType.fp32)[1] == 2


# ---- arg reductions: value and index must be identical (NaN wins, lowest index among equals) ----

def _reference_arg(is_max, x3):
    outer, red, inner = x3.shape
    in_dtype = {torch.float32: DataType.fp32, torch.float16: DataType.fp16, torch.bfloat16: DataType.bf16}[x3.dtype]
    path, ws_bytes = o.reference_cub_argreduce_workspace(is_max, int(in_dtype), outer, red, inner, o.UINT32)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    val = torch.full((outer * inner,), float("nan"), device="cuda")
    idx = torch.full((outer * inner,), -1, dtype=torch.int32, device="cuda")
    o.reference_cub_argreduce(is_max, path, x3.data_ptr(), int(in_dtype), val.data_ptr(), o.FP32, idx.data_ptr(), o.UINT32, outer, red, inner, ws.data_ptr(), ws_bytes,
                              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return val.cpu().numpy(), idx.cpu().numpy().view(np.uint32)


ARG_SHAPES = [(1, 100003, 1), (1, 9, 1), (4096, 4096, 1), (333, 1000, 1), (10000, 36, 1), (1, 2048, 1000), (8, 100, 64), (5, 333, 7), (2, 50, 4096)]


@pytest.mark.skipif(o.reference_cub_reduce_lib() is None or not hasattr(o.reference_cub_reduce_lib(), "thor_ref_cub_argreduce"), reason="no build of the reference's arg reductions")
@pytest.mark.parametrize("outer,red,inner", ARG_SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("is_max", [True, False])
def test_arg_reductions_match_the_reference_device_code(is_max, dtype, outer, red, inner):
    from thor_b200.reductions import CubArgReduction, CubArgReductionOp

    g = torch.Generator(device="cuda").manual_seed(outer + red * 3 + inner * 5)
    # few distinct values, so that ties are everywhere; some NaN and infinities
    x = torch.randint(-6, 7, (outer, red, inner), device="cuda", generator=g).to(torch.float32) * 0.5
    flat = x.reshape(-1)
    n = flat.numel()
    pick = torch.randint(0, n, (max(1, n // 5000),), device="cuda", generator=g)
    flat[pick[::3]] = float("nan")
    flat[pick[1::3]] = float("inf")
    flat[pick[2::3]] = float("-inf")
    x = x.to(dtype)
    want_v, want_i = _reference_arg(is_max, x)
    s = CubArgReduction(CubArgReductionOp.ArgMax if is_max else CubArgReductionOp.ArgMin, [1]).stamp(x)
    s.run()
    torch.cuda.synchronize()
    got_i = s.index.cpu().numpy().reshape(-1).astype(np.uint32)
    got_v = s.value.float().cpu().numpy().reshape(-1)
    assert np.array_equal(got_i, want_i), int((got_i != want_i).sum())
    assert np.array_equal(got_v, want_v, equal_nan=True)
