"""The allocation-free full reduction (thor_b200_reduce_full_noalloc) against the planned reduction.

Some users of this library never get a chance to allocate device memory: all of it was handed out when the
process started, or they run as a plug-in that may not call the allocator, or a cudaMalloc (which
synchronises the device) is not acceptable inside their loop.  For them one entry point keeps its
scratch in a fixed array inside the library.  This file is collected last on purpose, so that a failure
here cannot hide the result of any other test in a stop-at-first-failure run.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from thor_b200 import DataType, _native
from thor_b200.reductions import CubReduction, CubReductionOp

pytestmark = pytest.mark.gpu

_lib = _native.lib
_lib.thor_b200_reduce_full_noalloc.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_uint64, C.c_void_p, C.c_int, C.c_float, C.c_void_p]
_lib.thor_b200_reduce_full_noalloc.restype = C.c_int


def _noalloc(op, x, out_dtype=torch.float32, scale=1.0):
    out = torch.empty(1, dtype=out_dtype, device="cuda")
    from thor_b200.dtypes import from_torch

    _native.check(_lib.thor_b200_reduce_full_noalloc(int(op), x.data_ptr(), int(from_torch(x.dtype)), x.numel(), out.data_ptr(), int(from_torch(out_dtype)),
                                                     C.c_float(scale), _native.stream_handle()))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_two_calls_in_a_row_match_the_planned_reduction(dtype):
    """Same arithmetic as thor_b200_reduce_launch (tolerance of the reduction tests: 1e-5 relative; min / max exact).
    The second call uses other data and another length, so values left in the shared scratch by the first call
    would show up as an error."""
    gen = torch.Generator(device="cuda").manual_seed(1)
    for n in ((1 << 22) + 5, (1 << 20) - 3):
        x = (torch.randn(n, device="cuda", generator=gen) + 0.01).to(dtype)
        for op in (CubReductionOp.Sum, CubReductionOp.Mean, CubReductionOp.Max, CubReductionOp.Min, CubReductionOp.L1Norm, CubReductionOp.L2Norm):
            ref = CubReduction(op, [0], DataType.fp32).stamp(x)
            ref.run()
            got = _noalloc(op, x)
            torch.cuda.synchronize()
            want = ref.output.reshape(1)
            if op in (CubReductionOp.Max, CubReductionOp.Min):
                assert torch.equal(got, want), op
            else:
                assert torch.allclose(got, want, rtol=1e-5, atol=1e-6), (op, float(got), float(want))


@pytest.mark.parametrize("n", [1000, (1 << 21) + 17, 1 << 24])
def test_against_an_independent_fp64_sum_and_torch_extremes(n):
    """Not the library against itself: float64 sums and torch's own max / min of the same values, including an fp8 input
    (converted to fp32 per element, accumulated in fp32 like the reduction seam) and sizes on both sides of the point
    where the two-phase form needs its fold."""
    gen = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(n, device="cuda", generator=gen) + 0.01
    for t in (x, x.bfloat16(), x.to(torch.float8_e4m3fn)):
        wide = t.double() if t.dtype != torch.float8_e4m3fn else t.float().double()
        got = float(_noalloc(CubReductionOp.Sum, t))
        assert abs(got - float(wide.sum())) <= 1e-5 * abs(float(wide.sum())) + 2e-7 * float(wide.abs().sum())
        assert float(_noalloc(CubReductionOp.Max, t)) == float(wide.max()) and float(_noalloc(CubReductionOp.Min, t)) == float(wide.min())
        want_l2 = float(wide.pow(2).sum().sqrt())
        assert abs(float(_noalloc(CubReductionOp.L2Norm, t)) - want_l2) <= 1e-5 * want_l2


def test_small_input_and_output_scale_and_dtype():
    x = torch.tensor([-2.0, 3.0, -4.0], device="cuda")
    assert float(_noalloc(CubReductionOp.Sum, x)) == -3.0
    assert float(_noalloc(CubReductionOp.Product, x)) == 24.0
    assert float(_noalloc(CubReductionOp.Sum, x, scale=0.5)) == -1.5
    assert float(_noalloc(CubReductionOp.L1Norm, x, out_dtype=torch.float16)) == 9.0


def test_sizes_beyond_the_fixed_scratch_are_rejected_before_any_launch():
    x = torch.zeros(8, device="cuda")
    out = torch.zeros(1, device="cuda")
    too_many = 65536 * 4096 * 4 + 1  # one element more than the fp32 limit; the pointer is never dereferenced
    rc = _lib.thor_b200_reduce_full_noalloc(0, x.data_ptr(), int(DataType.fp32), too_many, out.data_ptr(), int(DataType.fp32), C.c_float(1.0), _native.stream_handle())
    assert rc == 1
    msg = _lib.thor_b200_last_error().decode()
    assert "exceed the fixed scratch" in msg and "thor_b200_reduce_launch" in msg
    with pytest.raises(_native.ThorB200InvalidArgument):
        _native.check(_lib.thor_b200_reduce_full_noalloc(0, x.data_ptr(), int(DataType.fp32), 0, out.data_ptr(), int(DataType.fp32), C.c_float(1.0), None))


def test_the_call_allocates_no_device_memory():
    x = torch.randn(1 << 22, device="cuda")
    _noalloc(CubReductionOp.Sum, x)  # first call on this device resolves the scratch address
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        _noalloc(CubReductionOp.Sum, x)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    # `out` comes from torch's caching allocator (already reserved); the driver-level free memory must not move
    assert free_after == free_before
