"""Our fused stages against the kernels that the REFERENCE's own emitter generates for the same expressions
(CudaSourceEmitter::emitFlat compiled from the reference checkout into oracle/_ref, NVRTC with the reference's
flags), on the same device buffers.  16-bit stages use the same pair intrinsics and must agree bit for bit;
fp32 stages call the same libdevice functions under -fmad=true and must agree within 2 fp32 ulp with almost
all elements identical (the compiler may place a fused multiply-add differently in the two sources)."""
import numpy as np
import pytest
import torch

import oracle as o
from oracle import expr_oracle as eo
from thor_b200 import DataType
from thor_b200.expression import Expression as ex

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(o.reference_emitter_lib() is None, reason="the reference's emitter is not built (oracle/_ref)")]

from oracle.refkernel import ReferenceBroadcastKernel, run_reference_flat  # noqa: E402

_T = {o.FP32: torch.float32, o.FP16: torch.float16, o.BF16: torch.bfloat16}


def _ours(program: str, tensors, scalars):
    """The same postfix program through this repository's Expression API."""
    from _exprutil import build_postfix

    plan = ex.compile(build_postfix(program)).stamp({**tensors, **scalars})
    plan.run()
    return plan


PROGRAMS = [
    ("c2", "in:a in:x mul rs:b add lit:0 max in:z sigmoid mul", {"b": 0.1}),
    ("affine_tanh", "in:x in:a mul in:z add tanh", {}),
    ("softplus_swish", "in:x softplus in:z swish mul", {}),
    ("gelu_selu", "in:x gelu in:z selu add", {}),
    ("exp_log", "in:x exp lit:1 add ln in:a abs sqrt mul", {}),
    ("div_pow", "in:x in:a abs lit:0.5 add div in:z abs lit:1.5 pow add", {}),
    ("minmax_neg", "in:x in:z min in:a neg max lit:0.25 mul", {}),
    ("erf_expm1", "in:x erf in:z lit:0.5 mul expm1 sub", {}),
    # constant subtrees (folded in double to one float literal) and identities (x + 0, x * 1, x / 1 compute nothing):
    # CudaSourceEmitter.cpp:1965-2076, 3745-3782 -- in 16-bit stages a per-node evaluation would round differently
    ("const_fold", "in:x lit:0.1 lit:3 mul mul in:z lit:0.7 neg lit:3 div mul mul", {}),  # products only: no fused multiply-add to place differently
    ("identities", "in:x lit:0 add lit:1 mul in:z lit:2 lit:1 sub div mul lit:0 in:a add mul", {}),
]


@pytest.mark.parametrize("dtype", [o.FP16, o.BF16, o.FP32])
@pytest.mark.parametrize("name,program,scalars", PROGRAMS, ids=[p[0] for p in PROGRAMS])
def test_fused_stage_matches_the_reference_emitted_kernel(dtype, name, program, scalars):
    n, pad = (1 << 18) + 24, 64
    g = torch.Generator(device="cuda").manual_seed(11)
    tensors = {k: torch.randn(n + pad, device="cuda", generator=g).to(_T[dtype]) for k in ("a", "x", "z") if f"in:{k}" in program}
    dts = {k: dtype for k in tensors}
    dts.update({k: o.FP32 for k in scalars})
    theirs, out_dtype = run_reference_flat(program, {**tensors, **scalars}, dts, n, pad)
    plan = _ours(program, {k: v[:n] for k, v in tensors.items()}, scalars)
    torch.cuda.synchronize()
    ours = plan.output()
    # a literal subtree is an fp32 value in the reference's dtype resolution and promotes the stage to fp32
    promoted = name in ("const_fold", "identities")
    assert int(out_dtype) == (o.FP32 if promoted else dtype) and ours.dtype == _T[int(out_dtype)]
    a = ours.float().cpu().numpy().astype(np.float64)
    b = theirs[:n].float().cpu().numpy().astype(np.float64)
    assert np.array_equal(np.isnan(a), np.isnan(b))
    if int(out_dtype) in (o.FP16, o.BF16):
        same = ours.view(torch.int16).cpu().numpy() == theirs[:n].view(torch.int16).cpu().numpy()
        assert bool((same | np.isnan(a)).all()), f"{(~same).sum()} of {n} elements differ from the reference kernel"
    else:
        d = eo.ulp_distance(a, b, o.FP32)
        assert float(d.max()) <= 2.0, float(d.max())
        assert float((d == 0).mean()) > 0.999


def test_mixed_dtypes_and_casts_match_the_reference_emitted_kernel():
    n, pad = 100003, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(n + pad, device="cuda", generator=g).half()
    y = torch.randn(n + pad, device="cuda", generator=g).bfloat16()
    program = "in:x in:y add lit:2 mul cast:10"  # fp16 + bf16 -> fp32, stored as fp16
    theirs, out_dtype = run_reference_flat(program, {"x": x, "y": y}, {"x": o.FP16, "y": o.BF16}, n, pad)
    plan = _ours(program, {"x": x[:n], "y": y[:n]}, {})
    torch.cuda.synchronize()
    assert int(out_dtype) == o.FP16
    assert torch.equal(plan.output().view(torch.int16), theirs[:n].view(torch.int16))


@pytest.mark.parametrize("rows,cols", [(512, 8192), (8192, 8192)])
def test_configuration_2_matches_the_reference_broadcast_kernel_bit_for_bit(rows, cols):
    """relu(a*x + b) * sigmoid(z) with a broadcast over the rows: the kernel CudaSourceEmitter::emitSpecializedBroadcast
    generates for these shapes (one half2 per thread, shapes baked in) against our tiled stage, same buffers."""
    program = "in:a in:x mul rs:b add lit:0 max in:z sigmoid mul"
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(rows, cols, device="cuda", generator=g).half()
    z = torch.randn(rows, cols, device="cuda", generator=g).half()
    a = (torch.rand(cols, device="cuda", generator=g) + 0.5).half()
    ref = ReferenceBroadcastKernel(program, {"a": o.FP16, "x": o.FP16, "b": o.FP32, "z": o.FP16}, {"a": (cols,), "x": (rows, cols), "z": (rows, cols)})
    assert ref.ept == 2 and ref.numel == rows * cols and ref.out_dtype == o.FP16
    theirs = torch.empty(rows, cols, device="cuda", dtype=torch.float16)
    ref.launch({"a": a, "x": x, "b": 0.1, "z": z}, theirs)
    plan = _ours(program, {"a": a, "x": x, "z": z}, {"b": 0.1})
    torch.cuda.synchronize()
    assert plan.physical_stage_names() == ["bcast_tiled_v2"]
    assert torch.equal(plan.output().view(torch.int16), theirs.view(torch.int16))


def test_row_and_column_broadcasts_in_fp32_match_the_reference_broadcast_kernel():
    program = "in:x in:r sub exp in:c mul"
    rows, cols = 300, 1000
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(rows, cols, device="cuda", generator=g)
    r = torch.randn(rows, 1, device="cuda", generator=g)
    c = torch.randn(cols, device="cuda", generator=g)
    ref = ReferenceBroadcastKernel(program, {"x": o.FP32, "r": o.FP32, "c": o.FP32}, {"x": (rows, cols), "r": (rows, 1), "c": (cols,)})
    theirs = torch.empty(rows, cols, device="cuda")
    ref.launch({"x": x, "r": r, "c": c}, theirs)
    plan = _ours(program, {"x": x, "r": r, "c": c}, {})
    torch.cuda.synchronize()
    d = eo.ulp_distance(plan.output().double().cpu().numpy(), theirs.double().cpu().numpy(), o.FP32)
    assert float(d.max()) <= 2.0 and float((d == 0).mean()) > 0.999


def test_reference_stage_lists_compute_what_our_row_programs_compute():
    """The benchmark's reference stage-list baselines (reference-emitted fused kernels + the reference's own CUB
    reductions where oracle/_ref holds them, ours standing in otherwise) produce the results our single row programs
    produce, so their times compare like with like."""
    import bench

    class _Single:
        rank, world, enabled, local_rank = 0, 1, False, 0

    sm = bench.C3ReferenceStagePipeline(_Single(), 1.0 / 256)
    sm.setup()
    sm.step(0)
    xi = ex.input("x")
    e = (xi - xi.reduce_max([1])).exp()
    ours = ex.compile(e / e.reduce_sum([1])).stamp({"x": sm.x})
    ours.run()
    torch.cuda.synchronize()
    np.testing.assert_allclose(sm.y.cpu().numpy(), ours.output().cpu().numpy(), rtol=1e-5, atol=1e-12)

    ln = bench.C5FwdReferenceStagePipeline(_Single(), 1.0 / 256)
    ln.setup()
    ln.step(0)
    ours = ex.compile({"y": bench._layernorm_expr(ex)}).stamp({"x": ln.x, "gamma": ln.gamma, "beta": ln.beta})
    ours.run()
    torch.cuda.synchronize()
    a, b = ours.output("y").float().cpu().numpy().astype(np.float64), ln.y.float().cpu().numpy().astype(np.float64)
    d = eo.ulp_distance(a, b, o.BF16)
    d = np.where(np.abs(a - b) <= 1e-7, 0.0, d)  # results that cancel to ~0: the fp32 noise of the two summation orders, not a bf16 step
    assert float(d.max()) <= 1.0 and float((d == 0).mean()) > 0.99

    if o.reference_cub_reduce_lib() is not None:
        st = bench.C4ReferenceStagePipeline(_Single(), 1.0 / 256)
        st.setup()
        st.step(0)
        x = st.x[: st.N]
        xi = ex.input("x")
        ours = ex.compile({"sum": xi.reduce_sum(), "sumsq": (xi * xi).reduce_sum(), "max": xi.reduce_max()}).stamp({"x": x})
        ours.run()
        torch.cuda.synchronize()
        mag = float(x.double().abs().sum())
        assert abs(float(ours.output("sum")) - float(st.outs[0])) <= 1e-5 * abs(float(st.outs[0])) + 1e-6 * mag
        assert abs(float(ours.output("sumsq")) - float(st.outs[1])) <= 1e-5 * float(st.outs[1])
        assert float(ours.output("max")) == float(st.outs[2])


@pytest.mark.parametrize("dtype", [o.FP8_E4M3, o.FP8_E5M2])
@pytest.mark.parametrize("program", ["in:x in:z add lit:0.5 mul", "in:x sigmoid in:z mul", "in:x in:z max exp"])
def test_fp8_stages_match_the_reference_emitted_kernel_bit_for_bit(dtype, program):
    """fp8 storage computes in fp16 and is rounded to fp8 only at the store; the reference's vectorised fp8 kernels
    (16 elements per thread) and ours must produce the same bytes."""
    n, pad = (1 << 16) + 48, 64
    tdt = torch.float8_e4m3fn if dtype == o.FP8_E4M3 else torch.float8_e5m2
    g = torch.Generator(device="cuda").manual_seed(21)
    tensors = {k: (torch.randn(n + pad, device="cuda", generator=g) * 2.0).to(tdt) for k in ("x", "z")}
    theirs, out_dtype = run_reference_flat(program, tensors, {k: dtype for k in tensors}, n, pad)
    plan = _ours(program, {k: v[:n] for k, v in tensors.items()}, {})
    torch.cuda.synchronize()
    assert int(out_dtype) == dtype and plan.output().dtype == tdt
    a, b = plan.output().view(torch.uint8).cpu().numpy(), theirs[:n].view(torch.uint8).cpu().numpy()
    nan = np.isnan(plan.output().float().cpu().numpy())
    assert bool(((a == b) | nan).all()), f"{int((a != b).sum())} of {n} bytes differ from the reference kernel"


LAYOUTS = [
    ("col_vector", "in:x in:c mul in:x add", {"x": (64, 300), "c": (300,)}),
    ("middle_axis", "in:x in:m sub in:r mul", {"x": (8, 32, 64), "m": (8, 1, 64), "r": (32, 1)}),
    ("two_way", "in:x in:y add tanh", {"x": (16, 1, 128), "y": (1, 24, 128)}),
    ("row_scalar_4d", "in:x in:s div in:b add", {"x": (4, 6, 10, 16), "s": (4, 6, 1, 1), "b": (16,)}),
]


@pytest.mark.parametrize("dtype", [o.FP16, o.BF16, o.FP32])
@pytest.mark.parametrize("name,program,dims", LAYOUTS, ids=[c[0] for c in LAYOUTS])
def test_broadcast_layouts_match_the_reference_broadcast_kernel(dtype, name, program, dims):
    g = torch.Generator(device="cuda").manual_seed(31)
    tensors = {k: (torch.randn(*shape, device="cuda", generator=g) + (2.0 if k == "s" else 0.0)).to(_T[dtype]) for k, shape in dims.items()}
    ref = ReferenceBroadcastKernel(program, {k: dtype for k in dims}, dims)
    out_shape = torch.broadcast_shapes(*dims.values())
    theirs = torch.zeros(out_shape, device="cuda", dtype=_T[dtype])
    ref.launch(tensors, theirs)
    plan = _ours(program, tensors, {})
    torch.cuda.synchronize()
    ours = plan.output()
    assert tuple(ours.shape) == tuple(out_shape) and ref.numel == theirs.numel()
    if dtype == o.FP32:
        d = eo.ulp_distance(ours.double().cpu().numpy(), theirs.double().cpu().numpy(), o.FP32)
        assert float(d.max()) <= 2.0 and float((d == 0).mean()) > 0.999
    else:
        assert torch.equal(ours.view(torch.int16), theirs.view(torch.int16)), plan.physical_stage_names()
