"""The dumper around the reference's own source emitter (oracle/_ref/libthor_ref_emit.so) needs no GPU: these checks
pin what the reference generates for the headline expression, i.e. the arithmetic our fused stage has to reproduce
(the GPU tests then run both kernels on the same buffers)."""
import pytest

import oracle as o

pytestmark = pytest.mark.skipif(o.reference_emitter_lib() is None, reason="the reference's emitter is not built (oracle/_ref)")

C2 = "in:a in:x mul rs:b add lit:0 max in:z sigmoid mul"


def test_reference_flat_kernel_for_the_headline_expression_uses_the_half2_intrinsics():
    src, ept, order, out_dtype = o.reference_emit_flat(C2, {"a": o.FP16, "x": o.FP16, "b": o.FP32, "z": o.FP16})
    assert ept == 8 and order == ["a", "x", "b", "z"] and out_dtype == o.FP16
    for needle in ("__hmul2", "__hadd2", "__hmax2", "h2exp", "__h2div", "half(in2)"):
        assert needle in src, needle
    assert src.count("h2exp(") == 8  # two exponentials per half2 pair, four pairs per thread


def test_reference_broadcast_kernel_for_configuration_2_is_one_half2_per_thread_with_baked_shapes():
    src, ept, order, out_dtype, numel = o.reference_emit_broadcast(C2, {"a": o.FP16, "x": o.FP16, "b": o.FP32, "z": o.FP16},
                                                                    {"a": (8192,), "x": (8192, 8192), "z": (8192, 8192)})
    assert ept == 2 and numel == 8192 * 8192 and out_dtype == o.FP16
    assert "numel" not in src.split("{")[0], "broadcast kernels take no shape argument"
    assert "33554432U" in src and "half2* out0" in src and src.count("h2exp(") == 2


def test_fp32_stage_uses_libdevice_functions_and_four_elements_per_thread():
    src, ept, _, out_dtype = o.reference_emit_flat("in:x sigmoid in:y tanh mul", {"x": o.FP32, "y": o.FP32})
    assert ept == 4 and out_dtype == o.FP32
    assert "expf(" in src and "tanhf(" in src and "fmaxf(" in src


def test_mixed_16_bit_inputs_promote_to_fp32_in_the_reference_too():
    _, _, _, out_dtype = o.reference_emit_flat("in:x in:y add", {"x": o.FP16, "y": o.BF16})
    assert out_dtype == o.FP32


RESOLUTION_CASES = [
    (C2, {"a": o.FP16, "x": o.FP16, "b": o.FP32, "z": o.FP16}),
    (C2, {"a": o.BF16, "x": o.BF16, "b": o.FP32, "z": o.BF16}),
    (C2, {"a": o.FP16, "x": o.FP32, "b": o.FP32, "z": o.BF16}),
    ("in:x in:y add lit:2 mul exp", {"x": o.FP8_E4M3, "y": o.FP8_E5M2}),
    ("in:x in:y add lit:2 mul exp", {"x": o.FP8_E4M3, "y": o.FP8_E4M3}),
    ("in:x in:y mul cast:24 in:z add tanh", {"x": o.FP16, "y": o.FP16, "z": o.FP32}),
    ("in:x softplus in:y gelu mul in:z selu sub", {"x": o.BF16, "y": o.FP16, "z": o.BF16}),
    ("in:x lit:0.5 pow in:y abs sqrt div cast:10", {"x": o.FP32, "y": o.BF16}),
    ("in:x in:y min in:z max neg expm1", {"x": o.FP8_E5M2, "y": o.BF16, "z": o.BF16}),
]


@pytest.mark.parametrize("program,dtypes", RESOLUTION_CASES)
def test_dtype_resolution_agrees_with_the_reference_node_for_node(program, dtypes):
    """Our resolveOutputsDTypesInPlace against the reference's own (ExpressionDTypeResolution.cpp:1012-1148): the set of
    (op, output dtype, compute dtype) over all nodes is identical (the reference keeps duplicate nodes that our builder
    shares, so multiplicities are not compared) and so is the output node."""
    from _exprutil import build_postfix
    from thor_b200 import DataType
    from thor_b200.expression import resolve_dtypes

    theirs = o.reference_resolve_dtypes(program, dtypes)
    ours = resolve_dtypes({"output": build_postfix(program)}, {k: DataType(v) for k, v in dtypes.items()})
    ours = [(int(op), int(out), int(comp)) for op, out, comp in ours]
    assert set(ours) == set(theirs), (sorted(set(ours) - set(theirs)), sorted(set(theirs) - set(ours)))
    assert ours[-1] == theirs[-1]
