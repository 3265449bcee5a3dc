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
