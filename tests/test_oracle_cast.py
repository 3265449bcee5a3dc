"""Pins the restated cast oracle: against the golden vectors produced by the reference's own CPU
converter (tests/golden/cast_golden.npz), and live against that converter when oracle/_ref exists."""
from pathlib import Path

import numpy as np
import pytest

import oracle as o
from thor_b200.workloads import cast_input

GOLDEN = np.load(Path(__file__).parent / "golden" / "cast_golden.npz")


def _bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(a.size, -1)


def _same(a, b, dt):
    """Bit equality; fp8 NaN payloads are compared as 'both NaN' (the CUDA host and device
    conversions differ in the e5m2 NaN payload they emit)."""
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    if dt in (o.FP8_E5M2, o.FP8_E4M3):
        fa, fb = o.to_float64(a.view(np.uint8), dt), o.to_float64(b.view(np.uint8), dt)
        nan = np.isnan(fa) & np.isnan(fb)
        return np.array_equal(a.view(np.uint8)[~nan], b.view(np.uint8)[~nan])
    return np.array_equal(_bits(a), _bits(b))


@pytest.mark.parametrize("dst", [o.FP16, o.BF16, o.FP8_E4M3, o.FP8_E5M2, o.FP64])
def test_f32_edges_match_reference_golden(dst):
    got = o.cast(GOLDEN["f32_in"], o.FP32, dst)
    assert _same(got, GOLDEN[f"f32_to_{o.NAMES[dst]}"], dst)


@pytest.mark.parametrize("dst", [o.FP16, o.BF16, o.FP8_E4M3, o.FP8_E5M2, o.FP32])
def test_f64_single_rounding_matches_reference_golden(dst):
    got = o.cast(GOLDEN["f64_in"], o.FP64, dst)
    assert _same(got, GOLDEN[f"f64_to_{o.NAMES[dst]}"], dst)


def test_all_16bit_and_8bit_patterns_widen_like_the_reference():
    all16 = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    for name, src, sdt, ddt in [("fp16_all_to_fp32", all16.view(np.float16), o.FP16, o.FP32), ("bf16_all_to_fp32", all16, o.BF16, o.FP32),
                                ("fp16_all_to_bf16", all16.view(np.float16), o.FP16, o.BF16), ("bf16_all_to_fp16", all16, o.BF16, o.FP16)]:
        got = o.cast(src, sdt, ddt)
        want = GOLDEN[name]
        if ddt == o.FP32:  # NaN payloads differ between the CUDA host and device widening: compare NaN-ness
            keep = ~np.isnan(want)
            assert np.array_equal(np.isnan(got), np.isnan(want)), name
            assert np.array_equal(got[keep].view(np.uint32), want[keep].view(np.uint32)), name
        else:
            assert np.array_equal(got.view(np.uint8), np.ascontiguousarray(want).view(np.uint8)), name
    all8 = np.arange(256, dtype=np.uint16).astype(np.uint8)
    for name, sdt in [("e4m3_all_to_fp32", o.FP8_E4M3), ("e5m2_all_to_fp32", o.FP8_E5M2)]:
        got = o.cast(all8, sdt, o.FP32)
        keep = ~np.isnan(GOLDEN[name])
        assert np.array_equal(np.isnan(got), np.isnan(GOLDEN[name])), name
        assert np.array_equal(got[keep].view(np.uint32), GOLDEN[name][keep].view(np.uint32)), name


@pytest.mark.parametrize("src", o.ALL_DTYPES, ids=lambda d: o.NAMES[d])
def test_representable_grid_all_pairs(src):
    """The reference's TypeConverterTest.cpp:10-765 runs every pair on exactly representable values."""
    s = GOLDEN[f"grid_{o.NAMES[src]}"]
    s = s.view(np.float16) if src == o.FP16 else s
    for dst in o.ALL_DTYPES:
        if dst == src:
            continue
        got = o.cast(s, src, dst)
        want = GOLDEN[f"grid_{o.NAMES[src]}_to_{o.NAMES[dst]}"]
        assert np.array_equal(got.view(np.uint8), np.ascontiguousarray(want).view(np.uint8)), (o.NAMES[src], o.NAMES[dst])


def test_probed_fp16_edge_values():
    x = np.array([1.00048828125, 65520.0, 2.0 ** -25, np.nextafter(np.float32(2.0 ** -25), np.float32(1)), np.nan, -0.0, 65519.996], np.float32)
    got = o.cast(x, o.FP32, o.FP16).view(np.uint16)
    assert [int(v) for v in got] == [0x3C00, 0x7C00, 0x0000, 0x0001, 0x7FFF, 0x8000, 0x7BFF]


@pytest.mark.skipif(o.reference_cast_lib() is None, reason="oracle/_ref not built (reference checkout absent)")
def test_configuration_1_input_matches_live_reference():
    x = cast_input(1 << 20, seed=0, edge_density=1e-2)
    assert np.array_equal(o.cast(x, o.FP32, o.FP16).view(np.uint16), o.reference_cast(x, o.FP32, o.FP16).view(np.uint16))
    assert np.array_equal(o.cast(x, o.FP32, o.BF16), o.reference_cast(x, o.FP32, o.BF16))


def test_numpy_float16_agrees_on_non_nan_values():
    x = cast_input(1 << 18, seed=3, edge_density=5e-2)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(o.cast(x, o.FP32, o.FP16).view(np.uint16), want)
