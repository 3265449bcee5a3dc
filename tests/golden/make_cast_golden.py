"""Generates tests/golden/cast_golden.npz from the REFERENCE's own CPU converter.

Needs oracle/_ref/libthor_ref_cast.so (built by oracle/build.py where the reference checkout is
present).  The fixture pins the restated oracle and the CUDA path wherever the reference itself
cannot travel.  Inputs: a fixed list of fp32/fp64 edge values plus a grid of exactly
representable values (multiples of 0.25, the input family of the reference's TypeConverterTest.cpp).
Run: python tests/golden/make_cast_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import oracle as o  # noqa: E402
from thor_b200.workloads import C1_EDGE_VALUES  # noqa: E402


def main():
    rng = np.random.default_rng(1234)
    out = {}
    f32 = np.concatenate([C1_EDGE_VALUES, np.array([np.nan], np.float32), rng.uniform(-70000, 70000, 512).astype(np.float32),
                          rng.uniform(-4, 4, 2048).astype(np.float32),
                          (rng.standard_normal(1024) * 2.0 ** rng.integers(-30, 18, 1024)).astype(np.float32)])
    out["f32_in"] = f32
    for dt in (o.FP16, o.BF16, o.FP8_E4M3, o.FP8_E5M2, o.FP64):
        out[f"f32_to_{o.NAMES[dt]}"] = o.reference_cast(f32, o.FP32, dt)
    f64 = np.concatenate([f32.astype(np.float64), np.array([1 + 2.0 ** -11 + 2.0 ** -40, 1 + 2.0 ** -11 - 2.0 ** -40, 65520 - 2.0 ** -30,
                                                             1 + 2.0 ** -8 + 2.0 ** -45, 1 + 2.0 ** -8 - 2.0 ** -45])])
    out["f64_in"] = f64
    for dt in (o.FP16, o.BF16, o.FP8_E4M3, o.FP8_E5M2, o.FP32):
        out[f"f64_to_{o.NAMES[dt]}"] = o.reference_cast(f64, o.FP64, dt)
    # every 16-bit pattern of fp16 and bf16 widened / cross-converted
    all16 = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    out["fp16_all_to_fp32"] = o.reference_cast(all16.view(np.float16), o.FP16, o.FP32)
    out["bf16_all_to_fp32"] = o.reference_cast(all16, o.BF16, o.FP32)
    out["fp16_all_to_bf16"] = o.reference_cast(all16.view(np.float16), o.FP16, o.BF16)
    out["bf16_all_to_fp16"] = o.reference_cast(all16, o.BF16, o.FP16).view(np.uint16)
    all8 = np.arange(256, dtype=np.uint16).astype(np.uint8)
    out["e4m3_all_to_fp32"] = o.reference_cast(all8, o.FP8_E4M3, o.FP32)
    out["e5m2_all_to_fp32"] = o.reference_cast(all8, o.FP8_E5M2, o.FP32)
    # representable grid through every pair (values k*0.25 for floats, small non-negative ints otherwise)
    grid = (rng.integers(0, 9, 256) * 1.0).astype(np.float32)  # 0..8: representable everywhere incl. bool-free pairs
    for s in o.ALL_DTYPES:
        src = o.reference_cast(grid, o.FP32, s) if s != o.FP32 else grid
        out[f"grid_{o.NAMES[s]}"] = src.view(np.uint16) if src.dtype == np.float16 else src
        for d in o.ALL_DTYPES:
            if d == s:
                continue
            r = o.reference_cast(src, s, d)
            out[f"grid_{o.NAMES[s]}_to_{o.NAMES[d]}"] = r.view(np.uint16) if r.dtype == np.float16 else r
    np.savez_compressed(Path(__file__).with_name("cast_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
