"""Writes tests/golden/autodiff_reference_graphs.json: the backward graphs that the REFERENCE's own autodiff builds.

Run in a checkout that has the reference beside it and oracle/_ref built (python oracle/build.py):
    python tests/golden/make_autodiff_golden.py
Each entry holds the forward program (postfix, oracle/ref_postfix.h), the input shapes and dtypes, the wrt list, the
upstream dtype and the dtype-resolved graph returned by buildBackwardOutputs (Utilities/Expression/AutoDiff.cpp:6210)
through oracle/ref_autodiff.cpp.  The tests read this file where oracle/_ref is not available.
"""
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402

BF16, FP16, FP32 = oracle.BF16, oracle.FP16, oracle.FP32
LAYERNORM = ("in:x in:x rmean:1 sub lit:1 in:x in:x rmean:1 sub in:x in:x rmean:1 sub mul rmean:1 lit:1e-05 add sqrt div mul "
             "in:gamma mul in:beta add cast:%d")

CASES = {
    "layernorm_bf16_64x256": (LAYERNORM % BF16, {"x": ((64, 256), BF16), "gamma": ((256,), BF16), "beta": ((256,), BF16)}, ["x", "gamma", "beta"], BF16),
    "layernorm_bf16_512x8192": (LAYERNORM % BF16, {"x": ((512, 8192), BF16), "gamma": ((8192,), BF16), "beta": ((8192,), BF16)}, ["x", "gamma", "beta"], BF16),
    "layernorm_bf16_32768x8192": (LAYERNORM % BF16, {"x": ((32768, 8192), BF16), "gamma": ((8192,), BF16), "beta": ((8192,), BF16)}, ["x", "gamma", "beta"], BF16),
    "layernorm_fp32_48x96": (LAYERNORM % FP32, {"x": ((48, 96), FP32), "gamma": ((96,), FP32), "beta": ((96,), FP32)}, ["x", "gamma", "beta"], FP32),
    "affine_tanh_fp16_40x72": ("in:a in:x mul in:b add tanh", {"a": ((72,), FP16), "x": ((40, 72), FP16), "b": ((40, 1), FP16)}, ["a", "x", "b"], FP16),
    "row_normalise_fp32_33x50": ("in:x in:x rsum:1 div", {"x": ((33, 50), FP32)}, ["x"], FP32),
    "mixed_exp_fp16_bf16_20x64": ("in:x in:w mul exp", {"x": ((20, 64), FP16), "w": ((64,), BF16)}, ["x", "w"], FP32),
    "softplus_sqrt_bf16_16x128": ("in:x softplus in:s mul sqrt", {"x": ((16, 128), BF16), "s": ((16, 1), BF16)}, ["x", "s"], BF16),
}


def main():
    out = {}
    for name, (program, inputs, wrt, upstream) in CASES.items():
        graph = oracle.reference_backward_graph(program, inputs, wrt, upstream)
        out[name] = {"program": program, "inputs": {k: [list(v[0]), int(v[1])] for k, v in inputs.items()}, "wrt": wrt, "upstream_dtype": int(upstream),
                     "graph": graph}
        print(name, len(graph["nodes"]), "nodes")
    (Path(__file__).parent / "autodiff_reference_graphs.json").write_text(json.dumps(out, separators=(",", ":")) + "\n")


if __name__ == "__main__":
    main()
