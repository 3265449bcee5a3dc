"""The host layer's reverse-mode differentiation against the REFERENCE's own (no GPU needed).

oracle/ref_autodiff.cpp links the reference's AutoDiff.cpp and dumps the dtype-resolved backward graph that its
buildBackwardOutputs (Utilities/Expression/AutoDiff.cpp:6210) builds; tests/golden/autodiff_reference_graphs.json holds
those graphs for the cases below (written by tests/golden/make_autodiff_golden.py), so the comparison also runs where the
reference is not available.  FusedEquation.graph() returns the host layer's graph in the same form.  Checked per case:
the gradient outputs carry the same names, dtypes and shapes, reductions that end a gradient reduce the same axes, and
both graphs evaluated node by node with the numpy oracle (oracle/graph_eval.py) give the same gradients -- bit for bit
in the output dtype except where the two graphs associate a product differently (at most one output ulp then).
"""
import json
import zlib
from pathlib import Path

import numpy as np
import pytest

import oracle as o
from oracle import graph_eval as ge
from oracle.expr_oracle import round_to, ulp_distance
from thor_b200.dtypes import DataType as DT
from thor_b200.expression import Expression as ex

GOLDEN = json.loads((Path(__file__).parent / "golden" / "autodiff_reference_graphs.json").read_text())
UPSTREAM = "__grad_output"


def _layernorm(out_dtype):
    x, gamma, beta = ex.input("x"), ex.input("gamma"), ex.input("beta")
    xc = x - x.reduce_mean([1])
    rstd = 1.0 / ((xc * xc).reduce_mean([1]) + 1e-5).sqrt()
    return (xc * rstd * gamma + beta).cast(out_dtype)


# the same forward expressions as the golden file's postfix programs, written with the host layer's Expression API
FORWARD = {
    "layernorm_bf16_64x256": lambda: _layernorm(DT.bf16),
    "layernorm_bf16_512x8192": lambda: _layernorm(DT.bf16),
    "layernorm_bf16_32768x8192": lambda: _layernorm(DT.bf16),
    "layernorm_fp32_48x96": lambda: _layernorm(DT.fp32),
    "affine_tanh_fp16_40x72": lambda: (ex.input("a") * ex.input("x") + ex.input("b")).tanh(),
    "row_normalise_fp32_33x50": lambda: ex.input("x") / ex.input("x").reduce_sum([1]),
    "mixed_exp_fp16_bf16_20x64": lambda: (ex.input("x") * ex.input("w")).exp(),
    "softplus_sqrt_bf16_16x128": lambda: (ex.input("x").softplus() * ex.input("s")).sqrt(),
}


def _ours(name):
    case = GOLDEN[name]
    shapes = {k: (tuple(v[0]), DT(v[1])) for k, v in case["inputs"].items()}
    out_shape = np.broadcast_shapes(*[s for s, _ in shapes.values()])
    shapes[UPSTREAM] = (tuple(out_shape), DT(case["upstream_dtype"]))
    return ex.compile({"output": FORWARD[name]()}).compile_backward(case["wrt"]).graph(shapes), shapes


def _data(shapes, seed):
    rng = np.random.default_rng(seed)
    data = {}
    for name, (shape, dtype) in shapes.items():
        if name in ("gamma", "s", "a"):
            v = rng.uniform(0.6, 1.4, shape)
        elif name == UPSTREAM:
            v = rng.normal(0.0, 0.05, shape)
        else:
            v = rng.standard_normal(shape)
        data[name] = round_to(v, int(dtype))
    return data


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_gradient_outputs_have_the_reference_names_dtypes_and_shapes(name):
    ref = GOLDEN[name]["graph"]
    ours, shapes = _ours(name)
    in_shapes = {k: v[0] for k, v in shapes.items()}
    ref_shapes, our_shapes = ge.node_shapes(ref, in_shapes), ge.node_shapes(ours, in_shapes)
    ref_out = {out["name"]: out["node"] for out in ref["outputs"]}
    our_out = {out["name"]: out["node"] for out in ours["outputs"]}
    assert set(ref_out) == set(our_out) == {w + "_grad" for w in GOLDEN[name]["wrt"]}
    for out_name in ref_out:
        rn, on = ref["nodes"][ref_out[out_name]], ours["nodes"][our_out[out_name]]
        assert rn["out"] == on["out"], f"{out_name}: stored as {on['out']}, the reference stores {rn['out']}"
        assert tuple(ref_shapes[ref_out[out_name]]) == tuple(our_shapes[our_out[out_name]]), out_name
        wrt = out_name[: -len("_grad")]
        assert rn["out"] == GOLDEN[name]["inputs"][wrt][1], "a gradient is stored in the dtype of the input it belongs to"
        if rn["op"] in ge._REDUCTIONS:  # an un-broadcast sum ends the gradient: same op, axes, squeeze and fp32 accumulation
            assert (on["op"], on["reduction_axes"], on["squeeze_axes"], on["compute"]) == (rn["op"], rn["reduction_axes"], rn["squeeze_axes"], rn["compute"])


@pytest.mark.parametrize("name", [n for n in sorted(GOLDEN) if "32768" not in n and "512x8192" not in n])
def test_both_graphs_compute_the_same_gradients(name):
    ref = GOLDEN[name]["graph"]
    ours, shapes = _ours(name)
    data = _data(shapes, seed=zlib.crc32(name.encode()))
    want, got = ge.evaluate(ref, data), ge.evaluate(ours, data)
    for out_name, w in want.items():
        dtype = ref["nodes"][{x["name"]: x["node"] for x in ref["outputs"]}[out_name]]["out"]
        g = got[out_name]
        assert g.shape == w.shape
        if dtype == o.FP32:
            # fp32 gradients are sums of terms that cancel: the graphs differ by re-association of fp32 products only,
            # a few fp32 roundings of the largest term
            assert float(np.abs(g - w).max()) <= 8 * 2.0 ** -24 * float(np.abs(w).max()), out_name
            continue
        d = ulp_distance(g, w, dtype)
        assert float(d.max()) <= 1.0, f"{out_name}: {float(d.max())} ulp apart"
        assert float((d == 0).mean()) >= 0.99, f"{out_name}: only {(d == 0).mean():.4f} of the values identical"


def test_the_layernorm_graph_differentiates_through_fp32_statistics_like_the_reference():
    """Per-node dtypes inside the backward graph: everything downstream of x - mean computes in fp32 in both graphs and no
    gradient leaves fp32 before its final store."""
    ref = GOLDEN["layernorm_bf16_64x256"]["graph"]
    ours, _ = _ours("layernorm_bf16_64x256")
    for graph in (ref, ours):
        outs = {x["node"] for x in graph["outputs"]}
        for k, node in enumerate(graph["nodes"]):
            if node["op"] in (ge.INPUT, ge.SCALAR_FP, ge.FILL) or k in outs:
                continue
            if node["op"] == ge.CAST and node["out"] == o.BF16:
                continue  # the forward output's own cast, recomputed for nothing but its dtype
            assert node["compute"] in (0, o.FP32) or node["op"] in ge._VIEWS, (k, node)


@pytest.mark.skipif(o.reference_autodiff_lib() is None, reason="the reference's autodiff is not built (oracle/_ref)")
@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_the_golden_graphs_are_what_the_reference_builds_today(name):
    case = GOLDEN[name]
    inputs = {k: (tuple(v[0]), v[1]) for k, v in case["inputs"].items()}
    assert o.reference_backward_graph(case["program"], inputs, case["wrt"], case["upstream_dtype"]) == case["graph"]


def test_the_reference_backward_graph_cuts_into_its_stage_list():
    """oracle/stage_cut.py applies the reference's planning rule (a reduction is a stage over a tensor in memory,
    EquationCompiler.cpp:684-688, 4088-4173) to its LayerNorm backward graph: the benchmark's reference baseline runs
    exactly these stages.  Equal nodes merge first (x - mean appears three times in the dump)."""
    from oracle import stage_cut

    case = GOLDEN["layernorm_bf16_32768x8192"]
    graph = stage_cut.merge_equal_nodes(case["graph"])
    assert len(case["graph"]["nodes"]) == 67 and len(graph["nodes"]) == 47
    shapes = {k: tuple(v[0]) for k, v in case["inputs"].items()}
    shapes[UPSTREAM] = (32768, 8192)
    stages = stage_cut.stage_list(graph, shapes)
    assert [s["kind"] for s in stages] == ["fused", "reduction"] + ["reduction", "fused"] * 6
    assert stages[0]["program"] == f"in:{UPSTREAM} cast:11" and stages[0]["dtype"] == o.FP32
    column_sums = [s for s in stages if s["kind"] == "reduction" and s["axes"] == [0]]
    assert [s["name"] for s in column_sums] == ["beta_grad", "gamma_grad"] and all(s["dtype"] == o.BF16 and s["shape"] == (8192,) for s in column_sums)
    row_stats = [s for s in stages if s["kind"] == "reduction" and s["axes"] == [1]]
    assert len(row_stats) == 5 and all(s["shape"] == (32768, 1) and s["dtype"] == o.FP32 for s in row_stats)
    last = stages[-1]
    assert last["name"] == "x_grad" and last["dtype"] == o.BF16 and set(last["inputs"]) >= {"gamma", "x"}
    # every fused stage reads only inputs and results of earlier stages
    known = set(shapes)
    for s in stages:
        assert set(s["inputs"] if s["kind"] == "fused" else [s["input"]]) <= known, s["name"]
        known.add(s["name"])
