"""Stage cut of a dtype-resolved expression graph by the reference's planning rule — BASELINE / TEST INFRASTRUCTURE ONLY.

The reference makes every reduction a stage of its own that reads exactly one tensor already in memory
(EquationCompiler.cpp:684-688, 4088-4173), so whatever feeds a reduction is written out by a fused stage before it, and a
fused stage walks back through every node that is not in memory, recomputing shared elementwise sub-trees
(EquationCompiler.cpp:3543-3635).  This module applies that rule to a graph in the JSON form of oracle/ref_autodiff.cpp:

* structurally equal nodes are merged first (the reference's stage-level common-subexpression pass,
  EquationCompiler.cpp:504-575);
* "in memory" = the graph's inputs, every reduction result, every reduction argument that is not an input, every output;
* every such node that is not an input becomes one stage, in graph order: a reduction stage, or a fused stage given as a
  postfix program for oracle/ref_postfix.h whose leaves are inputs and earlier stages' results (named t<node>).

One fused stage per materialised node: the reference may put several outputs that share a stage into one kernel; emitting
them one by one re-reads shared inputs, so a baseline built from this list can only overstate the fused part, never the
reductions.
"""
from . import graph_eval as ge

_BINARY = {ge.ADD: "add", ge.SUB: "sub", ge.MUL: "mul", ge.DIV: "div", ge.POW: "pow", ge.MIN: "min", ge.MAX: "max"}
_UNARY = {ge.NEG: "neg", ge.ABS: "abs", ge.EXP: "exp", ge.EXPM1: "expm1", ge.EXP2: "exp2", ge.EXP10: "exp10", ge.LN: "ln", ge.LOG1P: "log1p", ge.LOG2: "log2",
          ge.LOG10: "log10", ge.SQRT: "sqrt", ge.TANH: "tanh", ge.NORMCDF: "normcdf"}
_REDUCE_NAME = {ge.REDUCE_SUM: "sum", ge.REDUCE_AVG: "mean", ge.REDUCE_MAX: "max", ge.REDUCE_MIN: "min"}


def merge_equal_nodes(graph: dict) -> dict:
    """The graph with structurally equal nodes merged (parents precede children in the node list, so one pass is enough)."""
    remap, seen, nodes = {}, {}, []
    for k, n in enumerate(graph["nodes"]):
        parent = lambda p: remap[p] if p >= 0 else -1
        key = (n["op"], parent(n["lhs"]), parent(n["rhs"]), parent(n["aux"]), n["slot"], repr(n["scalar"]), n["out"], n["compute"], tuple(n["reduction_axes"]),
               tuple(n["squeeze_axes"]), tuple(n["unsqueeze_axes"]), tuple(n["reshape_dims"]), tuple(n["fill_dims"]))
        if key not in seen:
            seen[key] = len(nodes)
            nodes.append(dict(n, lhs=parent(n["lhs"]), rhs=parent(n["rhs"]), aux=parent(n["aux"])))
        remap[k] = seen[key]
    return {"inputs": graph["inputs"], "nodes": nodes, "outputs": [dict(o, node=remap[o["node"]]) for o in graph["outputs"]]}


def stage_list(graph: dict, input_shapes: dict) -> list:
    """Stages of `graph` (already merged) in execution order.  Each stage is a dict:
    {"node", "kind": "reduction" | "fused", "name": "t<node>" or the output's name, "shape", "dtype",
     reduction: "op" ("sum" / "mean" / ...), "axes", "input" (a tensor name);  fused: "program", "inputs" (tensor names)}."""
    nodes = graph["nodes"]
    slot_name = {i["slot"]: i["name"] for i in graph["inputs"]}
    shapes = ge.node_shapes(graph, input_shapes)
    out_name = {o["node"]: o["name"] for o in graph["outputs"]}
    reductions = [k for k, n in enumerate(nodes) if n["op"] in ge._REDUCTIONS]
    in_memory = set(reductions) | set(out_name)
    for k in reductions:
        arg = nodes[k]["lhs"]
        if nodes[arg]["op"] != ge.INPUT:
            in_memory.add(arg)
    tensor_name = lambda k: slot_name[nodes[k]["slot"]] if nodes[k]["op"] == ge.INPUT else out_name.get(k, f"t{k}")

    def program(k: int, root: bool, leaves: list) -> str:
        n = nodes[k]
        op = n["op"]
        if op == ge.INPUT or (not root and k in in_memory):
            if tensor_name(k) not in leaves:
                leaves.append(tensor_name(k))
            return "in:" + tensor_name(k)
        if op in (ge.SCALAR_FP, ge.FILL):
            return "lit:" + repr(float(n["scalar"]))
        if op == ge.CAST:
            return program(n["lhs"], False, leaves) + f" cast:{n['out']}"
        if op in _UNARY:
            return program(n["lhs"], False, leaves) + " " + _UNARY[op]
        if op in _BINARY:
            return program(n["lhs"], False, leaves) + " " + program(n["rhs"], False, leaves) + " " + _BINARY[op]
        raise NotImplementedError(f"stage cut: op {op} of node {k} has no postfix spelling")

    stages = []
    for k, n in enumerate(nodes):
        if k not in in_memory or n["op"] == ge.INPUT:
            continue
        stage = {"node": k, "name": tensor_name(k), "shape": tuple(shapes[k]), "dtype": n["out"]}
        if n["op"] in ge._REDUCTIONS:
            stage.update(kind="reduction", op=_REDUCE_NAME[n["op"]], axes=list(n["reduction_axes"]), input=tensor_name(n["lhs"]), input_shape=tuple(shapes[n["lhs"]]))
        else:
            leaves = []
            stage.update(kind="fused", program=program(k, True, leaves), inputs=leaves)
        stages.append(stage)
    return stages
