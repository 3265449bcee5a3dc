"""Numpy evaluation of a dtype-resolved expression graph — TEST INFRASTRUCTURE ONLY.

The graph is the JSON form that both dumpers produce: ``oracle/ref_autodiff.cpp`` for the graphs the REFERENCE's own
autodiff builds (buildBackwardOutputs, AutoDiff.cpp:6210) and ``FusedEquation::describeGraph`` for the host layer's.
Every node carries the reference's ExprOp integer (Expression.h:32-148), its parents and its resolved output / compute
dtypes.  Evaluation follows the per-node rule of the reference's kernels (CudaSourceEmitter.cpp:1610-1959,
2077-2083): a node converts its operands to its compute dtype, computes (here in float64, rounded ONCE to the
compute dtype: correctly rounded + - * / sqrt, ideal transcendentals), holds the value in the compute dtype and rounds
it to its output dtype where it is materialised (an output, the argument of a reduction or of a view).  Reductions
convert to fp32, accumulate (here in float64), finalise and round once to the output dtype
(CubReductionOperation.cuh:60-129, 186-198).
"""
from __future__ import annotations

import numpy as np
from scipy import special as _sp

from . import BF16, FP16, FP32
from .expr_oracle import round_to

# ExprOp integers of the reference (Utilities/Expression/Expression.h:32-148)
INPUT, RUNTIME_SCALAR, TENSOR_RUNTIME_SCALAR, SCALAR_FP, ADD, SUB, MUL, DIV, POW = 3, 4, 5, 6, 7, 8, 9, 10, 11
CAST, WHERE, NEG, ABS = 21, 22, 23, 24
EXP, EXPM1, EXP2, EXP10, LN, LOG1P, LOG2, LOG10, SQRT, TANH, NORMCDF = 48, 49, 50, 51, 52, 53, 54, 55, 56, 57, 58
FILL, RESHAPE, UNSQUEEZE, SQUEEZE = 61, 62, 65, 66
MIN, MAX, MIN_GRAD_LEFT, MIN_GRAD_RIGHT, MAX_GRAD_LEFT, MAX_GRAD_RIGHT = 69, 70, 71, 72, 73, 74
REDUCE_SUM, REDUCE_PROD, REDUCE_MIN, REDUCE_MAX, REDUCE_AVG, REDUCE_NORM1, REDUCE_NORM2 = 83, 84, 85, 86, 95, 96, 97
_COMPARE = {12: np.equal, 13: np.not_equal, 14: np.less, 15: np.less_equal, 16: np.greater, 17: np.greater_equal}
_UNARY = {NEG: np.negative, ABS: np.abs, 25: np.ceil, 26: np.floor, 28: np.trunc, 29: np.sin, 30: np.cos, 31: np.tan, 32: np.arcsin, 33: np.arccos,
          34: np.arctan, 35: np.sinh, 36: np.cosh, 37: np.arcsinh, 38: np.arccosh, 39: np.arctanh, 40: _sp.erf, 41: _sp.erfc, 42: _sp.erfcx,
          43: _sp.erfinv, 44: _sp.erfcinv, 45: _sp.gamma, 46: _sp.gammaln, 47: _sp.digamma, EXP: np.exp, EXPM1: np.expm1, EXP2: np.exp2,
          EXP10: lambda v: np.power(10.0, v), LN: np.log, LOG1P: np.log1p, LOG2: np.log2, LOG10: np.log10, SQRT: np.sqrt, TANH: np.tanh,
          NORMCDF: _sp.ndtr}
_REDUCTIONS = (REDUCE_SUM, REDUCE_PROD, REDUCE_MIN, REDUCE_MAX, REDUCE_AVG, REDUCE_NORM1, REDUCE_NORM2)
_VIEWS = (RESHAPE, UNSQUEEZE, SQUEEZE)


class _Value:
    """values (float64), the dtype they are held in (None: an untyped literal) and the node's output dtype."""

    def __init__(self, v, held, out):
        self.v, self.held, self.out = np.asarray(v, dtype=np.float64), held, out

    def materialised(self):
        return self.v if self.held == self.out or self.out == 0 else round_to(self.v, self.out)

    def as_operand(self, compute):
        # literals are rounded to the consumer's compute dtype first (CudaSourceEmitter.cpp:4034-4043); typed values convert
        return round_to(self.v, compute) if compute in (FP16, BF16, FP32) and self.held != compute else self.v


def evaluate(graph: dict, inputs: dict) -> dict:
    """inputs: name -> numpy array (float32 / float16 / bf16 bit patterns are NOT accepted: pass float64 or float32 values
    that are already representable in the input's dtype) or a python float for runtime scalars.  Returns name -> float64
    array holding each output rounded to its output dtype."""
    slot_name = {i["slot"]: i["name"] for i in graph["inputs"]}
    vals = []
    with np.errstate(all="ignore"):
        for node in graph["nodes"]:
            op, out, comp = node["op"], node["out"], node["compute"] or node["out"]
            par = [vals[node[k]] for k in ("lhs", "rhs", "aux") if node[k] >= 0]
            if op in (INPUT, TENSOR_RUNTIME_SCALAR):
                vals.append(_Value(np.asarray(inputs[slot_name[node["slot"]]], dtype=np.float64), out, out))
            elif op == RUNTIME_SCALAR:
                vals.append(_Value(np.float32(inputs[slot_name[node["slot"]]]), FP32, FP32))
            elif op == SCALAR_FP:
                vals.append(_Value(node["scalar"], None, out))
            elif op == FILL:
                vals.append(_Value(round_to(np.full(node["fill_dims"], node["scalar"]), out or FP32), out, out))
            elif op == CAST:
                vals.append(_Value(round_to(par[0].v, out), out, out))
            elif op in _VIEWS:
                v = par[0].materialised()
                if op == RESHAPE:
                    v = v.reshape(node["reshape_dims"])
                elif op == UNSQUEEZE:
                    for axis in sorted(node["unsqueeze_axes"]):
                        v = np.expand_dims(v, axis)
                else:
                    v = np.squeeze(v, axis=tuple(node["squeeze_axes"]))
                vals.append(_Value(v, par[0].out, out or par[0].out))
            elif op in _REDUCTIONS:
                v = round_to(par[0].materialised(), FP32)
                axes = tuple(node["reduction_axes"]) or tuple(range(v.ndim))
                if op == REDUCE_SUM: r = v.sum(axis=axes, keepdims=True)
                elif op == REDUCE_AVG: r = round_to(round_to(v.sum(axis=axes, keepdims=True), FP32) / np.prod([v.shape[a] for a in axes]), FP32)
                elif op == REDUCE_PROD: r = v.prod(axis=axes, keepdims=True)
                elif op == REDUCE_MIN: r = v.min(axis=axes, keepdims=True)
                elif op == REDUCE_MAX: r = v.max(axis=axes, keepdims=True)
                elif op == REDUCE_NORM1: r = np.abs(v).sum(axis=axes, keepdims=True)
                else: r = np.sqrt(round_to((v * v).sum(axis=axes, keepdims=True), FP32))
                sq = node["squeeze_axes"]
                if sq:
                    r = np.squeeze(r) if sq == [np.iinfo(np.uint64).max] else np.squeeze(r, axis=tuple(sq))
                    if r.ndim == 0:
                        r = r.reshape(1)
                vals.append(_Value(round_to(r, out), out, out))
            else:
                a = [p.as_operand(comp) for p in par]
                if op == ADD: r = a[0] + a[1]
                elif op == SUB: r = a[0] - a[1]
                elif op == MUL: r = a[0] * a[1]
                elif op == DIV: r = a[0] / a[1]
                elif op == POW: r = np.power(a[0], a[1])
                elif op == MIN: r = np.fmin(a[0], a[1])
                elif op == MAX: r = np.fmax(a[0], a[1])
                elif op in (MIN_GRAD_LEFT, MIN_GRAD_RIGHT, MAX_GRAD_LEFT, MAX_GRAD_RIGHT):
                    # 1 where this side is the selected one, 0.5 on ties, 0 otherwise (CudaSourceEmitter.cpp:1940-1954)
                    left = op in (MIN_GRAD_LEFT, MAX_GRAD_LEFT)
                    smaller = op in (MIN_GRAD_LEFT, MIN_GRAD_RIGHT)
                    mine, other = (a[0], a[1]) if left else (a[1], a[0])
                    wins = mine < other if smaller else mine > other
                    r = np.where(wins, 1.0, np.where(mine == other, 0.5, 0.0))
                elif op == WHERE: r = np.where(a[0] != 0, a[1], a[2])
                elif op in _COMPARE: r = _COMPARE[op](a[0], a[1]).astype(np.float64)
                elif op == 27: r = np.where(a[0] >= 0, np.floor(a[0] + 0.5), np.ceil(a[0] - 0.5))  # roundf: halves away from zero
                elif op in _UNARY: r = _UNARY[op](a[0])
                else: raise NotImplementedError(f"graph_eval: ExprOp {op}")
                vals.append(_Value(round_to(r, comp), comp, out))
    return {o["name"]: vals[o["node"]].materialised() for o in graph["outputs"]}


def node_shapes(graph: dict, input_shapes: dict) -> list:
    """Shape of every node (numpy broadcasting; reductions keep reduced axes as 1, then squeeze)."""
    zeros = {n: np.zeros(s) for n, s in input_shapes.items()}
    slot_name = {i["slot"]: i["name"] for i in graph["inputs"]}
    shapes = []
    for node in graph["nodes"]:
        op = node["op"]
        par = [shapes[node[k]] for k in ("lhs", "rhs", "aux") if node[k] >= 0]
        if op in (INPUT, TENSOR_RUNTIME_SCALAR): shapes.append(tuple(zeros[slot_name[node["slot"]]].shape))
        elif op in (RUNTIME_SCALAR, SCALAR_FP): shapes.append(())
        elif op == FILL: shapes.append(tuple(node["fill_dims"]))
        elif op == RESHAPE: shapes.append(tuple(node["reshape_dims"]))
        elif op == UNSQUEEZE:
            s = list(par[0])
            for axis in sorted(node["unsqueeze_axes"]): s.insert(axis, 1)
            shapes.append(tuple(s))
        elif op == SQUEEZE: shapes.append(tuple(d for i, d in enumerate(par[0]) if i not in node["squeeze_axes"]))
        elif op in _REDUCTIONS:
            axes = node["reduction_axes"] or list(range(len(par[0])))
            s = [1 if i in axes else d for i, d in enumerate(par[0])]
            sq = node["squeeze_axes"]
            if sq: s = [d for i, d in enumerate(s) if not (i in sq or (sq == [np.iinfo(np.uint64).max] and d == 1))] or [1]
            shapes.append(tuple(s))
        else: shapes.append(np.broadcast_shapes(*par) if par else ())
    return shapes
