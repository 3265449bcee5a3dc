"""Shared helpers of the expression tests: run one expression through the CUDA path and the oracle."""
from __future__ import annotations

from typing import Callable, Dict, Mapping

import numpy as np

import oracle as o
from oracle import expr_oracle as eo

TORCH_VIEW = {o.BF16: "bfloat16", o.FP8_E4M3: "float8_e4m3fn", o.FP8_E5M2: "float8_e5m2"}


def to_device(storage: np.ndarray, dtype: int):
    import torch

    t = torch.from_numpy(np.ascontiguousarray(storage)).cuda()
    if dtype in TORCH_VIEW:
        t = t.view(getattr(torch, TORCH_VIEW[dtype]))
    return t


def from_device(t, dtype: int) -> np.ndarray:
    """Device tensor -> float64 values."""
    import torch

    if dtype in TORCH_VIEW:
        raw = t.view(torch.uint16 if dtype == o.BF16 else torch.uint8).cpu().numpy()
        return o.to_float64(raw, dtype)
    if dtype == o.BOOLEAN:
        return t.cpu().numpy().astype(np.float64)
    return t.cpu().numpy().astype(np.float64)


class ThorNS:
    """Expression namespace backed by thor_b200.expression."""

    def __init__(self):
        from thor_b200.expression import Expression

        self.E = Expression

    def input(self, name): return self.E.input(name)
    def runtime_scalar(self, name): return self.E.runtime_scalar(name)
    def where(self, c, t, f): return self.E.where(c, t, f)
    def cast(self, e, dtype): return e.cast(dtype)


class OracleNS:
    """Expression namespace backed by the eager numpy oracle."""

    def __init__(self, values: Mapping[str, "eo.OTensor"], scalars: Mapping[str, float]):
        self.values, self.scalars = values, scalars

    def input(self, name): return self.values[name]
    def runtime_scalar(self, name): return float(np.float32(self.scalars[name]))
    def where(self, c, t, f): return eo.OTensor.where(c, t, f)
    def cast(self, e, dtype): return e.cast(int(dtype))


def make_inputs(spec: Mapping[str, tuple], seed: int = 0) -> Dict[str, tuple]:
    """spec: name -> (shape, dtype, low, high).  Returns name -> (storage array, dtype)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, (shape, dtype, lo, hi) in spec.items():
        vals = rng.uniform(lo, hi, shape).astype(np.float32)
        out[name] = (o.from_float32(vals.reshape(-1), dtype).reshape(shape), dtype)
    return out


def run_both(fn: Callable, inputs: Mapping[str, tuple], scalars: Mapping[str, float] | None = None, fuse_row_reductions: bool = True):
    """Runs fn(namespace) -> expression (or dict of named expressions) on the GPU and in the oracle.

    Returns (plan, {name: (got float64 array, want OTensor)})."""
    import torch

    from thor_b200.expression import Expression

    scalars = dict(scalars or {})
    expr = fn(ThorNS())
    named = {"output": expr} if not isinstance(expr, dict) else expr
    eq = Expression.compile(named, device_num=0, fuse_row_reductions=fuse_row_reductions)
    dev = {name: to_device(arr, dt) for name, (arr, dt) in inputs.items()}
    bind = dict(dev)
    bind.update(scalars)
    plan = eq.stamp(bind)
    plan.run()
    torch.cuda.synchronize()
    ovals = {name: eo.OTensor.input(o.to_float64(arr, dt), dt) for name, (arr, dt) in inputs.items()}
    want = fn(OracleNS(ovals, scalars))
    want = {"output": want} if not isinstance(want, dict) else want
    results = {}
    for name, w in want.items():
        got = from_device(plan.output(name), w.dtype)
        results[name] = (got.reshape(w.v.shape), w)
    return plan, results


def assert_ulp(got: np.ndarray, want: "eo.OTensor", max_ulp: float, frac_within_1: float = 0.0, atol: float = 0.0):
    d = eo.ulp_distance(got, want.v, want.dtype)
    if atol:
        d = np.where(np.abs(got - want.v) <= atol, 0.0, d)
    worst = float(d.max()) if d.size else 0.0
    assert worst <= max_ulp, f"max ulp distance {worst} > {max_ulp} (at {np.unravel_index(d.argmax(), d.shape)}: got {got.flat[d.argmax()]!r}, want {want.v.flat[d.argmax()]!r})"
    if frac_within_1:
        frac = float((d <= 1.0).mean())
        assert frac >= frac_within_1, f"only {frac:.6f} of the elements are within 1 ulp"


def build_postfix(program: str):
    """The postfix mini-language of the reference-emitter dumper (oracle/ref_emit.cpp) through this repository's Expression API."""
    from thor_b200 import DataType
    from thor_b200.expression import Expression as ex

    stack = []
    for tok in program.split():
        if tok.startswith("in:"):
            stack.append(ex.input(tok[3:]))
        elif tok.startswith("rs:"):
            stack.append(ex.runtime_scalar(tok[3:]))
        elif tok.startswith("lit:"):
            stack.append(ex.scalar(float(tok[4:])))
        elif tok.startswith("cast:"):
            stack.append(stack.pop().cast(DataType(int(tok[5:]))))
        elif tok in ("add", "sub", "mul", "div", "pow", "min", "max"):
            b, a = stack.pop(), stack.pop()
            stack.append({"add": lambda: a + b, "sub": lambda: a - b, "mul": lambda: a * b, "div": lambda: a / b, "pow": lambda: a.pow(b),
                          "min": lambda: a.min(b), "max": lambda: a.max(b)}[tok]())
        elif tok == "neg":
            stack.append(-stack.pop())
        else:
            stack.append(getattr(stack.pop(), tok)())
    assert len(stack) == 1
    return stack[0]
