"""Eager numpy restatement of the reference's expression semantics — TEST INFRASTRUCTURE ONLY.

An ``OTensor`` carries its output dtype plus the values as the reference's kernels hold them: leaves,
casts and reduction results in their output dtype, every other arithmetic node in its COMPUTE dtype
(CudaSourceEmitter.cpp:2077-2083) -- a value is rounded to its output dtype only where it is
materialised: read as a result (``.v``), consumed by a reduction, an arg reduction or a view.  Every
operation applies the reference's per-node rule (Utilities/Expression/ExpressionDTypeResolution.cpp:1012-1128):
pick the output dtype by promoting the TENSOR operands (scalars never promote, :506-515, :793-805) and compute
in toSupportedComputeDType(promote(input, output)) (fp8 computes in fp16, :95-220).  For fp16 / bf16 / fp32
graphs compute and output dtype coincide, so the distinction only shows with fp8 storage.  Arithmetic is done in float64 (exact for + - * on <= 24-bit significands) and
rounded ONCE to the compute dtype, which equals correctly-rounded fp16 / bf16 / fp32 arithmetic;
transcendental functions are evaluated in float64 and rounded, i.e. "ideal" libdevice results --
the CUDA functions differ from that by their documented ulp error, which is what the parity
tolerances in the tests absorb.

Reductions follow CubReductionOperation.cuh:60-129,186-198: convert to fp32, transform, combine
(here in float64, the 'fp64-accumulated oracle of the same rounded operands'), finalise, round once
to the output dtype (default fp32).  Arg reductions follow CubArgReductionOperation.cuh:31-73: NaN
wins, lowest index wins ties.

The same test expression can be written once as a Python function of an "expression namespace" and
run through ``thor_b200.expression.Expression`` and through this module.
"""
from __future__ import annotations

import math
from typing import Iterable, Optional, Sequence, Union

import numpy as np
from scipy import special as _sp

from . import BF16, BOOLEAN, FP16, FP32, FP8_E4M3, FP8_E5M2, UINT32, cast as _cast

_FLOATS = (FP16, BF16, FP32, FP8_E4M3, FP8_E5M2)


def round_to(values: np.ndarray, dtype: int) -> np.ndarray:
    """Round float64/float32 values to `dtype` (RNE) and return them widened again (float64)."""
    v = np.asarray(values, dtype=np.float64)
    if dtype == FP32:
        with np.errstate(over="ignore"):
            return v.astype(np.float32).astype(np.float64)
    if dtype == FP16:
        with np.errstate(over="ignore"):
            return v.astype(np.float16).astype(np.float64)  # numpy float64->float16 is a single RNE rounding
    if dtype in (BF16, FP8_E4M3, FP8_E5M2):
        from . import FP64

        shape = v.shape
        enc = _cast(np.ascontiguousarray(v.reshape(-1)), FP64, dtype)
        return _cast(enc, dtype, FP64).reshape(shape)
    if dtype == BOOLEAN:
        return (v != 0).astype(np.float64)
    if dtype == UINT32:
        return v
    raise ValueError(f"round_to: unsupported dtype {dtype}")


def promote(a: int, b: int) -> int:
    """promoteTensorValueDTypes (ExpressionDTypeResolution.cpp:277-307)."""
    if a == b:
        return a
    if {a, b} == {FP16, BF16}:
        return FP32
    if FP32 in (a, b):
        return FP32
    if BF16 in (a, b):
        return BF16
    return FP16


def compute_dtype_for(dtype: int) -> int:
    """toSupportedComputeDType for pointwise ops: fp8 computes in fp16."""
    return FP16 if dtype in (FP8_E4M3, FP8_E5M2, FP16) else dtype


class OTensor:
    def __init__(self, values, dtype: int, held: Optional[int] = None):
        self.dtype = dtype
        self.held = dtype if held is None else held
        self._h = round_to(values, self.held)

    @property
    def v(self) -> np.ndarray:
        """The materialised values: rounded to the output dtype."""
        return self._h if self.held == self.dtype else round_to(self._h, self.dtype)

    # ---- construction -------------------------------------------------------------------------------
    @staticmethod
    def input(values: np.ndarray, dtype: int) -> "OTensor":
        return OTensor(np.asarray(values, dtype=np.float64), dtype)

    @property
    def shape(self):
        return self.v.shape

    def storage(self) -> np.ndarray:
        """Storage array (see oracle.STORAGE) of the values."""
        from . import FP64

        if self.dtype == BOOLEAN:
            return self.v != 0
        if self.dtype == UINT32:
            return self.v.astype(np.uint32)
        return _cast(np.ascontiguousarray(self.v.reshape(-1)), FP64, self.dtype).reshape(self.v.shape)

    # ---- core ---------------------------------------------------------------------------------------
    def _binary(self, other, fn, swap=False, out_dtype: Optional[int] = None, compute: Optional[int] = None) -> "OTensor":
        if isinstance(other, OTensor):
            out = out_dtype or promote(self.dtype, other.dtype)
            cd = compute or compute_dtype_for(promote(promote(self.dtype, other.dtype), out))
            a, b = round_to(self._h, cd), round_to(other._h, cd)
        else:
            out = out_dtype or self.dtype
            cd = compute or compute_dtype_for(out)
            # literal: double -> float literal -> compute dtype (CudaSourceEmitter.cpp:4034-4043)
            a, b = round_to(self._h, cd), round_to(round_to(np.float64(other), FP32), cd)
        if swap:
            a, b = b, a
        with np.errstate(all="ignore"):
            r = fn(a, b)
        return OTensor(r, out, held=cd)

    def _unary(self, fn, compute: Optional[int] = None) -> "OTensor":
        cd = compute or compute_dtype_for(self.dtype)
        with np.errstate(all="ignore"):
            r = fn(round_to(self._h, cd))
        return OTensor(r, self.dtype, held=cd)

    def __add__(self, o): return self._binary(o, np.add)
    def __radd__(self, o): return self._binary(o, np.add, swap=True)
    def __sub__(self, o): return self._binary(o, np.subtract)
    def __rsub__(self, o): return self._binary(o, np.subtract, swap=True)
    def __mul__(self, o): return self._binary(o, np.multiply)
    def __rmul__(self, o): return self._binary(o, np.multiply, swap=True)
    def __truediv__(self, o): return self._binary(o, np.divide)
    def __rtruediv__(self, o): return self._binary(o, np.divide, swap=True)
    def __pow__(self, o): return self._binary(o, np.power)
    def __rpow__(self, o): return self._binary(o, np.power, swap=True)
    def __neg__(self): return self._unary(np.negative)
    def pow(self, o): return self.__pow__(o)
    def min(self, o): return self._binary(o, np.fmin)
    def max(self, o): return self._binary(o, np.fmax)

    def _compare(self, o, fn) -> "OTensor":
        if isinstance(o, OTensor):
            cd = compute_dtype_for(promote(self.dtype, o.dtype))
            a, b = round_to(self._h, cd), round_to(o._h, cd)
        else:
            cd = compute_dtype_for(self.dtype)
            a, b = round_to(self._h, cd), round_to(round_to(np.float64(o), FP32), cd)
        return OTensor(fn(a, b).astype(np.float64), BOOLEAN)

    def __lt__(self, o): return self._compare(o, np.less)
    def __le__(self, o): return self._compare(o, np.less_equal)
    def __gt__(self, o): return self._compare(o, np.greater)
    def __ge__(self, o): return self._compare(o, np.greater_equal)
    def equal(self, o): return self._compare(o, np.equal)
    def not_equal(self, o): return self._compare(o, np.not_equal)
    def logical_and(self, o): return OTensor(((self.v != 0) & (o.v != 0)).astype(np.float64), BOOLEAN)
    def logical_or(self, o): return OTensor(((self.v != 0) | (o.v != 0)).astype(np.float64), BOOLEAN)
    def logical_not(self): return OTensor((self.v == 0).astype(np.float64), BOOLEAN)
    def __invert__(self): return self.logical_not()

    @staticmethod
    def where(cond: "OTensor", t, f) -> "OTensor":
        branches = [x.dtype for x in (t, f) if isinstance(x, OTensor)]
        out = FP32 if not branches else (branches[0] if len(branches) == 1 else promote(branches[0], branches[1]))
        cd = compute_dtype_for(out)
        tv = t._h if isinstance(t, OTensor) else round_to(round_to(np.float64(t), FP32), out)
        fv = f._h if isinstance(f, OTensor) else round_to(round_to(np.float64(f), FP32), out)
        return OTensor(np.where(cond.v != 0, round_to(tv, cd), round_to(fv, cd)), out, held=cd)

    def cast(self, dtype: int) -> "OTensor":
        return OTensor(self._h, dtype)

    def abs(self): return self._unary(np.abs)
    def ceil(self): return self._unary(np.ceil)
    def floor(self): return self._unary(np.floor)
    def round(self): return self._unary(lambda a: np.sign(a) * np.floor(np.abs(a) + 0.5))  # roundf: half away from zero
    def trunc(self): return self._unary(np.trunc)
    def sin(self): return self._unary(np.sin)
    def cos(self): return self._unary(np.cos)
    def tan(self): return self._unary(np.tan)
    def asin(self): return self._unary(np.arcsin)
    def acos(self): return self._unary(np.arccos)
    def atan(self): return self._unary(np.arctan)
    def sinh(self): return self._unary(np.sinh)
    def cosh(self): return self._unary(np.cosh)
    def asinh(self): return self._unary(np.arcsinh)
    def acosh(self): return self._unary(np.arccosh)
    def atanh(self): return self._unary(np.arctanh)
    def erf(self): return self._unary(_sp.erf)
    def erfc(self): return self._unary(_sp.erfc)
    def erfcx(self): return self._unary(_sp.erfcx)
    def erfinv(self): return self._unary(_sp.erfinv)
    def erfcinv(self): return self._unary(_sp.erfcinv)
    def tgamma(self): return self._unary(_sp.gamma)
    def lgamma(self): return self._unary(lambda a: _sp.gammaln(a))
    def digamma(self): return self._unary(_sp.digamma)
    def exp(self): return self._unary(np.exp)
    def expm1(self): return self._unary(np.expm1)
    def exp2(self): return self._unary(np.exp2)
    def exp10(self): return self._unary(lambda a: np.power(10.0, a))
    def ln(self): return self._unary(np.log)
    def log1p(self): return self._unary(np.log1p)
    def log2(self): return self._unary(np.log2)
    def log10(self): return self._unary(np.log10)
    def sqrt(self): return self._unary(np.sqrt)
    def tanh(self): return self._unary(np.tanh)
    def normcdf(self): return self._unary(_sp.ndtr)

    # composites, spelled like Expression.h:1077-1115
    def sigmoid(self):
        neg = -self
        numerator = (-(neg.max(0.0))).exp()
        denominator = 1.0 + (-(self.abs())).exp()
        return numerator / denominator

    def softplus(self): return self.max(0.0) + (-(self.abs())).exp().log1p()
    def elu(self, alpha: float = 1.0): return self.max(0.0) + (self.min(0.0).expm1() * alpha)
    def selu(self): return (self.max(0.0) * 1.05070098) + (self.min(0.0).expm1() * 1.758099326)
    def gelu(self): return self * self.normcdf()
    def swish(self): return self * self.sigmoid()
    def relu(self): return self.max(0.0)
    def relu6(self): return self.max(0.0).min(6.0)
    def hard_tanh(self, lo=-1.0, hi=1.0): return self.max(lo).min(hi)
    def clamp(self, lo, hi): return self.max(lo).min(hi)

    # ---- shapes ---------------------------------------------------------------------------------------
    def reshape(self, dims): return OTensor(self.v.reshape(dims), self.dtype)
    def unsqueeze(self, axes):
        v = self.v
        for ax in sorted(axes):
            v = np.expand_dims(v, ax)
        return OTensor(v, self.dtype)
    def squeeze(self, axes): return OTensor(np.squeeze(self.v, tuple(axes)), self.dtype)

    # ---- reductions -------------------------------------------------------------------------------------
    def _reduce(self, kind: str, axes: Iterable[int], squeeze_axes: Iterable[int], out_dtype: Optional[int] = None) -> "OTensor":
        ax = tuple(axes) or tuple(range(self.v.ndim))
        x = round_to(self.v, FP32)  # input -> fp32 is exact for every supported storage dtype
        with np.errstate(all="ignore"):
            if kind in ("sum", "mean"):
                r = x.sum(axis=ax, keepdims=True, dtype=np.float64)
                if kind == "mean":
                    count = np.float32(np.prod([x.shape[a] for a in ax]))
                    r = round_to(r, FP32) / np.float64(count)
            elif kind == "prod":
                r = x.prod(axis=ax, keepdims=True, dtype=np.float64)
            elif kind == "min":
                r = np.min(x, axis=ax, keepdims=True)  # NaN-propagating
            elif kind == "max":
                r = np.max(x, axis=ax, keepdims=True)
            elif kind == "norm1":
                r = np.abs(x).sum(axis=ax, keepdims=True, dtype=np.float64)
            elif kind == "norm2":
                sq = round_to(x * x, FP32)  # SquareFp32 is an fp32 multiply
                r = np.sqrt(round_to(sq.sum(axis=ax, keepdims=True, dtype=np.float64), FP32))
            else:
                raise ValueError(kind)
        r = round_to(r, FP32)
        r = _apply_squeeze(r, squeeze_axes)
        return OTensor(r, out_dtype or FP32)

    def reduce_sum(self, axes=(), squeeze_axes=(), out_dtype=None): return self._reduce("sum", axes, squeeze_axes, out_dtype)
    def reduce_mean(self, axes=(), squeeze_axes=(), out_dtype=None): return self._reduce("mean", axes, squeeze_axes, out_dtype)
    def reduce_prod(self, axes=(), squeeze_axes=(), out_dtype=None): return self._reduce("prod", axes, squeeze_axes, out_dtype)
    def reduce_min(self, axes=(), squeeze_axes=(), out_dtype=None): return self._reduce("min", axes, squeeze_axes, out_dtype)
    def reduce_max(self, axes=(), squeeze_axes=(), out_dtype=None): return self._reduce("max", axes, squeeze_axes, out_dtype)
    def reduce_norm1(self, axes=(), squeeze_axes=(), out_dtype=None): return self._reduce("norm1", axes, squeeze_axes, out_dtype)
    def reduce_norm2(self, axes=(), squeeze_axes=(), out_dtype=None): return self._reduce("norm2", axes, squeeze_axes, out_dtype)

    def _arg(self, is_max: bool, axes: Iterable[int], squeeze_axes: Iterable[int]) -> "OTensor":
        ax = tuple(axes) or tuple(range(self.v.ndim))
        x = self.v
        # move reduced axes last and flatten them: index = row-major position inside the reduced domain
        keep = [a for a in range(x.ndim) if a not in ax]
        moved = np.transpose(x, keep + list(ax)).reshape([x.shape[a] for a in keep] + [-1])
        idx = arg_reduce_rows(moved.reshape(-1, moved.shape[-1]), is_max).reshape([x.shape[a] for a in keep])
        full_shape = [1 if a in ax else x.shape[a] for a in range(x.ndim)]
        r = idx.reshape(full_shape).astype(np.float64)
        return OTensor(_apply_squeeze(r, squeeze_axes), UINT32)

    def argmax(self, axes=(), squeeze_axes=()): return self._arg(True, axes, squeeze_axes)
    def argmin(self, axes=(), squeeze_axes=()): return self._arg(False, axes, squeeze_axes)


def _apply_squeeze(r: np.ndarray, squeeze_axes: Iterable[int]) -> np.ndarray:
    sq = list(squeeze_axes)
    if len(sq) == 1 and sq[0] == (1 << 64) - 1:
        r = r.reshape([d for d in r.shape if d != 1] or [1])
    elif sq:
        r = np.squeeze(r, tuple(sq))
        if r.ndim == 0:
            r = r.reshape(1)
    return r


def arg_reduce_rows(rows: np.ndarray, is_max: bool) -> np.ndarray:
    """Index of the arg-extremum of every row: NaN wins, the lowest index wins ties (incl. NaN vs NaN)."""
    rows = np.asarray(rows, dtype=np.float64)
    nan = np.isnan(rows)
    has_nan = nan.any(axis=1)
    first_nan = nan.argmax(axis=1)
    with np.errstate(all="ignore"):
        clean = np.where(nan, -np.inf if is_max else np.inf, rows)
        best = clean.argmax(axis=1) if is_max else clean.argmin(axis=1)  # numpy returns the first occurrence
    return np.where(has_nan, first_nan, best).astype(np.uint64)


def ulp_distance(got: np.ndarray, want: np.ndarray, dtype: int) -> np.ndarray:
    """|got - want| in units of the spacing of `dtype` at |want| (values given as floats; NaN pairs count as 0)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    man = {FP32: 23, FP16: 10, BF16: 7, FP8_E4M3: 3, FP8_E5M2: 2}[dtype]
    emin = {FP32: -126, FP16: -14, BF16: -126, FP8_E4M3: -6, FP8_E5M2: -14}[dtype]
    with np.errstate(all="ignore"):
        e = np.floor(np.log2(np.maximum(np.abs(want), 2.0 ** emin)))
        spacing = np.exp2(np.maximum(e, emin) - man)
        d = np.abs(got - want) / spacing
    both_nan = np.isnan(got) & np.isnan(want)
    same_inf = np.isinf(got) & np.isinf(want) & (np.sign(got) == np.sign(want))
    d = np.where(both_nan | same_inf, 0.0, d)
    return np.where(np.isnan(d), np.inf, d)
