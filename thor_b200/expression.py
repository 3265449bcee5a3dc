"""ctypes binding of the C++ host layer (Expression / FusedEquation / CubReduction).

Plays the role of the reference's ``thor.physical.Expression`` Python module
(bindings/python/src/core/physical/expression.cpp): expressions are built with Python operators,
``compile`` gives a FusedEquation, ``stamp`` binds torch CUDA tensors and returns a plan whose
``run()`` only launches kernels.  All numerics and planning live in the C++ host layer and the CUDA
library; nothing here computes.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Dict, Iterable, Mapping, Optional, Sequence, Union

import torch

from . import _native
from .dtypes import DataType, from_torch, to_torch

_HOST_PATH = Path(__file__).resolve().parent / "lib" / "libthor_b200_host.so"
if not _HOST_PATH.exists():
    raise ImportError(f"{_HOST_PATH} is missing: build it with `python -m thor_b200.build`")
_host = C.CDLL(str(_HOST_PATH))
_host.thb_last_error.restype = C.c_char_p
_host.thb_plan_strings.restype = C.c_char_p
_host.thb_plan_strings.argtypes = [C.c_void_p, C.c_int]
_host.thb_plan_intermediate_bytes.restype = C.c_uint64
_host.thb_plan_intermediate_bytes.argtypes = [C.c_void_p]
_host.thb_plan_launches.restype = C.c_uint64
_host.thb_plan_launches.argtypes = [C.c_void_p]
_host.thb_plan_waits_expired.restype = C.c_int
_host.thb_plan_waits_expired.argtypes = [C.c_void_p, C.POINTER(C.c_uint64)]
_host.thb_cub_reduction_kind.restype = C.c_char_p
_host.thb_cub_reduction_kind.argtypes = [C.c_void_p]
_host.thb_cub_reduction_workspace_bytes.restype = C.c_uint64
_host.thb_cub_reduction_workspace_bytes.argtypes = [C.c_void_p]
_host.thb_cub_empty_value.restype = C.c_float
_host.thb_expr_node_count.restype = C.c_uint32
_host.thb_expr_node_count.argtypes = [C.c_void_p]
for _name in ("thb_expr_free", "thb_equation_free", "thb_plan_free", "thb_cub_reduction_free"):
    getattr(_host, _name).argtypes = [C.c_void_p]
    getattr(_host, _name).restype = None


class _Binding(C.Structure):
    _fields_ = [("name", C.c_char_p), ("ptr", C.c_void_p), ("dtype", C.c_int32), ("rank", C.c_uint32), ("dims", C.c_uint64 * 8),
                ("is_scalar", C.c_int32), ("scalar", C.c_float)]


def _check(status: int) -> None:
    if status == 0:
        return
    msg = _host.thb_last_error().decode("utf-8", "replace")
    if status == 1:
        raise _native.ThorB200InvalidArgument(msg)
    raise _native.ThorB200Error(msg)


class ExprOp:
    """Integer values of ThorImplementation::ExprOp (Utilities/Expression/Expression.h:32-148)."""
    ADD, SUB, MUL, DIV, POW = 7, 8, 9, 10, 11
    EQUAL, NOT_EQUAL, LESS, LESS_EQUAL, GREATER, GREATER_EQUAL = 12, 13, 14, 15, 16, 17
    LOGICAL_AND, LOGICAL_OR, LOGICAL_NOT = 18, 19, 20
    NEG, ABS, CEIL, FLOOR, ROUND, TRUNC = 23, 24, 25, 26, 27, 28
    SIN, COS, TAN, ASIN, ACOS, ATAN, SINH, COSH, ASINH, ACOSH, ATANH = range(29, 40)
    ERF, ERFC, ERFCX, ERFINV, ERFCINV, TGAMMA, LGAMMA, DIGAMMA = range(40, 48)
    EXP, EXPM1, EXP2, EXP10, LN, LOG1P, LOG2, LOG10, SQRT, TANH, NORMCDF = range(48, 59)
    RESHAPE, UNSQUEEZE, SQUEEZE = 62, 65, 66
    MIN, MAX = 69, 70
    REDUCE_SUM, REDUCE_PROD, REDUCE_MIN, REDUCE_MAX, REDUCE_ARGMIN, REDUCE_ARGMAX = range(83, 89)
    REDUCE_AVG, REDUCE_NORM1, REDUCE_NORM2 = 95, 96, 97


SQUEEZE_ALL = (1 << 64) - 1

_Scalar = Union[int, float]


def _as_expr(v) -> "Expression":
    return v if isinstance(v, Expression) else Expression.scalar(float(v))


class Expression:
    """A node of a lazy expression DAG (ThorImplementation::Expression, Expression.h:516-1075)."""

    __slots__ = ("_h",)

    def __init__(self, handle: C.c_void_p):
        self._h = handle

    def __del__(self):
        try:
            if self._h:
                _host.thb_expr_free(self._h)
        except Exception:
            pass

    # ---- leaves -----------------------------------------------------------------------------------
    @staticmethod
    def _leaf(name: str, kind: int, compute_dtype, output_dtype) -> "Expression":
        out = C.c_void_p()
        _check(_host.thb_input(name.encode(), kind, int(compute_dtype or 0), int(output_dtype or 0), C.byref(out)))
        return Expression(out)

    @staticmethod
    def input(name: str, compute_dtype: Optional[DataType] = None, output_dtype: Optional[DataType] = None) -> "Expression":
        return Expression._leaf(name, 0, compute_dtype, output_dtype)

    @staticmethod
    def runtime_scalar(name: str, compute_dtype: Optional[DataType] = None, output_dtype: Optional[DataType] = None) -> "Expression":
        return Expression._leaf(name, 1, compute_dtype, output_dtype)

    @staticmethod
    def tensor_runtime_scalar(name: str, compute_dtype: Optional[DataType] = None, output_dtype: Optional[DataType] = None) -> "Expression":
        return Expression._leaf(name, 2, compute_dtype, output_dtype)

    @staticmethod
    def scalar(value: float) -> "Expression":
        out = C.c_void_p()
        _check(_host.thb_scalar(C.c_double(value), C.byref(out)))
        return Expression(out)

    # ---- helpers ----------------------------------------------------------------------------------
    def _unary(self, op: int) -> "Expression":
        out = C.c_void_p()
        _check(_host.thb_unary(op, self._h, C.byref(out)))
        return Expression(out)

    def _binary(self, op: int, other, swap: bool = False) -> "Expression":
        o = _as_expr(other)
        a, b = (o, self) if swap else (self, o)
        out = C.c_void_p()
        _check(_host.thb_binary(op, a._h, b._h, C.byref(out)))
        return Expression(out)

    def _composite(self, name: str, p0: float = 0.0, p1: float = 0.0) -> "Expression":
        out = C.c_void_p()
        _check(_host.thb_composite(name.encode(), self._h, C.c_double(p0), C.c_double(p1), C.byref(out)))
        return Expression(out)

    # ---- operators --------------------------------------------------------------------------------
    def __add__(self, o): return self._binary(ExprOp.ADD, o)
    def __radd__(self, o): return self._binary(ExprOp.ADD, o, swap=True)
    def __sub__(self, o): return self._binary(ExprOp.SUB, o)
    def __rsub__(self, o): return self._binary(ExprOp.SUB, o, swap=True)
    def __mul__(self, o): return self._binary(ExprOp.MUL, o)
    def __rmul__(self, o): return self._binary(ExprOp.MUL, o, swap=True)
    def __truediv__(self, o): return self._binary(ExprOp.DIV, o)
    def __rtruediv__(self, o): return self._binary(ExprOp.DIV, o, swap=True)
    def __pow__(self, o): return self._binary(ExprOp.POW, o)
    def __rpow__(self, o): return self._binary(ExprOp.POW, o, swap=True)
    def __neg__(self): return self._unary(ExprOp.NEG)
    def __invert__(self): return self._unary(ExprOp.LOGICAL_NOT)
    def __lt__(self, o): return self._binary(ExprOp.LESS, o)
    def __le__(self, o): return self._binary(ExprOp.LESS_EQUAL, o)
    def __gt__(self, o): return self._binary(ExprOp.GREATER, o)
    def __ge__(self, o): return self._binary(ExprOp.GREATER_EQUAL, o)
    def equal(self, o): return self._binary(ExprOp.EQUAL, o)
    def not_equal(self, o): return self._binary(ExprOp.NOT_EQUAL, o)
    def logical_and(self, o): return self._binary(ExprOp.LOGICAL_AND, o)
    def logical_or(self, o): return self._binary(ExprOp.LOGICAL_OR, o)
    def logical_not(self): return self._unary(ExprOp.LOGICAL_NOT)
    def min(self, o): return self._binary(ExprOp.MIN, o)
    def max(self, o): return self._binary(ExprOp.MAX, o)
    def pow(self, o): return self._binary(ExprOp.POW, o)

    def cast(self, dtype: DataType) -> "Expression":
        out = C.c_void_p()
        _check(_host.thb_cast(self._h, int(dtype), C.byref(out)))
        return Expression(out)

    def with_output_dtype(self, dtype: DataType) -> "Expression":
        out = C.c_void_p()
        _check(_host.thb_with_output_dtype(self._h, int(dtype), C.byref(out)))
        return Expression(out)

    @staticmethod
    def where(cond: "Expression", true_value, false_value) -> "Expression":
        out = C.c_void_p()
        t, f = _as_expr(true_value), _as_expr(false_value)
        _check(_host.thb_where(cond._h, t._h, f._h, C.byref(out)))
        return Expression(out)

    # ---- math -------------------------------------------------------------------------------------
    def abs(self): return self._unary(ExprOp.ABS)
    def ceil(self): return self._unary(ExprOp.CEIL)
    def floor(self): return self._unary(ExprOp.FLOOR)
    def round(self): return self._unary(ExprOp.ROUND)
    def trunc(self): return self._unary(ExprOp.TRUNC)
    def sin(self): return self._unary(ExprOp.SIN)
    def cos(self): return self._unary(ExprOp.COS)
    def tan(self): return self._unary(ExprOp.TAN)
    def asin(self): return self._unary(ExprOp.ASIN)
    def acos(self): return self._unary(ExprOp.ACOS)
    def atan(self): return self._unary(ExprOp.ATAN)
    def sinh(self): return self._unary(ExprOp.SINH)
    def cosh(self): return self._unary(ExprOp.COSH)
    def asinh(self): return self._unary(ExprOp.ASINH)
    def acosh(self): return self._unary(ExprOp.ACOSH)
    def atanh(self): return self._unary(ExprOp.ATANH)
    def erf(self): return self._unary(ExprOp.ERF)
    def erfc(self): return self._unary(ExprOp.ERFC)
    def erfcx(self): return self._unary(ExprOp.ERFCX)
    def erfinv(self): return self._unary(ExprOp.ERFINV)
    def erfcinv(self): return self._unary(ExprOp.ERFCINV)
    def tgamma(self): return self._unary(ExprOp.TGAMMA)
    def lgamma(self): return self._unary(ExprOp.LGAMMA)
    def digamma(self): return self._unary(ExprOp.DIGAMMA)
    def exp(self): return self._unary(ExprOp.EXP)
    def expm1(self): return self._unary(ExprOp.EXPM1)
    def exp2(self): return self._unary(ExprOp.EXP2)
    def exp10(self): return self._unary(ExprOp.EXP10)
    def ln(self): return self._unary(ExprOp.LN)
    def log1p(self): return self._unary(ExprOp.LOG1P)
    def log2(self): return self._unary(ExprOp.LOG2)
    def log10(self): return self._unary(ExprOp.LOG10)
    def sqrt(self): return self._unary(ExprOp.SQRT)
    def tanh(self): return self._unary(ExprOp.TANH)
    def normcdf(self): return self._unary(ExprOp.NORMCDF)
    def sigmoid(self): return self._composite("sigmoid")
    def softplus(self): return self._composite("softplus")
    def elu(self, alpha: float = 1.0): return self._composite("elu", alpha)
    def selu(self): return self._composite("selu")
    def gelu(self): return self._composite("gelu")
    def swish(self): return self._composite("swish")
    def relu(self): return self._composite("relu")
    def relu6(self): return self._composite("relu6")
    def hard_tanh(self, lo: float = -1.0, hi: float = 1.0): return self._composite("hard_tanh", lo, hi)
    def clamp(self, lo: float, hi: float): return self._composite("clamp", lo, hi)

    # cudnnSoftmaxAlgorithm_t / cudnnSoftmaxMode_t values of the reference's softmax op
    SOFTMAX_FAST, SOFTMAX_ACCURATE, SOFTMAX_LOG = 0, 1, 2
    SOFTMAX_MODE_INSTANCE, SOFTMAX_MODE_CHANNEL = 0, 1

    def softmax(self, algorithm: int = 1, mode: int = 1) -> "Expression":
        """Softmax over axis 1 (channel mode) or over every axis but the first (instance mode), computed in
        fp32 and stored in the operand's dtype; runs as one row program."""
        return self._composite("softmax", float(algorithm), float(mode))

    def log_softmax(self, mode: int = 1) -> "Expression":
        return self._composite("log_softmax", 2.0, float(mode))

    # ---- shapes and reductions --------------------------------------------------------------------
    def _shape_op(self, op: int, values: Sequence[int]) -> "Expression":
        arr = (C.c_uint64 * max(1, len(values)))(*values)
        out = C.c_void_p()
        _check(_host.thb_shape_op(self._h, op, arr, len(values), C.byref(out)))
        return Expression(out)

    def reshape(self, dims: Sequence[int]): return self._shape_op(ExprOp.RESHAPE, dims)
    def unsqueeze(self, axes: Sequence[int]): return self._shape_op(ExprOp.UNSQUEEZE, axes)
    def squeeze(self, axes: Sequence[int]): return self._shape_op(ExprOp.SQUEEZE, axes)

    def _reduce(self, op: int, axes: Iterable[int] = (), squeeze_axes: Iterable[int] = (), compute_dtype: Optional[DataType] = None) -> "Expression":
        ax, sq = list(axes), list(squeeze_axes)
        a = (C.c_uint64 * max(1, len(ax)))(*ax)
        s = (C.c_uint64 * max(1, len(sq)))(*sq)
        out = C.c_void_p()
        _check(_host.thb_reduce(self._h, op, a, len(ax), s, len(sq), int(compute_dtype or 0), C.byref(out)))
        return Expression(out)

    def reduce_sum(self, axes=(), squeeze_axes=(), compute_dtype=None): return self._reduce(ExprOp.REDUCE_SUM, axes, squeeze_axes, compute_dtype)
    def reduce_prod(self, axes=(), squeeze_axes=(), compute_dtype=None): return self._reduce(ExprOp.REDUCE_PROD, axes, squeeze_axes, compute_dtype)
    def reduce_min(self, axes=(), squeeze_axes=(), compute_dtype=None): return self._reduce(ExprOp.REDUCE_MIN, axes, squeeze_axes, compute_dtype)
    def reduce_max(self, axes=(), squeeze_axes=(), compute_dtype=None): return self._reduce(ExprOp.REDUCE_MAX, axes, squeeze_axes, compute_dtype)
    def reduce_mean(self, axes=(), squeeze_axes=(), compute_dtype=None): return self._reduce(ExprOp.REDUCE_AVG, axes, squeeze_axes, compute_dtype)
    def reduce_norm1(self, axes=(), squeeze_axes=(), compute_dtype=None): return self._reduce(ExprOp.REDUCE_NORM1, axes, squeeze_axes, compute_dtype)
    def reduce_norm2(self, axes=(), squeeze_axes=(), compute_dtype=None): return self._reduce(ExprOp.REDUCE_NORM2, axes, squeeze_axes, compute_dtype)
    def argmin(self, axes=(), squeeze_axes=(), compute_dtype=None): return self._reduce(ExprOp.REDUCE_ARGMIN, axes, squeeze_axes, compute_dtype)
    def argmax(self, axes=(), squeeze_axes=(), compute_dtype=None): return self._reduce(ExprOp.REDUCE_ARGMAX, axes, squeeze_axes, compute_dtype)

    def node_count(self) -> int:
        return int(_host.thb_expr_node_count(self._h))

    # ---- compilation ------------------------------------------------------------------------------
    @staticmethod
    def compile(expr: Union["Expression", Mapping[str, "Expression"]], device_num: Optional[int] = None, use_fast_math: bool = False,
                fuse_row_reductions: bool = True, row_program: Optional[Mapping[str, int]] = None,
                unrounded_column_sums: bool = False, branch_streams: bool = True) -> "FusedEquation":
        """FusedEquation::compile: one Expression (output named "output") or a dict of named outputs.
        device_num defaults to the current CUDA device of the calling process.  row_program sets fields of
        FusedEquationOptions::row_program (ROW_PROGRAM_TUNING_FIELDS; layout choices of row programs, all computing the same
        values), which backward equations compiled from this one inherit.  unrounded_column_sums (for callers that hold
        one shard of the rows): row programs with column reductions also deliver those sums as the fp32 output
        "__column_sums" [reductions, cols], rows named by StampedExecutionPlan.column_sum_names().  branch_streams: stages
        that do not depend on each other run on helper streams joined by events (StampedExecutionPlan.stage_lanes()) when the
        plan's tensor inputs hold at least 64 MiB (the joins cost about 4 us per run); "always" uses them at any size."""
        named = {"output": expr} if isinstance(expr, Expression) else dict(expr)
        if device_num is None:
            device_num = torch.cuda.current_device() if torch.cuda.is_available() else 0
        return FusedEquation(named, device_num, use_fast_math, fuse_row_reductions, row_program, unrounded_column_sums, branch_streams)


def _bind_tensor(name: str, t: torch.Tensor, dtype: Optional[DataType] = None) -> _Binding:
    if not t.is_cuda:
        raise _native.ThorB200InvalidArgument(f"'{name}': tensors must live on a CUDA device")
    if not t.is_contiguous():
        raise _native.ThorB200InvalidArgument(f"'{name}': tensors must be contiguous")
    if t.dim() > 8:
        raise _native.ThorB200InvalidArgument(f"'{name}': rank above 8")
    b = _Binding()
    b.name = name.encode()
    b.ptr = t.data_ptr()
    b.dtype = int(dtype if dtype is not None else from_torch(t.dtype))
    b.rank = t.dim()
    for i, d in enumerate(t.shape):
        b.dims[i] = d
    b.is_scalar = 0
    return b


class StampedExecutionPlan:
    """A stamped plan: run() launches every stage; nothing is allocated or compiled at run time."""

    def __init__(self, handle, keep, plan_only: bool = False):
        self._h = handle
        self._keep = keep  # torch tensors whose memory the plan points at
        self._plan_only = plan_only

    def __del__(self):
        try:
            if self._h:
                _host.thb_plan_free(self._h)
        except Exception:
            pass

    def run(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        _check(_host.thb_plan_run(self._h, _native.stream_handle(stream) if stream is not None else None))

    def set_runtime_scalar(self, name: str, value: float) -> None:
        _check(_host.thb_plan_set_scalar(self._h, name.encode(), C.c_float(value)))

    def _strings(self, kind: int):
        raw = _host.thb_plan_strings(self._h, kind).decode("utf-8", "replace")
        return raw.split("\x1e") if raw else []

    def stage_kind_names(self): return self._strings(0)
    def physical_stage_names(self): return self._strings(1)
    def stage_sources(self): return self._strings(2)
    def output_names(self): return self._strings(3)
    def column_sum_names(self): return self._strings(4)

    def stage_lanes(self):
        """Lane of every physical stage: 0 = the caller's stream, 1.. = helper streams of independent branches."""
        buf = (C.c_uint32 * 256)()
        n = int(_host.thb_plan_stage_lanes(self._h, buf, 256))
        return [int(buf[i]) for i in range(min(n, 256))]
    def output_spec(self, name: str = "output"):
        """(shape, DataType) of the named output."""
        b = _Binding()
        _check(_host.thb_plan_output(self._h, name.encode(), C.byref(b)))
        return [int(b.dims[i]) for i in range(b.rank)], DataType(b.dtype)

    def intermediate_bytes(self) -> int: return int(_host.thb_plan_intermediate_bytes(self._h))
    def kernel_launches_per_run(self) -> int: return int(_host.thb_plan_launches(self._h))

    def waits_expired(self) -> int:
        """Bounded device-side waits that ran out in the launches so far (synchronises); 0 on a healthy run."""
        count = C.c_uint64(0)
        _check(_host.thb_plan_waits_expired(self._h, C.byref(count)))
        return int(count.value)

    def output(self, name: str = "output") -> torch.Tensor:
        """The named output as a torch tensor aliasing the plan's memory (valid while the plan lives)."""
        b = _Binding()
        _check(_host.thb_plan_output(self._h, name.encode(), C.byref(b)))
        if self._plan_only:
            raise _native.ThorB200Error("plan-only plans own no memory")
        for t in self._keep:
            if t.data_ptr() == b.ptr:
                return t
        dt = DataType(b.dtype)
        shape = [int(b.dims[i]) for i in range(b.rank)]
        n = 1
        for d in shape:
            n *= d
        from .dtypes import SIZE

        nbytes = n * SIZE[dt]
        holder = self

        class _Owner:
            __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(b.ptr), False), "version": 3}
            _plan = holder

        raw = torch.as_tensor(_Owner(), device="cuda")
        return raw.view(to_torch(dt)).reshape(shape)


ROW_PROGRAM_TUNING_FIELDS = ("ring_buffers", "pipeline_round_one", "copy_warpgroup", "keep_values", "reciprocal_division", "wait_limit_ms", "test_skip_fill", "reserve_sms")


class FusedEquation:
    def __init__(self, named: Mapping[str, Expression], device_num: int, use_fast_math: bool, fuse_row_reductions: bool, row_program=None, unrounded_column_sums=False, branch_streams=True, _handle=None):
        self.device_num = device_num
        if _handle is not None:
            self._h = _handle
            return
        names = list(named.keys())
        arr_n = (C.c_char_p * len(names))(*[n.encode() for n in names])
        arr_e = (C.c_void_p * len(names))(*[named[n]._h for n in names])
        out = C.c_void_p()
        tuning = None
        if row_program:
            unknown = set(row_program) - set(ROW_PROGRAM_TUNING_FIELDS)
            if unknown:
                raise _native.ThorB200InvalidArgument(f"unknown row_program field(s): {sorted(unknown)}")
            tuning = (C.c_int32 * len(ROW_PROGRAM_TUNING_FIELDS))(*[int(row_program.get(f, 0)) for f in ROW_PROGRAM_TUNING_FIELDS])
        _check(_host.thb_compile(arr_n, arr_e, len(names), device_num, int(use_fast_math), int(fuse_row_reductions), tuning, int(unrounded_column_sums), 2 if branch_streams == "always" else int(bool(branch_streams)), C.byref(out)))
        self._h = out

    def __del__(self):
        try:
            if self._h:
                _host.thb_equation_free(self._h)
        except Exception:
            pass

    def compile_backward(self, wrt: Sequence[str], upstream_prefix: str = "__grad_output") -> "FusedEquation":
        arr = (C.c_char_p * len(wrt))(*[w.encode() for w in wrt])
        out = C.c_void_p()
        _check(_host.thb_compile_backward(self._h, arr, len(wrt), upstream_prefix.encode(), C.byref(out)))
        return FusedEquation({}, self.device_num, False, True, None, False, True, _handle=out)

    def stamp(self, inputs: Mapping[str, Union[torch.Tensor, float]], stream: Optional[torch.cuda.Stream] = None,
              outputs: Optional[Mapping[str, torch.Tensor]] = None, dtypes: Optional[Mapping[str, DataType]] = None) -> StampedExecutionPlan:
        """Binds tensors / runtime scalars by name; `outputs` adopts caller tensors for named outputs;
        `dtypes` overrides the dtype of raw-storage tensors."""
        dtypes = dtypes or {}
        ins, keep = [], []
        for name, v in inputs.items():
            if isinstance(v, torch.Tensor):
                ins.append(_bind_tensor(name, v, dtypes.get(name)))
                keep.append(v)
            else:
                b = _Binding()
                b.name = name.encode()
                b.is_scalar = 1
                b.scalar = float(v)
                ins.append(b)
        outs = []
        for name, t in (outputs or {}).items():
            outs.append(_bind_tensor(name, t, dtypes.get(name)))
            keep.append(t)
        in_arr = (_Binding * max(1, len(ins)))(*ins)
        out_arr = (_Binding * max(1, len(outs)))(*outs)
        plan = C.c_void_p()
        with torch.cuda.device(self.device_num):
            _check(_host.thb_stamp(self._h, in_arr, len(ins), out_arr, len(outs), _native.stream_handle(stream), C.byref(plan)))
        return StampedExecutionPlan(plan, keep)

    def graph(self, inputs: Mapping[str, Union[tuple, float]]) -> dict:
        """The dtype-resolved SSA graph this equation evaluates for tensors of the given (shape, DataType): inputs by slot,
        named outputs and every node (ExprOp integer, parents, literal, axes lists, output / compute dtype).  For a backward
        equation it is the differentiated graph for those forward shapes.  Needs no GPU."""
        import json

        in_arr, n = self._shape_bindings(inputs)
        text = C.c_char_p()
        _check(_host.thb_equation_graph(self._h, in_arr, n, C.byref(text)))
        return json.loads(text.value.decode())

    @staticmethod
    def _shape_bindings(inputs):
        ins = []
        for name, v in inputs.items():
            b = _Binding()
            b.name = name.encode()
            if isinstance(v, (int, float)):
                b.is_scalar = 1
                b.scalar = float(v)
            else:
                shape, dtype = v
                if len(shape) > 8:
                    raise _native.ThorB200InvalidArgument(f"'{name}': rank above 8")
                b.dtype = int(dtype)
                b.rank = len(shape)
                for i, d in enumerate(shape):
                    b.dims[i] = int(d)
                b.is_scalar = 0
            ins.append(b)
        return (_Binding * max(1, len(ins)))(*ins), len(ins)

    def plan(self, inputs: Mapping[str, Union[tuple, float]]) -> StampedExecutionPlan:
        """Stamps without a GPU: `inputs` maps each tensor name to (shape, DataType) and each runtime
        scalar to a float.  The returned plan lists its stages, kernel shapes, emitted sources and
        intermediate bytes exactly as a real stamp on those shapes would; run() and output() refuse."""
        in_arr, n_in = self._shape_bindings(inputs)
        plan = C.c_void_p()
        _check(_host.thb_stamp_plan_only(self._h, in_arr, n_in, C.byref(plan)))
        return StampedExecutionPlan(plan, [], plan_only=True)

    def run(self, inputs: Mapping[str, Union[torch.Tensor, float]], output: Union[torch.Tensor, Mapping[str, torch.Tensor]],
            stream: Optional[torch.cuda.Stream] = None) -> None:
        """Convenience path of the reference (single fused stage only): stamp, check, launch."""
        outs = {"output": output} if isinstance(output, torch.Tensor) else dict(output)
        plan = self.stamp(inputs, stream, outs)
        kinds = plan.stage_kind_names()
        if kinds != ["FusedKernel"]:
            raise _native.ThorB200InvalidArgument("FusedEquation.run supports single fused-stage expressions only; use stamp() for staged reductions")
        plan.run(stream)


def resolve_dtypes(named: Mapping[str, Expression], input_dtypes: Mapping[str, DataType]):
    """(op, output_dtype, compute_dtype) of every node after dtype resolution -- needs no GPU."""
    names = list(named.keys())
    arr_n = (C.c_char_p * len(names))(*[n.encode() for n in names])
    arr_e = (C.c_void_p * len(names))(*[named[n]._h for n in names])
    in_names = list(input_dtypes.keys())
    arr_in = (C.c_char_p * max(1, len(in_names)))(*[n.encode() for n in in_names])
    arr_dt = (C.c_int32 * max(1, len(in_names)))(*[int(input_dtypes[n]) for n in in_names])
    cap = 4096
    buf = (C.c_int32 * (3 * cap))()
    n_nodes = C.c_uint32()
    _check(_host.thb_resolve_dtypes(arr_n, arr_e, len(names), arr_in, arr_dt, len(in_names), buf, cap, C.byref(n_nodes)))
    return [(buf[3 * k], DataType(buf[3 * k + 1]), DataType(buf[3 * k + 2])) for k in range(n_nodes.value)]


def build_execution_schedule(dependencies: Sequence[Sequence[int]]):
    """The pure lane-assignment function of stamped plans (the reference's detail::buildStampedExecutionSchedule,
    StampedEquation.h:1634-1646): dependencies[s] lists the stages that stage s consumes.  Returns (lanes per stage,
    completion-event flags per stage, number of lanes, needs_caller_ready_event).  Needs no GPU."""
    flat, offsets = [], [0]
    for d in dependencies:
        flat += list(d)
        offsets.append(len(flat))
    n = len(dependencies)
    lanes = (C.c_uint32 * max(1, n))()
    events = (C.c_uint8 * max(1, n))()
    n_lanes, ready = C.c_uint32(), C.c_int32()
    _host.thb_plan_stage_lanes.restype = C.c_uint32
    _check(_host.thb_build_schedule((C.c_uint32 * max(1, len(flat)))(*flat), (C.c_uint32 * len(offsets))(*offsets), n, lanes, events, C.byref(n_lanes), C.byref(ready)))
    return [int(lanes[i]) for i in range(n)], [bool(events[i]) for i in range(n)], int(n_lanes.value), bool(ready.value)
