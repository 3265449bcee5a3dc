"""Binding of the reduction seam, named after the reference's CubReduction / CubArgReduction
(Utilities/TensorOperations/Cub/CubReduction.h:176-447): describe, stamp (plan + allocate), run."""
from __future__ import annotations

import ctypes as C
import enum
from typing import Optional, Sequence, Union

import torch

from . import _native
from .dtypes import DataType, from_torch, to_torch
from .expression import _Binding, _bind_tensor, _check, _host

_lib = _native.lib


class _ReduceDesc(C.Structure):
    _fields_ = [("op", C.c_int32), ("input_dtype", C.c_int32), ("output_dtype", C.c_int32), ("flags", C.c_uint32), ("outer", C.c_uint64),
                ("reduction", C.c_uint64), ("inner", C.c_uint64), ("out_stride_outer", C.c_uint64), ("out_stride_inner", C.c_uint64)]


class _ArgDesc(C.Structure):
    _fields_ = [("op", C.c_int32), ("input_dtype", C.c_int32), ("value_dtype", C.c_int32), ("index_dtype", C.c_int32), ("outer", C.c_uint64),
                ("reduction", C.c_uint64), ("inner", C.c_uint64)]


_lib.thor_b200_reduce_plan_create.argtypes = [C.POINTER(_ReduceDesc), C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]
_lib.thor_b200_reduce_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_void_p]
_lib.thor_b200_reduce_plan_kind.argtypes = [C.c_void_p]
_lib.thor_b200_reduce_plan_kind.restype = C.c_char_p
_lib.thor_b200_reduce_plan_destroy.argtypes = [C.c_void_p]
_lib.thor_b200_reduce_plan_destroy.restype = None
_lib.thor_b200_argreduce_plan_create.argtypes = [C.POINTER(_ArgDesc), C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]
_lib.thor_b200_argreduce_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
_lib.thor_b200_argreduce_plan_destroy.argtypes = [C.c_void_p]
_lib.thor_b200_argreduce_plan_destroy.restype = None


class _StridedDesc(C.Structure):
    _fields_ = [("op", C.c_int32), ("arg_op", C.c_int32), ("input_dtype", C.c_int32), ("output_dtype", C.c_int32), ("rank", C.c_uint32),
                ("has_strides", C.c_uint32), ("dims", C.c_uint64 * 8), ("reduced", C.c_uint8 * 8), ("strides", C.c_uint64 * 8)]


_lib.thor_b200_strided_reduce_launch.argtypes = [C.POINTER(_StridedDesc), C.c_void_p, C.c_void_p, C.c_float, C.c_void_p]


def _strided_desc(shape, axes, op: int, arg_op: int, in_dt: DataType, out_dt: DataType) -> _StridedDesc:
    if len(shape) > 8:
        raise _native.ThorB200InvalidArgument("reductions over non-adjacent axes support rank <= 8")
    d = _StridedDesc()
    d.op, d.arg_op, d.input_dtype, d.output_dtype, d.rank = int(op), int(arg_op), int(in_dt), int(out_dt), len(shape)
    for i, v in enumerate(shape):
        d.dims[i] = int(v)
        d.reduced[i] = 1 if i in axes else 0
    return d


class CubReductionOp(enum.IntEnum):
    Sum = 0
    Min = 1
    Max = 2
    Product = 3
    Mean = 4
    L1Norm = 5
    L2Norm = 6


class CubArgReductionOp(enum.IntEnum):
    ArgMin = 0
    ArgMax = 1


class CubReductionPath(enum.IntEnum):
    DeviceTransformReduce = 0
    ContiguousFixedSegment = 1
    TiledFixedSegment = 2
    StridedFixedSegment = 3


def analyze_geometry(dims: Sequence[int], axes: Sequence[int]):
    """(outer, reduction, inner, path) like CubReduction::analyzeGeometry (CubReduction.cpp:755-912); needs no GPU."""
    d = (C.c_uint64 * max(1, len(dims)))(*dims)
    a = (C.c_uint32 * max(1, len(axes)))(*axes)
    ori = (C.c_uint64 * 3)()
    path = C.c_int32()
    _check(_host.thb_reduction_geometry(d, len(dims), a, len(axes), ori, C.byref(path)))
    return int(ori[0]), int(ori[1]), int(ori[2]), CubReductionPath(path.value)


def analyze_geometry_full(dims: Sequence[int], axes: Sequence[int], strides: Optional[Sequence[int]] = None) -> dict:
    """Every field of CubReduction::analyzeGeometry for a dense tensor or, with element `strides`, a view of storage
    (permutation-aware tiled geometry, output strides, affine rank-1 views; CubReduction.h:107-153).  Needs no GPU."""
    import json

    d = (C.c_uint64 * max(1, len(dims)))(*dims)
    s = (C.c_uint64 * max(1, len(dims)))(*strides) if strides is not None else None
    a = (C.c_uint32 * max(1, len(axes)))(*axes)
    text = C.c_char_p()
    _check(_host.thb_reduction_geometry_json(d, s, len(dims), a, len(axes), C.byref(text)))
    return json.loads(text.value.decode())


def map_logical_reduction_index(dims: Sequence[int], axes: Sequence[int], output_index: int, reduction_index: int, strides: Optional[Sequence[int]] = None) -> int:
    """CubReduction::mapLogicalReductionIndexToPhysicalIndex: element offset of one element of one output's reduction domain."""
    d = (C.c_uint64 * max(1, len(dims)))(*dims)
    s = (C.c_uint64 * max(1, len(dims)))(*strides) if strides is not None else None
    a = (C.c_uint32 * max(1, len(axes)))(*axes)
    out = C.c_uint64()
    _check(_host.thb_reduction_map_index(d, s, len(dims), a, len(axes), C.c_uint64(output_index), C.c_uint64(reduction_index), C.byref(out)))
    return int(out.value)


def empty_reduction_value(op: CubReductionOp) -> float:
    return float(_host.thb_cub_empty_value(int(op)))


class StampedCubReduction:
    def __init__(self, handle, input_t, output_t):
        self._h, self._in, self.output = handle, input_t, output_t

    def __del__(self):
        try:
            _host.thb_cub_reduction_free(self._h)
        except Exception:
            pass

    def run(self) -> None:
        _check(_host.thb_cub_reduction_run(self._h))

    def kernel_kind(self) -> str:
        return _host.thb_cub_reduction_kind(self._h).decode()

    def workspace_bytes(self) -> int:
        return int(_host.thb_cub_reduction_workspace_bytes(self._h))


class CubReduction:
    def __init__(self, op: CubReductionOp, axes: Union[int, Sequence[int]], output_dtype: Optional[DataType] = None, output_scale: float = 1.0):
        self.op = CubReductionOp(op)
        self.axes = [axes] if isinstance(axes, int) else list(axes)
        self.output_dtype = output_dtype
        self.output_scale = float(output_scale)

    def stamp(self, input_t: torch.Tensor, stream=None, input_dtype: Optional[DataType] = None, output: Optional[torch.Tensor] = None) -> StampedCubReduction:
        in_dt = DataType(input_dtype) if input_dtype is not None else from_torch(input_t.dtype)
        out_dt = DataType(self.output_dtype) if self.output_dtype is not None else in_dt
        out_shape = [1 if i in self.axes else d for i, d in enumerate(input_t.shape)]
        if output is None:
            output = torch.empty(out_shape, dtype=to_torch(out_dt), device=input_t.device)
        ob = _bind_tensor("output", output, out_dt)
        axes = (C.c_uint32 * max(1, len(self.axes)))(*self.axes)
        h = C.c_void_p()
        if not input_t.is_contiguous():
            # a view of storage (permuted, sliced with a step, expanded ...): stamped as it is, nothing is copied
            ib = _Binding()
            ib.name, ib.ptr, ib.dtype, ib.rank, ib.is_scalar = b"input", input_t.data_ptr(), int(in_dt), input_t.dim(), 0
            for i, d in enumerate(input_t.shape):
                ib.dims[i] = d
            strides = (C.c_uint64 * max(1, input_t.dim()))(*input_t.stride())
            with torch.cuda.device(input_t.device):
                _check(_host.thb_cub_reduction_stamp_view(int(self.op), axes, len(self.axes), int(self.output_dtype or 0), C.c_float(self.output_scale),
                                                          C.byref(ib), strides, C.byref(ob), _native.stream_handle(stream), input_t.device.index or 0, C.byref(h)))
            return StampedCubReduction(h, input_t, output)
        ib = _bind_tensor("input", input_t, in_dt)
        with torch.cuda.device(input_t.device):
            _check(_host.thb_cub_reduction_stamp(int(self.op), axes, len(self.axes), int(self.output_dtype or 0), C.c_float(self.output_scale),
                                                 C.byref(ib), C.byref(ob), _native.stream_handle(stream), input_t.device.index or 0, C.byref(h)))
        return StampedCubReduction(h, input_t, output)


class StampedCubArgReduction:
    def __init__(self, plan, input_t, index, value, workspace, ws_bytes, stream):
        self._plan, self._in, self.index, self.value, self._ws, self._ws_bytes, self._stream = plan, input_t, index, value, workspace, ws_bytes, stream

    def __del__(self):
        try:
            _lib.thor_b200_argreduce_plan_destroy(self._plan)
        except Exception:
            pass

    def run(self) -> None:
        _native.check(_lib.thor_b200_argreduce_launch(self._plan, self._in.data_ptr(), self.value.data_ptr() if self.value is not None else None,
                                                      self.index.data_ptr() if self.index is not None else None, self._ws.data_ptr(), self._ws_bytes,
                                                      _native.stream_handle(self._stream)))


class StampedStridedCubArgReduction:
    """Arg reduction over non-adjacent axes (StridedFixedSegment): stateless launches, the winner's value is the
    NaN-propagating min / max of the segment."""

    def __init__(self, index_desc, value_desc, input_t, index, value, stream):
        self._index_desc, self._value_desc, self._in, self.index, self.value, self._stream = index_desc, value_desc, input_t, index, value, stream

    def run(self) -> None:
        st = _native.stream_handle(self._stream)
        if self._index_desc is not None:
            _native.check(_lib.thor_b200_strided_reduce_launch(C.byref(self._index_desc), self._in.data_ptr(), self.index.data_ptr(), C.c_float(1.0), st))
        if self._value_desc is not None:
            _native.check(_lib.thor_b200_strided_reduce_launch(C.byref(self._value_desc), self._in.data_ptr(), self.value.data_ptr(), C.c_float(1.0), st))


class CubArgReduction:
    def __init__(self, op: CubArgReductionOp, axes: Union[int, Sequence[int]], produce_value: bool = True, produce_index: bool = True,
                 index_dtype: DataType = DataType.uint32):
        self.op = CubArgReductionOp(op)
        self.axes = [axes] if isinstance(axes, int) else list(axes)
        self.produce_value, self.produce_index, self.index_dtype = produce_value, produce_index, DataType(index_dtype)

    def stamp(self, input_t: torch.Tensor, stream=None, input_dtype: Optional[DataType] = None) -> StampedCubArgReduction:
        in_dt = DataType(input_dtype) if input_dtype is not None else from_torch(input_t.dtype)
        if not input_t.is_contiguous():
            # the reference's arg reductions take dense tensors only (CubReduction.cpp:1310, requireDenseContiguousGpuTensor)
            raise _native.ThorB200InvalidArgument("input must be dense contiguous.")
        outer, red, inner, path = analyze_geometry(list(input_t.shape), self.axes)
        if path == CubReductionPath.StridedFixedSegment:
            out_shape = [1 if i in self.axes else d for i, d in enumerate(input_t.shape)]
            index = torch.empty(out_shape, dtype=to_torch(self.index_dtype), device=input_t.device) if self.produce_index else None
            value = torch.empty(out_shape, dtype=input_t.dtype, device=input_t.device) if self.produce_value else None
            idesc = _strided_desc(input_t.shape, self.axes, 0, int(self.op), in_dt, self.index_dtype) if self.produce_index else None
            vop = CubReductionOp.Max if self.op == CubArgReductionOp.ArgMax else CubReductionOp.Min
            vdesc = _strided_desc(input_t.shape, self.axes, int(vop), -1, in_dt, in_dt) if self.produce_value else None
            return StampedStridedCubArgReduction(idesc, vdesc, input_t, index, value, stream)
        desc = _ArgDesc(int(self.op), int(in_dt), int(in_dt) if self.produce_value else 0, int(self.index_dtype), outer, red, inner)
        plan = C.c_void_p()
        ws = C.c_size_t()
        with torch.cuda.device(input_t.device):
            _native.check(_lib.thor_b200_argreduce_plan_create(C.byref(desc), C.byref(plan), C.byref(ws)))
        out_shape = [1 if i in self.axes else d for i, d in enumerate(input_t.shape)]
        index = torch.empty(out_shape, dtype=to_torch(self.index_dtype), device=input_t.device) if self.produce_index else None
        value = torch.empty(out_shape, dtype=input_t.dtype, device=input_t.device) if self.produce_value else None
        workspace = torch.empty(max(16, ws.value), dtype=torch.uint8, device=input_t.device)
        return StampedCubArgReduction(plan, input_t, index, value, workspace, ws.value, stream)


# ---- backward of dense min / max reductions ---------------------------------------------------------
class _MinMaxBackwardDesc(C.Structure):
    _fields_ = [("is_max", C.c_int32), ("input_dtype", C.c_int32), ("grad_output_dtype", C.c_int32), ("grad_input_dtype", C.c_int32),
                ("outer", C.c_uint64), ("reduction", C.c_uint64), ("inner", C.c_uint64), ("grad_mode", C.c_int32), ("grad_value", C.c_float)]


_lib.thor_b200_minmax_backward_plan_create.argtypes = [C.POINTER(_MinMaxBackwardDesc), C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]
_lib.thor_b200_minmax_backward_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
_lib.thor_b200_minmax_backward_plan_destroy.argtypes = [C.c_void_p]
_lib.thor_b200_minmax_backward_plan_destroy.restype = None


class ReduceMinMaxBackward:
    """Routes the gradient of a min / max reduction over `[outer, reduction, inner]` to each segment's winner
    (the reference stamps a zero fill, an arg reduction and launchReduceMinMaxBackwardScatter for this,
    Utilities/Expression/ReduceMinMaxBackwardKernel.h:28-34)."""

    def __init__(self, is_max: bool, input_t: torch.Tensor, grad_output: torch.Tensor, outer: int, reduction: int, inner: int,
                 grad_input_dtype: Optional[DataType] = None, stream=None):
        if input_t.numel() != outer * reduction * inner or grad_output.numel() != outer * inner:
            raise _native.ThorB200InvalidArgument("ReduceMinMaxBackward: tensor sizes do not match [outer, reduction, inner]")
        self._input, self._grad_output, self._stream = input_t, grad_output, stream
        gi = grad_input_dtype if grad_input_dtype is not None else from_torch(input_t.dtype)
        d = _MinMaxBackwardDesc(int(bool(is_max)), int(from_torch(input_t.dtype)), int(from_torch(grad_output.dtype)), int(gi), outer, reduction, inner, 0, 0.0)
        self._plan = C.c_void_p()
        ws = C.c_size_t()
        _native.check(_lib.thor_b200_minmax_backward_plan_create(C.byref(d), C.byref(self._plan), C.byref(ws)))
        self._ws_bytes = ws.value
        self._workspace = torch.empty(max(1, ws.value), dtype=torch.uint8, device=input_t.device)
        self.grad_input = torch.empty(input_t.shape, dtype=to_torch(gi), device=input_t.device)

    def __del__(self):
        try:
            if self._plan:
                _lib.thor_b200_minmax_backward_plan_destroy(self._plan)
        except Exception:
            pass

    def run(self) -> torch.Tensor:
        _native.check(_lib.thor_b200_minmax_backward_launch(self._plan, self._input.data_ptr(), self._grad_output.data_ptr(), self.grad_input.data_ptr(),
                                                            self._workspace.data_ptr(), self._ws_bytes, _native.stream_handle(self._stream)))
        return self.grad_input


# ---- flat scatter-add without atomics ------------------------------------------------------------------
class _ScatterAddDesc(C.Structure):
    _fields_ = [("value_dtype", C.c_int32), ("index_policy", C.c_int32), ("num_updates", C.c_uint64), ("output_numel", C.c_uint64)]


_lib.thor_b200_scatter_add_workspace_bytes.argtypes = [C.POINTER(_ScatterAddDesc), C.POINTER(C.c_size_t)]
_lib.thor_b200_scatter_add_launch.argtypes = [C.POINTER(_ScatterAddDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
_lib.thor_b200_scatter_add_launch_count.argtypes = [C.POINTER(_ScatterAddDesc)]


class FlatScatterAddIndexPolicy(enum.IntEnum):
    CanonicalizeDuplicatesAndSkipInvalid = 0
    IndicesAreUniqueAndValid = 1


def scatter_add_workspace_bytes(num_updates: int, output_numel: int, policy=FlatScatterAddIndexPolicy.CanonicalizeDuplicatesAndSkipInvalid,
                                value_dtype: DataType = DataType.fp32) -> int:
    """Workspace a FlatScatterAdd of this size needs; validates the description (no GPU needed)."""
    d = _ScatterAddDesc(int(value_dtype), int(policy), num_updates, output_numel)
    ws = C.c_size_t()
    _native.check(_lib.thor_b200_scatter_add_workspace_bytes(C.byref(d), C.byref(ws)))
    return int(ws.value)


class FlatScatterAdd:
    """output[:] = 0; output[indices[i]] += updates[i] for every valid i, duplicates added in the order of i, no atomics
    (the reference's prepareFlatScatterAdd / runFlatScatterAdd, Utilities/Expression/FlatScatterAddKernel.h:61-74).
    The plan owns its workspace; run() allocates nothing."""

    def __init__(self, updates: torch.Tensor, flat_indices: torch.Tensor, output: torch.Tensor,
                 index_policy=FlatScatterAddIndexPolicy.CanonicalizeDuplicatesAndSkipInvalid, stream=None):
        if flat_indices.dtype != torch.uint32:
            raise _native.ThorB200InvalidArgument("Flat scatter-add indices must be UINT32.")
        if updates.dtype != output.dtype:
            raise _native.ThorB200InvalidArgument("Flat scatter-add updates and output must have the same dtype.")
        if tuple(updates.shape) != tuple(flat_indices.shape):
            raise _native.ThorB200InvalidArgument("Flat scatter-add updates and indices must have the same shape.")
        if not (updates.device == flat_indices.device == output.device):
            raise _native.ThorB200InvalidArgument("Flat scatter-add updates, indices, and output must be on the same placement.")
        self.index_policy = FlatScatterAddIndexPolicy(index_policy)
        self._desc = _ScatterAddDesc(int(from_torch(updates.dtype)), int(self.index_policy), updates.numel(), output.numel())
        ws = C.c_size_t()
        _native.check(_lib.thor_b200_scatter_add_workspace_bytes(C.byref(self._desc), C.byref(ws)))
        self.workspace_bytes = int(ws.value) if self.index_policy == FlatScatterAddIndexPolicy.CanonicalizeDuplicatesAndSkipInvalid else 0
        self._ws_bytes = int(ws.value)
        self._workspace = torch.empty(max(16, self._ws_bytes), dtype=torch.uint8, device=output.device)
        self._stream = stream
        self.kernel_launches = int(_lib.thor_b200_scatter_add_launch_count(C.byref(self._desc)))

    def run(self, updates: torch.Tensor, flat_indices: torch.Tensor, output: torch.Tensor, stream=None) -> torch.Tensor:
        if updates.numel() != self._desc.num_updates or flat_indices.numel() != self._desc.num_updates or output.numel() != self._desc.output_numel:
            raise _native.ThorB200InvalidArgument("Flat scatter-add runtime tensors do not match the prepared plan shape.")
        if int(from_torch(updates.dtype)) != self._desc.value_dtype or updates.dtype != output.dtype or flat_indices.dtype != torch.uint32:
            raise _native.ThorB200InvalidArgument("Flat scatter-add runtime tensor dtypes do not match the prepared plan.")
        _native.check(_lib.thor_b200_scatter_add_launch(C.byref(self._desc), updates.data_ptr(), flat_indices.data_ptr(), output.data_ptr(),
                                                        self._workspace.data_ptr(), self._ws_bytes, _native.stream_handle(stream if stream is not None else self._stream)))
        return output
