"""Binding of the cast seam, named after the reference's TypeConverter
(Utilities/TensorOperations/DataTypeConversions/TypeConverter.h:17-34)."""
from __future__ import annotations

import ctypes

import torch

from . import _native
from .dtypes import DataType, from_torch


class TypeConverter:
    @staticmethod
    def convert_type_raw(src_ptr: int, dst_ptr: int, src_dtype: DataType, dst_dtype: DataType, num_elements: int, stream=None) -> None:
        """TypeConverter::convertType on raw device pointers (asynchronous on `stream`)."""
        _native.check(_native.lib.thor_b200_cast_launch(ctypes.c_void_p(src_ptr), ctypes.c_void_p(dst_ptr), int(src_dtype), int(dst_dtype),
                                                        int(num_elements), _native.stream_handle(stream)))

    @staticmethod
    def convert_type(src: torch.Tensor, dst: torch.Tensor, src_dtype: DataType | None = None, dst_dtype: DataType | None = None,
                     stream=None) -> torch.Tensor:
        """Cast `src` into `dst` (same element count).  Dtypes default to the tensors' own; pass them
        explicitly for raw-storage tensors (e.g. bf16 carried as uint16)."""
        if not (src.is_cuda and dst.is_cuda):
            raise _native.ThorB200InvalidArgument("TypeConverter: both tensors must live on a CUDA device (no CPU path in this library)")
        if not (src.is_contiguous() and dst.is_contiguous()):
            raise _native.ThorB200InvalidArgument("TypeConverter: tensors must be contiguous")
        if src.numel() != dst.numel():
            raise _native.ThorB200InvalidArgument("TypeConverter: element counts differ")
        sd = DataType(src_dtype) if src_dtype is not None else from_torch(src.dtype)
        dd = DataType(dst_dtype) if dst_dtype is not None else from_torch(dst.dtype)
        with torch.cuda.device(src.device):
            TypeConverter.convert_type_raw(src.data_ptr(), dst.data_ptr(), sd, dd, src.numel(), stream)
        return dst

    @staticmethod
    def stamp(src: torch.Tensor, dst: torch.Tensor, src_dtype: DataType | None = None, dst_dtype: DataType | None = None,
              stream=None) -> "StampedConversion":
        """The same conversion with everything resolved once: run() is a single call into the library."""
        return StampedConversion(src, dst, src_dtype, dst_dtype, stream)


class StampedConversion:
    """A cast bound to its tensors, dtypes and stream (the current one when none is given) at construction, for callers
    that repeat it: run() makes one C call and no Python-side checks, which matters when the cast itself takes a few
    microseconds.  The tensors must stay alive and the device current at construction must be current at run()."""

    def __init__(self, src: torch.Tensor, dst: torch.Tensor, src_dtype=None, dst_dtype=None, stream=None):
        if not (src.is_cuda and dst.is_cuda):
            raise _native.ThorB200InvalidArgument("TypeConverter: both tensors must live on a CUDA device (no CPU path in this library)")
        if not (src.is_contiguous() and dst.is_contiguous()):
            raise _native.ThorB200InvalidArgument("TypeConverter: tensors must be contiguous")
        if src.numel() != dst.numel():
            raise _native.ThorB200InvalidArgument("TypeConverter: element counts differ")
        if src.device != dst.device or src.device.index != torch.cuda.current_device():
            raise _native.ThorB200InvalidArgument("TypeConverter.stamp: both tensors must live on the current device")
        self.src, self.dst = src, dst
        self._args = (ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(dst.data_ptr()), int(DataType(src_dtype) if src_dtype is not None else from_torch(src.dtype)),
                      int(DataType(dst_dtype) if dst_dtype is not None else from_torch(dst.dtype)), ctypes.c_int64(src.numel()), _native.stream_handle(stream))
        self._launch = _native.lib.thor_b200_cast_launch

    def run(self) -> torch.Tensor:
        status = self._launch(*self._args)
        if status:
            _native.check(status)
        return self.dst


def tensor_copy_from(dst: torch.Tensor, src: torch.Tensor, dst_dtype: DataType | None = None, src_dtype: DataType | None = None, stream=None) -> torch.Tensor:
    """Tensor::copyFromAsync of the reference (Tensor.cpp:700-860) through the host layer: `dst` and `src` hold the same
    number of elements; either may be a pinned host tensor.  A dtype change across placements copies in the source dtype
    and converts in place on the destination GPU (refused when the destination dtype is the smaller one, like the
    reference; conversions into host memory are refused because this library has no CPU path).  Pass dtypes explicitly for
    raw storage (a bf16 tensor whose first half holds fp8 bytes and the like)."""
    import ctypes as C

    from .expression import _Binding, _check, _host

    def bind(t, dt):
        b = _Binding()
        b.name = b"t"
        b.ptr = t.data_ptr()
        b.dtype = int(dt if dt is not None else from_torch(t.dtype))
        b.rank = 1
        b.dims[0] = t.numel()
        b.is_scalar = 0
        return b

    if not (dst.is_contiguous() and src.is_contiguous()):
        raise _native.ThorB200InvalidArgument("tensor_copy_from: tensors must be contiguous")
    device = lambda t: t.device.index if t.is_cuda else -1
    d, s = bind(dst, dst_dtype), bind(src, src_dtype)
    on = dst.device if dst.is_cuda else src.device
    with torch.cuda.device(on):
        _check(_host.thb_tensor_copy_from(C.byref(d), device(dst), C.byref(s), device(src), _native.stream_handle(stream)))
    return dst
