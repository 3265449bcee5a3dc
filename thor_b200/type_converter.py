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
