"""DataType tokens with the reference's integer values (DeepLearning/Implementation/Tensor/DataType.h:7-26)."""
from __future__ import annotations

import enum

import torch


class DataType(enum.IntEnum):
    fp16 = 10
    fp32 = 11
    fp64 = 12
    int8 = 13
    int16 = 14
    int32 = 15
    int64 = 16
    uint8 = 17
    uint16 = 18
    uint32 = 19
    uint64 = 20
    boolean = 21
    fp8_e4m3 = 22
    fp8_e5m2 = 23
    bf16 = 24


_TORCH = {
    DataType.fp16: torch.float16, DataType.fp32: torch.float32, DataType.fp64: torch.float64, DataType.int8: torch.int8,
    DataType.int16: torch.int16, DataType.int32: torch.int32, DataType.int64: torch.int64, DataType.uint8: torch.uint8,
    DataType.uint16: torch.uint16, DataType.uint32: torch.uint32, DataType.uint64: torch.uint64, DataType.boolean: torch.bool,
    DataType.fp8_e4m3: torch.float8_e4m3fn, DataType.fp8_e5m2: torch.float8_e5m2, DataType.bf16: torch.bfloat16,
}
_FROM_TORCH = {v: k for k, v in _TORCH.items()}

SIZE = {DataType.fp16: 2, DataType.bf16: 2, DataType.int16: 2, DataType.uint16: 2, DataType.fp32: 4, DataType.int32: 4, DataType.uint32: 4,
        DataType.fp64: 8, DataType.int64: 8, DataType.uint64: 8, DataType.int8: 1, DataType.uint8: 1, DataType.boolean: 1,
        DataType.fp8_e4m3: 1, DataType.fp8_e5m2: 1}


def to_torch(dtype: DataType) -> torch.dtype:
    return _TORCH[DataType(dtype)]


def from_torch(dtype: torch.dtype) -> DataType:
    return _FROM_TORCH[dtype]
