"""CPU checkers for the hot path — TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import this
package.  The product (``thor_b200``) never does: it fails loudly when its CUDA library is missing
instead of falling back to anything here.

Contents:
* ``thor_oracle.c``  — plain-C restatement (casts, reductions, fused row ops), loaded via ctypes.
* ``expr_oracle.py`` — numpy interpreter for expression DAGs with the reference's per-node dtypes.
* ``_ref/``          — the reference's own CPU cast path compiled from its checkout (optional).
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

# ThorImplementation::DataType integers (DeepLearning/Implementation/Tensor/DataType.h:7-26).
FP16, FP32, FP64, INT8, INT16, INT32, INT64, UINT8, UINT16, UINT32, UINT64, BOOLEAN, FP8_E4M3, FP8_E5M2, BF16 = range(10, 25)

ALL_DTYPES = [FP16, FP32, FP64, INT8, INT16, INT32, INT64, UINT8, UINT16, UINT32, UINT64, BOOLEAN, FP8_E4M3, FP8_E5M2, BF16]
FLOAT_DTYPES = [FP16, BF16, FP32, FP64, FP8_E4M3, FP8_E5M2]
NAMES = {FP16: "fp16", FP32: "fp32", FP64: "fp64", INT8: "int8", INT16: "int16", INT32: "int32", INT64: "int64", UINT8: "uint8",
         UINT16: "uint16", UINT32: "uint32", UINT64: "uint64", BOOLEAN: "boolean", FP8_E4M3: "fp8_e4m3", FP8_E5M2: "fp8_e5m2", BF16: "bf16"}

# Storage arrays: formats numpy lacks (bf16, fp8) are carried as raw unsigned integers.
STORAGE = {FP16: np.float16, FP32: np.float32, FP64: np.float64, INT8: np.int8, INT16: np.int16, INT32: np.int32, INT64: np.int64,
           UINT8: np.uint8, UINT16: np.uint16, UINT32: np.uint32, UINT64: np.uint64, BOOLEAN: np.bool_, FP8_E4M3: np.uint8,
           FP8_E5M2: np.uint8, BF16: np.uint16}


def _load(path: Path) -> ctypes.CDLL:
    if not path.exists():
        from . import build as _build  # compile on first use (gcc is part of the image)
        _build.build_oracle()
    return ctypes.CDLL(str(path))


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = _load(HERE / "_build" / "libthor_oracle.so")
        _lib.tor_cast.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int64]
        _lib.tor_cast.restype = ctypes.c_int
        _lib.tor_cast_f32_f16.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        _lib.tor_cast_f32_f16.restype = None
        for name in ("tor_round_f32_to_f16_array", "tor_round_f32_to_bf16_array"):
            getattr(_lib, name).argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
            getattr(_lib, name).restype = None
    return _lib


_ref = None


def reference_cast_lib():
    """The reference's own cpuConvertTypeImpl, or None when oracle/_ref was not built."""
    global _ref
    if _ref is None:
        path = HERE / "_ref" / "libthor_ref_cast.so"
        if not path.exists():
            return None
        _ref = ctypes.CDLL(str(path))
        _ref.thor_ref_cpu_convert.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_long]
        _ref.thor_ref_cpu_convert.restype = ctypes.c_int
        _ref.thor_ref_omp_threads_for.argtypes = [ctypes.c_long]
        _ref.thor_ref_omp_threads_for.restype = ctypes.c_int
    return _ref


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def cast(src: np.ndarray, src_dtype: int, dst_dtype: int) -> np.ndarray:
    """Restated cast of a storage array (see STORAGE) to the storage array of dst_dtype."""
    src = np.ascontiguousarray(src)
    assert src.dtype == STORAGE[src_dtype], (src.dtype, NAMES[src_dtype])
    dst = np.empty(src.shape, dtype=STORAGE[dst_dtype])
    rc = lib().tor_cast(_ptr(src), _ptr(dst), src_dtype, dst_dtype, src.size)
    assert rc == 0
    return dst


def reference_cast(src: np.ndarray, src_dtype: int, dst_dtype: int) -> np.ndarray:
    """Same cast through the reference's own CPU code (requires oracle/_ref)."""
    ref = reference_cast_lib()
    assert ref is not None, "oracle/_ref/libthor_ref_cast.so has not been built"
    src = np.ascontiguousarray(src)
    dst = np.empty(src.shape, dtype=STORAGE[dst_dtype])
    rc = ref.thor_ref_cpu_convert(_ptr(src), _ptr(dst), src_dtype, dst_dtype, src.size)
    assert rc == 0
    return dst


def to_float64(a: np.ndarray, dtype: int) -> np.ndarray:
    """Decode any storage array to float64 values (exact for every supported dtype but 64-bit ints)."""
    if dtype in (BF16, FP8_E4M3, FP8_E5M2):
        return cast(a, dtype, FP64)
    return np.asarray(a).astype(np.float64)


def from_float32(a: np.ndarray, dtype: int) -> np.ndarray:
    """Encode float32 values into the storage array of dtype with one RNE rounding."""
    return cast(np.ascontiguousarray(a, dtype=np.float32), FP32, dtype) if dtype != FP32 else np.ascontiguousarray(a, dtype=np.float32)
