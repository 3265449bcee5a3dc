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


_ref_gpu = None


def reference_gpu_cast_lib():
    """The reference's own GPU cast kernels (TypeConverter::gpuConvertType), or None when oracle/_ref holds no build of them."""
    global _ref_gpu
    if _ref_gpu is None:
        path = HERE / "_ref" / "libthor_ref_gpu_cast.so"
        if not path.exists():
            return None
        _ref_gpu = ctypes.CDLL(str(path))
        _ref_gpu.thor_ref_gpu_convert.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_long, ctypes.c_void_p]
        _ref_gpu.thor_ref_gpu_convert.restype = ctypes.c_int
    return _ref_gpu


def reference_gpu_cast(src_ptr: int, dst_ptr: int, src_dtype: int, dst_dtype: int, n: int, stream: int = 0) -> None:
    """Launches the reference's GPU conversion of n elements between two device buffers (asynchronous on `stream`).
    The reference's kernels may read up to 7 elements past n (they rely on padded tensors): give it padded buffers."""
    ref = reference_gpu_cast_lib()
    assert ref is not None, "oracle/_ref/libthor_ref_gpu_cast.so has not been built"
    rc = ref.thor_ref_gpu_convert(ctypes.c_void_p(src_ptr), ctypes.c_void_p(dst_ptr), src_dtype, dst_dtype, n, ctypes.c_void_p(stream))
    assert rc == 0, f"reference GPU conversion failed ({rc})"


_ref_cub = None


def reference_cub_reduce_lib():
    """The reference's own value reductions (its fp32 operators, CUB calls and tiled kernels), or None when oracle/_ref
    holds no build of them."""
    global _ref_cub
    if _ref_cub is None:
        path = HERE / "_ref" / "libthor_ref_cub_reduce.so"
        if not path.exists():
            return None
        _ref_cub = ctypes.CDLL(str(path))
        c = ctypes
        _ref_cub.thor_ref_cub_reduce.argtypes = [c.c_int, c.c_int, c.c_void_p, c.c_int, c.c_void_p, c.c_int, c.c_ulonglong, c.c_ulonglong, c.c_ulonglong, c.c_void_p,
                                                 c.POINTER(c.c_size_t), c.c_void_p]
        _ref_cub.thor_ref_cub_reduce.restype = c.c_int
        if hasattr(_ref_cub, "thor_ref_cub_argreduce"):
            _ref_cub.thor_ref_cub_argreduce.argtypes = [c.c_int, c.c_int, c.c_void_p, c.c_int, c.c_void_p, c.c_int, c.c_void_p, c.c_int, c.c_ulonglong, c.c_ulonglong,
                                                        c.c_ulonglong, c.c_void_p, c.POINTER(c.c_size_t), c.c_void_p]
            _ref_cub.thor_ref_cub_argreduce.restype = c.c_int
    return _ref_cub


REF_REDUCE_OPS = {"sum": 0, "mean": 1, "max": 2, "min": 3}


def reference_cub_reduce_workspace(op: str, input_dtype: int, output_dtype: int, outer: int, reduction: int, inner: int) -> tuple[int, int]:
    """(path, workspace bytes) of the reference's reduction of a dense [outer, reduction, inner] input over the middle
    axis.  The path follows its geometry analysis (CubReduction.cpp:755-912): one output -> DeviceTransformReduce (0),
    inner == 1 -> ContiguousFixedSegment (1), otherwise TiledFixedSegment (2)."""
    ref = reference_cub_reduce_lib()
    assert ref is not None, "oracle/_ref/libthor_ref_cub_reduce.so has not been built"
    path = 0 if outer * inner == 1 else (1 if inner == 1 else 2)
    size = ctypes.c_size_t(0)
    rc = ref.thor_ref_cub_reduce(REF_REDUCE_OPS[op], path, None, input_dtype, None, output_dtype, outer, reduction, inner, None, ctypes.byref(size), None)
    assert rc == 0, f"reference reduction workspace query failed ({rc})"
    return path, int(size.value)


def reference_cub_reduce(op: str, path: int, in_ptr: int, input_dtype: int, out_ptr: int, output_dtype: int, outer: int, reduction: int, inner: int, temp_ptr: int,
                         temp_bytes: int, stream: int = 0) -> None:
    """Launches the reference's reduction on device buffers (asynchronous on `stream`); workspace from reference_cub_reduce_workspace."""
    ref = reference_cub_reduce_lib()
    assert ref is not None, "oracle/_ref/libthor_ref_cub_reduce.so has not been built"
    size = ctypes.c_size_t(temp_bytes)
    rc = ref.thor_ref_cub_reduce(REF_REDUCE_OPS[op], path, ctypes.c_void_p(in_ptr), input_dtype, ctypes.c_void_p(out_ptr), output_dtype, outer, reduction, inner,
                                 ctypes.c_void_p(temp_ptr), ctypes.byref(size), ctypes.c_void_p(stream))
    assert rc == 0, f"reference reduction failed ({rc})"


def reference_cub_argreduce_workspace(is_max: bool, input_dtype: int, outer: int, reduction: int, inner: int, index_dtype: int) -> tuple[int, int]:
    """(path, workspace bytes) of the reference's arg reduction of a dense [outer, reduction, inner] input over the middle axis."""
    ref = reference_cub_reduce_lib()
    assert ref is not None and hasattr(ref, "thor_ref_cub_argreduce"), "oracle/_ref holds no build of the reference's arg reductions"
    path = 0 if outer * inner == 1 else (1 if inner == 1 else 2)
    size = ctypes.c_size_t(0)
    rc = ref.thor_ref_cub_argreduce(int(is_max), path, None, input_dtype, None, FP32, None, index_dtype, outer, reduction, inner, None, ctypes.byref(size), None)
    assert rc == 0, f"reference arg reduction workspace query failed ({rc})"
    return path, int(size.value)


def reference_cub_argreduce(is_max: bool, path: int, in_ptr: int, input_dtype: int, value_ptr: int, value_dtype: int, index_ptr: int, index_dtype: int, outer: int,
                            reduction: int, inner: int, temp_ptr: int, temp_bytes: int, stream: int = 0) -> None:
    """Launches the reference's arg reduction on device buffers (value_ptr or index_ptr may be 0)."""
    ref = reference_cub_reduce_lib()
    assert ref is not None and hasattr(ref, "thor_ref_cub_argreduce"), "oracle/_ref holds no build of the reference's arg reductions"
    size = ctypes.c_size_t(temp_bytes)
    rc = ref.thor_ref_cub_argreduce(int(is_max), path, ctypes.c_void_p(in_ptr), input_dtype, ctypes.c_void_p(value_ptr or None), value_dtype,
                                    ctypes.c_void_p(index_ptr or None), index_dtype, outer, reduction, inner, ctypes.c_void_p(temp_ptr), ctypes.byref(size),
                                    ctypes.c_void_p(stream))
    assert rc == 0, f"reference arg reduction failed ({rc})"


_ref_emit = None


def reference_emitter_lib():
    """The reference's own flat fused-kernel emitter behind a dumper, or None when oracle/_ref holds no build of it."""
    global _ref_emit
    if _ref_emit is None:
        path = HERE / "_ref" / "libthor_ref_emit.so"
        if not path.exists():
            return None
        _ref_emit = ctypes.CDLL(str(path))
        c = ctypes
        _ref_emit.thor_ref_emit_flat.argtypes = [c.c_char_p, c.POINTER(c.c_char_p), c.POINTER(c.c_int), c.c_int, c.POINTER(c.c_char_p), c.POINTER(c.c_uint),
                                                 c.POINTER(c.c_int), c.POINTER(c.c_int)]
        _ref_emit.thor_ref_emit_flat.restype = c.c_int
        _ref_emit.thor_ref_emit_broadcast.argtypes = [c.c_char_p, c.POINTER(c.c_char_p), c.POINTER(c.c_int), c.POINTER(c.c_ulonglong), c.c_int, c.POINTER(c.c_char_p),
                                                      c.POINTER(c.c_uint), c.POINTER(c.c_int), c.POINTER(c.c_int), c.POINTER(c.c_ulonglong)]
        _ref_emit.thor_ref_emit_broadcast.restype = c.c_int
    return _ref_emit


def reference_resolve_dtypes(program: str, input_dtypes: dict):
    """(op, output dtype, compute dtype) of every node after the reference's resolveOutputsDTypesInPlace, in its node order."""
    lib_ = reference_emitter_lib()
    assert lib_ is not None, "oracle/_ref/libthor_ref_emit.so has not been built"
    c = ctypes
    lib_.thor_ref_resolve_dtypes.argtypes = [c.c_char_p, c.POINTER(c.c_char_p), c.POINTER(c.c_int), c.c_int, c.POINTER(c.c_int), c.c_int]
    lib_.thor_ref_resolve_dtypes.restype = c.c_int
    names = list(input_dtypes.keys())
    arr_n = (c.c_char_p * len(names))(*[n.encode() for n in names])
    arr_d = (c.c_int * len(names))(*[int(input_dtypes[n]) for n in names])
    cap = 1024
    buf = (c.c_int * (3 * cap))()
    n = lib_.thor_ref_resolve_dtypes(program.encode(), arr_n, arr_d, len(names), buf, cap)
    if n < 0:
        raise RuntimeError("reference dtype resolution failed")
    return [(buf[3 * k], buf[3 * k + 1], buf[3 * k + 2]) for k in range(n)]


def reference_emit_broadcast(program: str, input_dtypes: dict, input_dims: dict):
    """CUDA source that the reference's CudaSourceEmitter::emitSpecializedBroadcast generates for `program` with
    concrete dense input shapes (`input_dims[name]`, () for runtime scalars).  Returns
    (source, elements_per_thread, input names in kernel-parameter order, output dtype, output numel)."""
    lib_ = reference_emitter_lib()
    assert lib_ is not None, "oracle/_ref/libthor_ref_emit.so has not been built"
    names = list(input_dtypes.keys())
    c = ctypes
    arr_n = (c.c_char_p * len(names))(*[n.encode() for n in names])
    arr_d = (c.c_int * len(names))(*[int(input_dtypes[n]) for n in names])
    flat = []
    for n in names:
        dims = tuple(input_dims.get(n, ()))
        flat += [len(dims), *dims]
    arr_dims = (c.c_ulonglong * max(1, len(flat)))(*flat)
    src, ept, out_dt, numel = c.c_char_p(), c.c_uint(), c.c_int(), c.c_ulonglong()
    order = (c.c_int * max(1, len(names)))(*([-1] * max(1, len(names))))
    rc = lib_.thor_ref_emit_broadcast(program.encode(), arr_n, arr_d, arr_dims, len(names), c.byref(src), c.byref(ept), order, c.byref(out_dt), c.byref(numel))
    text = src.value.decode()
    if rc != 0:
        raise RuntimeError("reference emitter: " + text)
    return text, int(ept.value), [names[i] for i in order if i >= 0], int(out_dt.value), int(numel.value)


def reference_emit_flat(program: str, input_dtypes: dict):
    """CUDA source that the reference's CudaSourceEmitter::emitFlat generates for a postfix `program`
    (tokens: in:<name> rs:<name> lit:<value> cast:<dtype> add sub mul div pow min max and the unary op names).
    `input_dtypes` maps every tensor input / fp32 runtime scalar name to its dtype.
    Returns (source, elements_per_thread, input names in kernel-parameter order, output dtype)."""
    lib_ = reference_emitter_lib()
    assert lib_ is not None, "oracle/_ref/libthor_ref_emit.so has not been built"
    names = list(input_dtypes.keys())
    c = ctypes
    arr_n = (c.c_char_p * len(names))(*[n.encode() for n in names])
    arr_d = (c.c_int * len(names))(*[int(input_dtypes[n]) for n in names])
    src, ept, out_dt = c.c_char_p(), c.c_uint(), c.c_int()
    order = (c.c_int * max(1, len(names)))(*([-1] * max(1, len(names))))
    rc = lib_.thor_ref_emit_flat(program.encode(), arr_n, arr_d, len(names), c.byref(src), c.byref(ept), order, c.byref(out_dt))
    text = src.value.decode()
    if rc != 0:
        raise RuntimeError("reference emitter: " + text)
    return text, int(ept.value), [names[i] for i in order if i >= 0], int(out_dt.value)


_ref_autodiff = None


def reference_autodiff_lib():
    """The reference's own reverse-mode differentiation behind a graph dumper, or None when oracle/_ref holds no build of it."""
    global _ref_autodiff
    if _ref_autodiff is None:
        path = HERE / "_ref" / "libthor_ref_autodiff.so"
        if not path.exists():
            return None
        _ref_autodiff = ctypes.CDLL(str(path))
        c = ctypes
        _ref_autodiff.thor_ref_backward_graph.argtypes = [c.c_char_p, c.POINTER(c.c_char_p), c.POINTER(c.c_int), c.POINTER(c.c_ulonglong), c.c_int,
                                                          c.POINTER(c.c_char_p), c.c_int, c.c_int, c.POINTER(c.c_char_p)]
        _ref_autodiff.thor_ref_backward_graph.restype = c.c_int
    return _ref_autodiff


def reference_backward_graph(program: str, inputs: dict, wrt, upstream_dtype: int) -> dict:
    """The dtype-resolved backward graph that the reference's buildBackwardOutputs (AutoDiff.cpp:6210) produces for the
    forward `program` (postfix, ref_postfix.h) with `inputs` = {name: (dims, dtype)}: {"inputs", "outputs", "nodes"}."""
    import json

    lib_ = reference_autodiff_lib()
    assert lib_ is not None, "oracle/_ref/libthor_ref_autodiff.so has not been built"
    c = ctypes
    names = list(inputs)
    flat = []
    for n in names:
        dims = inputs[n][0]
        flat += [len(dims), *dims]
    text = c.c_char_p()
    rc = lib_.thor_ref_backward_graph(program.encode(), (c.c_char_p * len(names))(*[n.encode() for n in names]),
                                      (c.c_int * len(names))(*[int(inputs[n][1]) for n in names]), (c.c_ulonglong * max(1, len(flat)))(*flat), len(names),
                                      (c.c_char_p * len(wrt))(*[w.encode() for w in wrt]), len(wrt), int(upstream_dtype), c.byref(text))
    if rc != 0:
        raise RuntimeError("reference buildBackwardOutputs: " + text.value.decode())
    return json.loads(text.value.decode())


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


# ---- workload-sized loops of thor_oracle.c --------------------------------------------------------
def _setup_workloads():
    L = lib()
    if getattr(L, "_workloads_ready", False):
        return L
    c = ctypes
    L.tor_c2_fused.argtypes = [c.c_void_p, c.c_void_p, c.c_float, c.c_void_p, c.c_void_p, c.c_int64, c.c_int64, c.c_int, c.c_int]
    L.tor_c2_fused.restype = None
    L.tor_softmax_rows_f32.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int64, c.c_int64, c.c_int]
    L.tor_softmax_rows_f32.restype = None
    L.tor_c4_stats_bf16.argtypes = [c.c_void_p, c.c_int64, c.POINTER(c.c_double), c.POINTER(c.c_double), c.POINTER(c.c_float), c.c_int]
    L.tor_c4_stats_bf16.restype = None
    L.tor_layernorm_fwd_bf16.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_float, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int64, c.c_int64, c.c_int]
    L.tor_layernorm_fwd_bf16.restype = None
    L.tor_layernorm_bwd_bf16.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_float, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int64, c.c_int64, c.c_int]
    L.tor_layernorm_bwd_bf16.restype = None
    L._workloads_ready = True
    return L


def host_threads() -> int:
    import os

    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def c2_fused(a: np.ndarray, x: np.ndarray, b: float, z: np.ndarray, fuse_mul_add: bool = False, threads: int = 0) -> np.ndarray:
    """relu(a*x + b) * sigmoid(z), every node fp16; arrays are np.float16 ([cols], [rows, cols], [rows, cols])."""
    L = _setup_workloads()
    rows, cols = x.shape
    a, x, z = (np.ascontiguousarray(v, dtype=np.float16) for v in (a, x, z))
    y = np.empty((rows, cols), np.float16)
    L.tor_c2_fused(_ptr(a), _ptr(x), float(b), _ptr(z), _ptr(y), rows, cols, int(fuse_mul_add), threads or host_threads())
    return y


def softmax_rows(x: np.ndarray, want_softmax: bool = True, want_argmax: bool = True, threads: int = 0):
    L = _setup_workloads()
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    y = np.empty_like(x) if want_softmax else None
    idx = np.empty(rows, np.uint32) if want_argmax else None
    L.tor_softmax_rows_f32(_ptr(x), _ptr(y) if y is not None else None, _ptr(idx) if idx is not None else None, rows, cols, threads or host_threads())
    return y, idx


def c4_stats(x_bf16: np.ndarray, threads: int = 0):
    """(sum, sum of bf16-rounded squares, max) of a bf16 vector given as uint16 storage; fp64 accumulation."""
    L = _setup_workloads()
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    s, q, m = ctypes.c_double(), ctypes.c_double(), ctypes.c_float()
    L.tor_c4_stats_bf16(_ptr(x), x.size, ctypes.byref(s), ctypes.byref(q), ctypes.byref(m), threads or host_threads())
    return s.value, q.value, m.value


def layernorm_fwd(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray, eps: float = 1e-5, threads: int = 0):
    """bf16 storage (uint16) in, bf16 y out plus fp32 mean / rstd per row."""
    L = _setup_workloads()
    rows, cols = x.shape
    y = np.empty((rows, cols), np.uint16)
    mean, rstd = np.empty(rows, np.float32), np.empty(rows, np.float32)
    L.tor_layernorm_fwd_bf16(_ptr(np.ascontiguousarray(x)), _ptr(np.ascontiguousarray(gamma)), _ptr(np.ascontiguousarray(beta)), eps, _ptr(y), _ptr(mean),
                             _ptr(rstd), rows, cols, threads or host_threads())
    return y, mean, rstd


def layernorm_bwd(x: np.ndarray, gamma: np.ndarray, dy: np.ndarray, eps: float = 1e-5, threads: int = 0):
    """bf16 storage in; returns dx (bf16 storage), dgamma, dbeta (float64)."""
    L = _setup_workloads()
    rows, cols = x.shape
    dx = np.empty((rows, cols), np.uint16)
    dg, db = np.empty(cols, np.float64), np.empty(cols, np.float64)
    L.tor_layernorm_bwd_bf16(_ptr(np.ascontiguousarray(x)), _ptr(np.ascontiguousarray(gamma)), _ptr(np.ascontiguousarray(dy)), eps, _ptr(dx), _ptr(dg),
                             _ptr(db), rows, cols, threads or host_threads())
    return dx, dg, db
