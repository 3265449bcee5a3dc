"""Runs kernels that the REFERENCE's own emitter generated (oracle/_ref/libthor_ref_emit.so) on the GPU:
NVRTC with the reference's flags (-fmad=true; --std=c++20 because NVRTC 12.9 knows no c++23; compiled straight to
sm_100a instead of LTO-IR + link, EquationCompiler.cpp:1864-1908) and the reference's launch geometry
(grid = ceil(numel / elements_per_thread / 256) x 256 threads, EquationRunner.cpp:274-289).
TEST AND BASELINE INFRASTRUCTURE ONLY: imported by the tests and by the benchmark's reference-GPU baseline leg, never by the product."""
from __future__ import annotations

import ctypes
import os
import re
from typing import Dict, Union

import numpy as np
import torch

from . import reference_emit_broadcast, reference_emit_flat

_cache: dict = {}


def _cuda_include() -> str:
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and os.path.exists(os.path.join(root, "include", "cuda_fp16.h")):
            return os.path.join(root, "include")
    raise RuntimeError("CUDA headers not found")


def _check(res, what):
    err = res[0]
    if int(err) != 0:
        raise RuntimeError(f"{what} failed: {err}")
    return res[1:] if len(res) > 2 else (res[1] if len(res) == 2 else None)


def compile_reference_kernel(source: str):
    from cuda.bindings import driver, nvrtc

    if source in _cache:
        return _cache[source]
    torch.cuda.init()
    torch.zeros(1, device="cuda")  # primary context current
    prog = _check(nvrtc.nvrtcCreateProgram(source.encode(), b"fused.cu", 0, [], []), "nvrtcCreateProgram")
    opts = [b"--gpu-architecture=sm_100a", b"--std=c++20", b"-fmad=true", ("--include-path=" + _cuda_include()).encode()]
    res = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    if int(res[0]) != 0:
        size = _check(nvrtc.nvrtcGetProgramLogSize(prog), "log size")
        log = b" " * size
        nvrtc.nvrtcGetProgramLog(prog, log)
        raise RuntimeError("NVRTC rejected the reference-emitted kernel:\n" + log.decode(errors="replace"))
    size = _check(nvrtc.nvrtcGetCUBINSize(prog), "cubin size")
    cubin = b" " * size
    _check(nvrtc.nvrtcGetCUBIN(prog, cubin), "cubin")
    module = _check(driver.cuModuleLoadData(np.frombuffer(cubin, dtype=np.uint8).ctypes.data), "cuModuleLoadData")
    func = _check(driver.cuModuleGetFunction(module, b"fused_kernel"), "cuModuleGetFunction")
    m = re.search(r"void\s+fused_kernel\s*\(([^)]*)\)", source)
    params = [p.strip() for p in m.group(1).split(",")]
    _cache[source] = (func, params, module, cubin)
    return _cache[source]


def _launch(source, ept, order, out, inputs, numel, stream=None):
    from cuda.bindings import driver

    func, params, _, _ = compile_reference_kernel(source)
    holders = []
    for i, p in enumerate(params):
        if i < len(order):
            v = inputs[order[i]]
            if "*" in p:
                assert isinstance(v, torch.Tensor)
                holders.append(ctypes.c_void_p(v.data_ptr()))
            else:
                assert p.startswith("float"), p
                holders.append(ctypes.c_float(float(v)))
        elif "*" in p:
            holders.append(ctypes.c_void_p(out.data_ptr()))
        elif "long long" in p:
            holders.append(ctypes.c_ulonglong(numel))
        else:
            holders.append(ctypes.c_uint(numel))
    argv = (ctypes.c_void_p * len(holders))(*[ctypes.cast(ctypes.pointer(h), ctypes.c_void_p) for h in holders])
    launch_numel = -(-numel // ept)
    block = min(launch_numel, 256)
    grid = max(1, -(-launch_numel // block))
    st = stream if stream is not None else torch.cuda.current_stream().cuda_stream
    _check(driver.cuLaunchKernel(func, grid, 1, 1, block, 1, 1, 0, st, ctypes.addressof(argv), 0), "cuLaunchKernel")
    return holders, argv


class ReferenceBroadcastKernel:
    """The reference's specialized-broadcast kernel for `program` and concrete dense shapes, ready to launch repeatedly."""

    def __init__(self, program: str, input_dtypes: Dict[str, int], input_dims: Dict[str, tuple]):
        from thor_b200.dtypes import DataType, to_torch

        self.source, self.ept, self.order, self.out_dtype, self.numel = reference_emit_broadcast(program, input_dtypes, input_dims)
        self.torch_out_dtype = to_torch(DataType(self.out_dtype))
        compile_reference_kernel(self.source)

    def launch(self, inputs: Dict[str, Union[torch.Tensor, float]], out: torch.Tensor, stream=None) -> None:
        _launch(self.source, self.ept, self.order, out, inputs, self.numel, stream)


class ReferenceFlatKernel:
    """The reference's flat (same-shape) fused kernel for `program`, ready to launch repeatedly on caller-provided buffers;
    every tensor must hold numel + 64 elements (the reference's kernels read whole packs and rely on padded tensors)."""

    def __init__(self, program: str, input_dtypes: Dict[str, int], numel: int):
        from thor_b200.dtypes import DataType, to_torch

        self.source, self.ept, self.order, self.out_dtype = reference_emit_flat(program, input_dtypes)
        self.torch_out_dtype = to_torch(DataType(self.out_dtype))
        self.numel = numel
        compile_reference_kernel(self.source)

    def launch(self, inputs: Dict[str, Union[torch.Tensor, float]], out: torch.Tensor, stream=None) -> None:
        _launch(self.source, self.ept, self.order, out, inputs, self.numel, stream)


def run_reference_flat(program: str, inputs: Dict[str, Union[torch.Tensor, float]], input_dtypes: Dict[str, int], numel: int, pad: int = 64):
    """Emits, compiles and launches the reference's flat kernel for `program`; tensors must hold numel + pad elements
    (the reference's kernels read whole packs and rely on padded tensors).  Returns (output tensor incl. padding, output dtype)."""
    from cuda.bindings import driver

    from thor_b200.dtypes import DataType, to_torch

    source, ept, order, out_dtype = reference_emit_flat(program, input_dtypes)
    func, params, _, _ = compile_reference_kernel(source)
    out = torch.zeros(numel + pad, dtype=to_torch(DataType(out_dtype)), device="cuda")
    holders = []
    for i, p in enumerate(params):
        if i < len(order):
            v = inputs[order[i]]
            if "*" in p:
                assert isinstance(v, torch.Tensor) and v.numel() >= numel + pad, f"input '{order[i]}' needs numel + pad elements"
                holders.append(ctypes.c_void_p(v.data_ptr()))
            else:
                assert p.startswith("float"), p
                holders.append(ctypes.c_float(float(v)))
        elif "*" in p:
            holders.append(ctypes.c_void_p(out.data_ptr()))
        elif "long long" in p:
            holders.append(ctypes.c_ulonglong(numel))
        else:
            holders.append(ctypes.c_uint(numel))
    argv = (ctypes.c_void_p * len(holders))(*[ctypes.cast(ctypes.pointer(h), ctypes.c_void_p) for h in holders])
    grid = max(1, -(-numel // (ept * 256)))
    stream = torch.cuda.current_stream().cuda_stream
    _check(driver.cuLaunchKernel(func, grid, 1, 1, 256, 1, 1, 0, stream, ctypes.addressof(argv), 0), "cuLaunchKernel")
    return out, out_dtype
