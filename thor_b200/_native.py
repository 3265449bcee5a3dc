"""ctypes loader for libthor_b200.so.  Import fails loudly when the library has not been built."""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "lib"
LIB_PATH = LIB_DIR / "libthor_b200.so"


class ThorB200Error(RuntimeError):
    """CUDA / JIT failure below the C ABI (the reference throws std::runtime_error here)."""


class ThorB200InvalidArgument(ValueError):
    """Contract violation by the caller (the reference throws std::logic_error here)."""


if not LIB_PATH.exists():
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m thor_b200.build` (needs nvcc). "
        "thor_b200 has no CPU or PyTorch fallback."
    )

lib = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_GLOBAL)

_c = ctypes
lib.thor_b200_abi_version.restype = _c.c_int
lib.thor_b200_last_error.restype = _c.c_char_p
lib.thor_b200_dtype_size.argtypes = [_c.c_int]
lib.thor_b200_dtype_size.restype = _c.c_size_t
lib.thor_b200_launch_count.restype = _c.c_uint64
lib.thor_b200_cast_launch.argtypes = [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int64, _c.c_void_p]
lib.thor_b200_cast_launch.restype = _c.c_int


def check(status: int) -> None:
    if status == 0:
        return
    msg = lib.thor_b200_last_error().decode("utf-8", "replace")
    if status in (1, 4):
        raise ThorB200InvalidArgument(msg)
    raise ThorB200Error(msg)


def launch_count() -> int:
    """Kernels launched by libthor_b200 in this process so far."""
    return int(lib.thor_b200_launch_count())


def stream_handle(stream=None) -> ctypes.c_void_p:
    """cudaStream_t of a torch stream (current stream when None)."""
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)
