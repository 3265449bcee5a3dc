"""In-tree build of the native libraries (no cmake, no JIT cache).

``python -m thor_b200.build`` compiles every ``csrc/*.cu`` for sm_100a with nvcc and links
``thor_b200/lib/libthor_b200.so`` (the C ABI declared in ``include/thor_b200.h``), then compiles
the C++ host layer in ``thor_b200/host`` into ``thor_b200/lib/libthor_b200_host.so``, which talks to
the first library only through that C ABI.  Objects are rebuilt when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
HOST = PKG / "host"
LIB = PKG / "lib"
OBJ = CSRC / "_build"
INCLUDE = ROOT / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "-DTHOR_B200_BUILD",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libthor_b200 cannot be built")
    return exe


def _newest_header() -> float:
    stamps = [p.stat().st_mtime for p in list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))]
    return max(stamps) if stamps else 0.0


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))
    if os.environ.get("THOR_B200_BUILD_VERBOSE") and (proc.stdout or proc.stderr):
        sys.stderr.write(proc.stdout + proc.stderr)


def build_kernels(force: bool = False, extra_flags: list[str] | None = None) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB.mkdir(parents=True, exist_ok=True)
    hdr = _newest_header()
    sources = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr):
            cmd = [_nvcc(), *NVCC_FLAGS, *(extra_flags or []), "-I", str(INCLUDE), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            if src.suffix == ".cpp":
                cmd.insert(1, "-x")
                cmd.insert(2, "cu")
            jobs.append(cmd)
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        list(pool.map(_run, jobs))
    out = LIB / "libthor_b200.so"
    if jobs or not out.exists():
        # cudart is linked statically; libcuda / libnvrtc are dlopen'ed at first use so that the
        # library loads (and exports its symbols) on a machine without a driver.
        _run([_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-cudart", "static", "-ldl", "-lpthread"])
    return out


def build_host(force: bool = False) -> Path | None:
    sources = sorted(HOST.glob("*.cpp"))
    if not sources:
        return None
    out = LIB / "libthor_b200_host.so"
    newest = max(p.stat().st_mtime for p in sources + list(HOST.glob("*.h")) + list(INCLUDE.glob("*.h")))
    if force or not out.exists() or out.stat().st_mtime < newest:
        cxx = shutil.which("g++") or "g++"
        _run([cxx, "-O2", "-std=c++20", "-fPIC", "-shared", "-fvisibility=hidden", "-I", str(INCLUDE), "-I", str(HOST),
              *map(str, sources), "-o", str(out), "-L", str(LIB), "-lthor_b200", "-Wl,-rpath,$ORIGIN", "-ldl", "-lpthread"])
    return out


def build_all(force: bool = False) -> None:
    build_kernels(force)
    build_host(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built:", *(str(p) for p in sorted(LIB.glob("*.so"))))
