"""Builds the CPU checkers (test infrastructure, never the product).

* ``_build/libthor_oracle.so``  — the plain-C restatement in ``thor_oracle.c`` (gcc, OpenMP).
* ``_ref/libthor_ref_cast.so``   — the REFERENCE's own CPU cast path, compiled from the reference
  checkout where it lies (only when that checkout is present; the output is git-ignored and is
  carried to the GPU machine as a built file).  Nothing is copied out of the reference tree.
* ``_ref/libthor_ref_emit.so``  — the REFERENCE's own expression builder, dtype resolution and CUDA source emitter
  (three host sources, g++) behind a dumper: the tests compile the kernels it emits with NVRTC and run them
  beside ours on the same buffers.
* ``_ref/libthor_ref_gpu_cast.so`` — the REFERENCE's own GPU cast kernels (TypeConverterKernels.cu,
  nvcc for sm_100a, about 90 s), same rules; the parity tests compare against it bit for bit and the
  benchmark times it beside our kernel.

* ``_ref/libthor_ref_autodiff.so`` — the REFERENCE's own reverse-mode differentiation (AutoDiff.cpp) behind a graph
  dumper: the tests compare the host layer's backward graphs with it and use its graphs as a second gradient oracle.

Run as ``python oracle/build.py``.  The reference checkout is looked up in ``$THOR_REFERENCE_DIR``, else in a folder
named ``reference`` beside this repository.
"""
from __future__ import annotations

import os
import shutil
import site
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
BUILD = HERE / "_build"
REF_OUT = HERE / "_ref"
def _reference_dir() -> Path:
    """The reference checkout: $THOR_REFERENCE_DIR, else a folder named `reference` beside this repository.  When neither
    exists the _ref libraries are simply not (re)built and prebuilt ones are used as they are."""
    env = os.environ.get("THOR_REFERENCE_DIR")
    return Path(env) if env else HERE.parent.parent / "reference"


REFERENCE_DIR = _reference_dir()
CUDA_INCLUDE = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), proc.stdout, proc.stderr))


def _stale(out: Path, deps: list[Path]) -> bool:
    return not out.exists() or out.stat().st_mtime < max(p.stat().st_mtime for p in deps)


def build_oracle(force: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    out = BUILD / "libthor_oracle.so"
    srcs = sorted(HERE.glob("*.c"))
    if force or _stale(out, srcs):
        _run(["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-fvisibility=hidden", "-ffp-contract=off",
              *map(str, srcs), "-o", str(out), "-lm"])
    return out


def _site_include_dirs() -> list[Path]:
    dirs = []
    for sp in site.getsitepackages() + [sysconfig.get_paths()["purelib"]]:
        base = Path(sp)
        for rel in ("include/cudnn_frontend/thirdparty", "include", "nvidia/cudnn/include", "nvidia/cublas/include"):
            if (base / rel).is_dir():
                dirs.append(base / rel)
    return dirs


def build_reference_cast(force: bool = False) -> Path | None:
    """Compile the reference's CPU TypeConverter into _ref/; returns None when it cannot be built here."""
    out = REF_OUT / "libthor_ref_cast.so"
    src = HERE / "ref_cast.cpp"
    ref_src = REFERENCE_DIR / "Utilities/TensorOperations/DataTypeConversions/TypeConverter.cpp"
    if not ref_src.exists():
        return out if out.exists() else None
    REF_OUT.mkdir(exist_ok=True)
    if not force and not _stale(out, [src, ref_src]):
        return out
    verdir = REF_OUT / "generated"
    verdir.mkdir(exist_ok=True)
    # ThorVersion.h is produced by the reference's cmake from ThorVersion.h.in; give it the same two macros.
    (verdir / "ThorVersion.h").write_text('#pragma once\n#define THOR_VERSION "0.0.33"\n#define THOR_GIT_VERSION "unknown"\n')
    cmd = ["g++", "-std=c++23", "-O2", "-fopenmp", "-fPIC", "-shared", "-fvisibility=hidden", "-ffunction-sections", "-fdata-sections",
           "-Wl,--gc-sections", "-Wl,-z,defs", "-I", str(REFERENCE_DIR), "-I", str(verdir), "-I", str(CUDA_INCLUDE)]
    for d in _site_include_dirs():
        cmd += ["-I", str(d)]
    cmd += [str(src), "-o", str(out)]
    _run(cmd)
    return out


def build_reference_gpu_cast(force: bool = False) -> Path | None:
    """Compile the reference's GPU TypeConverter kernels into _ref/; None when they cannot be built here."""
    out = REF_OUT / "libthor_ref_gpu_cast.so"
    src = HERE / "ref_gpu_cast.cu"
    ref_src = REFERENCE_DIR / "Utilities/TensorOperations/DataTypeConversions/TypeConverterKernels.cu"
    nvcc = shutil.which("nvcc") or str(Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc")
    if not ref_src.exists() or not Path(nvcc).exists():
        return out if out.exists() else None
    REF_OUT.mkdir(exist_ok=True)
    if not force and not _stale(out, [src, ref_src]):
        return out
    verdir = REF_OUT / "generated"
    verdir.mkdir(exist_ok=True)
    (verdir / "ThorVersion.h").write_text('#pragma once\n#define THOR_VERSION "0.0.33"\n#define THOR_GIT_VERSION "unknown"\n')
    cmd = [nvcc, "-std=c++20", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
           "-Xlinker", "-z,defs", "-I", str(REFERENCE_DIR), "-I", str(verdir)]
    for d in _site_include_dirs():
        cmd += ["-I", str(d)]
    cmd += [str(src), "-o", str(out)]
    _run(cmd)
    return out


def _cccl3_include_dirs() -> list[Path]:
    """A CCCL 3.x header tree (the reference's reductions need <cuda/iterator>, which the toolkit's own CCCL 2.x lacks);
    some Python wheels carry one."""
    for sp in site.getsitepackages() + [sysconfig.get_paths()["purelib"]]:
        base = Path(sp) / "flashinfer" / "data" / "cccl"
        if (base / "libcudacxx" / "include" / "cuda" / "iterator").exists():
            return [base / "libcudacxx" / "include", base / "cub", base / "thrust"]
    return []


def build_reference_cub_reduce(force: bool = False) -> Path | None:
    """Compile the reference's reduction templates (CubReductionOperation.cuh: its fp32 operators, output iterator,
    CUB calls and tiled kernels) behind the C symbol of ref_cub_reduce.cu into _ref/ (nvcc, about 4 minutes); None when
    the reference checkout, nvcc or a CCCL 3.x header tree is missing."""
    out = REF_OUT / "libthor_ref_cub_reduce.so"
    src = HERE / "ref_cub_reduce.cu"
    ref_src = REFERENCE_DIR / "Utilities/TensorOperations/Cub/CubReductionOperation.cuh"
    nvcc = shutil.which("nvcc") or str(Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc")
    cccl = _cccl3_include_dirs()
    if not ref_src.exists() or not Path(nvcc).exists() or not cccl:
        return out if out.exists() else None
    REF_OUT.mkdir(exist_ok=True)
    if not force and not _stale(out, [src, ref_src]):
        return out
    verdir = REF_OUT / "generated"
    verdir.mkdir(exist_ok=True)
    (verdir / "ThorVersion.h").write_text('#pragma once\n#define THOR_VERSION "0.0.33"\n#define THOR_GIT_VERSION "unknown"\n')
    cmd = [nvcc, "-std=c++20", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
           "-Xlinker", "-z,defs"]
    for d in cccl:
        cmd += ["-I", str(d)]
    cmd += ["-I", str(REFERENCE_DIR), "-I", str(verdir)]
    for d in _site_include_dirs():
        cmd += ["-I", str(d)]
    cmd += [str(src), "-o", str(out)]
    _run(cmd)
    return out


def build_reference_emitter(force: bool = False) -> Path | None:
    """Compile the reference's expression builder, dtype resolution and CUDA source emitter (three host sources,
    g++ -std=c++23, about 15 s) with the dumper in ref_emit.cpp into _ref/; None when that cannot be done here."""
    out = REF_OUT / "libthor_ref_emit.so"
    shim = HERE / "ref_emit.cpp"
    ref_srcs = [REFERENCE_DIR / "Utilities/Expression" / n for n in ("CudaSourceEmitter.cpp", "Expression.cpp", "ExpressionDTypeResolution.cpp")]
    if not all(p.exists() for p in ref_srcs):
        return out if out.exists() else None
    REF_OUT.mkdir(exist_ok=True)
    if not force and not _stale(out, [shim, HERE / "ref_postfix.h", *ref_srcs]):
        return out
    verdir = REF_OUT / "generated"
    verdir.mkdir(exist_ok=True)
    (verdir / "ThorVersion.h").write_text('#pragma once\n#define THOR_VERSION "0.0.33"\n#define THOR_GIT_VERSION "unknown"\n')
    objdir = REF_OUT / "obj"
    objdir.mkdir(exist_ok=True)
    common = ["g++", "-std=c++23", "-O1", "-fopenmp", "-fPIC", "-fvisibility=hidden", "-ffunction-sections", "-fdata-sections",
              "-I", str(REFERENCE_DIR), "-I", str(HERE), "-I", str(verdir), "-I", str(CUDA_INCLUDE)]
    for d in _site_include_dirs():
        common += ["-I", str(d)]
    objs = []
    for src in [shim, *ref_srcs]:
        obj = objdir / (src.stem + ".o")
        _run(common + ["-c", str(src), "-o", str(obj)])
        objs.append(obj)
    # only the dumper's entry point is exported; everything it cannot reach is dropped, and -z defs proves the rest resolves
    _run(["g++", "-shared", "-fopenmp", "-o", str(out), *map(str, objs), "-Wl,--gc-sections", "-Wl,-z,defs"])
    shutil.rmtree(objdir, ignore_errors=True)
    return out


def build_reference_autodiff(force: bool = False) -> Path | None:
    """Compile the reference's reverse-mode differentiation (AutoDiff.cpp with the expression builder, dtype resolution,
    SqueezeAxes.cpp and BatchedMatmulPlan.cpp it calls; five host sources, g++ -std=c++23, about 25 s) with the graph dumper
    in ref_autodiff.cpp into _ref/; None when that cannot be done here."""
    out = REF_OUT / "libthor_ref_autodiff.so"
    shim = HERE / "ref_autodiff.cpp"
    ref_srcs = [REFERENCE_DIR / "Utilities/Expression" / n
                for n in ("AutoDiff.cpp", "Expression.cpp", "ExpressionDTypeResolution.cpp", "SqueezeAxes.cpp", "BatchedMatmulPlan.cpp")]
    if not all(p.exists() for p in ref_srcs):
        return out if out.exists() else None
    REF_OUT.mkdir(exist_ok=True)
    if not force and not _stale(out, [shim, HERE / "ref_postfix.h", *ref_srcs]):
        return out
    verdir = REF_OUT / "generated"
    verdir.mkdir(exist_ok=True)
    (verdir / "ThorVersion.h").write_text('#pragma once\n#define THOR_VERSION "0.0.33"\n#define THOR_GIT_VERSION "unknown"\n')
    objdir = REF_OUT / "obj_autodiff"
    objdir.mkdir(exist_ok=True)
    common = ["g++", "-std=c++23", "-O1", "-fopenmp", "-fPIC", "-fvisibility=hidden", "-ffunction-sections", "-fdata-sections",
              "-I", str(REFERENCE_DIR), "-I", str(HERE), "-I", str(verdir), "-I", str(CUDA_INCLUDE)]
    for d in _site_include_dirs():
        common += ["-I", str(d)]
    objs = []
    procs = []
    for src in [shim, *ref_srcs]:
        obj = objdir / (src.stem + ".o")
        procs.append(subprocess.Popen(common + ["-c", str(src), "-o", str(obj)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
        objs.append(obj)
    for proc in procs:
        log, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError("compiling the reference's autodiff failed:\n" + log[-4000:])
    _run(["g++", "-shared", "-fopenmp", "-o", str(out), *map(str, objs), "-Wl,--gc-sections", "-Wl,-z,defs"])
    shutil.rmtree(objdir, ignore_errors=True)
    return out


def build_all(force: bool = False) -> dict:
    result = {"oracle": str(build_oracle(force))}
    try:
        emit = build_reference_emitter(force)
        result["reference_emitter"] = str(emit) if emit else None
    except RuntimeError as exc:
        result["reference_emitter"] = None
        result["reference_emitter_error"] = str(exc)[-2000:]
    try:
        ad = build_reference_autodiff(force)
        result["reference_autodiff"] = str(ad) if ad else None
    except RuntimeError as exc:
        result["reference_autodiff"] = None
        result["reference_autodiff_error"] = str(exc)[-2000:]
    try:
        ref_gpu = build_reference_gpu_cast(force)
        result["reference_gpu_cast"] = str(ref_gpu) if ref_gpu else None
    except RuntimeError as exc:
        result["reference_gpu_cast"] = None
        result["reference_gpu_cast_error"] = str(exc)[-2000:]
    try:
        ref_red = build_reference_cub_reduce(force)
        result["reference_cub_reduce"] = str(ref_red) if ref_red else None
    except RuntimeError as exc:
        result["reference_cub_reduce"] = None
        result["reference_cub_reduce_error"] = str(exc)[-2000:]
    try:
        ref = build_reference_cast(force)
        result["reference_cast"] = str(ref) if ref else None
    except RuntimeError as exc:  # the reference needs headers this machine lacks
        result["reference_cast"] = None
        result["reference_cast_error"] = str(exc)[-2000:]
    return result


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv))
