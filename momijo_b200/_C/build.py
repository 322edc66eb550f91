"""In-tree build of the native libraries.

``libmomijo_b200.so``  : every CUDA kernel, compiled for sm_100a only, C ABI (loaded with ctypes)
``libmomijo_host.so``  : host-side C++ runtime (checkpoint blob I/O, samplers, CSV, image loops)

The build is incremental (per-object timestamps) and parallel. It needs only ``nvcc`` and
``g++``; there is no dependency on the torch headers, so a full rebuild takes seconds and the
resulting libraries can be loaded from any process (Python through ctypes, or C/C++ directly).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB_CUDA = HERE / "libmomijo_b200.so"
LIB_HOST = HERE / "libmomijo_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]
# Approximate division / square root / exp are fine where results are rounded to bf16 (GEMM epilogues,
# attention, activations); the optimizer and the collectives that carry the optimizer update keep IEEE
# division and sqrtf, so the update matches a plain fp32 AdamW bit for bit.
FAST_MATH = ["--use_fast_math"]
EXACT_MATH_SOURCES = {"loss_optim.cu", "comm.cu"}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    return r.stdout + r.stderr


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False,
          debug_bounds: bool = None) -> dict:
    """Compile all sources; returns {'cuda': path, 'host': path, 'log': str}. ``debug_bounds`` (default:
    the MOMIJO_DEBUG_BOUNDS environment variable) builds the bounds-checked variant of the kernel library
    beside the normal one (``libmomijo_b200_dbg.so``, own object directory)."""
    if debug_bounds is None:
        debug_bounds = os.environ.get("MOMIJO_DEBUG_BOUNDS", "0") == "1"
    obj_dir = HERE / "build_dbg" if debug_bounds else OBJ
    lib_cuda = HERE / "libmomijo_b200_dbg.so" if debug_bounds else LIB_CUDA
    obj_dir.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    cu = sorted(CSRC.glob("*.cu"))
    cpp = [c for c in sorted(CSRC.glob("*.cpp")) if not c.name.endswith("_selftest.cpp")]
    nvcc = _nvcc()
    log = []

    def compile_cu(src: Path):
        obj = obj_dir / (src.stem + ".o")
        if not force and _newer(obj, [src, *headers]):
            return obj
        flags = list(NVCC_FLAGS)
        if src.name not in EXACT_MATH_SOURCES:
            flags += FAST_MATH
        if debug_bounds:
            flags += ["-DMMJ_DEBUG_BOUNDS"]
        if ptxas_info:
            flags += ["-Xptxas", "-v"]
        log.append(_run([nvcc, *flags, "-c", src, "-o", obj], verbose))
        return obj

    def compile_cpp(src: Path):
        obj = obj_dir / (src.stem + ".host.o")
        if not force and _newer(obj, [src, *headers]):
            return obj
        log.append(_run(["g++", "-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread",
                         "-c", src, "-o", obj], verbose))
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        cu_objs = list(ex.map(compile_cu, cu))
        cpp_objs = list(ex.map(compile_cpp, cpp))

    if cu_objs and (force or not _newer(lib_cuda, cu_objs)):
        log.append(_run([nvcc, "-shared", "-o", lib_cuda, *cu_objs, "-cudart", "static",
                         "-gencode", "arch=compute_100a,code=sm_100a"], verbose))
    if cpp_objs and (force or not _newer(LIB_HOST, cpp_objs)):
        log.append(_run(["g++", "-shared", "-pthread", "-o", LIB_HOST, *cpp_objs], verbose))
    return {"cuda": str(lib_cuda), "host": str(LIB_HOST), "log": "\n".join(log)}


SANITIZERS = {
    "asan_ubsan": ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer"],
    "tsan": ["-fsanitize=thread"],
}


def build_sanitized(kind: str, out_dir=None, verbose: bool = False) -> Path:
    """Build the host runtime together with its self-test driver (``csrc/host_runtime_selftest.cpp``) under
    a sanitizer: ``kind`` is "asan_ubsan" (AddressSanitizer + UndefinedBehaviorSanitizer) or "tsan"
    (ThreadSanitizer). Returns the executable; running it exits non-zero on a failed check or a sanitizer
    report. The device library has its own checked variant (``debug_bounds``)."""
    flags = SANITIZERS[kind]
    out_dir = Path(out_dir) if out_dir is not None else (HERE / "build")
    out_dir.mkdir(exist_ok=True)
    exe = out_dir / f"host_runtime_selftest_{kind}"
    srcs = [CSRC / "host_runtime.cpp", CSRC / "host_runtime_selftest.cpp"]
    _run(["g++", "-O1", "-g", "-std=c++17", "-pthread", *flags, *srcs, "-o", exe], verbose)
    return exe


if __name__ == "__main__":
    out = build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(out["log"])
    print("built:", out["cuda"], out["host"])
