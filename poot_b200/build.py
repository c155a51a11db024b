"""In-tree build of the native libraries.

Two shared objects are produced under ``poot_b200/lib``:

* ``libpoot_kernels.so`` - every CUDA kernel under ``csrc/kernels`` compiled with
  ``nvcc -gencode arch=compute_100a,code=sm_100a`` (cross-compiles without a GPU).
* ``libpoot_host.so`` - the C++ runtime pieces under ``csrc/host`` (quant codecs, GGUF /
  safetensors readers, block pool and prefix cache, oracle inner loops).

Both expose a plain C ABI and are loaded with :mod:`ctypes`, so no torch headers are needed and a
full build takes well under a minute.  Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIB_DIR = ROOT / "poot_b200" / "lib"
OBJ_DIR = ROOT / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-pthread", "-fvisibility=hidden", "-Wall", "-Wno-unused-function"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build command failed: {' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    return r.stdout + r.stderr


def build_kernels(verbose: bool = False, force: bool = False, ptxas_info: bool = False,
                  debug_bounds: bool = False) -> Path:
    """``debug_bounds``: the checked flavour (``-DPOOT_DEBUG_BOUNDS``: every data-dependent index is compared with its
    bound and a miss is recorded for the host instead of trapping), built beside the release library as
    ``libpoot_kernels_dbg.so`` and loaded instead of it when ``POOT_DEBUG_BOUNDS=1`` is in the environment."""
    src_dir = CSRC / "kernels"
    sources = sorted(src_dir.glob("*.cu"))
    headers = sorted(src_dir.glob("*.cuh")) + sorted(src_dir.glob("*.h"))
    obj_dir = OBJ_DIR.parent / "obj_dbg" if debug_bounds else OBJ_DIR
    obj_dir.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    out = LIB_DIR / ("libpoot_kernels_dbg.so" if debug_bounds else "libpoot_kernels.so")
    nvcc = _nvcc()
    jobs = []
    objs = []
    extra = ["-DPOOT_DEBUG_BOUNDS"] if debug_bounds else []
    for s in sources:
        o = obj_dir / (s.stem + ".o")
        objs.append(o)
        if force or _newer(o, [s, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(src_dir), "-c", str(s), "-o", str(o)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)
    logs = []
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            logs = list(ex.map(lambda c: _run(c, verbose), jobs))
    if jobs or force or _newer(out, objs):
        _run([nvcc, "-shared", "-o", str(out), *map(str, objs), "-cudart", "static",
              "-gencode", "arch=compute_100a,code=sm_100a"], verbose)
    if ptxas_info:
        print("\n".join(logs))
    return out


def build_host(verbose: bool = False, force: bool = False) -> Path:
    src_dir = CSRC / "host"
    sources = sorted(src_dir.glob("*.cpp"))
    headers = sorted(src_dir.glob("*.h")) + sorted(src_dir.glob("*.hpp"))
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    out = LIB_DIR / "libpoot_host.so"
    cxx = os.environ.get("CXX", "g++")
    jobs, objs = [], []
    for s in sources:
        o = OBJ_DIR / ("host_" + s.stem + ".o")
        objs.append(o)
        if force or _newer(o, [s, *headers]):
            jobs.append([cxx, *CXX_FLAGS, "-I", str(src_dir), "-c", str(s), "-o", str(o)])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    if sources and (jobs or force or _newer(out, objs)):
        _run([cxx, "-shared", "-pthread", "-o", str(out), *map(str, objs)], verbose)
    return out


def build_kernels_checked(verbose: bool = False, force: bool = False) -> Path:
    return build_kernels(verbose, force, debug_bounds=True)


def build_all(verbose: bool = False, force: bool = False, checked: bool = False) -> None:
    build_host(verbose, force)
    build_kernels(verbose, force)
    if checked:
        build_kernels_checked(verbose, force)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv, force="-f" in sys.argv, checked="--checked" in sys.argv)
    if "--ptxas" in sys.argv:
        build_kernels(verbose=False, force=True, ptxas_info=True)
    print("built:", *(p.name for p in LIB_DIR.glob("*.so")))
