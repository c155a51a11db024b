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
import json
import os
import re
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


_ENTRY = re.compile(r"Compiling entry function '([^']+)' for 'sm_100a'")
_SPILL = re.compile(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads")
_USED = re.compile(r"Used (\d+) registers(?:, used (\d+) barriers)?")
_SMEM = re.compile(r"(\d+) bytes smem")


def parse_ptxas_info(text: str) -> dict:
    """``ptxas -v`` output of one translation unit -> ``{mangled entry: {registers, barriers, static_smem, stack,
    spill_stores, spill_loads}}``.  The static shared memory is what the kernel declares; a kernel that takes dynamic
    shared memory gets the rest from its launcher."""
    out, cur = {}, None
    for line in text.splitlines():
        m = _ENTRY.search(line)
        if m:
            cur = out.setdefault(m.group(1), {"registers": 0, "barriers": 0, "static_smem": 0, "stack": 0, "spill_stores": 0, "spill_loads": 0})
            continue
        if cur is None:
            continue
        m = _SPILL.search(line)
        if m:
            cur["stack"], cur["spill_stores"], cur["spill_loads"] = (int(x) for x in m.groups())
            continue
        m = _USED.search(line)
        if m:
            sm = _SMEM.search(line)               # a stack-size note may stand between the barriers and the shared memory
            cur["registers"], cur["barriers"], cur["static_smem"] = int(m.group(1)), int(m.group(2) or 0), int(sm.group(1)) if sm else 0
            cur = None
    return out


def _demangle(names) -> dict:
    names = list(names)
    tool = shutil.which("c++filt")
    if not tool or not names:
        return {n: n for n in names}
    r = subprocess.run([tool], input="\n".join(names), capture_output=True, text=True)
    plain = r.stdout.splitlines()
    return dict(zip(names, plain)) if r.returncode == 0 and len(plain) == len(names) else {n: n for n in names}


def write_resource_table(obj_dir: Path, out: Path) -> dict:
    """Merge the per-object resource records into the table ``plan/register_feedback.py`` reads: one row per kernel
    entry with its source file, the readable signature and what ``ptxas`` reported for it."""
    rows = {}
    for rec in sorted(obj_dir.glob("*.res.json")):
        for mangled, r in json.loads(rec.read_text()).items():
            rows[mangled] = {"source": rec.name[:-len(".res.json")] + ".cu", **r}
    plain = _demangle(rows)
    table = {"arch": "sm_100a", "kernels": [{"entry": m, "signature": plain[m], **r} for m, r in sorted(rows.items())]}
    out.write_text(json.dumps(table, indent=0))
    return table


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
            jobs.append([nvcc, "-Xptxas", "-v", *NVCC_FLAGS, *extra, "-I", str(src_dir), "-c", str(s), "-o", str(o)])
    logs = []
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            logs = list(ex.map(lambda c: _run(c, verbose), jobs))
        for cmd, log in zip(jobs, logs):          # what the compiler reported per entry, kept beside the object
            Path(cmd[-1]).with_suffix(".res.json").write_text(json.dumps(parse_ptxas_info(log)))
    if not debug_bounds and (jobs or force or not (LIB_DIR / "kernel_resources.json").exists()):
        write_resource_table(obj_dir, LIB_DIR / "kernel_resources.json")
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
