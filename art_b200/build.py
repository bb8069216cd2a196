"""In-tree build of the native libraries.

Two shared objects are produced under ``art_b200/_native``:

* ``libartb_kernels.so``  every ``csrc/kernels/*.cu`` and ``csrc/comm/*.cu``, compiled by
  nvcc for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``).  The kernels are
  exported with a plain C ABI and called through :mod:`ctypes` with raw device pointers
  and the current CUDA stream, so neither the build nor the call path needs the PyTorch
  C++ headers.
* ``libartb_runtime.so``  the host runtime (paged-KV block manager, continuous-batching
  scheduler, packer) from ``csrc/engine/*.cpp``, compiled by g++.

``python -m art_b200.build`` rebuilds what is out of date; ``build_all(force=True)``
rebuilds everything.  Object files are cached under ``art_b200/_native/obj``.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT = ROOT / "_native"
OBJ = OUT / "obj"

KERNEL_LIB = OUT / "libartb_kernels.so"
CHECKED_KERNEL_LIB = OUT / "libartb_kernels_checked.so"
RUNTIME_LIB = OUT / "libartb_runtime.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-I", str(CSRC / "include"),
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-I", str(CSRC / "include")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install CUDA 12.8+")


def _digest(src: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(src.read_bytes())
    for hdr in sorted((CSRC / "include").glob("*")):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _compile_one(src: Path, cmd_prefix: list[str], flags: list[str], verbose: bool, obj_dir: Path | None = None) -> Path:
    obj_dir = obj_dir or OBJ
    obj = obj_dir / f"{src.stem}.{_digest(src, flags)}.o"
    if obj.exists():
        return obj
    for stale in obj_dir.glob(f"{src.stem}.*.o"):
        stale.unlink()
    cmd = cmd_prefix + flags + ["-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {src}\n{res.stdout}\n{res.stderr}")
    if verbose and res.stderr.strip():
        print(res.stderr, flush=True)
    return obj


def kernel_sources() -> list[Path]:
    return sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu"))


def runtime_sources() -> list[Path]:
    # *_selftest.cpp are stand-alone sanitizer test programs (they define main), not part of the library
    return sorted(p for p in (CSRC / "engine").glob("*.cpp") if not p.name.endswith("_selftest.cpp"))


def build_all(force: bool = False, verbose: bool = False, ptxas_info: bool = False, checked: bool = False) -> None:
    OBJ.mkdir(parents=True, exist_ok=True)
    if force:
        for o in OBJ.glob("*.o"):
            o.unlink()
    nvcc = _nvcc()
    nv_flags = NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else [])
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        kjobs = [pool.submit(_compile_one, s, [nvcc], nv_flags, verbose or ptxas_info) for s in kernel_sources()]
        rjobs = [pool.submit(_compile_one, s, ["g++"], CXX_FLAGS, verbose) for s in runtime_sources()]
        kobjs = [j.result() for j in kjobs]
        robjs = [j.result() for j in rjobs]

    def _link(lib: Path, objs: list[Path], cmd: list[str]) -> None:
        if not objs:
            return
        if lib.exists() and not force and all(lib.stat().st_mtime >= o.stat().st_mtime for o in objs):
            return
        tmp = lib.with_suffix(".so.tmp")
        res = subprocess.run(cmd + [str(o) for o in objs] + ["-o", str(tmp)], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed: {lib}\n{res.stdout}\n{res.stderr}")
        os.replace(tmp, lib)

    _link(KERNEL_LIB, kobjs, [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"])
    _link(RUNTIME_LIB, robjs, ["g++", "-shared", "-fPIC", "-pthread"])
    if checked:
        # the same kernels with device-side index checks compiled in (csrc/include/bounds_check.cuh); loaded instead of
        # the normal library when ARTB_BOUNDS_CHECK=1 is set in the environment
        cdir = OBJ / "checked"
        cdir.mkdir(parents=True, exist_ok=True)
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            cjobs = [pool.submit(_compile_one, s, [nvcc], nv_flags + ["-DARTB_BOUNDS_CHECK"], verbose, cdir)
                     for s in kernel_sources()]
            cobjs = [j.result() for j in cjobs]
        _link(CHECKED_KERNEL_LIB, cobjs, [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"])


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv,
              checked="--checked" in sys.argv)
    print("built:", KERNEL_LIB, RUNTIME_LIB, *([CHECKED_KERNEL_LIB] if "--checked" in sys.argv else []))
