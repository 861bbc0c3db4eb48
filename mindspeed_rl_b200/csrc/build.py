"""In-tree build of the CUDA kernel library for sm_100a.

``python -m mindspeed_rl_b200.csrc.build`` compiles every ``*.cu`` under this directory
with ``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` into objects and links them
into ``mindspeed_rl_b200/_C/libmsrl_b200.so`` (plain ``extern "C"`` entry points, loaded with
ctypes -- no Python or torch headers involved, so a full rebuild takes seconds).  C++-only
sources (``*.cpp``: block manager, host runtime helpers) are compiled with g++ into the same
library.  Objects are rebuilt only when their source or a header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path
from typing import List

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
OUT_DIR = PKG / "_C"
OBJ_DIR = OUT_DIR / "obj"
LIB_PATH = OUT_DIR / "libmsrl_b200.so"
HOST_LIB_PATH = OUT_DIR / "libmsrl_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return cand


def _newest_header() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.hpp"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile_one(src: Path, force: bool, log_dir: Path) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = max(src.stat().st_mtime, _newest_header(), Path(__file__).stat().st_mtime)
    if not force and obj.exists() and obj.stat().st_mtime >= stamp:
        return obj
    if src.suffix == ".cu":
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", *CXX_FLAGS, "-I", str(CSRC), "-I", "/usr/local/cuda/include", "-c", str(src),
               "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (log_dir / (src.stem + ".log")).write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"compilation of {src.name} failed:\n{res.stdout}\n{res.stderr}")
    return obj


def sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    log_dir = OUT_DIR / "logs"
    log_dir.mkdir(exist_ok=True)
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as pool:
        objs = list(pool.map(lambda s: _compile_one(s, force, log_dir), srcs))
    cu_objs = [o for s, o in zip(srcs, objs) if s.suffix == ".cu"]
    host_objs = [o for s, o in zip(srcs, objs) if s.suffix == ".cpp"]

    def stale(lib, deps):
        return force or not lib.exists() or any(o.stat().st_mtime > lib.stat().st_mtime for o in deps)

    if cu_objs and stale(LIB_PATH, cu_objs):
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, cu_objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-Xcompiler", "-fPIC",
               "-Xlinker", "-z,noexecstack"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if host_objs and stale(HOST_LIB_PATH, host_objs):
        # host-only runtime pieces (block manager, ...) load on machines without CUDA
        cmd = ["g++", "-shared", "-o", str(HOST_LIB_PATH), *map(str, host_objs), "-pthread"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"host link failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        for s in srcs:
            log = log_dir / (s.stem + ".log")
            if log.exists():
                sys.stdout.write(f"== {s.name}\n{log.read_text()}\n")
    return LIB_PATH


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(p)
