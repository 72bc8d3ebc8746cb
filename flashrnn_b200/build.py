"""Ahead-of-time build of libfrnn_b200.so (sm_100a only) with nvcc.

Replaces the reference's per-shape JIT (flashrnn/flashrnn/cuda_init.py:95-168 and
cuda_init_parametric.py:92-358): one library, built once, no compile at call time.

    python -m flashrnn_b200.build [--force] [--jobs N]
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "_build"
LIB = PKG / "libfrnn_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; libfrnn_b200.so cannot be built")
    return exe


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(out: Path, deps: list[Path]) -> bool:
    return not out.exists() or any(d.stat().st_mtime > out.stat().st_mtime for d in deps)


def _compile(src: Path, headers: list[Path], force: bool, f16: bool = False) -> Path:
    """One object per (source, element type): as is = bfloat16, with -DFRNN_F16 = float16 (csrc/frnn_elem.cuh)."""
    stem = src.stem + ("_f16" if f16 else "")
    obj = OBJ / (stem + ".o")
    if force or _stale(obj, [src] + headers):
        cmd = [_nvcc(), *NVCC_FLAGS, *(["-DFRNN_F16"] if f16 else []), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        (OBJ / (stem + ".log")).write_text(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stderr[-4000:]}")
    return obj


def build(force: bool = False, jobs: int | None = None, extra_flags: tuple[str, ...] = (), lib: Path | None = None,
          obj_dir: Path | None = None) -> Path:
    """Compile every .cu under csrc/ for sm_100a and link the shared library next to the package.
    ``extra_flags`` / ``lib`` / ``obj_dir`` build a variant (e.g. with development macros) somewhere else."""
    global OBJ, LIB, NVCC_FLAGS
    if extra_flags or lib or obj_dir:
        saved = (OBJ, LIB, NVCC_FLAGS)
        OBJ, LIB, NVCC_FLAGS = Path(obj_dir or OBJ), Path(lib or LIB), [*NVCC_FLAGS, *extra_flags]
        try:
            return build(force, jobs)
        finally:
            OBJ, LIB, NVCC_FLAGS = saved
    OBJ.mkdir(exist_ok=True, parents=True)
    headers = sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "frnn.h"]
    srcs = _sources()
    units = [(s, f16) for f16 in (False, True) for s in srcs]
    jobs = jobs or min(len(units), os.cpu_count() or 4)
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        objs = list(ex.map(lambda u: _compile(u[0], headers, force, u[1]), units))
    if force or _stale(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stderr[-4000:]}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    a = ap.parse_args()
    print(build(a.force, a.jobs))
    sys.exit(0)
