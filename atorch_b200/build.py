"""Builds the CUDA library of atorch_b200 for sm_100a.

Every ``csrc/*.cu`` file is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a`` into an
object file and the objects are linked into one shared library, ``atorch_b200/_C/libatb.so``, that
exposes plain ``extern "C"`` launchers (loaded with ctypes by :mod:`atorch_b200._lib`). nvcc
cross-compiles, so the build needs no GPU. Objects are rebuilt only when a source or header is newer.

Plays the role of the JIT op builder of the reference (atorch/ops/op_builder/builder.py:120-681),
but ahead of time and for one architecture only.

Usage: ``python -m atorch_b200.build [--force] [--verbose]``
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT_DIR = ROOT / "_C"
OBJ_DIR = OUT_DIR / "obj"
LIB = OUT_DIR / "libatb.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def _newest_header_mtime() -> float:
    return max((p.stat().st_mtime for p in CSRC.glob("*.cuh")), default=0.0)


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    return res.stderr if verbose else ""


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    hdr_m = _newest_header_mtime()
    todo, objs = [], []
    for src in sources():
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m):
            todo.append((src, obj))
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            futs = {ex.submit(_compile_one, nvcc, s, o, verbose): s for s, o in todo}
            for f in cf.as_completed(futs):
                log = f.result()
                if verbose and log:
                    print(f"--- {futs[f].name}\n{log}")
    if todo or not LIB.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args(argv)
    lib = build(force=args.force, verbose=args.verbose)
    print(f"built {lib} ({lib.stat().st_size / 1e6:.1f} MB) from {len(sources())} sources")
    return 0


if __name__ == "__main__":
    sys.exit(main())
