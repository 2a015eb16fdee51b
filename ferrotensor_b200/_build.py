"""Builds libft_cuda.so in-tree with nvcc for sm_100a.

    python -m ferrotensor_b200._build [--force] [--verbose]

Objects and the shared library are written next to the sources (`csrc/build/`,
`libft_cuda.so`); a source is recompiled when it or a header is newer than its object.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "build"
LIB = PKG / "libft_cuda.so"
INCLUDE = PKG.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libft_cuda.so cannot be built")
    return exe


def sources():
    return sorted(CSRC.glob("*.cu"))


def _stale(src: Path, obj: Path, headers) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *headers])


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    # objects built with other flags (FT_NVCC_EXTRA) are stale whatever their age
    stamp = OBJ / "flags.txt"
    flags_now = " ".join(NVCC_FLAGS + os.environ.get("FT_NVCC_EXTRA", "").split())
    if not stamp.exists() or stamp.read_text() != flags_now:
        force = True
    jobs = []
    for src in sources():
        obj = OBJ / (src.stem + ".o")
        if force or _stale(src, obj, headers):
            jobs.append((src, obj))

    extra = os.environ.get("FT_NVCC_EXTRA", "").split()   # e.g. -DFT_ATTN_TIMING, -DFT_DEBUG_MARKERS

    def compile_one(job):
        src, obj = job
        cmd = [nvcc(), *NVCC_FLAGS, *extra, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, r in ex.map(compile_one, jobs):
                if verbose or r.returncode != 0:
                    sys.stderr.write(f"--- {src.name}\n{r.stdout}{r.stderr}\n")
                (OBJ / (src.stem + ".ptxas.log")).write_text(r.stderr)
                if r.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {src.name}")
        stamp.write_text(flags_now)
    objs = [OBJ / (s.stem + ".o") for s in sources()]
    if jobs or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-lcudart", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of libft_cuda.so failed")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
