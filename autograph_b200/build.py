"""Builds libautograph_b200.so (the C-ABI library) with nvcc for sm_100a.

Usage: ``python -m autograph_b200.build [--force] [--verbose]``.
Objects go to ``autograph_b200/_build``; the shared library is written next to
this file so that it ships with the source tree.  No GPU is needed to build.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "_build"
LIB = HERE / "libautograph_b200.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# Extra compiler flags (e.g. AG_NVCC_EXTRA=-DAG_PHASE_STAMPS for the phase timestamps that the
# profile summaries quote) and where to put the result (AG_LIB_OUT=<path>: a side build that
# leaves the product library alone).
EXTRA = os.environ.get("AG_NVCC_EXTRA", "").split()
if os.environ.get("AG_LIB_OUT"):
    LIB = Path(os.environ["AG_LIB_OUT"]).resolve()
    BUILD = LIB.parent / (LIB.stem + "_build")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden",
          "--expt-relaxed-constexpr", "-Xptxas", "-v", *EXTRA]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted((CSRC / "host").glob("*.cu"))


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.hpp")) +
                    [HERE.parent / "include" / "autograph_b200.h"]):
        h.update(p.read_bytes())
    h.update(" ".join(ARCH + CFLAGS).encode())
    return h.hexdigest()


def _compile(src: Path, digest: str, force: bool, verbose: bool) -> Path:
    obj = BUILD / (src.stem + ".o")
    stamp = BUILD / (src.stem + ".stamp")
    key = hashlib.sha256(src.read_bytes() + digest.encode()).hexdigest()
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == key:
        return obj
    cmd = [NVCC, *ARCH, *CFLAGS, "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (BUILD / (src.stem + ".ptxas.log")).write_text(res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stderr[-6000:]}")
    if verbose:
        sys.stderr.write(res.stderr)
    stamp.write_text(key)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    digest = _headers_digest()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, digest, force, verbose), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    if force or not LIB.exists() or LIB.stat().st_mtime < newest:
        cmd = [NVCC, *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stderr[-4000:]}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
