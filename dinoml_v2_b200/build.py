"""Builds libdinoml_b200_gguf.so in-tree with nvcc for sm_100a.

    python -m dinoml_v2_b200.build [--force] [--verbose]

Each csrc/*.cu is compiled to build/<name>.o (in parallel, rebuilt when the source or a header is
newer) and linked into dinoml_v2_b200/lib/libdinoml_b200_gguf.so.  `-Xptxas -v` output (registers,
spills, shared memory per kernel) is kept in build/ptxas_<name>.log.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG / "build"
LIB_DIR = PKG / "lib"
LIB_NAME = "libdinoml_b200_gguf.so"
LIB_PATH = LIB_DIR / LIB_NAME

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v", "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build the sm_100a kernels")
    return exe


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((PKG.parent / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def _compile(src: Path, force: bool) -> tuple[Path, bool]:
    obj = BUILD / (src.stem + ".o")
    stamp = max(src.stat().st_mtime, _newest_header(), Path(__file__).stat().st_mtime)
    if not force and obj.exists() and obj.stat().st_mtime >= stamp:
        return obj, False
    cmd = [nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    (BUILD / f"ptxas_{src.stem}.log").write_text(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return obj, True


def build(force: bool = False, verbose: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(lambda s: _compile(s, force), sources))
    objs = [o for o, _ in results]
    changed = any(c for _, c in results)
    if changed or not LIB_PATH.exists():
        # default visibility only for the extern "C" entry points (marked in the sources)
        cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB_PATH), *map(str, objs)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        for src in sources:
            log = BUILD / f"ptxas_{src.stem}.log"
            if log.exists():
                sys.stdout.write(log.read_text())
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    print(build(args.force, args.verbose))
