"""Builds libkd_attention.so (hand-written sm_100a CUDA behind a C ABI) in-tree with nvcc.

Usage: ``python -m kerneldev_b200.build [--force]``.  nvcc cross-compiles for sm_100a, so the
build works on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "_lib"
LIB_PATH = LIB_DIR / "libkd_attention.so"
INCLUDE_DIR = PKG_DIR.parent / "include"

SOURCES = ["capi.cu", "plan.cu", "attn_fwd.cu", "attn_bwd.cu", "attn_bwd_fused.cu", "hadamard.cu", "metadata.cu", "cocktail.cu"]
HEADERS = sorted(p.name for p in (Path(__file__).resolve().parent / "csrc").glob("*.cuh"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--use_fast_math",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libkd_attention.so cannot be built")
    return exe


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    deps = [CSRC / s for s in SOURCES + HEADERS] + [INCLUDE_DIR / "kd_attention.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, extra_flags=(), name=None) -> Path:
    """Compiles every CUDA source for sm_100a and links the shared library. Returns its path.

    ``name`` + ``extra_flags`` build a variant of the same sources as libkd_attention_<name>.so (the
    wait time-out test builds one with a short wait limit); the package itself loads only the
    default library unless KD_LIB_PATH says otherwise."""
    lib_path = LIB_PATH
    if name:
        lib_path = LIB_DIR / f"libkd_attention_{name}.so"
        deps = [CSRC / s for s in SOURCES + HEADERS] + [INCLUDE_DIR / "kd_attention.h"]
        if not force and lib_path.exists() and all(d.stat().st_mtime <= lib_path.stat().st_mtime for d in deps):
            return lib_path
    elif not force and not _stale():
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / (f"obj_{name}" if name else "obj")
    obj_dir.mkdir(exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: str) -> Path:
        obj = obj_dir / (src + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    cmd = [nvcc, "-shared", "-o", str(lib_path), *map(str, objs), "-cudart", "shared"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib_path


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(p)
