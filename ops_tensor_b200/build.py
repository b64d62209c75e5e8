"""Builds libops_tensor_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m ops_tensor_b200.build [--force] [--verbose]

Sources: csrc/*.cu (kernels and the C-ABI launch layer) and csrc/host/*.cpp (the acltensor* host API).  Objects are
cached under build/ and rebuilt when a source or any header is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = ROOT / "build"
LIB_PATH = PKG_DIR / "libops_tensor_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", f"-I{ROOT / 'include'}",
          f"-I{CSRC}", f"-I{CSRC / 'host'}"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def _sources():
    return sorted(CSRC.glob("*.cu")) + sorted((CSRC / "host").glob("*.cpp"))


def _headers():
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((CSRC / "host").glob("*.hpp"))
    hs += list((ROOT / "include").rglob("*.h"))
    return hs


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > t for p in _sources() + _headers())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB_PATH
    nvcc = _nvcc()
    BUILD_DIR.mkdir(exist_ok=True)
    newest_header = max((p.stat().st_mtime for p in _headers()), default=0.0)

    def compile_one(src: Path) -> Path:
        obj = BUILD_DIR / (src.stem + ".o")
        if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, newest_header):
            return obj
        cmd = [nvcc, *ARCH_FLAGS, *COMMON, "-x", "cu" if src.suffix == ".cu" else "c++", "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose and r.stderr:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, _sources()))
    link = [nvcc, *ARCH_FLAGS, "-shared", "-cudart", "static", "-o", str(LIB_PATH), *map(str, objs)]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
