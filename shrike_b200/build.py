"""Builds libshrike_b200.so (sm_100a) in-tree with nvcc.

Usage: python -m shrike_b200.build [--force]
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT_DIR = ROOT / "_lib"
LIB = OUT_DIR / "libshrike_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _newest_input() -> float:
    deps = list(CSRC.glob("*")) + [ROOT.parent / "include" / "shrike_b200.h"]
    return max(p.stat().st_mtime for p in deps)


def needs_build() -> bool:
    return not LIB.exists() or LIB.stat().st_mtime < _newest_input()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (cand == "nvcc" or Path(cand).exists()):
            return cand
    raise RuntimeError("nvcc not found")


def _compile(src: Path, verbose: bool) -> Path:
    obj = OUT_DIR / (src.stem + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    OUT_DIR.mkdir(exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), sources()))
    cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


HARNESS = OUT_DIR / "harness"


def build_harness(force: bool = False) -> Path:
    """Compiles the C++ host harness (shrike_b200/host) against the library with g++."""
    src = ROOT / "host" / "harness.cpp"
    hdr = ROOT / "host" / "shrike_moe.hpp"
    build()
    if not force and HARNESS.exists() and HARNESS.stat().st_mtime >= max(src.stat().st_mtime, hdr.stat().st_mtime,
                                                                         LIB.stat().st_mtime):
        return HARNESS
    cuda = Path(_nvcc()).resolve().parent.parent if _nvcc() != "nvcc" else Path("/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-O2", str(src), "-o", str(HARNESS), f"-I{cuda / 'include'}",
           f"-L{OUT_DIR}", "-lshrike_b200", f"-L{cuda / 'lib64'}", "-lcudart",
           f"-Wl,-rpath,{OUT_DIR}", f"-Wl,-rpath,{cuda / 'lib64'}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"g++ failed on harness.cpp:\n{res.stdout}\n{res.stderr}")
    return HARNESS


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
