"""Builds libretro_b200.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

Usage: python -m retrograd_b200.build [--force] [--checked]
Objects are cached under retrograd_b200/build/ and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "libretro_b200.so"
OBJ = HERE / "build"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _gcc_libdir() -> str:
    try:
        path = subprocess.check_output(["g++", "-print-libgcc-file-name"], text=True).strip()
        return str(Path(path).parent)
    except Exception:
        return ""


def _flags() -> list[str]:
    host = ["-fPIC", "-fopenmp", "-O3"]
    libdir = _gcc_libdir()
    if libdir:
        host.append(f"-B{libdir}")
    return ["-std=c++17", "-O3", "-lineinfo", *ARCH, "-Xcompiler", ",".join(host), "-I", str(HERE.parent / "include")]


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _newest_header() -> float:
    headers = list(CSRC.glob("*.hpp")) + list(CSRC.glob("*.cuh")) + list((HERE.parent / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> Path:
    """`checked`: the bounds-checked build (-DRETRO_B200_CHECKED) into libretro_b200_checked.so."""
    global OBJ, OUT
    if checked:
        saved = OBJ, OUT
        OBJ, OUT = HERE / "build_checked", HERE / "libretro_b200_checked.so"
        try:
            return _build(force, verbose, ["-DRETRO_B200_CHECKED=1"])
        finally:
            OBJ, OUT = saved
    return _build(force, verbose, [])


def _build(force: bool, verbose: bool, defines: list[str]) -> Path:
    OBJ.mkdir(exist_ok=True)
    flags = _flags() + defines
    header_time = _newest_header()
    jobs = []
    objects = []
    for src in sources():
        obj = OBJ / (src.name + ".o")
        objects.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_time):
            cmd = [NVCC, *flags, "-x", "cu", "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd: list[str]) -> None:
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
        if verbose and proc.stderr:
            print(proc.stderr)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(run, jobs))
    if jobs or force or not OUT.exists():
        link = [NVCC, "-shared", *ARCH, "-Xcompiler", "-fPIC", "-o", str(OUT), *map(str, objects), "-lgomp"]
        libdir = _gcc_libdir()
        if libdir:
            link += ["-L", libdir]
        run(link)
    return OUT


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, checked="--checked" in sys.argv)
    print(path)
