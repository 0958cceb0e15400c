"""Builds the CUDA library in-tree (padra_b200/libpadra_b200.so, sm_100a only) and the C++ host tool above its C ABI
(padra_b200/host/padra_host_tool, g++ -std=c++20).

Run as `python -m padra_b200.build` (or call build()).  nvcc cross-compiles without a GPU."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libpadra_b200.so"
HOST = HERE / "host"
HOST_TOOL = HOST / "padra_host_tool"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
CUDA_HOME = Path(NVCC).resolve().parent.parent
FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.glob("*")) + [HERE.parent / "include" / "padra_b200.h"])
    return newest > LIB.stat().st_mtime


def build_host_tool(force: bool = False) -> Path:
    """The C++ host tool: artifact reader/writer/binder and one decode layer through the C ABI."""
    sources_ = [HOST / "host_tool.cpp", HOST / "artifact.cpp"]
    newest = max(p.stat().st_mtime for p in list(HOST.glob("*.?pp")) + [LIB, HERE.parent / "include" / "padra_b200.h"])
    if not force and HOST_TOOL.exists() and HOST_TOOL.stat().st_mtime >= newest:
        return HOST_TOOL
    subprocess.check_call([CXX, "-std=c++20", "-O2", "-Wall", "-Wextra", f"-I{CUDA_HOME / 'include'}", *map(str, sources_), "-o",
                           str(HOST_TOOL), f"-L{HERE}", "-lpadra_b200", f"-L{CUDA_HOME / 'lib64'}", "-lcudart",
                           "-Wl,-rpath,$ORIGIN/..", f"-Wl,-rpath,{CUDA_HOME / 'lib64'}"])
    return HOST_TOOL


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        build_host_tool()
        return LIB
    objects = []
    build_dir = HERE / "build"
    build_dir.mkdir(exist_ok=True)
    procs = []
    for src in sources():
        obj = build_dir / (src.stem + ".o")
        cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if out.strip() and (verbose or p.returncode):
            print(f"--- {src.name}\n{out}", file=sys.stderr)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([NVCC, "-shared", "-o", str(LIB), *map(str, objects), "-lcudart"])
    build_host_tool(force=True)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
