"""Builds libpoplibs_b200.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

    python -m poplibs_b200.build [--force]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libpoplibs_b200.so")
OBJ_DIR = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    inc = os.path.join(ROOT, "include")
    for d, _, fs in os.walk(inc):
        hs += [os.path.join(d, f) for f in fs if f.endswith((".h", ".hpp"))]
    return hs


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libpoplibs_b200.so")
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = _headers()
    objs = []
    procs = []
    for src in _sources():
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        if not force and _newer(obj, [path] + headers):
            continue
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose and out:
            print(out)
    if force or procs or not _newer(OUT, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", OUT] + objs
        subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))


POPLIN_OUT = os.path.join(HERE, "libpoplin_b200.so")
POPLIN_DIRS = [os.path.join(CSRC, "poplar"), os.path.join(CSRC, "poplin")]
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]


def build_poplin(force: bool = False) -> str:
    """The C++ poplar / poplin layer over the C ABI -> libpoplin_b200.so."""
    build()
    cxx = shutil.which("g++") or "g++"
    objs, procs = [], []
    headers = _headers()
    for d in POPLIN_DIRS:
        headers += [os.path.join(d, f) for f in os.listdir(d) if f.endswith((".hpp", ".h"))]
    for d in POPLIN_DIRS:
        for src in sorted(f for f in os.listdir(d) if f.endswith(".cpp")):
            path = os.path.join(d, src)
            obj = os.path.join(OBJ_DIR, "poplin_" + os.path.splitext(src)[0] + ".o")
            objs.append(obj)
            if not force and _newer(obj, [path] + headers):
                continue
            procs.append((src, subprocess.Popen([cxx] + CXX_FLAGS + ["-c", path, "-o", obj],
                                                stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"g++ failed on {src}:\n{out}")
    if force or procs or not _newer(POPLIN_OUT, objs + [OUT]):
        subprocess.run([cxx, "-shared", "-o", POPLIN_OUT] + objs +
                       ["-L" + HERE, "-lpoplibs_b200", "-Wl,-rpath,$ORIGIN"], check=True)
    return POPLIN_OUT


TOOLS_DIR = os.path.join(HERE, "tools")
TOOLS_BIN = os.path.join(TOOLS_DIR, "bin")


def build_tools(force: bool = False):
    """The driver tools (ports of the reference's single_conv_layer and
    general_matrix_multiply) -> poplibs_b200/tools/bin/."""
    build_poplin()
    cxx = shutil.which("g++") or "g++"
    os.makedirs(TOOLS_BIN, exist_ok=True)
    built = []
    deps = _headers() + [os.path.join(TOOLS_DIR, "tool_util.hpp"), POPLIN_OUT]
    for src in sorted(f for f in os.listdir(TOOLS_DIR) if f.endswith(".cpp")):
        exe = os.path.join(TOOLS_BIN, os.path.splitext(src)[0])
        path = os.path.join(TOOLS_DIR, src)
        if force or not _newer(exe, [path] + deps):
            subprocess.run([cxx] + CXX_FLAGS + ["-I" + TOOLS_DIR, path, "-o", exe, "-L" + HERE,
                            "-lpoplin_b200", "-lpoplibs_b200", "-Wl,-rpath,$ORIGIN/../.."], check=True)
        built.append(exe)
    return built
