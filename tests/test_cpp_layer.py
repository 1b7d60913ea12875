"""The C++ poplar / poplin layer: host-only checks (graph construction, options,
ConvParams algebra) run here without a GPU; the tool ports run on the GPU and
their dumped tensors are compared with the oracle."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "poplibs_b200")


def compile_cpp(source, output):
    from poplibs_b200 import build
    build.build_poplin()
    cmd = ["g++", "-std=c++17", "-O1", "-I" + os.path.join(ROOT, "include"), source, "-o", output,
           "-L" + LIBDIR, "-lpoplin_b200", "-lpoplibs_b200", "-Wl,-rpath," + LIBDIR]
    subprocess.run(cmd, check=True)


def test_poplin_host_layer(tmp_path):
    exe = str(tmp_path / "test_poplin_host")
    compile_cpp(os.path.join(ROOT, "tests", "cpp", "test_poplin_host.cpp"), exe)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "all host checks passed" in out.stdout
