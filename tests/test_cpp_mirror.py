"""The C++ mirror of the Backend interface (include/hc_cuda.hpp): it compiles and links against
the C-ABI library on a machine without a GPU, and on a GPU its conformance program - the
reference's known-answer tests in C++ - passes."""
import os
import subprocess

import pytest

from honeycrisp_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "backend_conformance")


def build_conformance():
    _lib.load()
    libdir = os.path.dirname(_lib.lib_path())
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", f"-I{ROOT}/include",
           os.path.join(ROOT, "tests", "cpp", "backend_conformance.cpp"), "-o", BIN, f"-L{libdir}", "-lhccuda",
           f"-Wl,-rpath,{libdir}", "-ldl", "-lpthread", "-lrt"]
    subprocess.check_call(cmd)
    return BIN


GROUP_BIN = os.path.join(ROOT, "tests", "cpp", "group_conformance")


def build_group_conformance():
    _lib.load()
    libdir = os.path.dirname(_lib.lib_path())
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", f"-I{ROOT}/include",
           os.path.join(ROOT, "tests", "cpp", "group_conformance.cpp"), "-o", GROUP_BIN, f"-L{libdir}", "-lhccuda",
           f"-Wl,-rpath,{libdir}", "-ldl", "-lpthread", "-lrt"]
    subprocess.check_call(cmd)
    return GROUP_BIN


def test_group_program_compiles_and_links_without_python_or_torch():
    assert os.path.exists(build_group_conformance())


@pytest.mark.gpu
def test_group_program_passes_on_every_visible_device():
    """The multi-device entry points driven from plain C++ threads, one per GPU (up to four, to
    keep it short; a single GPU runs a group of one)."""
    exe = build_group_conformance()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([exe, "4"], capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "group conformance ok" in out.stdout


def test_cpp_mirror_compiles_and_links():
    assert os.path.exists(build_conformance())


@pytest.mark.gpu
def test_cpp_conformance_program_passes_on_the_device():
    exe = build_conformance()
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "conformance ok" in out.stdout
