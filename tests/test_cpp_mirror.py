"""The C++ host mirror (include/MetalDSP.hpp) compiled with g++ against the C-ABI library.
CPU: it builds, links and its host logic / no-device behaviour hold.  GPU: its known-answer tests
pass on the device."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "mirror_test.cpp")
EXE = os.path.join(ROOT, "tests", "cpp", "mirror_test")


@pytest.fixture(scope="module")
def exe(lib):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not available")
    libdir = os.path.join(ROOT, "metalaudio_b200")
    deps = [SRC, os.path.join(ROOT, "include", "MetalDSP.hpp"), os.path.join(ROOT, "include", "metalaudio_cuda.h")]
    if not os.path.exists(EXE) or any(os.path.getmtime(d) > os.path.getmtime(EXE) for d in deps):
        subprocess.run([gxx, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), SRC, "-o", EXE,
                        "-L", libdir, "-l:libmetalaudio_cuda.so", f"-Wl,-rpath,{libdir}"], check=True)
    return EXE


def test_cpp_mirror_host_logic(exe):
    r = subprocess.run([exe, "--host-only"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_cpp_mirror_on_gpu(exe):
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout + r.stderr
