"""The C++ host mirror (include/fusor_cuda.hpp) against the reference's own test cases (tests/cpp/reference_cases.cpp).
CPU: the header and the test program compile and the host-only checks pass.  GPU: the full program passes."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "reference_cases")


def _build():
    from floneum_b200 import build
    lib = build.build()
    src = os.path.join(ROOT, "tests", "cpp", "reference_cases.cpp")
    if not os.path.exists(EXE) or os.path.getmtime(EXE) < max(os.path.getmtime(src), os.path.getmtime(lib),
                                                               os.path.getmtime(os.path.join(ROOT, "include", "fusor_cuda.hpp"))):
        subprocess.run(["/usr/bin/g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), src, "-o", EXE,
                        "-L", os.path.dirname(lib), "-lfusor_cuda", "-Wl,-rpath," + os.path.dirname(lib)], check=True)
    return EXE


def test_cpp_mirror_compiles_and_host_checks_pass():
    exe = _build()
    res = subprocess.run([exe, "--no-gpu"], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr


@pytest.mark.gpu
def test_cpp_mirror_reference_cases_on_gpu():
    exe = _build()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "all reference cases passed" in res.stdout
