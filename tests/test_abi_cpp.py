"""The C ABI from C++: `tests/abi/abi_check.cpp` is compiled against `include/frink_b200.h` and linked to
`libfrink_b200.so` (no Python in the process that calls the library).  Without a GPU the program runs the
calls that need no device; on a GPU it runs matvecs through the host-buffer surface."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build(tmp_path):
    from frink_b200 import build as fb
    fb.build()
    libdir = os.path.join(ROOT, "frink_b200")
    exe = str(tmp_path / "abi_check")
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", os.path.join(ROOT, "tests", "abi", "abi_check.cpp"), "-I", os.path.join(ROOT, "include"),
           "-L", libdir, "-lfrink_b200", f"-Wl,-rpath,{libdir}", "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_cpp_program_links_and_runs_without_a_device(tmp_path):
    exe = build(tmp_path)
    r = subprocess.run([exe, "nogpu"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "abi_check: ok" in r.stdout


@pytest.mark.gpu
def test_cpp_program_runs_matvecs_through_the_host_buffer_surface(tmp_path):
    exe = build(tmp_path)
    r = subprocess.run([exe, "gpu"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "abi_check: ok" in r.stdout
