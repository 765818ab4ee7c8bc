"""The C++ host mirror (nabla_b200/host/nabla_optim.hpp): compiles on CPU; on a GPU it runs the reference's
own optimizer tests (tests/host_kat.cpp, after nabla-train/tests/optim.rs and tests/trainer.rs)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = "/usr/local/cuda"


def build(tmp_path, nbo_lib):
    exe = str(tmp_path / "host_kat")
    libdir = os.path.join(ROOT, "nabla_b200")
    cmd = ["/usr/bin/g++", "-std=c++17", "-Wall", "-Werror", f"-I{CUDA}/include", "-o", exe,
           os.path.join(ROOT, "tests", "host_kat.cpp"), f"-L{libdir}", "-lnabla_optim_b200",
           f"-L{CUDA}/lib64", "-lcudart", f"-Wl,-rpath,{libdir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_cpp_host_mirror_compiles_and_links(tmp_path, nbo_lib):
    build(tmp_path, nbo_lib)


@pytest.mark.gpu
def test_reference_kats_through_the_cpp_mirror(tmp_path, nbo_lib):
    exe = build(tmp_path, nbo_lib)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "HOST_KAT_OK" in r.stdout, r.stdout + r.stderr
