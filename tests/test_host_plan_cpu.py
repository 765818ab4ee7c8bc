"""CPU: the slice planner of the host-streamed step (nabla_b200/csrc/host_plan.h) against a chunk-by-chunk
restatement of the kernels' chunk geometry (tests/host_plan_test.cpp)."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_slice_plan_covers_every_element_exactly_once(tmp_path):
    exe = str(tmp_path / "host_plan_test")
    r = subprocess.run(["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-o", exe,
                        os.path.join(ROOT, "tests", "host_plan_test.cpp")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "HOST_PLAN_OK" in r.stdout, r.stdout + r.stderr
