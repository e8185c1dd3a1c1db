"""The header-only C++ front end (include/cinn_b200_frontend.hpp): tests/cpp/computation_test.cc, written the way
the reference's cinn/frontend/computation_test.cc is, compiled with g++ against the library.  Planned on CPU (no
GPU touched), executed on the GPU."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build(tmp_path):
    import cinn_b200
    cinn_b200.lib()   # builds the library if needed
    exe = str(tmp_path / "computation_test")
    gxx = shutil.which("g++")
    if not gxx:
        pytest.skip("no g++")
    libdir = os.path.join(ROOT, "cinn_b200")
    subprocess.run([gxx, "-std=c++17", "-O1", "-Wall", "-I" + os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "computation_test.cc"), "-o", exe, "-L" + libdir, "-lcinn_b200",
                    "-Wl,-rpath," + libdir], check=True)
    return exe


def test_cpp_program_plans_without_a_gpu(tmp_path):
    out = subprocess.run([build(tmp_path), "plan"], capture_output=True, text=True)
    assert out.returncode == 0 and "PLANNED" in out.stdout, out.stdout + out.stderr
    assert "transpose_vec_b4" in out.stdout and "row_reduce" in out.stdout and "ew_chain_bool" in out.stdout


@pytest.mark.gpu
def test_cpp_program_runs_and_checks_itself(tmp_path):
    out = subprocess.run([build(tmp_path), "run"], capture_output=True, text=True)
    assert out.returncode == 0 and "PASSED" in out.stdout, out.stdout + out.stderr
