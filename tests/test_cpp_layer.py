"""Runs the C++ operator layer's own test program (cuda-inference_b200/cpp/tests/test_api.cu) and examples on the GPU.
The program restates the hot-path subset of the reference's C++ tests against this library's registry."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "cuda-inference_b200", "cpp")
OUT = os.path.join(CPP, "build")


def _built():
    if not os.path.exists(os.path.join(OUT, "gie_api_tests")):
        subprocess.check_call([sys.executable, os.path.join(CPP, "build_cpp.py")])
    return OUT


def test_cpp_layer_builds_without_a_gpu():
    out = _built()
    for name in ("libgie.so", "libgie_testing.so", "gie_api_tests", "example_quickstart"):
        assert os.path.exists(os.path.join(out, name)), name
    syms = subprocess.check_output(["nm", "-DC", "--defined-only", os.path.join(out, "libgie.so")], text=True)
    for needed in ("gie::Conv2D::forward", "gie::Conv2D::workspace_size", "gie::ExecutionPlan::create", "gie::ExecutionPlan::execute_unchecked",
                   "gie::CudaGraphExecutor::capture", "gie::rmsnorm_forward", "gie::validate_problem", "gie::kernel_registry",
                   "gie::find_kernel", "gie::Dispatcher::select", "gie::launch_bias_act", "gie::DeviceInfo::get"):
        assert needed in syms, needed


@pytest.mark.gpu
def test_cpp_api_test_program():
    out = _built()
    r = subprocess.run([os.path.join(out, "gie_api_tests")], capture_output=True, text=True, timeout=900)
    sys.stdout.write(r.stdout[-6000:])
    sys.stderr.write(r.stderr[-6000:])
    assert r.returncode == 0, "C++ layer tests failed"
    assert " 0 failures" in r.stdout


@pytest.mark.gpu
def test_cpp_quickstart_examples():
    out = _built()
    for exe in ("example_quickstart", "reference_quickstart"):
        path = os.path.join(out, exe)
        if not os.path.exists(path):
            continue  # the reference's own quickstart is only compiled where the reference checkout exists
        r = subprocess.run([path], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, exe + ": " + r.stdout + r.stderr
        assert "output [" in r.stdout
