"""The C++ operator API on top of the C ABI: the reference library's OWN host layer (plan cache, ExecutionPlan, dispatcher,
CUDA-graph executor, autotuner, tune cache), compiled unmodified from the reference checkout with ONE file of this
repository (cuda-inference_b200/cpp/src/b200_family.cpp) in place of its kernels.  Run here: the reference's own test
programs and example (the tests in them that address kernels through the plug-in table rather than by legacy kernel
names), and this repository's restatement of the name-bound ones (cpp/tests/test_api.cu).

The programs are built where the reference checkout exists (build_refhost.py); the built files travel with the tree.
Where neither the checkout nor the built files exist, these tests skip."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "cuda-inference_b200", "cpp")
OUT = os.path.join(CPP, "build")

# program -> name filters of the tests to run (None = all).  The reference's harness runs the tests whose name contains
# its first argument (tests/test_util.h:99-103).  Left out: tests that look kernels up by legacy names
# ("im2col_gemm_fp32", "tcmma_...") or assert properties of the legacy WMMA kernel (no workspace).
REFERENCE_PROGRAMS = {
    "ref_test_cpu_reference": [None],
    "ref_test_rmsnorm": [None],
    "ref_test_tensor_core": ["tensor_core_fp16_bf16_all_configs", "tensor_core_unsupported_for_fp32",
                             "tensor_core_vector_and_scalar_weight_paths", "tensor_core_large_reduction_k4608"],
    "ref_test_implicit_gemm": ["implicit_gemm_fp32_fp16_all_configs", "implicit_gemm_all_distributions_one_shape"],
}


def _built():
    if not os.path.exists(os.path.join(OUT, "libgie_refhost.so")):
        sys.path.insert(0, CPP)
        import build_refhost
        if not build_refhost.available():
            pytest.skip("neither the reference checkout nor the built C++ layer is present")
        build_refhost.build()
    return OUT


def _run(path, *args, timeout=1200):
    r = subprocess.run([path, *args], capture_output=True, text=True, timeout=timeout)
    sys.stdout.write(r.stdout[-3000:])
    sys.stderr.write(r.stderr[-3000:])
    return r


def test_cpp_layer_builds_without_a_gpu():
    out = _built()
    for name in ("libgie_refhost.so", "gie_api_tests", "example_quickstart", "ref_quickstart", *REFERENCE_PROGRAMS):
        assert os.path.exists(os.path.join(out, name)), name
    syms = subprocess.check_output(["nm", "-DC", "--defined-only", os.path.join(out, "libgie_refhost.so")], text=True)
    for needed in ("gie::Conv2D::forward", "gie::Conv2D::workspace_size", "gie::ExecutionPlan::create", "gie::ExecutionPlan::execute_unchecked",
                   "gie::CudaGraphExecutor::capture", "gie::rmsnorm_forward", "gie::validate_problem", "gie::kernel_registry",
                   "gie::find_kernel", "gie::Dispatcher::select", "gie::launch_bias_act", "gie::DeviceInfo::get",
                   "gie::kernels::register_b200_family", "gie::Autotuner::tune"):
        assert needed in syms, needed
    # the CPU oracle tests of the reference need no GPU
    r = _run(os.path.join(out, "ref_test_cpu_reference"))
    assert r.returncode == 0 and " 0 failures" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("program", sorted(REFERENCE_PROGRAMS))
def test_reference_test_programs(program):
    """The reference's own tests, compiled unchanged, pass on the sm_100a family through the reference's own host code and
    against the reference's own oracle and tolerance policy."""
    out = _built()
    for flt in REFERENCE_PROGRAMS[program]:
        r = _run(os.path.join(out, program), *([flt] if flt else []))
        assert r.returncode == 0, f"{program} {flt or ''}: {r.stdout[-1500:]}"
        assert " 0 failures" in r.stdout


@pytest.mark.gpu
def test_cpp_api_test_program():
    out = _built()
    r = _run(os.path.join(out, "gie_api_tests"), timeout=900)
    assert r.returncode == 0, "C++ layer tests failed"
    assert " 0 failures" in r.stdout


@pytest.mark.gpu
def test_cpp_quickstart_examples():
    out = _built()
    for exe in ("example_quickstart", "ref_quickstart"):
        r = _run(os.path.join(out, exe), timeout=300)
        assert r.returncode == 0, exe + ": " + r.stdout + r.stderr
        assert "output [" in r.stdout
