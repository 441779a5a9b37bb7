"""Builds the reference library's OWN host layer, unmodified, on top of libgie_b200.so (no GPU needed).

Where the reference checkout exists (the directory GIE_REFERENCE_DIR names), its host sources -- plan cache,
ExecutionPlan, dispatcher and cost model, CUDA-graph executor, autotuner and tune cache, timing, CPU oracle, test helpers --
are compiled from where they lie, with plain nvcc (its CMake build is not used), together with ONE file of this
repository, cpp/src/b200_family.cpp, which stands in for the reference's kernels/*.cu, transformer/rmsnorm.cu and
kernels/elementwise.cu.  Nothing of the reference is copied.  Outputs, all under cpp/build/ (built artefacts: they travel
to a GPU machine with the tree, the checkout does not have to):
  libgie_refhost.so        the reference's C++ API with the sm_100a family behind its plug-in table
  ref_<name>               the reference's own test programs and quickstart example, compiled unchanged against it
                           (the ones that do not name legacy kernels: see REF_TESTS)
Usage: python build_refhost.py [--force]"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
OUT = os.path.join(HERE, "build")
REF = os.environ.get("GIE_REFERENCE_DIR", "/root/reference")
NVCC = os.environ.get("NVCC") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else "nvcc")

# The reference's host layer: every source of its library target except the legacy kernels (src/kernels/*_conv.cu,
# im2col.cu, implicit_gemm.cu, tensor_core_*.cu, elementwise.cu) and src/transformer/rmsnorm.cu.  build_info.cpp includes
# a header the reference's CMake build generates from cmake/gie_build_info.h.in; write_build_info() fills the same
# template here.
REF_SOURCES = [
    "src/cpu/cpu_reference.cpp", "src/runtime/error.cpp", "src/runtime/tensor.cpp", "src/runtime/device_info.cpp",
    "src/runtime/conv2d.cpp", "src/runtime/registry.cpp", "src/runtime/execution_plan.cpp", "src/runtime/dispatcher.cpp",
    "src/runtime/perf_model.cpp", "src/runtime/timing.cpp", "src/runtime/json_lite.cpp", "src/runtime/cuda_graph.cpp", "src/runtime/build_info.cpp",
    "src/runtime/reference.cu", "src/runtime/testing.cu", "src/kernels/conv_common.cu", "src/autotuner/tune_cache.cpp",
    "src/autotuner/autotuner.cpp", "src/profiling/ceilings.cu",
]
# Test programs of the reference that address kernels through the plug-in table's generic queries (backend, precision)
# and not by the names of legacy kernels; they are compiled unchanged.
REF_TESTS = ["tests/test_cpu_reference.cpp", "tests/test_rmsnorm.cpp", "tests/test_tensor_core.cpp", "tests/test_implicit_gemm.cpp"]
REF_EXAMPLES = ["examples/quickstart.cpp"]

COMMON = ["-std=c++17", "-O2", "-Xcompiler", "-fPIC,-fopenmp", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"]


def available() -> bool:
    return os.path.exists(os.path.join(REF, "src", "runtime", "registry.cpp"))


def stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("build step failed")


def write_build_info(gen_dir):
    """configure_file(cmake/gie_build_info.h.in ... @ONLY) of the reference's CMakeLists.txt:110, done by hand."""
    os.makedirs(gen_dir, exist_ok=True)
    with open(os.path.join(REF, "cmake", "gie_build_info.h.in")) as f:
        text = f.read()
    try:
        nvcc_version = subprocess.run([NVCC, "--version"], capture_output=True, text=True).stdout.strip().splitlines()[-2].split("release")[-1].strip()
    except Exception:
        nvcc_version = "unknown"
    values = {"GIE_SOURCE_FINGERPRINT": "reference host sources + b200_family.cpp", "CMAKE_BUILD_TYPE": "Release", "GIE_CUDA_ARCHS_STR": "100a",
              "CMAKE_CUDA_COMPILER_VERSION": nvcc_version, "CMAKE_CXX_COMPILER_ID": "GNU", "CMAKE_CXX_COMPILER_VERSION": "",
              "GIE_CUDA_FLAGS_FULL": " ".join(COMMON), "GIE_CXX_FLAGS_FULL": ""}
    for k, v in values.items():
        text = text.replace("@" + k + "@", v)
    path = os.path.join(gen_dir, "gie_build_info.h")
    if not os.path.exists(path) or open(path).read() != text:
        with open(path, "w") as f:
            f.write(text)


def build(force=False):
    if not available():
        return None
    os.makedirs(OUT, exist_ok=True)
    gen = os.path.join(OUT, "refhost_generated")
    write_build_info(gen)
    core = os.path.join(PKG, "libgie_b200.so")
    if not os.path.exists(core):
        subprocess.check_call([sys.executable, os.path.join(PKG, "build.py")])
    inc = ["-I" + os.path.join(REF, "include"), "-I" + os.path.join(ROOT, "include"), "-I" + gen]
    rpath = ["-Xlinker", "-rpath," + OUT, "-Xlinker", "-rpath," + PKG]
    family = os.path.join(HERE, "src", "b200_family.cpp")
    lib = os.path.join(OUT, "libgie_refhost.so")
    srcs = [os.path.join(REF, s) for s in REF_SOURCES]
    if force or stale(lib, srcs + [family, core, os.path.join(ROOT, "include", "gie_b200.h")]):
        run([NVCC] + COMMON + inc + ["-DGIE_B200_REPLACES_LEGACY_BACKENDS", "-shared", "-cudart", "shared", "-o", lib] + srcs
            + [family, "-L" + PKG, "-lgie_b200", "-lgomp"] + rpath)
    link = ["-L" + OUT, "-lgie_refhost", "-L" + PKG, "-lgie_b200", "-cudart", "shared", "-lgomp"] + rpath
    tinc = inc + ["-I" + os.path.join(REF, "tests")]
    for rel in REF_TESTS + REF_EXAMPLES:
        src = os.path.join(REF, rel)
        exe = os.path.join(OUT, "ref_" + os.path.splitext(os.path.basename(rel))[0])
        if os.path.exists(src) and (force or stale(exe, [src, lib])):
            run([NVCC] + COMMON + tinc + ["-o", exe, src] + link)
    # this repository's own test program of the C++ layer (the reference's test cases that name kernels, restated for the
    # names of this family) and its example, against the same headers and library
    own = [(os.path.join(HERE, "tests", "test_api.cu"), "gie_api_tests"), (os.path.join(HERE, "examples", "quickstart.cpp"), "example_quickstart")]
    hdrs = [os.path.join(HERE, "tests", n) for n in ("check.h", "test_support.h")]
    for src, name in own:
        exe = os.path.join(OUT, name)
        if force or stale(exe, [src, lib] + hdrs):
            run([NVCC] + COMMON + inc + ["-I" + os.path.join(HERE, "tests"), "-o", exe, src] + link)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
