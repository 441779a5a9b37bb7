"""Builds the C++ operator layer on top of libgie_b200.so (no GPU needed):
  cpp/build/libgie.so            the drop-in C++ API (namespace gie, headers in cpp/include)
  cpp/build/libgie_testing.so    TEST SUPPORT: reference.h / testing.h surface on top of the C test oracle
  cpp/build/gie_api_tests        GPU tests of the C++ layer (run by tests/test_cpp_layer.py)
  cpp/build/example_quickstart   the example in cpp/examples
  cpp/build/reference_quickstart the reference's own examples/quickstart.cpp compiled UNCHANGED against these headers,
                                 only where the reference checkout exists (drop-in check; nothing is copied)
Usage: python build_cpp.py [--force]"""
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

INC = ["-I" + os.path.join(HERE, "include"), "-I" + os.path.join(ROOT, "include")]
TEST_INC = INC + ["-I" + os.path.join(HERE, "testing", "include"), "-I" + os.path.join(HERE, "tests")]
COMMON = ["-std=c++17", "-O2", "-Xcompiler", "-fPIC,-Wall", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"]
RPATH = ["-Xlinker", "-rpath," + OUT, "-Xlinker", "-rpath," + PKG, "-Xlinker", "-rpath," + os.path.join(ROOT, "oracle")]


def stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def files(*dirs, ext=(".h", ".cpp", ".cu", ".c")):
    out = []
    for d in dirs:
        for base, _, names in os.walk(d):
            out += [os.path.join(base, n) for n in names if n.endswith(ext)]
    return out


def run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("build step failed")


def build(force=False):
    os.makedirs(OUT, exist_ok=True)
    core = os.path.join(PKG, "libgie_b200.so")
    if not os.path.exists(core):
        subprocess.check_call([sys.executable, os.path.join(PKG, "build.py")])
    oracle = os.path.join(ROOT, "oracle", "libgie_oracle.so")
    if not os.path.exists(oracle):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle")], stdout=subprocess.DEVNULL)
    hdrs = files(os.path.join(HERE, "include"), os.path.join(HERE, "testing", "include"), os.path.join(HERE, "tests"), ext=(".h",))
    hdrs.append(os.path.join(ROOT, "include", "gie_b200.h"))

    libgie = os.path.join(OUT, "libgie.so")
    srcs = sorted(files(os.path.join(HERE, "src"), ext=(".cpp",)))
    if force or stale(libgie, srcs + hdrs + [core]):
        run([NVCC] + COMMON + INC + ["-shared", "-cudart", "shared", "-o", libgie] + srcs + [core] + RPATH)

    libtest = os.path.join(OUT, "libgie_testing.so")
    tsrc = os.path.join(HERE, "testing", "testing.cpp")
    if force or stale(libtest, [tsrc, libgie, oracle] + hdrs):
        run([NVCC] + COMMON + TEST_INC + ["-shared", "-cudart", "shared", "-o", libtest, tsrc, libgie, oracle] + RPATH)

    link = [libtest, libgie, core, oracle, "-cudart", "shared"] + RPATH
    tests = os.path.join(OUT, "gie_api_tests")
    tcu = os.path.join(HERE, "tests", "test_api.cu")
    if force or stale(tests, [tcu, libtest, libgie] + hdrs):
        run([NVCC] + COMMON + TEST_INC + ["-o", tests, tcu] + link)
    ex = os.path.join(OUT, "example_quickstart")
    exsrc = os.path.join(HERE, "examples", "quickstart.cpp")
    if force or stale(ex, [exsrc, libtest, libgie] + hdrs):
        run([NVCC] + COMMON + TEST_INC + ["-o", ex, exsrc] + link)
    refq = os.path.join(REF, "examples", "quickstart.cpp")
    if os.path.exists(refq):
        exe = os.path.join(OUT, "reference_quickstart")
        if force or stale(exe, [refq, libtest, libgie] + hdrs):
            run([NVCC] + COMMON + TEST_INC + ["-o", exe, refq] + link)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
