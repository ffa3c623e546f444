"""Build recipe for the native pieces: explicit nvcc / g++ command lines, outputs in-tree.

  libcudarl.so          cudarl-arena_b200/csrc/{kernels.cu,context.cu,update_static.cu,facade.cpp}  (sm_100a only)
  cudarl_core*.so       pybind11 module with the reference's `cudarl_core` surface
  oracle/liboracle.so   the CPU oracle (test infrastructure)
  oracle/_ref/libref.so the reference's own kernels, compiled from the reference checkout when it
                        is present on this machine (never copied into this repository)
  tests/cpp/facade_consumer   C++ test program written against the reference's header names (csrc/compat/)
  oracle/_ref/ref_main_demo   the reference's own src/main.cu, compiled unmodified against csrc/compat/ (same condition)

Run as a script (`python cudarl-arena_b200/build.py`) or through `__graft_entry__.build()`.
"""
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcudarl.so")
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_LIB = os.path.join(ORACLE_DIR, "liboracle.so")
REF_DIR = os.path.join(ORACLE_DIR, "_ref")
REF_LIB = os.path.join(REF_DIR, "libref.so")
# The reference checkout is only read, and only at build time: CUDARL_REFERENCE_SRC names its src/ directory (default: a
# checkout called `reference` beside this repository).
REFERENCE_SRC = os.environ.get("CUDARL_REFERENCE_SRC", os.path.join(os.path.dirname(ROOT), "reference", "src"))
CONSUMER = os.path.join(ROOT, "tests", "cpp", "facade_consumer")
REF_DEMO = os.path.join(REF_DIR, "ref_main_demo")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "-Xptxas", "-v"] + ARCH


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd, log=None):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log:
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("build command failed: " + " ".join(cmd))
    return r.stdout


def build_lib(force=False):
    srcs = [os.path.join(CSRC, f) for f in ("kernels.cu", "tile_engine.cu", "context.cu", "update_static.cu", "facade.cpp")]
    deps = srcs + [os.path.join(CSRC, "kernels.cuh"), os.path.join(CSRC, "rules.cuh"), os.path.join(CSRC, "facade.h"), os.path.join(ROOT, "include", "cudarl.h")]
    deps = [d for d in deps if os.path.exists(d)]
    srcs = [s for s in srcs if os.path.exists(s)]
    if not force and _newer(LIB, deps):
        return LIB
    cmd = [_nvcc()] + NVCC_FLAGS + ["-shared", "-o", LIB] + srcs + ["-I" + os.path.join(ROOT, "include"), "-ldl"]
    _run(cmd, log=os.path.join(HERE, "build_libcudarl.log"))
    return LIB


def pybind_module_path():
    return os.path.join(HERE, "cudarl_core" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_pybind(force=False):
    src = os.path.join(CSRC, "pybind_module.cpp")
    if not os.path.exists(src):
        return None
    out = pybind_module_path()
    deps = [src, os.path.join(CSRC, "facade.h"), LIB]
    if not force and _newer(out, deps):
        return out
    import pybind11
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", src, "-o", out,
           "-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"], "-I" + os.path.join(ROOT, "include"),
           "-L" + HERE, "-lcudarl", "-Wl,-rpath,$ORIGIN"]
    _run(cmd)
    return out


def build_oracle(force=False):
    src = os.path.join(ORACLE_DIR, "oracle.cpp")
    if not force and _newer(ORACLE_LIB, [src, os.path.join(ROOT, "include", "cudarl.h")]):
        return ORACLE_LIB
    # -ffp-contract=off: the fused multiply-adds of the oracle are the explicit fmaf calls only.
    _run(["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-fPIC", "-shared", "-pthread", "-o", ORACLE_LIB, src])
    return ORACLE_LIB


def build_ref(force=False):
    """The reference's own step / TD-update kernels + a small launcher, for cross-checks on a GPU.
    Built only where the reference checkout exists; the prebuilt .so travels with the tree."""
    harness = os.path.join(ORACLE_DIR, "ref_harness.cu")
    if not os.path.isdir(REFERENCE_SRC) or not os.path.exists(harness):
        return REF_LIB if os.path.exists(REF_LIB) else None
    srcs = [harness, os.path.join(REFERENCE_SRC, "kernels.cu"), os.path.join(REFERENCE_SRC, "environment.cu"),
            os.path.join(REFERENCE_SRC, "gpu", "kernels.cu")]   # the last three are #included by the harness
    if not force and _newer(REF_LIB, srcs):
        return REF_LIB
    os.makedirs(REF_DIR, exist_ok=True)
    # the reference's own flags (CMakeLists.txt:67-72) except the architecture list
    cmd = [_nvcc(), "-O2", "-std=c++17", "--use_fast_math", "-Xcompiler", "-fPIC", "-shared"] + ARCH + \
          ["-I" + REFERENCE_SRC, "-o", REF_LIB, harness]
    _run(cmd)
    return REF_LIB


def build_consumer(force=False):
    """tests/cpp/facade_consumer: a C++ program written against the reference's header names, linked with libcudarl.so."""
    src = os.path.join(ROOT, "tests", "cpp", "facade_consumer.cpp")
    if not os.path.exists(src):
        return None
    deps = [src, os.path.join(CSRC, "facade.h"), LIB]
    if not force and _newer(CONSUMER, deps):
        return CONSUMER
    _run(["g++", "-O1", "-std=c++17", src, "-o", CONSUMER, "-I" + os.path.join(CSRC, "compat"), "-L" + HERE, "-lcudarl",
          "-Wl,-rpath,$ORIGIN/../../cudarl-arena_b200"])
    return CONSUMER


def build_ref_demo(force=False):
    """The reference's own demo program src/main.cu, compiled UNMODIFIED from where it lies against this library's
    compatibility headers (same include names).  Only where the reference checkout exists; the binary travels."""
    src = os.path.join(REFERENCE_SRC, "main.cu")
    if not os.path.exists(src):
        return REF_DEMO if os.path.exists(REF_DEMO) else None
    if not force and _newer(REF_DEMO, [src, os.path.join(CSRC, "facade.h"), LIB]):
        return REF_DEMO
    os.makedirs(REF_DIR, exist_ok=True)
    # `#include "environment.h"` looks beside the including file first, which would find the reference's own headers: the file
    # is therefore compiled from a scratch directory outside this repository (byte-identical, removed afterwards).
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        scratch = os.path.join(tmp, "main.cu")
        shutil.copyfile(src, scratch)
        _run([_nvcc(), "-O1", "-std=c++17"] + ARCH + ["-I" + os.path.join(CSRC, "compat"), "-o", REF_DEMO, scratch, "-L" + HERE, "-lcudarl",
              "-Xlinker", "-rpath,$ORIGIN/../../cudarl-arena_b200"])
    return REF_DEMO


def build_all(force=False):
    out = {"lib": build_lib(force), "oracle": build_oracle(force)}
    out["pybind"] = build_pybind(force)
    out["consumer"] = build_consumer(force)
    try:
        out["ref_demo"] = build_ref_demo(force)
    except RuntimeError as e:
        out["ref_demo"] = None
        sys.stderr.write("reference demo not built: %s\n" % e)
    try:
        out["ref"] = build_ref(force)
    except RuntimeError as e:  # the reference cross-check is optional
        out["ref"] = None
        sys.stderr.write("reference harness not built: %s\n" % e)
    return out


if __name__ == "__main__":
    for k, v in build_all(force="--force" in sys.argv).items():
        print(k, "->", v)
