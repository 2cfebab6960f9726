"""Builds every native artefact of the repository, in-tree.

  cudadma_b200/libcudadma_b200.so      the product: kernels + C ABI (nvcc, sm_100a)
  tests/csrc/libcudadma_apitest.so     test kernels that drive the object API one CTA at a time
  oracle/liboracle.so                  CPU oracle (gcc)
  oracle/_ref/libcudadma_ref.so        the benchmark workloads through the reference CudaDMA
                                       headers compiled for sm_100a (only where the reference
                                       checkout is present; `make -C oracle ref-apitest` adds the
                                       API harness against the reference, which takes very long)

nvcc cross-compiles without a GPU; nothing here needs one.
"""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-shared"] + ARCH
REFERENCE_INCLUDE = os.environ.get("CUDADMA_REFERENCE_INCLUDE", "/root/reference/include")


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def _run(cmd):
    print("[build]", " ".join(cmd), flush=True)
    subprocess.check_call(cmd, cwd=ROOT)


def _glob(*dirs):
    out = []
    for d in dirs:
        p = os.path.join(ROOT, d)
        for f in sorted(os.listdir(p)):
            if f.endswith((".cu", ".cuh", ".h", ".c")):
                out.append(os.path.join(p, f))
    return out


def build_library(force=False):
    target = os.path.join(ROOT, "cudadma_b200", "libcudadma_b200.so")
    srcs = _glob("cudadma_b200/csrc", "include", "include/cudadma")
    if force or _newer(target, srcs):
        _run([NVCC] + NVCC_FLAGS + ["-Iinclude", "-Iinclude/cudadma", "-Icudadma_b200/csrc", "-o", target,
                                    "cudadma_b200/csrc/capi.cu"])
    return target


def build_apitest(force=False):
    target = os.path.join(ROOT, "tests", "csrc", "libcudadma_apitest.so")
    srcs = _glob("tests/csrc", "include/cudadma")
    if force or _newer(target, srcs):
        _run([NVCC] + NVCC_FLAGS + ["-Iinclude/cudadma", "-Icudadma_b200/csrc", "-DAPITEST_PREFIX=apitest_",
                                    "-o", target, "tests/csrc/api_harness.cu"])
    return target


def build_checked_probe(force=False):
    """One small kernel against the -DCUDADMA_CHECKED build of the header (tests/csrc/checked_probe.cu)."""
    target = os.path.join(ROOT, "tests", "csrc", "libcudadma_checked_probe.so")
    srcs = [os.path.join(ROOT, "tests", "csrc", "checked_probe.cu")] + _glob("include/cudadma")
    if force or _newer(target, srcs):
        _run([NVCC] + NVCC_FLAGS + ["-Iinclude/cudadma", "-o", target, "tests/csrc/checked_probe.cu"])
    return target


def build_oracle(force=False):
    target = os.path.join(ROOT, "oracle", "liboracle.so")
    srcs = [os.path.join(ROOT, "oracle", "oracle.c")]
    if force or _newer(target, srcs):
        _run(["make", "-C", "oracle", "liboracle.so"])
    return target


def build_reference(force=False):
    """The reference classes compiled for sm_100a from the checkout, outputs into oracle/_ref/."""
    if not os.path.isdir(REFERENCE_INCLUDE):
        return None
    _run(["make", "-C", "oracle", "ref", "REFERENCE_INCLUDE=" + REFERENCE_INCLUDE] + (["-B"] if force else []))
    return os.path.join(ROOT, "oracle", "_ref")


def build_all(force=False, reference=True):
    out = [build_library(force), build_apitest(force), build_checked_probe(force), build_oracle(force)]
    if reference:
        out.append(build_reference(force))
    return out


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
