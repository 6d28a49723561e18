"""Build recipe for the CUDA library (nvcc, sm_100a only, in-tree output)."""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libb200gemm.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "b200gemm.h"))
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu under csrc/ into libb200gemm.so for sm_100a."""
    if not force and not needs_build():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB_PATH, *sources()]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    env = dict(os.environ)
    # The image exports CC/CXX pointing at a compiler wrapper; nvcc must use the system g++.
    for var in ("CC", "CXX"):
        env.pop(var, None)
    subprocess.check_call(cmd, env=env)
    return LIB_PATH


COMPARATOR_SRC = os.path.join(HERE, "comparator", "cublaslt_compare.cpp")
COMPARATOR_LIB = os.path.join(HERE, "comparator", "libcublaslt_compare.so")


def build_comparator(force: bool = False) -> str | None:
    """The benchmark's cuBLASLt column (never loaded by the package).  Returns None where the
    toolkit has no cuBLASLt to link against."""
    cuda = os.path.dirname(os.path.dirname(_nvcc()))
    if not os.path.exists(os.path.join(cuda, "include", "cublasLt.h")):
        return None
    if (not force and os.path.exists(COMPARATOR_LIB)
            and os.path.getmtime(COMPARATOR_LIB) >= os.path.getmtime(COMPARATOR_SRC)):
        return COMPARATOR_LIB
    env = dict(os.environ)
    for var in ("CC", "CXX"):
        env.pop(var, None)
    lib_dir = os.path.join(cuda, "lib64")
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")
    subprocess.check_call([gxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
                           "-I" + os.path.join(cuda, "include"), "-o", COMPARATOR_LIB, COMPARATOR_SRC,
                           "-L" + lib_dir, "-lcublasLt", "-lcudart", "-Wl,-rpath," + lib_dir], env=env)
    return COMPARATOR_LIB


if __name__ == "__main__":
    print(build(force=True, verbose=True))
