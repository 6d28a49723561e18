"""CPU checks of the boundary: the library loads without a GPU, exports every
symbol the header declares, the ctypes table matches the header, and the C++
host mirror compiles against it."""
import ctypes as C
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200gemm.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"B200GEMM_API\s+[\w\s\*]+?\b(b200gemm_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared_symbols()
    for must in ("b200gemm_create", "b200gemm_destroy", "b200gemm_gemm", "b200gemm_gemm_host",
                 "b200gemm_launch_config", "b200gemm_sgemm", "b200gemm_grouped_gemm",
                 "b200gemm_lmhead_ce_forward", "b200gemm_lmhead_ce_backward", "b200gemm_moe_route",
                 "b200gemm_device_status"):
        assert must in names


def test_library_loads_on_cpu_and_exports_every_declared_symbol(pkg):
    lib = pkg._lib.load()
    raw = C.CDLL(pkg._lib.LIB_PATH)
    for name in _declared_symbols():
        assert hasattr(raw, name), f"{name} is declared in b200gemm.h but not exported"
        assert name in pkg._lib.SIGNATURES, f"{name} has no ctypes signature"
    for name in pkg._lib.SIGNATURES:
        assert name in _declared_symbols(), f"{name} is bound but not declared in the header"
    assert lib.b200gemm_version() >= 100
    assert lib.b200gemm_last_error_string() is not None


def test_descriptor_struct_matches_the_c_layout(pkg):
    # b200gemm_desc_t: 3 pointers, 6 int64, 6 int32, 3 int64, 2 uint32 = 112 bytes, no padding surprises
    assert C.sizeof(pkg.GemmDesc) == 3 * 8 + 6 * 8 + 6 * 4 + 3 * 8 + 2 * 4
    probe = r'''
    #include <stdio.h>
    #include <stddef.h>
    #include "b200gemm.h"
    int main(void) {
      printf("%zu %zu %zu %zu\n", sizeof(b200gemm_desc_t), offsetof(b200gemm_desc_t, a_layout),
             offsetof(b200gemm_desc_t, batch_stride_a), offsetof(b200gemm_desc_t, flags));
      return 0;
    }'''
    gcc = shutil.which("gcc") or "/usr/bin/gcc"
    tmp = os.path.join(ROOT, "tests", "_abi_probe")
    try:
        with open(tmp + ".c", "w") as f:
            f.write(probe)
        env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
        subprocess.check_call([gcc, "-I", os.path.join(ROOT, "include"), tmp + ".c", "-o", tmp], env=env)
        size, off_layout, off_bsa, off_flags = map(int, subprocess.check_output([tmp]).split())
    finally:
        for ext in (".c", ""):
            if os.path.exists(tmp + ext):
                os.remove(tmp + ext)
    D = pkg.GemmDesc
    assert size == C.sizeof(D)
    assert off_layout == D.a_layout.offset
    assert off_bsa == D.batch_stride_a.offset
    assert off_flags == D.flags.offset


def test_cpp_host_mirror_compiles():
    gxx = shutil.which("g++") or "/usr/bin/g++"
    src = r'''
    #include "b200gemm.hpp"
    int use(void* stream) {
      b200gemm::Operand a, b;
      a.rows = 256; a.k = 64; b.rows = 256; b.k = 64;
      b200gemm::Tcgen05Gemm* g = nullptr;
      (void)g; (void)stream;
      return b200gemm::TC_M_TILE + (int)sizeof(b200gemm::Tcgen05Gemm);
    }'''
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    subprocess.run([gxx, "-std=c++17", "-fsyntax-only", "-Wall", "-I", os.path.join(ROOT, "include"),
                    "-x", "c++", "-"], input=src.encode(), check=True, env=env)


def test_create_fails_loudly_without_a_gpu(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError):
        pkg.Tcgen05Gemm()
    h = C.c_void_p()
    rc = pkg._lib.load().b200gemm_create(0, C.byref(h))
    assert rc != pkg._lib.OK and not h.value              # no device, no handle, no fallback
