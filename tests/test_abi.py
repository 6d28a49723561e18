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


def test_descriptor_struct_matches_the_c_layout(pkg, tmp_path):
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
    src, exe = tmp_path / "abi_probe.c", tmp_path / "abi_probe"
    src.write_text(probe)
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    subprocess.check_call([gcc, "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], env=env)
    size, off_layout, off_bsa, off_flags = map(int, subprocess.check_output([str(exe)]).split())
    D = pkg.GemmDesc
    assert size == C.sizeof(D)
    assert off_layout == D.a_layout.offset
    assert off_bsa == D.batch_stride_a.offset
    assert off_flags == D.flags.offset


def test_cpp_host_mirror_compiles_links_and_covers_the_header(pkg, tmp_path):
    """The header-only C++ mirror calls every entry point the C header declares (except the
    three that take no handle or create one), and a program using it links against the library."""
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    hpp = open(os.path.join(ROOT, "include", "b200gemm.hpp")).read()
    missing = [sym for sym in _declared_symbols() if sym + "(" not in hpp]
    assert missing == [], missing
    src = tmp_path / "use.cpp"
    src.write_text(r'''
    #include "b200gemm.hpp"
    #include <cstdio>
    // Never called: forces every inline method used here to be instantiated and type-checked.
    int use(b200gemm::Tcgen05Gemm& g, void* stream, void* p, float* f, const int32_t* i) {
      b200gemm::Operand a, b;
      a.ptr = p; b.ptr = p; a.rows = 256; a.k = 64; b.rows = 256; b.k = 64;
      int rc = g.f32_store_with_bf16_copy(stream, a, b, f, p);
      rc |= g.grouped_gemm_swiglu(stream, a, b, 1, i, p, 0, p, 0, i, 1, 128);
      rc |= g.grouped_gemm_indexed(stream, a, b, 1, i, p, 0, i, 1, 0);
      rc |= g.set_scheduler(true) | g.set_sm_limit(0) | g.set_exchange_ctas(0, false) | g.device_status(stream);
      rc |= g.convert_f32_to_bf16(stream, f, p, 8) | g.transpose_bf16(stream, p, p, 8, 8);
      rc |= g.sgemm(stream, 0, false, f, f, f, 4, 4, 4);
      return rc;
    }
    int main() { std::printf("%d\n", b200gemm::Tcgen05Gemm::version()); return 0; }
    ''')
    exe = tmp_path / "use"
    lib_dir = os.path.dirname(pkg._lib.LIB_PATH)
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    cuda_lib = "/usr/local/cuda/lib64"
    subprocess.run([gxx, "-std=c++17", "-Wall", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", lib_dir, "-lb200gemm", "-Wl,-rpath," + lib_dir, "-Wl,-rpath," + cuda_lib], check=True, env=env)
    out = subprocess.run([str(exe)], check=True, capture_output=True, env=env).stdout.decode().strip()
    assert int(out) == pkg._lib.load().b200gemm_version()


def test_create_fails_loudly_without_a_gpu(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError):
        pkg.Tcgen05Gemm()
    h = C.c_void_p()
    rc = pkg._lib.load().b200gemm_create(0, C.byref(h))
    assert rc != pkg._lib.OK and not h.value              # no device, no handle, no fallback
