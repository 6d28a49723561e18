"""The fp32 GEMM family, the bf16 staging converts and the packed transpose.

fp32 ladder shape and tolerance from the reference's gate (gpu/gemm/src/main.rs:393-513:
73 x 91 x 47 against a CPU product, 2e-5; gpu/tensor-gpu/src/main.rs:557-605: 19 x 23 x 29).
Here the kernels round every product and add in ascending k like the CPU loops, so the
comparison is exact."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gemm(pkg):
    g = pkg.Tcgen05Gemm()
    yield g
    g.close()


@pytest.mark.parametrize("m,n,k", [(73, 91, 47), (19, 23, 29), (1, 1, 1), (64, 64, 16), (130, 65, 200)])
def test_fp32_family_is_bit_exact_with_the_cpu_loops(pkg, oracle, gemm, m, n, k):
    import torch
    L = pkg._lib
    a = oracle.uniform(m * k, 1).reshape(m, k)
    b = oracle.uniform(k * n, 2).reshape(k, n)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    assert np.array_equal(gemm.matmul(da, db).cpu().numpy(), oracle.matmul(a, b))
    bt = np.ascontiguousarray(b.T)
    assert np.array_equal(gemm.matmul_nt(da, torch.from_numpy(bt).cuda()).cpu().numpy(), oracle.matmul_nt(a, bt))
    at = np.ascontiguousarray(a.T)                                  # [k, m]
    assert np.array_equal(gemm.matmul_tn(torch.from_numpy(at).cuda(), db).cpu().numpy(), oracle.matmul_tn(at, b))
    # accumulate forms (register_gemm_accumulate / tn_accumulate, gpu/gemm/src/fp32.rs:141-191)
    c0 = oracle.uniform(m * n, 3).reshape(m, n)
    c = torch.from_numpy(c0.copy()).cuda()
    gemm.sgemm(L.OP_NN, da, db, c, accumulate=True)
    assert np.array_equal(c.cpu().numpy(), (c0 + oracle.matmul(a, b)).astype(np.float32))
    assert gemm.device_status() == 0


def test_converts_round_to_nearest_even_and_widen_exactly(pkg, oracle, gemm):
    import torch
    for n in (8, 1000, 4099, 1 << 20):
        x = oracle.normal(n, 7, 0.0, 3.0)
        dx = torch.from_numpy(x).cuda()
        y = gemm.convert_f32_to_bf16(dx)
        got = y.view(torch.int16).cpu().numpy().view(np.uint16)
        assert np.array_equal(got, oracle.bf16_bits(x))
        back = gemm.convert_bf16_to_f32(y)
        assert np.array_equal(back.cpu().numpy(), oracle.bf16_round(x))
    ties = np.array([0x3F808000, 0x3F818000, 0x3F808001, 0xBF808000] * 2, np.uint32).view(np.float32)
    got = gemm.convert_f32_to_bf16(torch.from_numpy(ties.copy()).cuda()).view(torch.int16).cpu().numpy().view(np.uint16)
    assert got[:4].tolist() == [0x3F80, 0x3F82, 0x3F81, 0xBF80]


@pytest.mark.parametrize("rows,cols", [(64, 64), (1536, 4608), (100, 37), (1, 513)])
def test_transpose_bf16(pkg, oracle, gemm, rows, cols):
    import torch
    x = torch.arange(rows * cols, device="cuda", dtype=torch.float32).remainder(251).to(torch.bfloat16).view(rows, cols)
    y = gemm.transpose_bf16(x)
    assert torch.equal(y, x.t().contiguous())


def test_launch_config_reports_the_persistent_grid(pkg, gemm):
    import torch
    a = torch.zeros((32768, 1536), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((1536, 4608), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((32768, 4608), dtype=torch.float32, device="cuda")
    cfg = gemm.launch_config(a, w, c, transposed_b=True)
    assert cfg["cluster"] == 2 and cfg["grid"] == 148 and cfg["split_k"] == 1       # 2304 tiles on 74 clusters
    dw = torch.zeros((1536, 1536), dtype=torch.float32, device="cuda")
    cfg = gemm.launch_config(a, a, dw, transposed_a=True, transposed_b=True, accumulate=True)
    assert cfg["split_k"] > 1                          # 36 tiles cannot fill 74 clusters: split the token reduction
    small = gemm.launch_config(a[:128], w, c[:128], transposed_b=True)
    assert small["cluster"] == 1                       # 128 rows: single-CTA tiles
    gemm.set_sm_limit(100)
    assert gemm.launch_config(a, w, c, transposed_b=True)["grid"] == 100
    gemm.set_sm_limit(0)
    assert gemm.launch_config(a, w, c, transposed_b=True)["grid"] == 148
