"""One transformer block's GEMMs (forward + input gradient + weight gradient) against
the CPU oracle in full: B=2, T=1024 (2048 tokens), D=1536, QKV 1536->4608,
attention-out 1536->1536, MLP up 1536->4096, MLP down 4096->1536.  Activations
~N(0,1), weights ~N(0,0.02), upstream gradients ~N(0,1e-2), seed 0, bf16 operands,
fp32 accumulation.  Tolerance: relative Frobenius <= 1e-2 and per element
|d| <= 2e-2 (1 + |ref|); the fp32 outputs in fact agree to ~1e-6."""
import numpy as np
import pytest

from _util import THREADS, assert_gemm_close, bf16_operand

pytestmark = pytest.mark.gpu

TOKENS = 2048
PROJECTIONS = [("qkv", 1536, 4608), ("attn_out", 1536, 1536), ("mlp_up", 1536, 4096), ("mlp_down", 4096, 1536)]


@pytest.fixture(scope="module")
def gemm(pkg):
    g = pkg.Tcgen05Gemm()
    yield g
    g.close()


@pytest.mark.parametrize("name,d_in,d_out", PROJECTIONS)
def test_block_projection_forward_and_gradients(pkg, oracle, gemm, name, d_in, d_out):
    import torch
    seed = 0
    x, xv = bf16_operand(oracle, (TOKENS, d_in), seed * 100 + 1)
    w, wv = bf16_operand(oracle, (d_in, d_out), seed * 100 + 2, std=0.02)        # [IN, OUT], read in place
    dy, dyv = bf16_operand(oracle, (TOKENS, d_out), seed * 100 + 3, std=0.01)

    # forward  y = x W          (crates/nn/src/linear.rs:42-44)
    y = torch.empty((TOKENS, d_out), dtype=torch.float32, device="cuda")
    gemm.f32_store(x, w, y, transposed_b=True)
    assert_gemm_close(y.cpu().numpy(), oracle.matmul(xv, wv, THREADS), f"{name} forward")
    # input gradient  dx = dy W^T   (linear.rs:48)
    dx = torch.empty((TOKENS, d_in), dtype=torch.float32, device="cuda")
    gemm.f32_store(dy, w, dx)
    assert_gemm_close(dx.cpu().numpy(), oracle.matmul_nt(dyv, wv, THREADS), f"{name} input grad")
    # weight gradient  dW += x^T dy   (linear.rs:47), accumulated twice into a zeroed buffer
    dw = torch.zeros((d_in, d_out), dtype=torch.float32, device="cuda")
    gemm.f32_accumulate_transposed(x, dy, dw)
    ref_dw = oracle.matmul_tn(xv, dyv, THREADS)
    assert_gemm_close(dw.cpu().numpy(), ref_dw, f"{name} weight grad")
    gemm.f32_accumulate_transposed(x, dy, dw)
    assert_gemm_close(dw.cpu().numpy(), 2 * ref_dw, f"{name} weight grad, second accumulation")
    assert gemm.device_status() == 0
    # the fp32 results differ from the oracle only by summation order
    assert np.linalg.norm(y.cpu().numpy() - oracle.matmul(xv, wv, THREADS)) / np.linalg.norm(y.cpu().numpy()) < 1e-5


def test_full_step_shape_sampled_rows_and_linearity(pkg, oracle, gemm):
    """The 32768-token QKV projection: sampled rows against the oracle (full K per
    element) and linearity C(a1 + a2) = C(a1) + C(a2) on exactly representable inputs."""
    import torch
    m, k, n = 32768, 1536, 4608
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    x = torch.randn((m, k), generator=gen, device="cuda").to(torch.bfloat16)
    w = (torch.randn((k, n), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    y = torch.empty((m, n), dtype=torch.float32, device="cuda")
    gemm.f32_store(x, w, y, transposed_b=True)
    rows = np.array([0, 255, 256, 4097, 16383, 20000, 32767])
    ref = oracle.matmul_rows(x.float().cpu().numpy(), w.float().cpu().numpy(), rows, THREADS)
    assert_gemm_close(y[rows].cpu().numpy(), ref, "sampled rows", rel_fro=1e-5, elem=1e-4)
    # linearity with small-integer operands (every partial sum exact in fp32)
    a1 = torch.randint(-3, 4, (m, k), generator=gen, device="cuda").to(torch.bfloat16)
    a2 = torch.randint(-3, 4, (m, k), generator=gen, device="cuda").to(torch.bfloat16)
    wi = torch.randint(-2, 3, (k, n), generator=gen, device="cuda").to(torch.bfloat16)
    y1 = torch.empty_like(y)
    y2 = torch.empty_like(y)
    y12 = torch.empty_like(y)
    gemm.f32_store(a1, wi, y1, transposed_b=True)
    gemm.f32_store(a2, wi, y2, transposed_b=True)
    gemm.f32_store((a1 + a2), wi, y12, transposed_b=True)
    assert torch.equal(y12, y1 + y2)
    assert gemm.device_status() == 0
