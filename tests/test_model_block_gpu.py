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


def _sampled_weight_grad(oracle, x, dy, dw, rows, cols, what):
    """dW[rows, cols] = x[:, rows]^T . dy[:, cols] over ALL tokens, against the oracle."""
    xs = np.ascontiguousarray(x[:, rows].float().cpu().numpy())
    ds = np.ascontiguousarray(dy[:, cols].float().cpu().numpy())
    ref = oracle.matmul_tn(xs, ds, THREADS)
    got = dw[rows][:, cols].cpu().numpy()
    assert_gemm_close(got, ref, what, rel_fro=1e-4, elem=1e-3)


def test_full_step_weight_gradient_over_all_tokens(pkg, oracle, gemm):
    """The 32768-token QKV weight gradient (both operands read MN-major, K = tokens split over
    CTA pairs that reduce-add into dW): sampled blocks of dW against the oracle's matmul_tn over
    every token, accumulation included."""
    import torch
    m, k, n = 32768, 1536, 4608
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2)
    x = torch.randn((m, k), generator=gen, device="cuda").to(torch.bfloat16)
    dy = (torch.randn((m, n), generator=gen, device="cuda") * 0.01).to(torch.bfloat16)
    dw = torch.zeros((k, n), dtype=torch.float32, device="cuda")
    gemm.f32_accumulate_transposed(x, dy, dw)
    assert gemm.launch_config(x, dy, dw, transposed_a=True, transposed_b=True, accumulate=True)["split_k"] > 1
    rows = torch.tensor([0, 127, 128, 255, 256, 777, 1535], device="cuda")
    cols = torch.tensor([0, 255, 256, 2303, 2304, 4607], device="cuda")
    _sampled_weight_grad(oracle, x, dy, dw, rows, cols, "qkv weight gradient")
    first = dw.clone()
    gemm.f32_accumulate_transposed(x, dy, dw)
    # the K slices add into dW in no fixed order: twice the gradient to fp32 rounding
    assert float((dw - 2 * first).norm() / (2 * first).norm()) < 1e-6
    assert gemm.device_status() == 0


def test_tensor_parallel_mlp_shapes_at_full_size(pkg, oracle, gemm):
    """The scaled MLP block's GEMMs on one GPU: M=65536 tokens, D=4096, one eighth of FF=16384
    (the 8-GPU shard) and the whole of it for the forward; x ~ N(0, 1), W ~ N(0, 0.015).
    Sampled rows / blocks against the oracle, the weight gradients over all 65536 tokens."""
    import torch
    m, d, ff = 65536, 4096, 16384
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    bf = torch.bfloat16
    x = torch.randn((m, d), generator=gen, device="cuda").to(bf)
    w1 = (torch.randn((d, ff), generator=gen, device="cuda") * 0.015).to(bf)
    rows = np.array([0, 255, 256, 32767, 32768, 65535])
    h = torch.empty((m, ff), dtype=bf, device="cuda")
    gemm.gemm(x, w1, h, transposed_b=True)                                   # up, full FF
    ref = oracle.matmul_rows(x[rows].float().cpu().numpy(), w1.float().cpu().numpy(), np.arange(len(rows)), THREADS)
    assert_gemm_close(h[rows].float().cpu().numpy(), ref, "up forward rows", rel_fro=4e-3, elem=8e-3)
    # one rank's shard of the block: FF / 8 columns
    cols = ff // 8
    hs = h[:, :cols].contiguous()
    w2 = (torch.randn((cols, d), generator=gen, device="cuda") * 0.015).to(bf)
    y = torch.empty((m, d), dtype=bf, device="cuda")
    gemm.gemm(hs, w2, y, transposed_b=True)                                  # down (partial sum of this shard)
    ref = oracle.matmul(hs[rows].float().cpu().numpy(), w2.float().cpu().numpy(), THREADS)
    assert_gemm_close(y[rows].float().cpu().numpy(), ref, "down forward rows", rel_fro=4e-3, elem=8e-3)
    dy = (torch.randn((m, d), generator=gen, device="cuda") * 0.01).to(bf)
    dw2 = torch.zeros((cols, d), dtype=torch.float32, device="cuda")
    gemm.f32_accumulate_transposed(hs, dy, dw2)                              # K = 65536 tokens
    pick_r = torch.tensor([0, 255, 256, 1000, cols - 1], device="cuda")
    pick_c = torch.tensor([0, 1, 2047, 2048, d - 1], device="cuda")
    _sampled_weight_grad(oracle, hs, dy, dw2, pick_r, pick_c, "down weight gradient, K = 65536")
    dh = torch.empty((m, cols), dtype=bf, device="cuda")
    gemm.gemm(dy, w2, dh)                                                    # dh = dy W2^T
    ref = oracle.matmul_nt(dy[rows].float().cpu().numpy(), w2.float().cpu().numpy(), THREADS)
    assert_gemm_close(dh[rows].float().cpu().numpy(), ref, "down input gradient rows", rel_fro=4e-3, elem=8e-3)
    dw1 = torch.zeros((d, cols), dtype=torch.float32, device="cuda")
    gemm.f32_accumulate_transposed(x, dh, dw1)
    _sampled_weight_grad(oracle, x, dh, dw1, pick_c, pick_r, "up weight gradient, K = 65536")
    assert gemm.device_status() == 0
