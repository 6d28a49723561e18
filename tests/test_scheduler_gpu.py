"""Dynamic tile scheduling (`b200gemm_set_scheduler`) against the static walk.

The two modes hand out the same work items; only which cluster computes which item
changes.  Every output element is produced by one item, so store-mode results must be
bit-identical; where split-K slices are reduce-added into C the order of the adds is
not fixed in either mode and the results are compared within the GEMM tolerance.
"""
import numpy as np
import pytest

from _util import THREADS, assert_gemm_close, bf16_operand, from_dev_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture()
def gemms(pkg):
    static, dynamic = pkg.Tcgen05Gemm(), pkg.Tcgen05Gemm()
    static.set_scheduler(False)
    dynamic.set_scheduler(True)
    yield static, dynamic
    assert static.device_status() == 0 and dynamic.device_status() == 0
    static.close()
    dynamic.close()


@pytest.mark.parametrize("m,n,k,tb,out", [
    (4096, 4608, 1536, True, "f32"),      # many more items than clusters
    (2048, 1536, 4096, False, "bf16"),
    (1000, 520, 200, True, "f32"),        # ragged edges
    (300, 256, 64, False, "bf16"),        # fewer items than clusters
    (257, 8, 72, False, "f32"),
])
def test_store_is_bit_identical(pkg, oracle, gemms, m, n, k, tb, out):
    import torch
    static, dynamic = gemms
    a, av = bf16_operand(oracle, (m, k), 201)
    b, bv = bf16_operand(oracle, (k, n) if tb else (n, k), 202, std=0.1)
    dt = torch.float32 if out == "f32" else torch.bfloat16
    c1 = torch.full((m, n), 5.0, dtype=dt, device="cuda")
    c2 = torch.full((m, n), 6.0, dtype=dt, device="cuda")
    static.gemm(a, b, c1, transposed_b=tb, split_k=1)
    for _ in range(3):                     # the counters must be back at zero after every launch
        c2.fill_(6.0)
        dynamic.gemm(a, b, c2, transposed_b=tb, split_k=1)
        assert torch.equal(c1, c2)
    rows = np.arange(0, m, max(1, m // 64))
    w = bv if tb else bv.T
    ref = oracle.matmul(av[rows], np.ascontiguousarray(w), THREADS)
    tol = dict(rel_fro=2e-5, elem=2e-4) if out == "f32" else dict(rel_fro=4e-3, elem=8e-3)
    assert_gemm_close(c2.float().cpu().numpy()[rows], ref, "dynamic vs oracle", **tol)


def test_weight_gradient_with_split_k(pkg, oracle, gemms):
    import torch
    static, dynamic = gemms
    tokens, i, o = 8192, 512, 768
    x, xv = bf16_operand(oracle, (tokens, i), 203)
    dy, dyv = bf16_operand(oracle, (tokens, o), 204, std=0.01)
    d1 = torch.zeros((i, o), dtype=torch.float32, device="cuda")
    d2 = torch.zeros((i, o), dtype=torch.float32, device="cuda")
    static.f32_accumulate_transposed(x, dy, d1)
    dynamic.f32_accumulate_transposed(x, dy, d2)
    ref = oracle.matmul_tn(xv, dyv, THREADS)
    assert_gemm_close(d1.cpu().numpy(), ref, "static", rel_fro=2e-5, elem=2e-4)
    assert_gemm_close(d2.cpu().numpy(), ref, "dynamic", rel_fro=2e-5, elem=2e-4)


def test_fused_head_and_grouped_gemm(pkg, oracle, gemms):
    import torch
    static, dynamic = gemms
    m, k, v, classes = 1536, 256, 2560, 2500
    h, _ = bf16_operand(oracle, (m, k), 205)
    w, _ = bf16_operand(oracle, (k, v), 206, std=0.2)
    t = torch.from_numpy((oracle.uniform(m, 207) * classes).astype(np.int32) % classes).cuda()
    outs = []
    for g in (static, dynamic):
        head = pkg.FusedLmHead(g, classes, "in_out")
        loss, lse, row = head.forward(h, w, t)
        dl, dh, dw = head.backward(h, w, t, lse)
        outs.append((loss, lse, row, dl, dh))
    for s_t, d_t in zip(outs[0][:4], outs[1][:4]):
        assert torch.equal(s_t, d_t)
    # d_hidden is a split-K product here: slices are reduce-added in no fixed order
    assert torch.allclose(outs[0][4], outs[1][4], atol=1e-6, rtol=1e-4)
    # ragged groups, SiLU and SwiGLU epilogues
    sizes = [300, 0, 17, 256, 1, 513, 128, 31]
    offsets = torch.from_numpy(np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)).cuda()
    rows, kk, ff = int(sum(sizes)), 192, 320
    a, _ = bf16_operand(oracle, (rows, kk), 208)
    b, _ = bf16_operand(oracle, (len(sizes), kk, ff), 209, std=0.1)
    bg, _ = bf16_operand(oracle, (len(sizes), kk, 2, ff), 210, std=0.1)
    y1 = pkg.moe.grouped_gemm(static, a, b, offsets, transposed_b=True, silu=True)
    y2 = pkg.moe.grouped_gemm(dynamic, a, b, offsets, transposed_b=True, silu=True)
    assert torch.equal(y1, y2)
    g1, p1 = pkg.moe.grouped_gemm_swiglu(static, a, bg, offsets, want_gate_up=True)
    g2, p2 = pkg.moe.grouped_gemm_swiglu(dynamic, a, bg, offsets, want_gate_up=True)
    assert torch.equal(g1, g2) and torch.equal(p1, p2)


def test_two_streams_at_once(pkg, oracle, gemms):
    """Launches on different streams may overlap on the GPU; each stream has its own counters."""
    import torch
    static, dynamic = gemms
    a, _ = bf16_operand(oracle, (4096, 1024), 211)
    b1, _ = bf16_operand(oracle, (1024, 1024), 212, std=0.1)
    b2, _ = bf16_operand(oracle, (2048, 1024), 213, std=0.1)
    want1 = torch.empty((4096, 1024), dtype=torch.float32, device="cuda")
    want2 = torch.empty((4096, 2048), dtype=torch.float32, device="cuda")
    static.gemm(a, b1, want1, split_k=1)
    static.gemm(a, b2, want2, split_k=1)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    got1, got2 = torch.zeros_like(want1), torch.zeros_like(want2)
    torch.cuda.synchronize()
    for _ in range(4):
        with torch.cuda.stream(s1):
            dynamic.gemm(a, b1, got1, split_k=1)
        with torch.cuda.stream(s2):
            dynamic.gemm(a, b2, got2, split_k=1)
    torch.cuda.synchronize()
    assert torch.equal(want1, got1) and torch.equal(want2, got2)


def test_dynamic_schedule_on_a_limited_number_of_sms(pkg, oracle, gemms):
    """`set_sm_limit` shrinks the grid; the counter still hands every item out exactly once."""
    import torch
    static, dynamic = gemms
    a, _ = bf16_operand(oracle, (2048, 512), 214)
    b, _ = bf16_operand(oracle, (512, 1280), 215, std=0.1)
    want = torch.empty((2048, 1280), dtype=torch.float32, device="cuda")
    static.gemm(a, b, want, transposed_b=True, split_k=1)
    for sms in (100, 6, 2, 0):
        dynamic.set_sm_limit(sms)
        got = torch.zeros_like(want)
        dynamic.gemm(a, b, got, transposed_b=True, split_k=1)
        assert torch.equal(want, got), sms
    dynamic.set_sm_limit(0)
