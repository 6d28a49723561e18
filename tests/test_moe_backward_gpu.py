"""GPU parity of the expert path's backward against the oracle, through the C ABI.

Reference: ``MoeFfn::backward`` (crates/nn/src/moe.rs:354-452), ``SwiGlu::backward``
(crates/nn/src/swiglu.rs:30-47) and the GPU drivers ``expert_linear_backward`` /
``GpuExpertFfn::backward_profiled`` (gpu/model/src/lib.rs:2011-2154, 2335-2425), whose
weight-gradient form (`f32_accumulate_transposed_batched`) is gated at 256^3 in
gpu/gemm/src/main.rs:343-391.  Here the groups are ragged, so the cases are chosen around
the group boundaries: an empty group, groups shorter than one K block, groups that end in
the middle of a K block, and one long enough to be cut into several chunks.
"""
import numpy as np
import pytest

from _moe_ref import MoeRef
from _util import THREADS, assert_gemm_close, bf16_operand, from_dev_bf16, to_dev_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gemm(pkg):
    g = pkg.Tcgen05Gemm()
    yield g
    g.close()


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


def _offsets(counts):
    import torch
    off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    return off, torch.from_numpy(off).cuda()


# ---- grouped weight gradient ---------------------------------------------------------------

RAGGED = [0, 37, 64, 300, 1, 0, 5000, 129, 63, 255]


@pytest.mark.parametrize("m,n", [(256, 256), (192, 328), (512, 264)])
def test_grouped_wgrad_ragged_groups(pkg, oracle, gemm, m, n):
    import torch
    off, off_dev = _offsets(RAGGED)
    rows, G = int(off[-1]), len(RAGGED)
    a, av = bf16_operand(oracle, (rows + 70, m), 11)               # rows past the last group exist and must not count,
    b, bv = bf16_operand(oracle, (rows + 70, n), 12, std=0.05)     # whatever they hold: uninitialised memory can be NaN
    a[rows:] = float("nan")
    b[rows:] = float("inf")
    ref = np.stack([oracle.matmul_tn(av[off[g]:off[g + 1]], bv[off[g]:off[g + 1]], THREADS)
                    if off[g + 1] > off[g] else np.zeros((m, n), np.float32) for g in range(G)])
    c = torch.full((G, m, n), 5.0, dtype=torch.float32, device="cuda")
    pkg.moe.grouped_wgrad(gemm, a, b, off_dev, c, accumulate=False)
    assert gemm.device_status() == 0
    got = c.cpu().numpy()
    for g in range(G):
        if RAGGED[g] == 0:
            assert not got[g].any(), f"empty group {g} must give a zero matrix"
        else:
            assert_gemm_close(got[g], ref[g], f"wgrad group {g} ({RAGGED[g]} rows)", rel_fro=2e-5, elem=2e-4)
    pkg.moe.grouped_wgrad(gemm, a, b, off_dev, c, accumulate=True)
    assert gemm.device_status() == 0
    assert_gemm_close(c.cpu().numpy(), 2 * ref, "wgrad accumulate", rel_fro=2e-5, elem=2e-4)


def test_grouped_wgrad_is_exact_on_integers_and_ignores_neighbours(pkg, oracle, gemm):
    """Small-integer operands make every partial sum exact in fp32, so the result must EQUAL the
    integer product whatever the order of the chunks' additions -- and any row of a neighbouring
    group that leaked through a group's last K block would show."""
    import torch
    counts = [70, 1, 130, 0, 2100, 64, 3]
    off, off_dev = _offsets(counts)
    rows, G, m, n = int(off[-1]), len(counts), 256, 256
    i, j = np.meshgrid(np.arange(rows), np.arange(m), indexing="ij")
    av = (((i * 5 + j * 3) % 7) - 3).astype(np.float32)
    i, j = np.meshgrid(np.arange(rows), np.arange(n), indexing="ij")
    bv = (((i * 4 + j * 5) % 5) - 2).astype(np.float32)
    a, b = to_dev_bf16(oracle.bf16_bits(av)), to_dev_bf16(oracle.bf16_bits(bv))
    c = torch.zeros((G, m, n), dtype=torch.float32, device="cuda")
    pkg.moe.grouped_wgrad(gemm, a, b, off_dev, c, accumulate=False)
    assert gemm.device_status() == 0
    got = c.cpu().numpy()
    for g in range(G):
        want = av[off[g]:off[g + 1]].astype(np.int64).T @ bv[off[g]:off[g + 1]].astype(np.int64)
        assert np.array_equal(got[g], want.astype(np.float32)), f"group {g}"


def test_grouped_wgrad_shared_matrices(pkg, oracle, gemm):
    """Several groups adding into one matrix: rows that arrived from several ranks for one expert."""
    import torch
    counts = [100, 260, 31, 400, 0, 77]
    index = np.array([0, 1, 2, 0, 1, 2], dtype=np.int32)
    off, off_dev = _offsets(counts)
    rows, m, n = int(off[-1]), 320, 256
    a, av = bf16_operand(oracle, (rows, m), 13)
    b, bv = bf16_operand(oracle, (rows, n), 14, std=0.05)
    ref = np.zeros((3, m, n), np.float32)
    for g, e in enumerate(index):
        if counts[g]:
            ref[e] += oracle.matmul_tn(av[off[g]:off[g + 1]], bv[off[g]:off[g + 1]], THREADS)
    c = torch.zeros((3, m, n), dtype=torch.float32, device="cuda")
    pkg.moe.grouped_wgrad(gemm, a, b, off_dev, c, accumulate=True, group_c_index=torch.from_numpy(index).cuda())
    assert gemm.device_status() == 0
    assert_gemm_close(c.cpu().numpy(), ref, "shared matrices", rel_fro=2e-5, elem=2e-4)


# ---- elementwise pieces ----------------------------------------------------------------------

def test_activation_backward(pkg, oracle, gemm):
    rows, ff = 777, 192
    g, gv = bf16_operand(oracle, (rows, 2, ff), 21)
    dy, dyv = bf16_operand(oracle, (rows, ff), 22, std=0.1)
    d = pkg.moe.activation_backward(gemm, "swiglu", g, dy)
    dg, du = oracle.swiglu_backward(gv[:, 0], gv[:, 1], dyv)
    got = from_dev_bf16(d)
    assert_gemm_close(got[:, 0], dg, "d_gate", rel_fro=4e-3, elem=8e-3)
    assert_gemm_close(got[:, 1], du, "d_up", rel_fro=4e-3, elem=8e-3)
    d1 = pkg.moe.activation_backward(gemm, "silu", g[:, 0].contiguous(), dy)
    assert_gemm_close(from_dev_bf16(d1), oracle.silu_backward(gv[:, 0], dyv), "silu'", rel_fro=4e-3, elem=8e-3)


def test_grouped_gemm_silu_keeps_the_values_before_the_activation(pkg, oracle, gemm):
    counts = [300, 0, 41, 515]
    off, off_dev = _offsets(counts)
    rows, k, n = int(off[-1]), 192, 320
    a, av = bf16_operand(oracle, (rows, k), 23)
    w, wv = bf16_operand(oracle, (len(counts), k, n), 24, std=0.1)
    y, before = pkg.moe.grouped_gemm_silu(gemm, a, w, off_dev)
    assert gemm.device_status() == 0
    plain = pkg.moe.grouped_gemm(gemm, a, w, off_dev, transposed_b=True)
    fused = pkg.moe.grouped_gemm(gemm, a, w, off_dev, transposed_b=True, silu=True)
    import torch
    assert torch.equal(before, plain) and torch.equal(y, fused)       # the same kernel arithmetic, bit for bit
    for g in range(len(counts)):
        if counts[g]:
            ref = oracle.matmul(av[off[g]:off[g + 1]], wv[g], THREADS)
            assert_gemm_close(from_dev_bf16(before[off[g]:off[g + 1]]), ref, f"before {g}", rel_fro=4e-3, elem=8e-3)


@pytest.mark.parametrize("activation,ff", [("silu", 200), ("swiglu", 128), ("swiglu", 320), ("silu", 768)])
def test_activation_backward_fused_into_the_input_gradient(pkg, oracle, gemm, activation, ff):
    """`d_saved = act'(saved) * (dy . W^T)` from one launch against the oracle's two steps (an
    input gradient by `matmul_nt`, then `SwiGlu::backward`), and against the two-launch GPU form."""
    counts = [130, 0, 517, 64, 33]
    off, off_dev = _offsets(counts)
    rows, d = int(off[-1]), 192
    dy, dyv = bf16_operand(oracle, (rows, d), 25, std=0.1)
    w, wv = bf16_operand(oracle, (len(counts), ff, d), 26, std=0.1)
    shape = (rows, 2, ff) if activation == "swiglu" else (rows, ff)
    saved, sv = bf16_operand(oracle, shape, 27)
    fused = pkg.moe.grouped_gemm_act_backward(gemm, dy, w, off_dev, activation, saved)
    assert gemm.device_status() == 0
    d_hidden = pkg.moe.grouped_gemm(gemm, dy, w, off_dev, transposed_b=False)
    two_pass = pkg.moe.activation_backward(gemm, activation, saved, d_hidden)
    got, other = from_dev_bf16(fused), from_dev_bf16(two_pass)
    for g in range(len(counts)):
        if not counts[g]:
            continue
        a, b = off[g], off[g + 1]
        dact = oracle.matmul_nt(dyv[a:b], wv[g], THREADS)
        if activation == "swiglu":
            dg, du = oracle.swiglu_backward(sv[a:b, 0], sv[a:b, 1], dact)
            assert_gemm_close(got[a:b, 0], dg, f"d_gate {g}", rel_fro=4e-3, elem=8e-3)
            assert_gemm_close(got[a:b, 1], du, f"d_up {g}", rel_fro=4e-3, elem=8e-3)
        else:
            assert_gemm_close(got[a:b], oracle.silu_backward(sv[a:b], dact), f"d_pre {g}", rel_fro=4e-3, elem=8e-3)
    # the two-launch form rounds d_hidden to bf16 in between: the same values to a bf16 ulp or two
    assert_gemm_close(got, other, "fused vs two launches", rel_fro=6e-3, elem=1.6e-2)


def test_combine_and_scatter_backward(pkg, oracle, gemm):
    import torch
    N, E, K, D, cap = 600, 6, 3, 136, 250            # the capacity forces drops
    probs = oracle.softmax_rows(oracle.normal(N * E, 31).reshape(N, E))
    r = pkg.moe.route(gemm, torch.from_numpy(probs).cuda(), K, cap)
    want = oracle.moe_route(probs, K, cap)
    assert int((want["slots"] == 0xFFFFFFFF).sum()) > 0
    rows = int(want["offsets"][E])
    yp, ypv = bf16_operand(oracle, (N * K, D), 32)
    for dy_dtype in ("f32", "bf16"):
        if dy_dtype == "f32":
            dyv = oracle.normal(N * D, 33, 0.0, 0.1).reshape(N, D)
            dy = torch.from_numpy(dyv).cuda()
        else:
            dy, dyv = bf16_operand(oracle, (N, D), 33, std=0.1)
        out = torch.full((N * K, D), 9.0, dtype=torch.bfloat16, device="cuda")
        dyp, gg = pkg.moe.combine_backward(gemm, dy, r, yp, out=out)
        ref_dyp, ref_gg = oracle.moe_combine_backward(dyv, ypv[:rows], want["dest_row"], want["gates"], K)
        assert_gemm_close(from_dev_bf16(dyp[:rows]), ref_dyp, f"dy_permuted {dy_dtype}", rel_fro=4e-3, elem=8e-3)
        assert np.all(from_dev_bf16(dyp[rows:]) == 9.0)                    # rows no pair maps to are untouched
        assert_gemm_close(gg.cpu().numpy(), ref_gg, f"gate_grad {dy_dtype}", rel_fro=1e-4, elem=1e-3)
        assert np.all(gg.cpu().numpy()[want["dest_row"] == 0xFFFFFFFF] == 0.0)
    dxp, dxpv = bf16_operand(oracle, (N * K, D), 34)
    dx = pkg.moe.scatter_backward(gemm, dxp, r)
    assert np.array_equal(dx.cpu().numpy(), oracle.moe_scatter_backward(dxpv[:rows], want["dest_row"], N, K))


def test_route_backward_and_router_logits(pkg, oracle, gemm):
    import torch
    N, D, E, K = 700, 136, 64, 8
    x, xv = bf16_operand(oracle, (N, D), 41)
    wr = oracle.normal(D * E, 42, 0.0, 0.3).reshape(D, E)
    logits = pkg.moe.router_logits(gemm, x, torch.from_numpy(wr).cuda())
    want_logits = oracle.matmul(xv, wr, THREADS)
    assert np.array_equal(logits.cpu().numpy(), want_logits)               # the CPU router's sums, bit for bit
    probs = oracle.softmax_rows(want_logits)
    r = pkg.moe.route(gemm, torch.from_numpy(probs).cuda(), K)
    want = oracle.moe_route(probs, K, N * K)
    assert np.array_equal(_u32(r.selected_experts), want["selected"])
    gg = oracle.normal(N * K, 43).astype(np.float32)
    got = pkg.moe.route_backward(gemm, torch.from_numpy(probs).cuda(), r, torch.from_numpy(gg).cuda(), 0.17)
    ref = oracle.moe_route_backward(probs, want["selected"], want["gates"], gg, want["assignment_counts"], 0.17, K)
    assert_gemm_close(got.cpu().numpy(), ref, "router dlogits", rel_fro=1e-5, elem=1e-5)
    # experts that do not fill a warp, top-1
    probs5 = oracle.softmax_rows(oracle.normal(50 * 5, 44).reshape(50, 5))
    r5 = pkg.moe.route(gemm, torch.from_numpy(probs5).cuda(), 1)
    w5 = oracle.moe_route(probs5, 1, 50)
    gg5 = oracle.normal(50, 45).astype(np.float32)
    got5 = pkg.moe.route_backward(gemm, torch.from_numpy(probs5).cuda(), r5, torch.from_numpy(gg5).cuda(), 0.0)
    ref5 = oracle.moe_route_backward(probs5, w5["selected"], w5["gates"], gg5, w5["assignment_counts"], 0.0, 1)
    assert_gemm_close(got5.cpu().numpy(), ref5, "router dlogits E=5", rel_fro=1e-5, elem=1e-5)


def test_loss_mean_with_aux(pkg, oracle, gemm):
    import ctypes as C
    import torch
    losses = oracle.normal(32768, 51, 10.0, 1.0).astype(np.float32)
    aux = np.array([1.01, 0.97, 1.2], dtype=np.float32)
    dl, da = torch.from_numpy(losses).cuda(), torch.from_numpy(aux).cuda()
    out = torch.zeros(1, device="cuda")
    L = pkg._lib
    L.check(gemm._lib.b200gemm_loss_mean_with_aux(gemm._h, torch.cuda.current_stream().cuda_stream, dl.data_ptr(),
                                                  losses.size, da.data_ptr(), 3, 0.01, out.data_ptr()))
    want = np.float32(losses.astype(np.float64).sum() / losses.size) + np.float32(0.01) * np.float32(
        (aux[0] + aux[1]) + aux[2])
    assert abs(float(out.item()) - float(want)) <= 1e-6 * abs(float(want))
    L.check(gemm._lib.b200gemm_loss_mean_with_aux(gemm._h, torch.cuda.current_stream().cuda_stream, dl.data_ptr(),
                                                  losses.size, None, 0, 0.0, out.data_ptr()))
    assert abs(float(out.item()) - float(np.float32(losses.astype(np.float64).mean()))) <= 1e-6 * 10


# ---- the whole block -------------------------------------------------------------------------

def _block(pkg, oracle, gemm, gated, N, D, FF, E, K, cap, seed, idle_expert=None):
    """Forward + backward of a whole expert block on the GPU and through MoeRef on the same bf16
    operands, MoeRef rounding its intermediates to bf16 where the GPU path stores them."""
    import torch
    x, xv = bf16_operand(oracle, (N, D), seed)
    logits = oracle.normal(N * E, seed + 1).reshape(N, E) * 1.5
    if idle_expert is not None:
        logits[:, idle_expert] -= 60.0                     # never among the top-k: the expert gets no rows
    probs = oracle.softmax_rows(logits)
    wd, wdv = bf16_operand(oracle, (E, FF, D), seed + 2, std=0.08)
    dy, dyv = bf16_operand(oracle, (N, D), seed + 3, std=0.1)
    if gated:
        wgu, wguv = bf16_operand(oracle, (E, D, 2, FF), seed + 4, std=0.08)
        ffn = pkg.GatedExpertFfn(gemm, wgu, wd)
        ref = MoeRef(oracle, None, np.ascontiguousarray(wguv[:, :, 0]), np.ascontiguousarray(wguv[:, :, 1]), wdv,
                     K, cap, threads=THREADS, round_to=oracle.bf16_round)
        d_up = torch.zeros((E, D, 2, FF), dtype=torch.float32, device="cuda")
    else:
        wu, wuv = bf16_operand(oracle, (E, D, FF), seed + 4, std=0.08)
        ffn = pkg.GroupedExpertFfn(gemm, wu, wd)
        ref = MoeRef(oracle, None, None, wuv, wdv, K, cap, threads=THREADS, round_to=oracle.bf16_round)
        d_up = torch.zeros((E, D, FF), dtype=torch.float32, device="cuda")
    d_down = torch.zeros((E, FF, D), dtype=torch.float32, device="cuda")
    kw = {"keep_gate_up": True} if gated else {"keep_for_backward": True}
    y, r = ffn.forward(x, torch.from_numpy(probs).cuda(), K, capacity=cap, **kw)
    dx, gg = ffn.backward(dy, d_up, d_down)
    assert gemm.device_status() == 0
    y_ref = ref.forward(xv, probs)
    g = ref.backward(dyv)
    assert np.array_equal(_u32(r.dest_row), ref.r["dest_row"])
    tol = dict(rel_fro=6e-3, elem=1.5e-2)
    assert_gemm_close(y.cpu().numpy(), y_ref, "forward", **tol)
    assert_gemm_close(dx.cpu().numpy(), g["dx"], "dx", **tol)
    assert_gemm_close(gg.cpu().numpy(), g["gate_grad"], "gate_grad", **tol)
    assert_gemm_close(d_down.cpu().numpy(), g["d_down"], "d_down", **tol)
    if gated:
        got = d_up.cpu().numpy()
        assert_gemm_close(got[:, :, 0], g["d_gate"], "d_gate", **tol)
        assert_gemm_close(got[:, :, 1], g["d_up"], "d_up", **tol)
    else:
        assert_gemm_close(d_up.cpu().numpy(), g["d_up"], "d_up", **tol)
    return ref


def test_gated_block_backward_with_drops_and_an_idle_expert(pkg, oracle, gemm):
    # the reference's own expert (SwiGLU); the capacity forces drops; expert 4 gets nothing
    ref = _block(pkg, oracle, gemm, True, N=700, D=192, FF=128, E=6, K=2, cap=200, seed=60, idle_expert=4)
    assert int((ref.r["slots"] == 0xFFFFFFFF).sum()) > 0
    assert int(ref.r["accepted_counts"][4]) == 0


def test_silu_block_backward(pkg, oracle, gemm):
    _block(pkg, oracle, gemm, False, N=900, D=136, FF=200, E=8, K=3, cap=900 * 3, seed=70)


def test_full_size_backward_on_sampled_experts(pkg, oracle, gemm):
    """32768 tokens, D=1536, E=64, top-8, FF=768 (Zipf-skewed): the weight gradients of the
    least loaded experts and the input gradient of a few tokens against the oracle."""
    import torch
    N, D, FF, E, K = 32768, 1536, 768, 64, 8
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    x = torch.randn((N, D), generator=gen, device="cuda").to(torch.bfloat16)
    w_up = (torch.randn((E, D, FF), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    w_dn = (torch.randn((E, FF, D), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    dy = (torch.randn((N, D), generator=gen, device="cuda") * 0.01).to(torch.bfloat16)
    bias = 0.5 * torch.log(1.0 / torch.arange(1, E + 1, device="cuda", dtype=torch.float32))
    logits = (torch.randn((N, E), generator=gen, device="cuda") + bias).contiguous()
    ffn = pkg.GroupedExpertFfn(gemm, w_up, w_dn)
    y, r = ffn.forward(x, logits, K, scores_are_logits=True, keep_for_backward=True)
    d_up = torch.zeros((E, D, FF), dtype=torch.float32, device="cuda")
    d_dn = torch.zeros((E, FF, D), dtype=torch.float32, device="cuda")
    dx, gg = ffn.backward(dy, d_up, d_dn)
    assert gemm.device_status() == 0
    c = ffn.ctx
    offs = _u32(r.offsets).astype(np.int64)
    counts = np.diff(offs)
    dest = _u32(r.dest_row).astype(np.int64)
    gates = r.gate_weights.cpu().numpy()
    dyv = dy.float().cpu().numpy()
    tol = dict(rel_fro=6e-3, elem=1.5e-2)
    for e in (int(np.argmin(counts)), E - 1):
        a, b = offs[e], offs[e + 1]
        # the rows the kernels saw, taken from the device; the arithmetic from the oracle
        hid = from_dev_bf16(c.hidden[a:b])
        xp = from_dev_bf16(c.x_permuted[a:b])
        pre = from_dev_bf16(c.saved[a:b])
        pairs = np.nonzero((dest >= a) & (dest < b))[0]
        dyp = np.zeros((b - a, D), np.float32)
        dyp[dest[pairs] - a] = gates[pairs, None] * dyv[pairs // K]         # moe.rs:371-373, one product per element
        dyp = oracle.bf16_round(dyp)
        assert_gemm_close(d_dn[e].cpu().numpy(), oracle.matmul_tn(hid, dyp, THREADS), f"d_down[{e}]", **tol)
        dact = oracle.bf16_round(oracle.matmul_nt(dyp, w_dn[e].float().cpu().numpy(), THREADS))
        dpre = oracle.bf16_round(oracle.silu_backward(pre, dact))
        assert_gemm_close(d_up[e].cpu().numpy(), oracle.matmul_tn(xp, dpre, THREADS), f"d_up[{e}]", **tol)
    assert torch.isfinite(dx).all() and torch.isfinite(gg).all()
    # linearity, at full size: twice the upstream gradient gives twice every gradient (the
    # activations are fixed), up to the bf16 rounding of the intermediates
    d_up2 = torch.zeros_like(d_up)
    d_dn2 = torch.zeros_like(d_dn)
    dx2, _ = ffn.backward((dy.float() * 2).to(torch.bfloat16), d_up2, d_dn2)
    assert gemm.device_status() == 0
    assert torch.equal(dx2, 2 * dx)
    # the chunks of a group add into its matrix in no fixed order, so these agree to fp32 rounding only
    for got, want in ((d_dn2, d_dn), (d_up2, d_up)):
        err = (got - 2 * want).norm() / (2 * want).norm()
        assert float(err) < 1e-5
