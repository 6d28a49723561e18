"""GPU parity of MoE routing (bit-exact integers) and the grouped expert GEMM.

Routing cases restate the reference's: the tie golden vector
(crates/nn/tests/moe.rs:182-197, gpu/ops/src/main.rs:1260-1283), the bin-assign
shape N=2500, E=5, K=2, C=720 with its formula routing (gpu/ops/src/main.rs:914-1036),
forced drops (crates/nn/tests/moe.rs:148-151) and the 64-expert top-8 configuration
with Zipf-skewed loads.
"""
import numpy as np
import pytest

from _util import THREADS, assert_gemm_close, bf16_operand, from_dev_bf16, to_dev_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gemm(pkg):
    g = pkg.Tcgen05Gemm()
    yield g
    g.close()


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


def _check_routing(pkg, oracle, gemm, probs, top_k, capacity):
    import torch
    want = oracle.moe_route(probs, top_k, capacity)
    r = pkg.moe.route(gemm, torch.from_numpy(probs).cuda(), top_k, capacity)
    assert np.array_equal(_u32(r.selected_experts), want["selected"])
    assert np.array_equal(_u32(r.slots), want["slots"])
    assert np.array_equal(_u32(r.assignment_counts), want["assignment_counts"])
    assert np.array_equal(_u32(r.accepted_counts), want["accepted_counts"])
    assert np.array_equal(_u32(r.offsets), want["offsets"])
    assert np.array_equal(_u32(r.dest_row), want["dest_row"])
    assert np.array_equal(r.gate_weights.cpu().numpy(), want["gates"])       # bit-exact gates too
    return r, want


def test_routing_tie_golden_vector(pkg, oracle, gemm):
    probs = oracle.softmax_rows(np.zeros((3, 3), np.float32))
    r, _ = _check_routing(pkg, oracle, gemm, probs, 2, 2)
    D = 0xFFFFFFFF
    assert _u32(r.selected_experts).tolist() == [0, 1, 0, 1, 0, 1]
    assert _u32(r.slots).tolist() == [0, 0, 1, 1, D, D]
    assert r.gate_weights.cpu().tolist() == [0.5] * 6


def test_bin_assign_reference_shape_with_drops(pkg, oracle, gemm):
    # gpu/ops/src/main.rs:935-937: token t prefers experts (t % E) and ((t * 3 + 1) % E).
    N, E, K, Cap = 2500, 5, 2, 720
    probs = np.full((N, E), 0.02, np.float32)
    t = np.arange(N)
    probs[t, t % E] += 0.5
    probs[t, (t * 3 + 1) % E] += 0.3
    probs /= probs.sum(1, keepdims=True)
    _, want = _check_routing(pkg, oracle, gemm, probs, K, Cap)
    assert int((want["slots"] == 0xFFFFFFFF).sum()) > 0          # the shape does force drops


@pytest.mark.parametrize("tokens,experts,top_k", [(4096, 64, 8), (1000, 8, 2), (257, 256, 16), (64, 3, 3)])
def test_routing_matches_oracle_with_ties_and_skew(pkg, oracle, gemm, tokens, experts, top_k):
    logits = oracle.normal(tokens * experts, 31).reshape(tokens, experts)
    logits += 0.5 * np.log(1.0 / np.arange(1, experts + 1, dtype=np.float32))   # Zipf-skewed loads
    probs = oracle.softmax_rows(logits)
    probs[5] = probs[5, 0]                       # a full tie row
    probs[7, 1] = probs[7, 2]                    # a pair tie
    _check_routing(pkg, oracle, gemm, probs, top_k, tokens * top_k)
    _check_routing(pkg, oracle, gemm, probs, top_k, max(1, tokens * top_k // (2 * experts)))


def test_routing_from_logits_agrees_with_probabilities(pkg, oracle, gemm):
    import torch
    tokens, experts, top_k = 2048, 64, 8
    logits = oracle.normal(tokens * experts, 32).reshape(tokens, experts)
    probs = oracle.softmax_rows(logits)
    a = pkg.moe.route(gemm, torch.from_numpy(logits).cuda(), top_k, scores_are_logits=True)
    want = oracle.moe_route(probs, top_k, tokens * top_k)
    # softmax is monotonic, so the selection agrees wherever probabilities did not round into a tie
    same = _u32(a.selected_experts) == want["selected"]
    assert same.mean() > 0.999
    assert np.allclose(a.gate_weights.cpu().numpy()[same], want["gates"][same], rtol=2e-6, atol=1e-7)


def _ragged_offsets(sizes):
    return np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)


@pytest.mark.parametrize("transposed_b", [False, True])
@pytest.mark.parametrize("silu", [False, True])
def test_grouped_gemm_ragged_groups(pkg, oracle, gemm, transposed_b, silu):
    import torch
    sizes = [300, 0, 17, 256, 1, 513, 128, 31]        # empty, tiny, exact-tile and straddling groups
    offsets = _ragged_offsets(sizes)
    rows, k, n, G = int(offsets[-1]), 192, 320, len(sizes)
    a, av = bf16_operand(oracle, (rows, k), 41)
    b, bv = bf16_operand(oracle, (G, k, n) if transposed_b else (G, n, k), 42, std=0.1)
    out = torch.full((rows + 8, n), 9.0, dtype=torch.bfloat16, device="cuda")   # canary rows at the end
    pkg.moe.grouped_gemm(gemm, a, b, torch.from_numpy(offsets).cuda(), out=out[:rows],
                         transposed_b=transposed_b, silu=silu)
    assert gemm.device_status() == 0
    got = from_dev_bf16(out)
    assert np.all(got[rows:] == 9.0)
    for g in range(G):
        lo, hi = offsets[g], offsets[g + 1]
        if lo == hi:
            continue
        w = bv[g] if transposed_b else bv[g].T            # [k, n]
        ref = oracle.matmul(av[lo:hi], np.ascontiguousarray(w), THREADS)
        if silu:
            ref = oracle.silu(ref)
        assert_gemm_close(got[lo:hi], ref, f"group {g}", rel_fro=4e-3, elem=8e-3)


@pytest.mark.parametrize("ff,want_panel", [(768, True), (192, True), (320, True), (200, False)])
def test_grouped_gemm_swiglu_matches_oracle(pkg, oracle, gemm, ff, want_panel):
    """silu(x W_gate) * (x W_up) over ragged groups in one launch, and the bf16 [rows, 2, ff]
    panel beside it (crates/nn/src/swiglu.rs:22-28 over the fused gate/up projection,
    crates/nn/src/moe.rs:76-90).  ff = 192, 320 and 200 leave a partly filled column tile."""
    import torch
    sizes = [300, 0, 17, 256, 1, 513, 128, 31]
    offsets = _ragged_offsets(sizes)
    rows, k, G = int(offsets[-1]), 192, len(sizes)
    a, av = bf16_operand(oracle, (rows, k), 45)
    w, wv = bf16_operand(oracle, (G, k, 2, ff), 46, std=0.1)
    y = torch.full((rows + 8, ff), 9.0, dtype=torch.bfloat16, device="cuda")
    panel = torch.full((rows + 8, 2, ff), 7.0, dtype=torch.bfloat16, device="cuda") if want_panel else None
    pkg.moe.grouped_gemm_swiglu(gemm, a, w, torch.from_numpy(offsets).cuda(), out=y[:rows],
                                gate_up=None if panel is None else panel[:rows])
    assert gemm.device_status() == 0
    got = from_dev_bf16(y)
    assert np.all(got[rows:] == 9.0)
    if want_panel:
        got_panel = from_dev_bf16(panel)
        assert np.all(got_panel[rows:] == 7.0)
    for g in range(G):
        lo, hi = offsets[g], offsets[g + 1]
        if lo == hi:
            continue
        gate = oracle.matmul(av[lo:hi], np.ascontiguousarray(wv[g, :, 0, :]), THREADS)
        up = oracle.matmul(av[lo:hi], np.ascontiguousarray(wv[g, :, 1, :]), THREADS)
        assert_gemm_close(got[lo:hi], oracle.swiglu(gate, up), f"group {g}", rel_fro=4e-3, elem=8e-3)
        if want_panel:
            assert_gemm_close(got_panel[lo:hi, 0], gate, f"gate {g}", rel_fro=4e-3, elem=8e-3)
            assert_gemm_close(got_panel[lo:hi, 1], up, f"up {g}", rel_fro=4e-3, elem=8e-3)


def test_grouped_gemm_swiglu_dense_and_indexed(pkg, oracle, gemm):
    """One group is the dense gated MLP; an index maps several groups onto one matrix."""
    import torch
    rows, k, ff = 700, 128, 256
    a, av = bf16_operand(oracle, (rows, k), 47)
    w, wv = bf16_operand(oracle, (2, k, 2, ff), 48, std=0.1)
    offsets = torch.tensor([0, rows], dtype=torch.int32, device="cuda")
    y = pkg.moe.grouped_gemm_swiglu(gemm, a, w[:1], offsets)
    ref0 = oracle.swiglu(oracle.matmul(av, np.ascontiguousarray(wv[0, :, 0, :]), THREADS),
                         oracle.matmul(av, np.ascontiguousarray(wv[0, :, 1, :]), THREADS))
    assert_gemm_close(from_dev_bf16(y), ref0, "dense", rel_fro=4e-3, elem=8e-3)
    # three groups: matrices 1, 0, 1
    offs = torch.tensor([0, 300, 301, rows], dtype=torch.int32, device="cuda")
    index = torch.tensor([1, 0, 1], dtype=torch.int32, device="cuda")
    y2 = from_dev_bf16(pkg.moe.grouped_gemm_swiglu(gemm, a, w, offs, group_b_index=index))
    ref1 = oracle.swiglu(oracle.matmul(av, np.ascontiguousarray(wv[1, :, 0, :]), THREADS),
                         oracle.matmul(av, np.ascontiguousarray(wv[1, :, 1, :]), THREADS))
    assert_gemm_close(y2[:300], ref1[:300], "group 0", rel_fro=4e-3, elem=8e-3)
    assert_gemm_close(y2[300:301], ref0[300:301], "group 1", rel_fro=4e-3, elem=8e-3)
    assert_gemm_close(y2[301:], ref1[301:], "group 2", rel_fro=4e-3, elem=8e-3)
    assert gemm.device_status() == 0
    with pytest.raises(pkg.B200GemmError):                      # a panel needs ff % 64 == 0
        w200, _ = bf16_operand(oracle, (1, k, 2, 200), 49)
        pkg.moe.grouped_gemm_swiglu(gemm, a, w200, offsets, want_gate_up=True)


def test_grouped_gemm_swiglu_k_major_weights(pkg, oracle, gemm):
    """The same product with the gate/up matrices stored [2 * ff, k] (K-major), through the C ABI."""
    import torch
    from oxide_train_b200 import _lib as L
    from oxide_train_b200.gemm import _stream_ptr
    sizes = [129, 300, 0, 64]
    offsets = _ragged_offsets(sizes)
    rows, k, ff, G = int(offsets[-1]), 128, 192, len(sizes)
    a, _ = bf16_operand(oracle, (rows, k), 61)
    w, _ = bf16_operand(oracle, (G, k, 2, ff), 62, std=0.1)
    offs = torch.from_numpy(offsets).cuda()
    want_y, want_panel = pkg.moe.grouped_gemm_swiglu(gemm, a, w, offs, want_gate_up=True)
    wk = w.permute(0, 2, 3, 1).contiguous().reshape(G, 2 * ff, k)          # [G, 2*ff, k]
    y = torch.zeros((rows, ff), dtype=torch.bfloat16, device="cuda")
    panel = torch.zeros((rows, 2, ff), dtype=torch.bfloat16, device="cuda")
    L.check(gemm._lib.b200gemm_grouped_gemm_swiglu(
        gemm._h, _stream_ptr(), a.data_ptr(), k, wk.data_ptr(), L.K_MAJOR, k, 2 * ff * k, G, None,
        y.data_ptr(), ff, panel.data_ptr(), 2 * ff, offs.data_ptr(), G, rows, ff, k))
    assert gemm.device_status() == 0
    assert torch.equal(y, want_y) and torch.equal(panel, want_panel)


def test_grouped_gemm_leaves_rows_outside_groups_untouched(pkg, oracle, gemm):
    import torch
    offsets = np.array([0, 100, 100, 260], np.int32)       # total 260 of 400 rows are routed
    rows, k, n = 400, 64, 256
    a, _ = bf16_operand(oracle, (rows, k), 43)
    b, _ = bf16_operand(oracle, (3, n, k), 44)
    out = torch.full((rows, n), 3.0, dtype=torch.bfloat16, device="cuda")
    pkg.moe.grouped_gemm(gemm, a, b, torch.from_numpy(offsets).cuda(), out=out)
    assert gemm.device_status() == 0
    assert torch.all(out[260:] == 3.0).item()
    assert not torch.all(out[:260] == 3.0).item()


def test_moe_forward_small_matches_oracle(pkg, oracle, gemm):
    """route -> scatter -> up + SiLU -> down -> combine against the CPU composition
    (crates/nn/src/moe.rs:283-352) with the same bf16 rounding points."""
    import torch
    N, D, FF, E, K = 600, 128, 192, 8, 2
    x, xv = bf16_operand(oracle, (N, D), 51)
    w_up, upv = bf16_operand(oracle, (E, D, FF), 52, std=0.1)
    w_dn, dnv = bf16_operand(oracle, (E, FF, D), 53, std=0.1)
    logits = oracle.normal(N * E, 54).reshape(N, E)
    probs = oracle.softmax_rows(logits)
    ffn = pkg.GroupedExpertFfn(gemm, w_up, w_dn)
    out, r = ffn.forward(x, torch.from_numpy(probs).cuda(), K, residual=x)
    assert gemm.device_status() == 0
    want = oracle.moe_route(probs, K, N * K)
    ref = xv.copy()
    sel = want["selected"].reshape(N, K)
    gates = want["gates"].reshape(N, K)
    for e in range(E):
        toks, ranks = np.nonzero(sel == e)
        if toks.size == 0:
            continue
        h = oracle.bf16_round(oracle.silu(oracle.matmul(xv[toks], upv[e], THREADS)))
        y = oracle.bf16_round(oracle.matmul(h, dnv[e], THREADS))
        for t, rk, row in zip(toks, ranks, y):
            ref[t] += gates[t, rk] * row                  # order differs from rank order only by fp32 rounding
    assert_gemm_close(out.cpu().numpy(), ref, "moe forward", rel_fro=5e-3, elem=1e-2)


def test_moe_full_size_properties(pkg, oracle, gemm):
    """The 64-expert configuration at full size: 32768 tokens, D=1536, E=64, top-8, FF=768."""
    import torch
    N, D, FF, E, K = 32768, 1536, 768, 64, 8
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4)
    x = torch.randn((N, D), generator=gen, device="cuda").to(torch.bfloat16)
    w_up = (torch.randn((E, D, FF), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    w_dn = (torch.randn((E, FF, D), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    bias = 0.5 * torch.log(1.0 / torch.arange(1, E + 1, device="cuda", dtype=torch.float32))
    logits = torch.randn((N, E), generator=gen, device="cuda") + bias
    ffn = pkg.GroupedExpertFfn(gemm, w_up, w_dn)
    out, r = ffn.forward(x, logits.contiguous(), K, scores_are_logits=True)
    assert gemm.device_status() == 0
    counts = _u32(r.assignment_counts).astype(np.int64)
    assert counts.sum() == N * K
    assert counts[0] > counts[-1]                                    # Zipf skew
    dest = _u32(r.dest_row).astype(np.int64)
    assert np.array_equal(np.sort(dest), np.arange(N * K))           # a permutation: nothing dropped
    offs = _u32(r.offsets).astype(np.int64)
    assert np.array_equal(offs, np.concatenate([[0], np.cumsum(counts)]))
    sel = _u32(r.selected_experts).reshape(N, K)
    g = r.gate_weights.cpu().numpy().reshape(N, K)
    assert np.allclose(g.sum(1), 1.0, atol=1e-5)
    # sampled tokens against the oracle composition
    xs = x.float().cpu().numpy()
    up = w_up.float().cpu().numpy()
    dn = w_dn.float().cpu().numpy()
    toks = np.array([0, 1, 777, 16384, 32767])
    ref = np.zeros((toks.size, D), np.float32)
    for i, t in enumerate(toks):
        for rk in range(K):
            e = sel[t, rk]
            h = oracle.bf16_round(oracle.silu(oracle.matmul(xs[t:t + 1], up[e], 1)))
            y = oracle.bf16_round(oracle.matmul(h, dn[e], 1))
            ref[i] += g[t, rk] * y[0]
    assert_gemm_close(out[toks].cpu().numpy(), ref, "sampled tokens", rel_fro=5e-3, elem=1e-2)
