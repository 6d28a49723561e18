"""GPU parity of the fused lm-head + softmax cross-entropy against the CPU oracle.

The oracle path is the reference's CPU one: ``Linear::forward`` (a matmul,
crates/nn/src/linear.rs:42-44) feeding ``SoftmaxCrossEntropy``
(crates/nn/src/cross_entropy.rs:28-72), then ``Linear::backward``.  Tolerances
follow the reference's classifier gate (gpu/ops/src/main.rs:1984-2110: loss
5e-5, dlogits 4e-3 relative, padded columns exactly zero) and the GEMM contract
for the two gradient products.
"""
import numpy as np
import pytest

from _util import THREADS, assert_gemm_close, bf16_operand, from_dev_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gemm(pkg):
    g = pkg.Tcgen05Gemm()
    yield g
    g.close()


def _oracle_head(oracle, hv, wv_kv, targets, classes):
    logits = oracle.matmul(hv, wv_kv, THREADS)
    loss, probs, row_loss = oracle.xent_forward(logits, targets, classes)
    dlogits = oracle.xent_backward(probs, targets, classes)
    z = logits[:, :classes].astype(np.float64)
    lse = np.log(np.exp(z - z.max(1, keepdims=True)).sum(1)) + z.max(1)
    return logits, loss, row_loss, lse, dlogits


@pytest.mark.parametrize("m,k,v,classes", [(512, 256, 1024, 1000), (300, 192, 520, 515), (256, 64, 256, 256)])
@pytest.mark.parametrize("layout", ["in_out", "out_in"])
def test_fused_head_matches_oracle(pkg, oracle, gemm, m, k, v, classes, layout):
    import torch
    h, hv = bf16_operand(oracle, (m, k), 21)
    w_kv, wv = bf16_operand(oracle, (k, v), 22, std=0.3)
    targets = (oracle.uniform(m, 23) * 0.5 + 0.5) * classes
    targets = np.clip(targets.astype(np.int32), 0, classes - 1)
    logits, loss, row_loss, lse, dlogits = _oracle_head(oracle, hv, wv, targets, classes)
    w = w_kv if layout == "in_out" else w_kv.t().contiguous()
    t = torch.from_numpy(targets).cuda()
    head = pkg.FusedLmHead(gemm, classes, layout)
    g_loss, g_lse, g_row = head.forward(h, w, t)
    assert gemm.device_status() == 0
    assert abs(float(g_loss.item()) - float(loss)) <= 5e-5 * max(1.0, abs(float(loss)))
    assert np.allclose(g_lse.cpu().numpy(), lse, atol=2e-4, rtol=1e-5)
    assert np.allclose(g_row.cpu().numpy(), row_loss, atol=2e-4, rtol=1e-5)

    g_dl, g_dh, g_dw = head.backward(h, w, t, g_lse)
    assert gemm.device_status() == 0
    dl = from_dev_bf16(g_dl)
    assert np.all(dl[:, classes:] == 0.0)                      # padded columns are exactly zero
    scale = np.abs(dlogits).max()
    assert np.max(np.abs(dl - dlogits)) <= 4e-3 * scale + 1e-8  # bf16 rounding of the gradient
    # gradient products, from the dlogits the kernel actually produced (bf16)
    dh_ref = oracle.matmul_nt(dl, wv, THREADS)                  # dlogits . W^T
    dw_ref = oracle.matmul_tn(hv, dl, THREADS)                  # hidden^T . dlogits, [k, v]
    assert_gemm_close(g_dh.cpu().numpy(), dh_ref, "d_hidden", rel_fro=1e-4, elem=1e-3)
    got_dw = g_dw.cpu().numpy() if layout == "in_out" else g_dw.cpu().numpy().T
    assert_gemm_close(got_dw, dw_ref, "d_weight", rel_fro=1e-4, elem=1e-3)
    # and against the full-precision oracle gradients, at the GEMM contract's tolerance
    assert_gemm_close(g_dh.cpu().numpy(), oracle.matmul_nt(dlogits, wv, THREADS), "d_hidden vs fp32 path")
    # accumulate into an existing d_weight
    _, _, g_dw2 = head.backward(h, w, t, g_lse, d_weight=g_dw.clone(), accumulate_dw=True, want_d_hidden=False)
    assert_gemm_close(g_dw2.cpu().numpy(), 2 * g_dw.cpu().numpy(), "d_weight accumulate", rel_fro=1e-5, elem=1e-4)


def test_fused_head_full_size_properties(pkg, oracle, gemm):
    """The 183M dense model's head at full size (32768 x 1536 x 50432, 50257 classes): sampled rows against the
    oracle and size-independent properties of the gradient."""
    import torch
    m, k, v, classes = 32768, 1536, 50432, 50257
    # The configuration's own inputs: SplitMix64 uniforms, Box-Muller normals on top, seed 1;
    # hidden ~ N(0, 1), weight ~ N(0, 0.02) with the padded columns masked, targets uniform.
    h, hv_all = bf16_operand(oracle, (m, k), 1)
    w_bits = oracle.bf16_bits(oracle.normal(k * v, 2, 0.0, 0.02)).reshape(k, v)
    w_bits[:, classes:] = 0
    from _util import to_dev_bf16
    w = to_dev_bf16(w_bits)
    tv_all = np.clip(((oracle.uniform(m, 3) * 0.5 + 0.5) * classes).astype(np.int32), 0, classes - 1)   # uniform is in [-1, 1)
    t = torch.from_numpy(tv_all).cuda()
    head = pkg.FusedLmHead(gemm, classes, "in_out")
    loss, lse, row_loss = head.forward(h, w, t)
    assert gemm.device_status() == 0
    rows = np.array([0, 1, 127, 128, 255, 256, 4095, 16384, 32767, 20001])
    hv = h[rows].float().cpu().numpy()
    wv = w.float().cpu().numpy()
    tv = t.cpu().numpy()
    logits = oracle.matmul(hv, wv, THREADS)
    _, probs, rl = oracle.xent_forward(logits, tv[rows], classes)
    assert np.allclose(row_loss.cpu().numpy()[rows], rl, atol=5e-4, rtol=1e-5)
    assert abs(float(loss.item()) - float(row_loss.double().mean().item())) < 1e-5
    # logits ~ N(0, k * 0.02^2): the expected loss is ln(classes) + variance / 2
    assert abs(float(loss.item()) - (np.log(classes) + 0.5 * k * 0.02 ** 2)) < 0.05
    dl, dh, dw = head.backward(h, w, t, lse)
    assert gemm.device_status() == 0
    assert torch.all(dl[:, classes:] == 0).item()
    sums = dl.float().sum(dim=1)
    assert float(sums.abs().max().item()) < 1e-5                     # rows of p - onehot sum to 0
    # the oracle divides by its own row count; rescale to the kernel's 1 / m
    ref_dl = oracle.xent_backward(probs, tv[rows], classes, dy=len(rows) / m)
    got = dl[rows].float().cpu().numpy()
    assert np.max(np.abs(got - ref_dl)) <= 4e-3 * np.abs(ref_dl).max()
    # d_hidden of the sampled rows from the kernel's own dlogits
    ref_dh = oracle.matmul_nt(got, wv, THREADS)
    assert_gemm_close(dh[rows].cpu().numpy(), ref_dh, "d_hidden rows", rel_fro=1e-4, elem=1e-3)
    # d_weight: sampled column blocks (one of them across the first padded column) against the
    # oracle's matmul_tn over all 32768 rows, from the dlogits the kernel produced
    for c0 in (0, 25000, 50240):
        cols = slice(c0, c0 + 24)
        ref_dw = oracle.matmul_tn(hv_all, np.ascontiguousarray(dl[:, cols].float().cpu().numpy()), THREADS)
        assert_gemm_close(dw[:, cols].cpu().numpy(), ref_dw, f"d_weight columns {c0}..", rel_fro=1e-4, elem=1e-3)
    assert not dw[:, classes:].any().item()                          # padded columns get no gradient


def test_target_outside_the_classes_is_reported(pkg, oracle, gemm):
    """A target index outside [0, classes) has no logit (the reference asserts on it,
    crates/nn/src/cross_entropy.rs:38): that row's loss and the mean are NaN and the device
    status says so, instead of a number built on whatever an earlier call left behind."""
    import torch
    m, k, v, classes = 512, 128, 512, 500
    h, _ = bf16_operand(oracle, (m, k), 26)
    w, _ = bf16_operand(oracle, (k, v), 27, std=0.3)
    t = torch.randint(0, classes, (m,), device="cuda", dtype=torch.int32)
    head = pkg.FusedLmHead(gemm, classes, "in_out")
    good_loss, _, good_rows = head.forward(h, w, t)
    assert gemm.device_status() == 0
    t_bad = t.clone()
    t_bad[7], t_bad[300] = -100, classes                          # an ignore-index style value, and one past the end
    loss, lse, rows = head.forward(h, w, t_bad)
    with pytest.raises(pkg.B200GemmError) as e:
        gemm.device_status()
    assert e.value.code == pkg._lib.ERR_DEVICE and "107" in str(e.value)
    r = rows.cpu().numpy()
    assert np.isnan(r[7]) and np.isnan(r[300]) and np.isnan(float(loss.item()))
    keep = np.ones(m, bool)
    keep[[7, 300]] = False
    assert np.array_equal(r[keep], good_rows.cpu().numpy()[keep])
    assert gemm.device_status() == 0
    assert float(head.forward(h, w, t)[0].item()) == float(good_loss.item())     # and the handle is fine afterwards


@pytest.mark.parametrize("world", [2, 5, 8])
def test_vocabulary_shards_emulated_on_one_gpu(pkg, oracle, gemm, world):
    """The sharded head with its ranks emulated one after another on one device: every shard's
    forward, the merge of their statistics, every shard's backward, and the sum of the partial
    input gradients -- against the ORACLE on the whole vocabulary.  13 column tiles split
    unevenly (5 ranks: 3,3,3,2,2; 8 ranks: 2,2,2,2,2,1,1,1), the last real column inside the
    last tile."""
    import torch
    par = pkg.parallel
    m, k, v, classes = 768, 192, 13 * 256, 13 * 256 - 41
    h, hv = bf16_operand(oracle, (m, k), 28)
    w, wv = bf16_operand(oracle, (k, v), 29, std=0.3)
    wv[:, classes:] = 0
    w[:, classes:] = 0
    targets = np.clip(((oracle.uniform(m, 30) * 0.5 + 0.5) * classes).astype(np.int32), 0, classes - 1)
    targets[:4] = [0, classes - 1, 255, 256]                      # shard and tile edges
    logits, loss, row_loss, lse, dlogits = _oracle_head(oracle, hv, wv, targets, classes)
    ops = par.DeviceOps(gemm)
    shards = par.vocab_shards(v, world)
    t = torch.from_numpy(targets).cuda()
    stats, locals_ = [], []
    for (c0, c1) in shards:
        cl = max(0, min(classes, c1) - c0)
        lt = (t - c0).to(torch.int32)
        locals_.append((c0, c1, cl, lt, w[:, c0:c1].contiguous()))
        stats.append(ops.head_forward_shard(h, locals_[-1][4], lt, cl, "in_out"))
    g_lse, g_rows, g_loss = ops.head_merge_shards(torch.stack(stats).contiguous())
    assert gemm.device_status() == 0
    assert abs(float(g_loss.item()) - float(loss)) <= 5e-5 * max(1.0, abs(float(loss)))
    assert np.allclose(g_lse.cpu().numpy(), lse, atol=2e-4, rtol=1e-5)
    assert np.allclose(g_rows.cpu().numpy(), row_loss, atol=2e-4, rtol=1e-5)
    # the header's merge formula in plain numpy gives the same rows
    st = torch.stack(stats).cpu().numpy().astype(np.float64)
    M = st[:, 0].max(0)
    S = (st[:, 1] * np.exp(st[:, 0] - M)).sum(0)
    assert np.allclose(M + np.log(S), lse, atol=2e-4, rtol=1e-5)
    dh_sum = np.zeros((m, k), np.float32)
    scale = np.abs(dlogits).max()
    for (c0, c1, cl, lt, ws) in locals_:
        head = pkg.FusedLmHead(gemm, cl, "in_out")
        dl, dh, dw = head.backward(h, ws, lt, g_lse)
        assert gemm.device_status() == 0
        got = from_dev_bf16(dl)
        assert np.max(np.abs(got - dlogits[:, c0:c1])) <= 4e-3 * scale + 1e-8
        assert np.all(got[:, cl:] == 0.0)
        assert_gemm_close(dw.cpu().numpy(), oracle.matmul_tn(hv, got, THREADS), f"d_weight shard {c0}", rel_fro=1e-4, elem=1e-3)
        dh_sum += dh.cpu().numpy()
    assert_gemm_close(dh_sum, oracle.matmul_nt(dlogits, wv, THREADS), "summed d_hidden")
