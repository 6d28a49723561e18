"""The sharded paths on real GPUs: 2 ranks over NCCL, compared with the CPU oracle (whole
matrices for the head, sampled rows for the expert and MLP paths) and with the same
computation done by the single-GPU kernels on each rank.  Needs two GPUs; skips itself
otherwise (the shard arithmetic itself is also covered on one GPU, ranks emulated, in the
lm-head and MoE-exchange tests).  Child processes, NVLS off, ranks leave only between steps."""
import os
import socket
import sys
import traceback

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORLD = 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, port, failures):
    try:
        import torch
        import torch.distributed as dist
        sys.path.insert(0, ROOT)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=dev)
        import __graft_entry__ as entry
        pkg = entry.load_package()
        import numpy as np
        from oracle import oracle as orc
        orc.lib()
        par = pkg.parallel
        gemm = pkg.Tcgen05Gemm(rank)
        ops = par.DeviceOps(gemm)
        gen = torch.Generator(device=dev)
        gen.manual_seed(5)                                   # same data on every rank
        bf = torch.bfloat16

        # ---- the barrier kernel: integers gathered on the way, data stored before it visible after it
        bar = par.PeerBarrier(ops, None, dev, payload_count=6)
        import torch.distributed._symmetric_memory as symm_mem
        box = symm_mem.empty((WORLD, 4096), dtype=torch.float32, device=dev)
        hbox = symm_mem.rendezvous(box, dist.group.WORLD.group_name)
        for step in range(1, 5):
            mine = torch.arange(6, dtype=torch.int32, device=dev) * (rank + 1) + 100 * step
            for r in range(WORLD):                            # my row of every rank's box
                hbox.get_buffer(r, (WORLD, 4096), torch.float32)[rank].copy_(
                    torch.full((4096,), float(step * 10 + rank), device=dev), non_blocking=True)
            got = bar.all_gather_i32(mine)
            for r in range(WORLD):
                assert got[r].tolist() == [j * (r + 1) + 100 * step for j in range(6)], (step, r)
                assert bool((box[r] == float(step * 10 + r)).all()), (step, r)
            bar.barrier()                                     # nobody overwrites a row a peer still reads
        assert gemm.device_status() == 0
        # a peer that never comes: the wait gives up, the host reads code 108, the context
        # stays usable (only rank 0 calls; its arrival word stays behind, so the object is dropped)
        lonely = par.PeerBarrier(ops, None, dev, limit_ms=100)
        if rank == 0:
            lonely.barrier()
            try:
                gemm.device_status()
                raise AssertionError("the wait should have run out")
            except pkg.B200GemmError as e:
                assert e.code == pkg._lib.ERR_DEVICE and "108" in str(e)
        assert gemm.device_status() == 0
        dist.barrier()
        del lonely

        # ---- vocabulary-parallel head vs the single-GPU fused head
        m, k, v, classes = 1024, 256, 2048, 2000
        h = torch.randn((m, k), generator=gen, device=dev).to(bf)
        w = (torch.randn((k, v), generator=gen, device=dev) * 0.2).to(bf)
        t = torch.randint(0, classes, (m,), generator=gen, device=dev, dtype=torch.int32)
        single = pkg.FusedLmHead(gemm, classes, "in_out")
        loss1, lse1, row1 = single.forward(h, w, t)
        _, dh1, dw1 = single.backward(h, w, t, lse1)
        head = par.VocabParallelHead(ops, classes, v)
        ws = head.shard_weight(w)
        loss2, lse2, row2 = head.forward(h, ws, t)
        assert abs(float(loss1.item()) - float(loss2.item())) < 5e-5
        assert torch.allclose(lse1, lse2, atol=2e-4, rtol=1e-5)
        _, dh2, dw2 = head.backward(h, ws, t, lse2)
        # partial sums cross the link as bf16: the GEMM contract's relative Frobenius bound
        assert float((dh1 - dh2).norm() / dh1.norm()) < 1e-2
        # (the weight-gradient GEMM leaves 16 SMs to the all-reduce in this variant)
        head32 = par.VocabParallelHead(ops, classes, v, reduce_dtype=torch.float32, reserve_sms=16)
        _, dh3, _ = head32.backward(h, ws, t, lse2)
        assert torch.allclose(dh1, dh3, atol=2e-5, rtol=2e-2), float((dh1 - dh3).abs().max())
        assert torch.allclose(dw1[:, head.c0:head.c1], dw2, atol=2e-5, rtol=2e-2)
        # d_hidden summed by copy-engine pushes + a local sum, all rows and this rank's rows only, twice
        for mode in ("all", "scatter", "all"):
            headc = par.VocabParallelHead(ops, classes, v, exchange="copy", d_hidden=mode, reserve_sms=4)
            _, dhc, dwc = headc.backward(h, ws, t, lse2)
            want_rows = dh1 if mode == "all" else dh1[rank * m // WORLD:(rank + 1) * m // WORLD]
            assert float((want_rows - dhc).norm() / want_rows.norm()) < 1e-2, mode
            assert torch.equal(dwc, dw2)
        # ... and against the oracle: Linear::forward + SoftmaxCrossEntropy + Linear::backward on the CPU
        hv, wv, tv = h.float().cpu().numpy(), w.float().cpu().numpy(), t.cpu().numpy()
        o_logits = orc.matmul(hv, wv, 8)
        o_loss, o_probs, o_rows = orc.xent_forward(o_logits, tv, classes)
        o_dl = orc.xent_backward(o_probs, tv, classes)
        assert abs(float(loss2.item()) - float(o_loss)) <= 5e-5 * max(1.0, abs(float(o_loss)))
        assert np.allclose(row2.cpu().numpy(), o_rows, atol=2e-4, rtol=1e-5)
        o_dh = orc.matmul_nt(o_dl, wv, 8)
        for name, got in (("bf16 partial sums", dh2), ("fp32 partial sums", dh3)):
            rel = np.linalg.norm(got.cpu().numpy() - o_dh) / np.linalg.norm(o_dh)
            assert rel <= 1e-2, (name, rel)
        o_dw = orc.matmul_tn(hv, np.ascontiguousarray(o_dl[:, head.c0:head.c1]), 8)
        rel = np.linalg.norm(dw2.cpu().numpy() - o_dw) / np.linalg.norm(o_dw)
        assert rel <= 1e-2, ("d_weight shard", rel)

        # ---- expert-parallel MoE vs the single-GPU grouped path on this rank's tokens
        n_local, d, ff, experts, top_k = 1024, 256, 384, 8, 2
        x = torch.randn((WORLD, n_local, d), generator=gen, device=dev).to(bf)
        up = (torch.randn((experts, d, ff), generator=gen, device=dev) * 0.1).to(bf)
        dn = (torch.randn((experts, ff, d), generator=gen, device=dev) * 0.1).to(bf)
        logits = torch.randn((WORLD, n_local, experts), generator=gen, device=dev)
        ref, _ = pkg.GroupedExpertFfn(gemm, up, dn).forward(x[rank].contiguous(), logits[rank].contiguous(),
                                                             top_k, scores_are_logits=True)
        local = experts // WORLD
        ep = par.ExpertParallelMoe(ops, experts, top_k, up[rank * local:(rank + 1) * local].contiguous(),
                                   dn[rank * local:(rank + 1) * local].contiguous())
        out = ep.forward(x[rank].contiguous(), logits[rank].contiguous(), scores_are_logits=True)
        assert torch.allclose(out, ref, atol=1e-5, rtol=1e-5), float((out - ref).abs().max())
        # sampled tokens against the oracle: route on the CPU, each selected expert's
        # down(silu(up(x))) with the bf16 roundings the kernels apply, gates in rank order
        xr = x[rank].float().cpu().numpy()
        probs = orc.softmax_rows(logits[rank].cpu().numpy())
        want = orc.moe_route(probs, top_k, n_local * top_k)
        upv, dnv = up.float().cpu().numpy(), dn.float().cpu().numpy()
        for tok in (0, 17, n_local - 1):
            acc = np.zeros(d, np.float32)
            for rk in range(top_k):
                e = int(want["selected"][tok * top_k + rk])
                hdn = orc.bf16_round(orc.silu(orc.matmul(xr[tok:tok + 1], upv[e], 1)))
                acc += want["gates"][tok * top_k + rk] * orc.bf16_round(orc.matmul(hdn, dnv[e], 1))[0]
            got = out[tok].cpu().numpy()
            assert np.max(np.abs(got - acc) / (1.0 + np.abs(acc))) <= 2e-2, tok
        # the same exchange by copy-engine pushes into peer memory, in two slices, twice in a row
        ep2 = par.ExpertParallelMoe(ops, experts, top_k, up[rank * local:(rank + 1) * local].contiguous(),
                                    dn[rank * local:(rank + 1) * local].contiguous(), pieces=2,
                                    use_peer_copies=True)
        for _ in range(2):
            out2 = ep2.forward(x[rank].contiguous(), logits[rank].contiguous(), scores_are_logits=True)
            assert ep2.last["exchange"] == "peer copies" and ep2.last["pieces"] == 2
            assert torch.allclose(out2, ref, atol=1e-5, rtol=1e-5), float((out2 - ref).abs().max())

        # the device-driven exchange (peer stores / peer loads, no host round trip), twice in a row
        ep3 = par.ExpertParallelMoe(ops, experts, top_k, up[rank * local:(rank + 1) * local].contiguous(),
                                    dn[rank * local:(rank + 1) * local].contiguous(), pieces=2, exchange="device")
        for _ in range(2):
            out3 = ep3.forward(x[rank].contiguous(), logits[rank].contiguous(), scores_are_logits=True)
            assert ep3.last["exchange"] == "device"
            assert torch.allclose(out3, ref, atol=1e-5, rtol=1e-5), float((out3 - ref).abs().max())
        # ... with NCCL's all-gather and one-element all-reduces in place of the barrier kernel
        ep6 = par.ExpertParallelMoe(ops, experts, top_k, up[rank * local:(rank + 1) * local].contiguous(),
                                    dn[rank * local:(rank + 1) * local].contiguous(), pieces=2, exchange="device",
                                    barrier="nccl")
        for _ in range(2):
            out6 = ep6.forward(x[rank].contiguous(), logits[rank].contiguous(), scores_are_logits=True)
            assert torch.equal(out6, out3)
        # ... in four slices whose middle dispatches and combines are the few-block bulk-copy kernels
        ep7 = par.ExpertParallelMoe(ops, experts, top_k, up[rank * local:(rank + 1) * local].contiguous(),
                                    dn[rank * local:(rank + 1) * local].contiguous(), pieces=4, exchange="device",
                                    exchange_ctas=6, exchange_bulk=True)
        ep7.reserve_sms = 8
        for _ in range(2):
            out7 = ep7.forward(x[rank].contiguous(), logits[rank].contiguous(), scores_are_logits=True)
            assert ep7.last["pieces"] == 4
            assert torch.equal(out7, out3)
        # ... with the results sent home by the owner's down-projection GEMM itself (peer stores from its epilogue)
        ep5 = par.ExpertParallelMoe(ops, experts, top_k, up[rank * local:(rank + 1) * local].contiguous(),
                                    dn[rank * local:(rank + 1) * local].contiguous(), pieces=2, exchange="device",
                                    return_path="push")
        for _ in range(2):
            out5 = ep5.forward(x[rank].contiguous(), logits[rank].contiguous(), scores_are_logits=True)
            assert ep5.last["return_path"] == "push"
            assert torch.allclose(out5, ref, atol=1e-5, rtol=1e-5), float((out5 - ref).abs().max())
        # ... and with token slices of different sizes (a short first and last slice)
        ep4 = par.ExpertParallelMoe(ops, experts, top_k, up[rank * local:(rank + 1) * local].contiguous(),
                                    dn[rank * local:(rank + 1) * local].contiguous(), pieces=[1, 2, 1], exchange="device")
        for _ in range(2):
            out4 = ep4.forward(x[rank].contiguous(), logits[rank].contiguous(), scores_are_logits=True)
            assert ep4.last["pieces"] == 3
            assert torch.allclose(out4, ref, atol=1e-5, rtol=1e-5), float((out4 - ref).abs().max())
        assert gemm.device_status() == 0

        # ---- tensor-parallel MLP vs the unsharded product of the same bf16 operands
        m, d, ff = 2048, 512, 1024
        x2 = torch.randn((m, d), generator=gen, device=dev).to(bf)
        w1 = (torch.randn((d, ff), generator=gen, device=dev) * 0.05).to(bf)
        w2 = (torch.randn((ff, d), generator=gen, device=dev) * 0.05).to(bf)
        cols = slice(rank * ff // WORLD, (rank + 1) * ff // WORLD)
        mlp = par.TensorParallelMlp(ops, w1[:, cols].contiguous(), w2[cols].contiguous(), chunks=2,
                                    partial_dtype=torch.float32, reserve_sms=8)
        y = mlp.forward(x2)
        # oracle on sampled rows: hidden = bf16(x W1) as each shard rounds it, y = hidden W2
        rows = mlp.owned_rows(m)
        pick = rows[[0, 1, len(rows) // 2, len(rows) - 1]]
        hid = orc.bf16_round(orc.matmul(x2[pick].float().cpu().numpy(), w1.float().cpu().numpy(), 4))
        full = orc.matmul(hid, w2.float().cpu().numpy(), 4)
        got = y[[0, 1, len(rows) // 2, len(rows) - 1]].cpu().numpy()
        assert np.max(np.abs(got - full) / (1.0 + np.abs(full))) <= 2e-2
        assert np.linalg.norm(got - full) / np.linalg.norm(full) <= 1e-2
        assert gemm.device_status() == 0
        # the same block with the exchanges done by copy-engine pushes into peer memory and a
        # local sum, forward and backward, twice in a row (the second step reuses every buffer)
        shard = (w1[:, cols].contiguous(), w2[cols].contiguous())
        mlp_nccl = par.TensorParallelMlp(ops, *shard, chunks=[1, 2, 1], partial_dtype=bf)
        mlp_copy = par.TensorParallelMlp(ops, *shard, chunks=[1, 2, 1], partial_dtype=bf, exchange="copy")
        mlp_copy_nccl = par.TensorParallelMlp(ops, *shard, chunks=[1, 2, 1], partial_dtype=bf, exchange="copy",
                                              barrier="nccl")
        dy_local = (torch.randn((m // WORLD, d), generator=gen, device=dev) * 0.1).to(bf)
        rows = mlp_copy.owned_rows(m)                          # short pieces at both ends: another ownership
        pick = rows[[0, 1, len(rows) // 2, len(rows) - 1]]
        hid = orc.bf16_round(orc.matmul(x2[pick].float().cpu().numpy(), w1.float().cpu().numpy(), 4))
        full = orc.matmul(hid, w2.float().cpu().numpy(), 4)
        outs = []
        for blk in (mlp_nccl, mlp_copy, mlp_copy, mlp_copy_nccl):
            dw1 = torch.zeros((d, ff // WORLD), device=dev, dtype=torch.float32)
            dw2 = torch.zeros((ff // WORLD, d), device=dev, dtype=torch.float32)
            yb = blk.forward(x2)
            dxb = blk.backward(x2, dy_local, dw1, dw2)
            torch.cuda.synchronize()
            outs.append((yb.float(), dxb.float(), dw1, dw2))
        assert mlp_copy._px is not None
        got = outs[1][0][[0, 1, len(rows) // 2, len(rows) - 1]].cpu().numpy()
        assert np.linalg.norm(got - full) / np.linalg.norm(full) <= 1e-2         # against the oracle rows above
        for a, b in ((outs[0], outs[1]), (outs[1], outs[2]), (outs[1], outs[3])):
            for u, v2, what in zip(a, b, ("y", "dx", "dw_up", "dw_down")):
                rel = float((u - v2).norm() / u.norm())
                assert rel <= (1e-2 if a is outs[0] else 1e-6), (what, rel)
        assert gemm.device_status() == 0
        dist.barrier()
        torch.cuda.synchronize()
        gemm.close()
        dist.destroy_process_group()
    except Exception:
        failures.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise


def test_sharded_paths_on_two_gpus():
    import torch
    if torch.cuda.device_count() < WORLD:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, failures)) for r in range(WORLD)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    msgs = []
    while not failures.empty():
        msgs.append(failures.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            msgs.append("a rank did not finish in time")
    assert not msgs, "\n".join(msgs)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
