"""The expert-parallel exchange kernels (plan / push / pull-combine) on ONE GPU.

`world` ranks are emulated by `world` sets of buffers on the same device and the phases
are launched rank after rank (none of these kernels waits on another, so the order of
launches is the only synchronisation needed).  Every rank's output must equal what the
single-GPU grouped path computes for that rank's tokens with all experts present; the
plan's integers are checked against their definition.
"""
import ctypes as C

import numpy as np
import pytest

from _util import bf16_operand

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,experts,top_k,tokens", [(4, 8, 2, 384), (2, 6, 3, 500), (8, 64, 8, 256)])
def test_emulated_ranks_match_single_gpu_moe(pkg, oracle, world, experts, top_k, tokens):
    import torch
    gemm = pkg.Tcgen05Gemm()
    ops = pkg.parallel.DeviceOps(gemm)
    d, ff, local = 128, 192, experts // world
    w_up, _ = bf16_operand(oracle, (experts, d, ff), 301, std=0.1)
    w_dn, _ = bf16_operand(oracle, (experts, ff, d), 302, std=0.1)
    xs = [bf16_operand(oracle, (tokens, d), 310 + r)[0] for r in range(world)]
    logits = [torch.from_numpy(oracle.normal(tokens * experts, 330 + r).reshape(tokens, experts)).cuda()
              for r in range(world)]
    want = [pkg.GroupedExpertFfn(gemm, w_up, w_dn).forward(xs[r], logits[r], top_k, scores_are_logits=True,
                                                           residual=xs[r])[0] for r in range(world)]

    routed = [ops.route(logits[r], top_k, True) for r in range(world)]
    counts = torch.stack([t.accepted_counts.to(torch.int32) for t in routed]).contiguous()      # [world, experts]
    plans = [ops.ep_plan(counts, world, r, experts) for r in range(world)]
    c = counts.cpu().numpy().astype(np.int64)
    for r, (dst_base, offsets, index) in enumerate(plans):
        # rows that rank j receives, laid out by (source rank, local expert)
        recv = c[:, r * local:(r + 1) * local]                               # [source, local expert]
        assert np.array_equal(offsets.cpu().numpy(), np.concatenate([[0], np.cumsum(recv.reshape(-1))]))
        assert np.array_equal(index.cpu().numpy(), np.tile(np.arange(local), world))
        base = dst_base.cpu().numpy()
        for e in range(experts):
            owner, le = divmod(e, local)
            own = c[:, owner * local:(owner + 1) * local]
            assert base[e] == own[:r].sum() + own[r, :le].sum()

    cap = tokens * top_k * world
    inbox = [torch.zeros((cap, d), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    result = [torch.zeros((cap, d), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    hidden = torch.empty((cap, ff), dtype=torch.bfloat16, device="cuda")
    ptr_in = (C.c_void_p * world)(*[t.data_ptr() for t in inbox])
    ptr_res = (C.c_void_p * world)(*[t.data_ptr() for t in result])
    for r in range(world):                                                   # phase 1: every rank pushes
        ops.ep_push(xs[r], routed[r], plans[r][0], ptr_in, cap, world, experts)
    for j in range(world):                                                   # phase 2: every rank multiplies
        _, offsets, index = plans[j]
        ops.grouped_indexed_into(inbox[j], w_up[j * local:(j + 1) * local], offsets, index, True, hidden)
        ops.grouped_indexed_into(hidden, w_dn[j * local:(j + 1) * local], offsets, index, False, result[j])
    for r in range(world):                                                   # phase 3: every rank pulls
        out = torch.empty((tokens, d), dtype=torch.float32, device="cuda")
        ops.ep_pull_combine(ptr_res, routed[r], plans[r][0], xs[r], cap, world, experts, d, out)
        assert torch.allclose(out, want[r], atol=1e-5, rtol=1e-5), float((out - want[r]).abs().max())
        # the few-block forms (stores from 3 or 16 blocks; rows fetched by bulk copies into a
        # shared-memory ring): the same sums in the same order, so the same bits, fp32 and bf16
        for ctas in (3, 16):
            gemm.set_exchange_ctas(ctas, bulk=True)
            for dtype in (torch.float32, torch.bfloat16):
                ref_out = torch.empty((tokens, d), dtype=dtype, device="cuda")
                gemm.set_exchange_ctas(0)
                ops.ep_pull_combine(ptr_res, routed[r], plans[r][0], xs[r], cap, world, experts, d, ref_out)
                gemm.set_exchange_ctas(ctas, bulk=True)
                few = torch.full((tokens, d), float("nan"), dtype=dtype, device="cuda")
                ops.ep_pull_combine(ptr_res, routed[r], plans[r][0], xs[r], cap, world, experts, d, few)
                assert torch.equal(few, ref_out), (ctas, dtype)
            few = torch.full((tokens, d), float("nan"), dtype=torch.float32, device="cuda")
            ops.ep_pull_combine(ptr_res, routed[r], plans[r][0], None, cap, world, experts, d, few)   # no residual
            gemm.set_exchange_ctas(0)
            ref_out = torch.empty((tokens, d), dtype=torch.float32, device="cuda")
            ops.ep_pull_combine(ptr_res, routed[r], plans[r][0], None, cap, world, experts, d, ref_out)
            assert torch.equal(few, ref_out), ctas
        gemm.set_exchange_ctas(0)
    assert gemm.device_status() == 0
    # pushes from a few blocks land the same rows
    gemm.set_exchange_ctas(5, bulk=True)
    inbox2 = [torch.zeros((cap, d), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ptr_in2 = (C.c_void_p * world)(*[t.data_ptr() for t in inbox2])
    for r in range(world):
        ops.ep_push(xs[r], routed[r], plans[r][0], ptr_in2, cap, world, experts)
    gemm.set_exchange_ctas(0)
    for a, b in zip(inbox, inbox2):
        assert torch.equal(a, b)
    # a result buffer that is too small for the bulk form too: rows beyond it are left out and reported
    gemm.set_exchange_ctas(4, bulk=True)
    few = torch.empty((tokens, d), dtype=torch.float32, device="cuda")
    ops.ep_pull_combine(ptr_res, routed[0], plans[0][0], xs[0], 1, world, experts, d, few)
    gemm.set_exchange_ctas(0)
    with pytest.raises(pkg.B200GemmError):
        gemm.device_status()
    assert gemm.device_status() == 0

    # The return leg fused into the expert GEMM: every owner's down projection stores its rows
    # straight into the buffer of the rank they came from; each rank then combines its own tokens
    # from its own buffer with the single-GPU combine.  Same result, to the last bit.
    pairs = tokens * top_k
    returned = [torch.full((pairs + 5, d), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ptr_back = (C.c_void_p * world)(*[t.data_ptr() for t in returned])
    for j in range(world):
        _, offsets, index = plans[j]
        dst_rank, dst_row = ops.ep_return_plan(counts, world, j, experts)
        assert np.array_equal(dst_rank.cpu().numpy(), np.repeat(np.arange(world), local))
        want_row = [c[s, :j * local + e].sum() for s in range(world) for e in range(local)]
        assert np.array_equal(dst_row.cpu().numpy(), np.array(want_row))
        ops.grouped_indexed_into(inbox[j], w_up[j * local:(j + 1) * local], offsets, index, True, hidden)
        ops.grouped_indexed_peer(hidden, w_dn[j * local:(j + 1) * local], offsets, index, ptr_back, world, d,
                                 pairs, dst_rank, dst_row)
    for r in range(world):
        assert torch.isnan(returned[r][pairs:]).all()                          # nothing written behind the routed rows
        out = ops.combine(returned[r][:pairs], routed[r], xs[r], torch.float32)
        assert torch.equal(out, pkg.moe.combine(gemm, returned[r][:pairs], routed[r], xs[r]))
        assert torch.allclose(out, want[r], atol=1e-5, rtol=1e-5), float((out - want[r]).abs().max())
    assert gemm.device_status() == 0
    # a return buffer that is too small: the rows beyond it are not written, the status word says so
    j = world - 1
    _, offsets, index = plans[j]
    dst_rank, dst_row = ops.ep_return_plan(counts, world, j, experts)
    ops.grouped_indexed_peer(hidden, w_dn[j * local:(j + 1) * local], offsets, index, ptr_back, world, d,
                             max(1, int(c[0, :j * local].sum())), dst_rank, dst_row)
    with pytest.raises(pkg.B200GemmError):
        gemm.device_status()
    assert gemm.device_status() == 0

    # an inbox that is too small: rows beyond it are dropped and the status word says so
    # (the last rank's rows come last in every inbox, so some of them must fall beyond the limit)
    small = max(1, int(c[:, :local].sum()) // 2)
    last = world - 1
    for ctas in (0, 4, 7):                                # the store-driven form, the bulk-copy form, few blocks
        gemm.set_exchange_ctas(ctas, bulk=ctas == 4)
        ops.ep_push(xs[last], routed[last], plans[last][0], ptr_in, small, world, experts)
        with pytest.raises(pkg.B200GemmError):
            gemm.device_status()
        assert gemm.device_status() == 0
    gemm.close()
