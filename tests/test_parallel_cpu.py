"""The sharded paths' exchange logic on CPU: world_size 2, ``gloo`` backend.

The compute kernels need a B200, so a CPU stand-in built on the oracle takes
their place here (``CpuOps``); what is under test is everything around them:
shard boundaries, the statistics merge, the counts exchange and split sizes of
the all-to-all, the (source rank, expert) grouping of received rows, the
reduce-scatter row ownership.  Each case compares against the single-process
oracle result.
"""
import os
import socket
import sys
import traceback

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORLD = 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Routing:
    pass


class CpuOps:
    """CPU stand-in for ``DeviceOps``: same methods, oracle / torch-CPU arithmetic."""

    def __init__(self, orc):
        self.orc = orc

    # ---- head
    def head_forward_shard(self, hidden, w_shard, local_targets, classes_local, w_layout):
        logits = hidden.float().numpy() @ w_shard.float().numpy()
        z = logits[:, :classes_local].astype(np.float64)
        mx = z.max(1)
        s = np.exp(z - mx[:, None]).sum(1)
        lt = local_targets.numpy()
        own = (lt >= 0) & (lt < classes_local)
        tl = np.where(own, logits[np.arange(len(lt)), np.clip(lt, 0, logits.shape[1] - 1)], 0.0)
        f = lambda a: torch.from_numpy(np.asarray(a, np.float32))
        return f(mx), f(s), f(tl)

    def head_backward_shard(self, hidden, w_shard, local_targets, lse, classes_local, w_layout, dy, d_weight, acc):
        h, w = hidden.float().numpy(), w_shard.float().numpy()
        logits = h @ w
        m = h.shape[0]
        p = np.exp(logits - lse.numpy()[:, None]) * (dy / m)
        p[:, classes_local:] = 0
        lt = local_targets.numpy()
        own = (lt >= 0) & (lt < classes_local)
        p[np.arange(m)[own], lt[own]] -= dy / m
        return torch.from_numpy(p), torch.from_numpy(p @ w.T), torch.from_numpy(h.T @ p)

    # ---- MoE
    def route(self, scores, top_k, scores_are_logits):
        probs = scores.numpy()
        want = self.orc.moe_route(probs, top_k, probs.shape[0] * top_k)
        r = _Routing()
        r.tokens, r.experts, r.top_k = probs.shape[0], probs.shape[1], top_k
        as_i32 = lambda a: torch.from_numpy(a.view(np.int32).copy())
        r.accepted_counts = as_i32(want["accepted_counts"])
        r.dest_row = torch.from_numpy(want["dest_row"].astype(np.int64))
        r.gate_weights = torch.from_numpy(want["gates"])
        r.offsets = as_i32(want["offsets"])
        return r

    def scatter(self, x, r):
        out = torch.zeros((r.tokens * r.top_k, x.shape[1]), dtype=x.dtype)
        out[r.dest_row] = x.repeat_interleave(r.top_k, 0)
        return out

    def combine(self, yp, r, residual, out_dtype):
        g = r.gate_weights.view(r.tokens, r.top_k, 1)
        rows = yp.float()[r.dest_row].view(r.tokens, r.top_k, -1)
        out = (g * rows).sum(1)
        return (out + residual.float()) if residual is not None else out

    def grouped_indexed(self, a, b, offsets, index, silu):
        out = torch.zeros((a.shape[0], b.shape[2]), dtype=torch.float32)
        off = offsets.tolist()
        for g, e in enumerate(index.tolist()):
            lo, hi = off[g], off[g + 1]
            if hi > lo:
                y = a[lo:hi].float() @ b[e].float()
                out[lo:hi] = y * torch.sigmoid(y) if silu else y
        return out

    # ---- dense
    def linear(self, x, w, out_dtype=None):
        return x.float() @ w.float()

    def linear_input_grad(self, dy, w, out_dtype=None):
        return dy.float() @ w.float().t()

    def linear_input_grad_into(self, dy, w, dx):
        dx.copy_(dy.float() @ w.float().t())

    def linear_weight_grad(self, x, dy, dw):
        dw += x.float().t() @ dy.float()


def _worker(rank, port, case, failures):
    try:
        sys.path.insert(0, ROOT)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=WORLD)
        import __graft_entry__ as entry
        from oracle import oracle as orc
        pkg = entry.load_package()
        CASES[case](rank, pkg.parallel, CpuOps(orc), orc)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        failures.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise


def _run(case):
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, case, failures)) for r in range(WORLD)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    msgs = []
    while not failures.empty():
        msgs.append(failures.get())
    assert not msgs, "\n".join(msgs)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]


# --------------------------------------------------------------------------- cases

def case_head(rank, par, ops, orc):
    m, k, v, classes = 96, 32, 1024, 1000
    h = orc.bf16_round(orc.normal(m * k, 1)).reshape(m, k)
    w = orc.bf16_round(orc.normal(k * v, 2, 0.0, 0.3)).reshape(k, v)
    t = np.clip(((orc.uniform(m, 3) * 0.5 + 0.5) * classes).astype(np.int32), 0, classes - 1)
    logits = orc.matmul(h, w)
    loss, probs, row_loss = orc.xent_forward(logits, t, classes)
    dl = orc.xent_backward(probs, t, classes)
    head = par.VocabParallelHead(ops, classes, v, reserve_sms=16)   # no SMs to reserve on the CPU: a no-op
    assert (head.c0, head.c1) == ((0, 512), (512, 1024))[rank]
    ws = head.shard_weight(torch.from_numpy(w))
    g_loss, lse, g_row = head.forward(torch.from_numpy(h), ws, torch.from_numpy(t))
    assert abs(float(g_loss) - float(loss)) < 1e-5
    assert np.allclose(g_row.numpy(), row_loss, atol=1e-4)
    _, dh, dw = head.backward(torch.from_numpy(h), ws, torch.from_numpy(t), lse)
    assert np.allclose(dh.numpy(), orc.matmul_nt(dl, w), atol=1e-5)              # summed over shards
    assert np.allclose(dw.numpy(), orc.matmul_tn(h, dl)[:, head.c0:head.c1], atol=1e-5)


def case_moe(rank, par, ops, orc):
    n_local, d, ff, experts, top_k = 40, 16, 24, 8, 2
    local = experts // WORLD
    x_all = orc.bf16_round(orc.normal(WORLD * n_local * d, 11)).reshape(WORLD, n_local, d)
    up = orc.bf16_round(orc.normal(experts * d * ff, 12, 0.0, 0.2)).reshape(experts, d, ff)
    dn = orc.bf16_round(orc.normal(experts * ff * d, 13, 0.0, 0.2)).reshape(experts, ff, d)
    probs_all = orc.softmax_rows(orc.normal(WORLD * n_local * experts, 14).reshape(-1, experts))
    probs_all = probs_all.reshape(WORLD, n_local, experts)
    moe = par.ExpertParallelMoe(ops, experts, top_k,
                                torch.from_numpy(up[rank * local:(rank + 1) * local]),
                                torch.from_numpy(dn[rank * local:(rank + 1) * local]))
    out = moe.forward(torch.from_numpy(x_all[rank]), torch.from_numpy(probs_all[rank]))
    # single-process oracle for this rank's tokens
    want = orc.moe_route(probs_all[rank], top_k, n_local * top_k)
    sel = want["selected"].reshape(n_local, top_k)
    gates = want["gates"].reshape(n_local, top_k)
    ref = np.zeros((n_local, d), np.float32)
    for tkn in range(n_local):
        for rk in range(top_k):
            e = sel[tkn, rk]
            hh = orc.silu(orc.matmul(x_all[rank][tkn:tkn + 1], up[e]))
            ref[tkn] += gates[tkn, rk] * orc.matmul(hh, dn[e])[0]
    assert np.allclose(out.numpy(), ref, atol=1e-4), np.abs(out.numpy() - ref).max()
    # rows received = rows every rank routed to this rank's experts
    routed_here = sum(int(np.isin(orc.moe_route(probs_all[s], top_k, n_local * top_k)["selected"],
                                  np.arange(rank * local, (rank + 1) * local)).sum()) for s in range(WORLD))
    assert moe.last["rows_received"] == routed_here
    assert moe.last["rows_sent"] == n_local * top_k


def case_tp_mlp(rank, par, ops, orc):
    for chunks in (2, [1, 3, 3, 1]):          # equal pieces; short pieces at both ends
        _tp_mlp_case(orc, par, ops, rank, chunks)


def _tp_mlp_case(orc, par, ops, rank, chunks):
    m, d, ff = 64, 16, 48
    x = orc.normal(m * d, 21).reshape(m, d)
    w1 = orc.normal(d * ff, 22, 0.0, 0.2).reshape(d, ff)
    w2 = orc.normal(ff * d, 23, 0.0, 0.2).reshape(ff, d)
    cols = slice(rank * ff // WORLD, (rank + 1) * ff // WORLD)
    mlp = par.TensorParallelMlp(ops, torch.from_numpy(w1[:, cols].copy()), torch.from_numpy(w2[cols].copy()),
                                chunks=chunks, partial_dtype=torch.float32, reserve_sms=8)
    y = mlp.forward(torch.from_numpy(x))
    full = (x @ w1) @ w2
    rows = mlp.owned_rows(m).numpy()
    assert y.shape == (m // WORLD, d)
    assert np.allclose(y.numpy(), full[rows], atol=1e-4)
    # every row is owned by exactly one rank
    owned = [torch.empty(m // WORLD, dtype=torch.int64) for _ in range(WORLD)]
    dist.all_gather(owned, mlp.owned_rows(m))
    assert sorted(torch.cat(owned).tolist()) == list(range(m))
    # backward: dy = ones on this rank's rows
    dy_full = orc.normal(m * d, 24).reshape(m, d)
    dw1 = torch.zeros(d, ff // WORLD)
    dw2 = torch.zeros(ff // WORLD, d)
    dx = mlp.backward(torch.from_numpy(x), torch.from_numpy(dy_full[rows].copy()), dw1, dw2)
    assert np.allclose(dx.numpy(), ((dy_full @ w2.T) @ w1.T)[rows], atol=1e-3)     # this rank's rows
    assert np.allclose(dw2.numpy(), ((x @ w1).T @ dy_full)[cols], atol=1e-3)
    assert np.allclose(dw1.numpy(), (x.T @ (dy_full @ w2.T))[:, cols], atol=1e-3)


CASES = {"head": case_head, "moe": case_moe, "tp_mlp": case_tp_mlp}


# --------------------------------------------------------------------------- tests

def test_vocab_shards_cover_the_vocabulary_in_whole_tiles():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    par = entry.load_package().parallel
    shards = par.vocab_shards(50432, 8)
    assert [(c1 - c0) // 256 for c0, c1 in shards] == [25, 25, 25, 25, 25, 24, 24, 24]
    assert shards[0][0] == 0 and shards[-1][1] == 50432
    assert all(a[1] == b[0] for a, b in zip(shards, shards[1:]))
    assert par.vocab_shards(50432, 1) == [(0, 50432)]
    assert par.vocab_shards(1000, 2) == [(0, 512), (512, 1000)]


def test_moe_token_slices_cover_every_token_once():
    """``ExpertParallelMoe._slices``: equal slices, weighted slices (the default tapers towards the
    end), and the fall-back to one slice when the weights do not divide the tokens or a slice
    would be shorter than 256 tokens."""
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    par = entry.load_package().parallel

    def slices(pieces, n):
        ep = par.ExpertParallelMoe.__new__(par.ExpertParallelMoe)
        ep.pieces = pieces
        return ep._slices(n)

    assert slices(4, 32768) == [(0, 8192), (8192, 8192), (16384, 8192), (24576, 8192)]
    assert slices([6, 5, 3, 2], 32768) == [(0, 12288), (12288, 10240), (22528, 6144), (28672, 4096)]
    assert slices(3, 32768) == [(0, 32768)]                  # 32768 is no multiple of 3
    assert slices([1, 2, 2, 1], 32768) == [(0, 32768)]       # sixths do not divide it either
    assert slices([6, 5, 3, 2], 1024) == [(0, 1024)]         # the last slice would hold 128 tokens
    assert slices(2, 300) == [(0, 300)]                      # slices shorter than 256 tokens
    for pieces, n in ((8, 32768), ([4, 4, 4, 2, 1, 1], 32768), ([6, 5, 3, 2], 16384)):
        got = slices(pieces, n)
        assert got[0][0] == 0 and sum(rows for _, rows in got) == n
        assert all(a[0] + a[1] == b[0] for a, b in zip(got, got[1:]))


def test_exchange_plan_offsets_are_consistent_between_ranks():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    par = entry.load_package().parallel
    world, experts = 4, 8
    rng = np.random.default_rng(3)
    counts = torch.from_numpy(rng.integers(0, 50, size=(world, experts)))
    plans = [par.exchange_plan(counts, r, world) for r in range(world)]
    per_dest = plans[0][4]
    for i in range(world):
        send_off, send_rows, inbox_off, back_off, _ = plans[i]
        assert send_rows == per_dest[i].tolist()
        assert send_off == [int(per_dest[i, :j].sum()) for j in range(world)]
        for j in range(world):
            # my block in j's inbox starts after the blocks of lower-ranked sources ...
            assert inbox_off[j] == int(per_dest[:i, j].sum())
            # ... which is exactly where j expects source i's rows
            assert plans[j][3][i] == inbox_off[j]
    # inbox blocks tile [0, total) without gaps
    for j in range(world):
        ends = [plans[i][2][j] + plans[i][1][j] for i in range(world)]
        assert ends[-1] == int(per_dest[:, j].sum())


@pytest.mark.parametrize("case", sorted(CASES))
def test_sharded_path_over_two_gloo_ranks(case):
    _run(case)
