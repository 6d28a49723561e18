"""A mixture-of-experts block assembled from the oracle's functions only, forward and backward.

Follows ``MoeFfn::{forward, backward}`` (crates/nn/src/moe.rs:283-452) step for step, but
over the permuted row layout the GPU path uses (rows of expert ``e`` are
``offsets[e] .. offsets[e+1]``, a pair's row is ``dest_row[pair]``) instead of one
capacity-padded bin per expert.  ``round_to`` lets a caller round intermediates to bf16 at
the places the GPU path stores them, so that both sides see the same operands.
"""
import numpy as np

DROPPED = 0xFFFFFFFF


def _identity(x):
    return x


class MoeRef:
    """``w_router [D, E]``; gated experts: ``w_gate, w_up [E, D, FF]``, ``w_down [E, FF, D]``;
    ``w_gate=None`` selects the plain ``down(silu(up(x)))`` expert."""

    def __init__(self, orc, w_router, w_gate, w_up, w_down, top_k, capacity, aux_coefficient=0.0,
                 threads=1, round_to=None):
        self.o, self.wr, self.wg, self.wu, self.wd = orc, w_router, w_gate, w_up, w_down
        self.k, self.cap, self.aux, self.threads = top_k, capacity, aux_coefficient, threads
        self.rnd = round_to or _identity

    # ------------------------------------------------------------------ forward
    def forward(self, x, probs=None):
        o, K = self.o, self.k
        N, D = x.shape
        E = self.wu.shape[0]
        if probs is None:
            self.logits = o.matmul(x, self.wr, self.threads)
            probs = o.softmax_rows(self.logits)
        self.probs = probs
        r = o.moe_route(probs, K, self.cap)
        self.r = r
        rows = int(r["offsets"][E])
        xp = np.zeros((rows, D), dtype=np.float32)
        for pair in range(N * K):
            if r["dest_row"][pair] != DROPPED:
                xp[r["dest_row"][pair]] = x[pair // K]
        self.x, self.xp = x, xp
        FF = self.wu.shape[2]
        self.gate = np.zeros((rows, FF), dtype=np.float32)
        self.up = np.zeros((rows, FF), dtype=np.float32)
        self.act = np.zeros((rows, FF), dtype=np.float32)
        yp = np.zeros((rows, self.wd.shape[2]), dtype=np.float32)
        for e in range(E):
            a, b = int(r["offsets"][e]), int(r["offsets"][e + 1])
            if a == b:
                continue
            self.up[a:b] = o.matmul(xp[a:b], self.wu[e], self.threads)
            if self.wg is not None:
                self.gate[a:b] = o.matmul(xp[a:b], self.wg[e], self.threads)
                self.act[a:b] = o.swiglu(self.gate[a:b], self.up[a:b])
            else:
                self.act[a:b] = o.silu(self.up[a:b])
            self.act[a:b] = self.rnd(self.act[a:b])
            yp[a:b] = o.matmul(self.act[a:b], self.wd[e], self.threads)
        # what the backward of the activation reads is the stored (rounded) panel
        self.gate, self.up = self.rnd(self.gate), self.rnd(self.up)
        self.yp = self.rnd(yp)
        y = np.zeros((N, self.wd.shape[2]), dtype=np.float32)
        for pair in range(N * K):
            if r["dest_row"][pair] != DROPPED:
                y[pair // K] += r["gates"][pair] * self.yp[r["dest_row"][pair]]
        mean_p = (probs.astype(np.float64).sum(0)).astype(np.float32) / np.float32(N)
        frac = r["assignment_counts"].astype(np.float32) / np.float32(N * K)
        self.aux_loss = np.float32(E) * np.float32((frac.astype(np.float64) * mean_p.astype(np.float64)).sum())
        return y

    # ------------------------------------------------------------------ backward
    def backward(self, dy):
        """Returns a dict of gradients: ``dx`` (without the router's part), ``gate_grad``,
        ``dlogits``, ``d_gate``/``d_up``/``d_down`` per expert, and the permuted intermediates."""
        o, K, r = self.o, self.k, self.r
        N = self.x.shape[0]
        E = self.wu.shape[0]
        dyp, gate_grad = o.moe_combine_backward(dy, self.yp, r["dest_row"], r["gates"], K)
        dyp = self.rnd(dyp)
        d_down = np.zeros_like(self.wd)
        d_up = np.zeros_like(self.wu)
        d_gate = np.zeros_like(self.wu) if self.wg is not None else None
        dact = np.zeros_like(self.act)
        dgate_rows = np.zeros_like(self.act)
        dup_rows = np.zeros_like(self.act)
        dxp = np.zeros_like(self.xp)
        for e in range(E):
            a, b = int(r["offsets"][e]), int(r["offsets"][e + 1])
            if a == b:
                continue
            d_down[e] = o.matmul_tn(self.act[a:b], dyp[a:b], self.threads)
            dact[a:b] = self.rnd(o.matmul_nt(dyp[a:b], self.wd[e], self.threads))
            if self.wg is not None:
                dg, du = o.swiglu_backward(self.gate[a:b], self.up[a:b], dact[a:b])
                dgate_rows[a:b], dup_rows[a:b] = self.rnd(dg), self.rnd(du)
                d_gate[e] = o.matmul_tn(self.xp[a:b], dgate_rows[a:b], self.threads)
                d_up[e] = o.matmul_tn(self.xp[a:b], dup_rows[a:b], self.threads)
                dxp[a:b] = (o.matmul_nt(dgate_rows[a:b], self.wg[e], self.threads)
                            + o.matmul_nt(dup_rows[a:b], self.wu[e], self.threads))
            else:
                dup_rows[a:b] = self.rnd(o.silu_backward(self.up[a:b], dact[a:b]))
                d_up[e] = o.matmul_tn(self.xp[a:b], dup_rows[a:b], self.threads)
                dxp[a:b] = o.matmul_nt(dup_rows[a:b], self.wu[e], self.threads)
        dxp = self.rnd(dxp)
        dx = o.moe_scatter_backward(dxp, r["dest_row"], N, K)
        dlogits = o.moe_route_backward(self.probs, r["selected"], r["gates"], gate_grad,
                                       r["assignment_counts"], self.aux, K)
        return {"dx": dx, "gate_grad": gate_grad, "dlogits": dlogits, "d_gate": d_gate, "d_up": d_up,
                "d_down": d_down, "dyp": dyp, "dact": dact, "dgate_rows": dgate_rows, "dup_rows": dup_rows,
                "dxp": dxp}

    def backward_with_router(self, dy):
        """The whole ``MoeFfn::backward``: adds the router's ``Linear::backward`` (moe.rs:446-447)."""
        g = self.backward(dy)
        g["d_router"] = self.o.matmul_tn(self.x, g["dlogits"], self.threads)
        g["dx_total"] = g["dx"] + self.o.matmul_nt(g["dlogits"], self.wr, self.threads)
        return g
