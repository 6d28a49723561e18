"""Pins the oracle's restatement of ``MoeFfn::backward`` the way the reference pins the original:
central differences on the reference's own 4-token fixture, with its step and tolerances
(crates/nn/tests/moe.rs:6-8, 10-37, 63-160), over every path -- no drops, forced drops,
an expert that receives nothing, and the router's gate path with the auxiliary loss off."""
import numpy as np
import pytest

from _moe_ref import MoeRef

EPS, ATOL, RTOL = 1e-3, 8e-3, 5e-2          # crates/nn/tests/moe.rs:6-8
N, D, FF, E = 4, 2, 3, 3

ROUTER = np.array([[1.2, -0.8, 0.2], [0.1, 0.9, -1.0]], dtype=np.float32)                  # moe.rs (tests):11-14
MIXED = np.array([[1.0, 0.2], [0.8, 0.4], [-0.7, 1.0], [-1.0, 0.6]], dtype=np.float32)     # :20-27
UNDERFULL = np.array([[1.0, 0.2], [0.9, 0.3], [1.1, 0.1], [0.8, 0.25]], dtype=np.float32)  # :29-36


def _experts(oracle):
    """``ExpertFfn::initialized(20 + 3 * expert)`` (crates/nn/src/moe.rs:47-58)."""
    hs, fs = np.float32(1.0) / np.sqrt(np.float32(D)), np.float32(1.0) / np.sqrt(np.float32(FF))
    wg = np.stack([oracle.uniform(D * FF, 20 + 3 * e).reshape(D, FF) * hs for e in range(E)])
    wu = np.stack([oracle.uniform(D * FF, 21 + 3 * e).reshape(D, FF) * hs for e in range(E)])
    wd = np.stack([oracle.uniform(FF * D, 22 + 3 * e).reshape(FF, D) * fs for e in range(E)])
    return wg.astype(np.float32), wu.astype(np.float32), wd.astype(np.float32)


def _objective(oracle, params, x, upstream, top_k, capacity, aux):
    wr, wg, wu, wd = params
    m = MoeRef(oracle, wr, wg, wu, wd, top_k, capacity, aux)
    y = m.forward(x)
    return np.float32((y.astype(np.float64) * upstream).sum()) + np.float32(aux) * m.aux_loss


def _numeric(f, t):
    g = np.zeros_like(t)
    flat, gf = t.reshape(-1), g.reshape(-1)
    for i in range(flat.size):
        orig = flat[i]
        flat[i] = orig + np.float32(EPS)
        plus = f()
        flat[i] = orig - np.float32(EPS)
        minus = f()
        flat[i] = orig
        gf[i] = (plus - minus) / np.float32(2 * EPS)
    return g


def _close(analytic, numeric, what):
    tol = ATOL + RTOL * np.abs(analytic)
    bad = np.abs(analytic - numeric) > tol
    assert not bad.any(), f"{what}: analytic {analytic[bad]} vs numeric {numeric[bad]}"


@pytest.mark.parametrize("top_k,capacity,x,aux,drop,underfull", [
    (2, 4, MIXED, 0.17, False, False),          # moe_gradchecks_every_path_without_drops
    (2, 1, MIXED, 0.17, True, False),           # ..._with_forced_drops
    (1, 4, UNDERFULL, 0.17, False, True),       # ..._with_underfull_experts
    (2, 4, MIXED, 0.0, False, False),           # router_gate_path_..._auxiliary_loss_disabled
], ids=["no_drops", "forced_drops", "underfull", "aux_off"])
def test_moe_backward_matches_central_differences(oracle, top_k, capacity, x, aux, drop, underfull):
    wg, wu, wd = _experts(oracle)
    wr = ROUTER.copy()
    x = x.copy()
    upstream = oracle.uniform(N * D, 92 if aux == 0.0 else 91).reshape(N, D).astype(np.float32)
    m = MoeRef(oracle, wr, wg, wu, wd, top_k, capacity, aux)
    m.forward(x)
    assert bool((m.r["slots"] == 0xFFFFFFFF).any()) == drop
    assert bool((m.r["accepted_counts"] == 0).any()) == underfull
    # the top-k margin must stay clear of the probe step (moe.rs (tests):46-61)
    srt = np.sort(m.logits, axis=1)[:, ::-1]
    assert np.all(srt[:, top_k - 1] - srt[:, top_k] > 20 * EPS)
    g = m.backward_with_router(upstream)
    params = [wr, wg, wu, wd]
    f = lambda: _objective(oracle, params, x, upstream, top_k, capacity, aux)
    _close(g["dx_total"], _numeric(f, x), "dx")
    _close(g["d_router"], _numeric(f, wr), "router weight")
    _close(g["d_gate"], _numeric(f, wg), "gate weights")
    _close(g["d_up"], _numeric(f, wu), "up weights")
    _close(g["d_down"], _numeric(f, wd), "down weights")


def test_silu_expert_backward_matches_central_differences(oracle):
    """The plain ``down(silu(up(x)))`` expert of the 64-expert configuration, same fixture."""
    _, wu, wd = _experts(oracle)
    wr, x = ROUTER.copy(), MIXED.copy()
    upstream = oracle.uniform(N * D, 91).reshape(N, D).astype(np.float32)
    m = MoeRef(oracle, wr, None, wu, wd, 2, 4, 0.17)
    m.forward(x)
    g = m.backward_with_router(upstream)
    params = [wr, None, wu, wd]
    f = lambda: _objective(oracle, params, x, upstream, 2, 4, 0.17)
    _close(g["dx_total"], _numeric(f, x), "dx")
    _close(g["d_router"], _numeric(f, wr), "router weight")
    _close(g["d_up"], _numeric(f, wu), "up weights")
    _close(g["d_down"], _numeric(f, wd), "down weights")


def test_auxiliary_loss_is_one_at_uniform_routing(oracle):
    """crates/nn/tests/moe.rs `auxiliary_loss_is_one_at_uniform_routing`: a zero router over two
    experts with top-2 routes everything everywhere."""
    hs, fs = np.float32(1.0) / np.sqrt(np.float32(D)), np.float32(1.0) / np.sqrt(np.float32(FF))
    wg = np.stack([oracle.uniform(D * FF, 70 + 3 * e).reshape(D, FF) * hs for e in range(2)]).astype(np.float32)
    wu = np.stack([oracle.uniform(D * FF, 71 + 3 * e).reshape(D, FF) * hs for e in range(2)]).astype(np.float32)
    wd = np.stack([oracle.uniform(FF * D, 72 + 3 * e).reshape(FF, D) * fs for e in range(2)]).astype(np.float32)
    m = MoeRef(oracle, np.zeros((D, 2), dtype=np.float32), wg, wu, wd, 2, 4, 0.1)
    m.forward(MIXED.copy())
    assert abs(float(m.aux_loss) - 1.0) < 1e-6
