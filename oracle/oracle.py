"""ctypes front end of the CPU oracle (``oracle/oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the test suite, the smoke check and the
CPU-baseline leg of the benchmark.  The product package never imports it.

Every function takes and returns numpy arrays; the arithmetic happens in the C
restatement of the reference's CPU crates (see the header of ``oracle.c`` for
the file:line each function follows).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
DROPPED = 0xFFFFFFFF


def build(force: bool = False) -> str:
    """Compile ``oracle.c`` into ``liboracle.so`` (gcc, no FMA contraction)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        cc = "gcc"
        for cand in ("/usr/bin/gcc", "/bin/gcc"):
            if os.path.exists(cand):
                cc = cand
                break
        subprocess.check_call(
            [cc, "-O2", "-ffp-contract=off", "-fno-fast-math", "-pthread", "-fPIC",
             "-fvisibility=hidden", "-shared", "-o", _LIB_PATH, src, "-lm"])
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


def _declare(L: C.CDLL) -> None:
    u64, sz, f32p, i32 = C.c_uint64, C.c_size_t, C.c_void_p, C.c_int
    L.orc_splitmix64.restype = u64
    L.orc_splitmix64.argtypes = [u64]
    L.orc_rng_next_u64.restype = u64
    L.orc_rng_next_u64.argtypes = [C.POINTER(u64)]
    L.orc_rng_next_uniform.restype = C.c_float
    L.orc_rng_next_uniform.argtypes = [C.POINTER(u64)]
    L.orc_uniform_fill.argtypes = [f32p, sz, u64]
    L.orc_normal_fill.argtypes = [f32p, sz, u64, C.c_float, C.c_float]
    L.orc_bf16_from_f32.restype = C.c_uint16
    L.orc_bf16_from_f32.argtypes = [C.c_float]
    L.orc_bf16_to_f32.restype = C.c_float
    L.orc_bf16_to_f32.argtypes = [C.c_uint16]
    L.orc_bf16_stochastic.restype = C.c_uint16
    L.orc_bf16_stochastic.argtypes = [C.c_float, C.c_uint32]
    L.orc_quantize_bf16.argtypes = [f32p, sz, C.c_void_p, C.c_void_p]
    for name in ("orc_matmul", "orc_matmul_tn", "orc_matmul_nt"):
        getattr(L, name).argtypes = [f32p, f32p, f32p, sz, sz, sz, i32]
        getattr(L, name).restype = None
    L.orc_transpose.argtypes = [f32p, f32p, sz, sz]
    L.orc_matmul_rows.argtypes = [f32p, f32p, f32p, C.c_void_p, sz, sz, sz, i32]
    L.orc_softmax_rows.argtypes = [f32p, f32p, sz, sz]
    L.orc_xent_forward.restype = C.c_float
    L.orc_xent_forward.argtypes = [f32p, C.c_void_p, sz, sz, sz, C.c_void_p, C.c_void_p]
    L.orc_xent_backward.argtypes = [f32p, C.c_void_p, sz, sz, sz, C.c_float, f32p]
    L.orc_moe_route.argtypes = [f32p, sz, sz, sz, sz] + [C.c_void_p] * 5
    L.orc_moe_offsets.argtypes = [C.c_void_p, sz, C.c_void_p]
    L.orc_moe_permutation.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, sz, C.c_void_p]
    L.orc_silu.argtypes = [f32p, f32p, sz]
    L.orc_swiglu.argtypes = [f32p, f32p, f32p, sz]
    L.orc_swiglu_backward.argtypes = [f32p] * 5 + [sz]
    L.orc_silu_backward.argtypes = [f32p] * 3 + [sz]
    L.orc_moe_combine_backward.argtypes = [f32p, f32p, C.c_void_p, f32p, sz, sz, sz, sz, f32p, f32p]
    L.orc_moe_scatter_backward.argtypes = [f32p, C.c_void_p, sz, sz, sz, f32p]
    L.orc_moe_route_backward.argtypes = [f32p, C.c_void_p, f32p, f32p, C.c_void_p, C.c_float, sz, sz, sz, f32p]


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# --------------------------------------------------------------------------- RNG / bf16

def splitmix64(state: int) -> int:
    return int(lib().orc_splitmix64(C.c_uint64(state & (2**64 - 1))))


def uniform(n: int, seed: int) -> np.ndarray:
    """``uniform_vec(n, seed)``: n draws in [-1, 1) from SplitMix64."""
    out = np.empty(n, dtype=np.float32)
    lib().orc_uniform_fill(_p(out), n, C.c_uint64(seed))
    return out


def normal(n: int, seed: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().orc_normal_fill(_p(out), n, C.c_uint64(seed), mean, std)
    return out


def bf16_bits(x) -> np.ndarray:
    """f32 -> bf16 words (uint16), round to nearest even."""
    x = _f32(x)
    bits = np.empty(x.shape, dtype=np.uint16)
    lib().orc_quantize_bf16(_p(x), x.size, _p(bits), None)
    return bits


def bf16_round(x) -> np.ndarray:
    """f32 -> bf16 -> f32: the values a bf16 operand actually holds."""
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.float32)
    lib().orc_quantize_bf16(_p(x), x.size, None, _p(out))
    return out


def bf16_to_f32(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    return (bits.astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------- matmul family

def matmul(a, b, threads: int = 1) -> np.ndarray:
    """``C[M,N] = A[M,K] . B[K,N]``."""
    a, b = _f32(a), _f32(b)
    (M, K), (K2, N) = a.shape, b.shape
    assert K == K2
    c = np.empty((M, N), dtype=np.float32)
    lib().orc_matmul(_p(a), _p(b), _p(c), M, K, N, threads)
    return c


def matmul_tn(a, b, threads: int = 1) -> np.ndarray:
    """``C[K,N] = A[M,K]^T . B[M,N]``."""
    a, b = _f32(a), _f32(b)
    (M, K), (M2, N) = a.shape, b.shape
    assert M == M2
    c = np.empty((K, N), dtype=np.float32)
    lib().orc_matmul_tn(_p(a), _p(b), _p(c), M, K, N, threads)
    return c


def matmul_nt(a, b, threads: int = 1) -> np.ndarray:
    """``C[M,N] = A[M,K] . B[N,K]^T``."""
    a, b = _f32(a), _f32(b)
    (M, K), (N, K2) = a.shape, b.shape
    assert K == K2
    c = np.empty((M, N), dtype=np.float32)
    lib().orc_matmul_nt(_p(a), _p(b), _p(c), M, K, N, threads)
    return c


def transpose(a) -> np.ndarray:
    a = _f32(a)
    M, K = a.shape
    out = np.empty((K, M), dtype=np.float32)
    lib().orc_transpose(_p(a), _p(out), M, K)
    return out


def matmul_rows(a, b, rows, threads: int = 1) -> np.ndarray:
    """Rows ``rows`` of ``matmul(a, b)``, full K per element."""
    a, b = _f32(a), _f32(b)
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    K, N = b.shape
    c = np.empty((rows.size, N), dtype=np.float32)
    lib().orc_matmul_rows(_p(a), _p(b), _p(c), _p(rows), rows.size, K, N, threads)
    return c


# --------------------------------------------------------------------------- softmax / CE

def softmax_rows(a) -> np.ndarray:
    a = _f32(a)
    out = np.empty_like(a)
    lib().orc_softmax_rows(_p(a), _p(out), a.shape[0], a.shape[1])
    return out


def xent_forward(logits, targets, classes: int | None = None):
    """Mean softmax cross entropy over the first ``classes`` columns.

    Returns ``(mean_loss_f32, probs[N, ld], row_loss_f64[N])``.
    """
    logits = _f32(logits)
    n, ld = logits.shape
    classes = ld if classes is None else classes
    targets = np.ascontiguousarray(targets, dtype=np.int32)
    probs = np.zeros_like(logits)
    row_loss = np.empty(n, dtype=np.float64)
    loss = lib().orc_xent_forward(_p(logits), _p(targets), n, classes, ld, _p(probs), _p(row_loss))
    return np.float32(loss), probs, row_loss


def xent_backward(probs, targets, classes: int | None = None, dy: float = 1.0) -> np.ndarray:
    probs = _f32(probs)
    n, ld = probs.shape
    classes = ld if classes is None else classes
    targets = np.ascontiguousarray(targets, dtype=np.int32)
    d = np.empty_like(probs)
    lib().orc_xent_backward(_p(probs), _p(targets), n, classes, ld, dy, _p(d))
    return d


# --------------------------------------------------------------------------- MoE routing

def moe_route(probs, top_k: int, capacity: int):
    """``MoeFfn::route``: returns a dict of selected/gates/slots/counts arrays."""
    probs = _f32(probs)
    N, E = probs.shape
    sel = np.empty(N * top_k, dtype=np.uint32)
    gates = np.empty(N * top_k, dtype=np.float32)
    slots = np.empty(N * top_k, dtype=np.uint32)
    assigned = np.empty(E, dtype=np.uint32)
    accepted = np.empty(E, dtype=np.uint32)
    lib().orc_moe_route(_p(probs), N, E, top_k, capacity, _p(sel), _p(gates), _p(slots),
                        _p(assigned), _p(accepted))
    offsets = np.empty(E + 1, dtype=np.uint32)
    lib().orc_moe_offsets(_p(accepted), E, _p(offsets))
    dest = np.empty(N * top_k, dtype=np.uint32)
    lib().orc_moe_permutation(_p(sel), _p(slots), _p(offsets), N * top_k, _p(dest))
    return {"selected": sel, "gates": gates, "slots": slots, "assignment_counts": assigned,
            "accepted_counts": accepted, "offsets": offsets, "dest_row": dest}


def silu(g) -> np.ndarray:
    g = _f32(g)
    out = np.empty_like(g)
    lib().orc_silu(_p(g), _p(out), g.size)
    return out


def swiglu(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().orc_swiglu(_p(gate), _p(up), _p(out), gate.size)
    return out


# --------------------------------------------------------------------------- MoE backward

def swiglu_backward(gate, up, dy):
    """``SwiGlu::backward``: returns ``(dgate, dup)``."""
    gate, up, dy = _f32(gate), _f32(up), _f32(dy)
    dg, du = np.empty_like(gate), np.empty_like(gate)
    lib().orc_swiglu_backward(_p(gate), _p(up), _p(dy), _p(dg), _p(du), gate.size)
    return dg, du


def silu_backward(g, dy) -> np.ndarray:
    g, dy = _f32(g), _f32(dy)
    dg = np.empty_like(g)
    lib().orc_silu_backward(_p(g), _p(dy), _p(dg), g.size)
    return dg


def moe_combine_backward(dy, y_permuted, dest_row, gates, top_k: int):
    """Backward of the combine: ``(dy_permuted [rows, D], gate_grad [N*K])``."""
    dy, y_permuted, gates = _f32(dy), _f32(y_permuted), _f32(gates)
    dest_row = np.ascontiguousarray(dest_row, dtype=np.uint32)
    n, d = dy.shape
    rows = y_permuted.shape[0]
    dyp = np.empty((rows, d), dtype=np.float32)
    gg = np.empty(n * top_k, dtype=np.float32)
    lib().orc_moe_combine_backward(_p(dy), _p(y_permuted), _p(dest_row), _p(gates), n, top_k, d, rows,
                                   _p(dyp), _p(gg))
    return dyp, gg


def moe_scatter_backward(dx_permuted, dest_row, tokens: int, top_k: int) -> np.ndarray:
    dx_permuted = _f32(dx_permuted)
    dest_row = np.ascontiguousarray(dest_row, dtype=np.uint32)
    d = dx_permuted.shape[1]
    dx = np.empty((tokens, d), dtype=np.float32)
    lib().orc_moe_scatter_backward(_p(dx_permuted), _p(dest_row), tokens, top_k, d, _p(dx))
    return dx


def moe_route_backward(probs, selected, gates, gate_grad, assignment_counts, aux_coefficient: float,
                       top_k: int) -> np.ndarray:
    probs, gates, gate_grad = _f32(probs), _f32(gates), _f32(gate_grad)
    selected = np.ascontiguousarray(selected, dtype=np.uint32)
    counts = np.ascontiguousarray(assignment_counts, dtype=np.uint32)
    n, e = probs.shape
    out = np.empty_like(probs)
    lib().orc_moe_route_backward(_p(probs), _p(selected), _p(gates), _p(gate_grad), _p(counts),
                                 aux_coefficient, n, e, top_k, _p(out))
    return out
