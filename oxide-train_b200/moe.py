"""Host mirror of the reference's MoE routing + expert path, over the C ABI.

Reference: ``MoeFfn::route`` / ``MoeFfn::forward`` (crates/nn/src/moe.rs:205-352)
and the GPU block in gpu/model/src/lib.rs:4971-5130 (router_softmax_topk ->
moe_bin_assign_parallel -> moe_scatter -> expert linears -> gather/combine).
Here the experts run as ONE variable-length grouped GEMM per projection over the
permuted rows, instead of fixed-capacity bins.
"""
from __future__ import annotations

import torch

from . import _lib as L
from .gemm import Tcgen05Gemm, _stream_ptr

DROPPED = 0xFFFFFFFF


class MoeRouting:
    """Device tensors produced by :func:`route` (names follow ``MoeRouting``, moe.rs:23-35)."""

    def __init__(self, tokens, experts, top_k, device):
        pairs = tokens * top_k
        i32 = torch.int32
        # uint32 values live in int32 storage; view them with ``.cpu().numpy().view(np.uint32)``.
        self.selected_experts = torch.empty(pairs, dtype=i32, device=device)
        self.gate_weights = torch.empty(pairs, dtype=torch.float32, device=device)
        self.slots = torch.empty(pairs, dtype=i32, device=device)
        self.assignment_counts = torch.empty(experts, dtype=i32, device=device)
        self.accepted_counts = torch.empty(experts, dtype=i32, device=device)
        self.offsets = torch.empty(experts + 1, dtype=i32, device=device)
        self.dest_row = torch.empty(pairs, dtype=i32, device=device)
        self.tokens, self.experts, self.top_k = tokens, experts, top_k


def route(gemm: Tcgen05Gemm, scores, top_k: int, capacity: int | None = None,
          scores_are_logits: bool = False) -> MoeRouting:
    """Top-k routing of ``scores[tokens, experts]`` (fp32)."""
    if scores.dtype != torch.float32 or not scores.is_contiguous():
        raise TypeError("scores must be dense fp32")
    tokens, experts = scores.shape
    capacity = tokens * top_k if capacity is None else capacity
    r = MoeRouting(tokens, experts, top_k, scores.device)
    L.check(gemm._lib.b200gemm_moe_route(
        gemm._h, _stream_ptr(), scores.data_ptr(), int(scores_are_logits), tokens, experts, top_k,
        capacity, r.selected_experts.data_ptr(), r.gate_weights.data_ptr(), r.slots.data_ptr(),
        r.assignment_counts.data_ptr(), r.accepted_counts.data_ptr(), r.offsets.data_ptr(),
        r.dest_row.data_ptr()))
    return r


def scatter(gemm: Tcgen05Gemm, x, routing: MoeRouting, rows: int | None = None):
    """Dispatch: permuted[dest_row] = x[token].  ``rows`` defaults to tokens * top_k."""
    tokens, d = x.shape
    rows = tokens * routing.top_k if rows is None else rows
    # every routed row is written; rows of dropped assignments (none when capacity is
    # tokens * top_k) are never read back by combine
    out = torch.empty((rows, d), dtype=torch.bfloat16, device=x.device)
    L.check(gemm._lib.b200gemm_moe_scatter(gemm._h, _stream_ptr(), x.data_ptr(),
                                           routing.dest_row.data_ptr(), tokens, routing.top_k, d,
                                           out.data_ptr()))
    return out


def combine(gemm: Tcgen05Gemm, y_permuted, routing: MoeRouting, residual=None, out_dtype=torch.float32):
    """out[token] = residual[token] + sum_rank gate * y_permuted[dest_row]."""
    d = y_permuted.shape[1]
    out = torch.empty((routing.tokens, d), dtype=out_dtype, device=y_permuted.device)
    L.check(gemm._lib.b200gemm_moe_combine(
        gemm._h, _stream_ptr(), y_permuted.data_ptr(), routing.dest_row.data_ptr(),
        routing.gate_weights.data_ptr(), residual.data_ptr() if residual is not None else None,
        routing.tokens, routing.top_k, d, out.data_ptr(),
        L.OUT_F32 if out_dtype == torch.float32 else L.OUT_BF16))
    return out


def grouped_gemm(gemm: Tcgen05Gemm, a, b, offsets, out=None, transposed_b: bool = False,
                 silu: bool = False):
    """Rows ``offsets[g]:offsets[g+1]`` of ``a`` times expert ``g``'s matrix.

    ``b`` is ``[groups, n, k]`` or, with ``transposed_b``, ``[groups, k, n]``."""
    rows, k = a.shape
    groups = b.shape[0]
    n = b.shape[2] if transposed_b else b.shape[1]
    if (b.shape[1] if transposed_b else b.shape[2]) != k:
        raise ValueError("reduction extents differ")
    if offsets.dtype != torch.int32 or offsets.numel() != groups + 1:
        raise TypeError("offsets must be int32 [groups + 1] on the device")
    if out is None:
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=a.device)
    L.check(gemm._lib.b200gemm_grouped_gemm(
        gemm._h, _stream_ptr(), a.data_ptr(), a.stride(0), b.data_ptr(),
        L.MN_MAJOR if transposed_b else L.K_MAJOR, b.stride(1), b.stride(0), out.data_ptr(),
        out.stride(0), offsets.data_ptr(), groups, rows, n, k, int(silu)))
    return out


def grouped_gemm_swiglu(gemm: Tcgen05Gemm, a, w_gate_up, offsets, out=None, gate_up=None,
                        want_gate_up: bool = False, group_b_index=None):
    """``silu(a . W_gate) * (a . W_up)`` per row group in one launch.

    ``w_gate_up`` is ``[matrices, k, 2, ff]`` (the reference's fused gate/up weight,
    read in place).  Returns ``y [rows, ff]`` and, with ``want_gate_up`` (or a
    ``gate_up`` buffer), the bf16 ``[rows, 2, ff]`` panel the activation's backward reads.
    ``group_b_index`` (int32 ``[groups]``) picks the matrix of each group; without it
    group ``g`` uses matrix ``g``."""
    rows, k = a.shape
    mats, kw, two, ff = w_gate_up.shape
    if two != 2 or kw != k:
        raise ValueError("w_gate_up must be [matrices, k, 2, ff] with a's reduction extent")
    if not w_gate_up.is_contiguous():
        raise ValueError("w_gate_up must be contiguous")
    groups = offsets.numel() - 1
    if offsets.dtype != torch.int32:
        raise TypeError("offsets must be int32 on the device")
    if group_b_index is None and groups != mats:
        raise ValueError("one group per matrix unless group_b_index is given")
    if out is None:
        out = torch.empty((rows, ff), dtype=torch.bfloat16, device=a.device)
    if gate_up is None and want_gate_up:
        gate_up = torch.empty((rows, 2, ff), dtype=torch.bfloat16, device=a.device)
    L.check(gemm._lib.b200gemm_grouped_gemm_swiglu(
        gemm._h, _stream_ptr(), a.data_ptr(), a.stride(0), w_gate_up.data_ptr(), L.MN_MAJOR,
        w_gate_up.stride(1), w_gate_up.stride(0), mats,
        None if group_b_index is None else group_b_index.data_ptr(), out.data_ptr(), out.stride(0),
        None if gate_up is None else gate_up.data_ptr(), 0 if gate_up is None else gate_up.stride(0),
        offsets.data_ptr(), groups, rows, ff, k))
    return (out, gate_up) if gate_up is not None else out


class GatedExpertFfn:
    """``y = down(silu(gate(x)) * up(x))`` per expert over routed rows -- the reference's
    own expert (crates/nn/src/moe.rs:76-90: SwiGLU over a fused gate/up projection).

    ``w_gate_up`` is ``[experts, d, 2, ff]``, ``w_down`` ``[experts, ff, d]``."""

    def __init__(self, gemm: Tcgen05Gemm, w_gate_up, w_down):
        self.gemm, self.w_gate_up, self.w_down = gemm, w_gate_up, w_down

    def forward(self, x, scores, top_k: int, scores_are_logits: bool = False, residual=None,
                out_dtype=torch.float32, keep_gate_up: bool = False):
        r = route(self.gemm, scores, top_k, scores_are_logits=scores_are_logits)
        xp = scatter(self.gemm, x, r)
        res = grouped_gemm_swiglu(self.gemm, xp, self.w_gate_up, r.offsets, want_gate_up=keep_gate_up)
        hidden, self.gate_up = res if keep_gate_up else (res, None)
        yp = grouped_gemm(self.gemm, hidden, self.w_down, r.offsets, transposed_b=True)
        return combine(self.gemm, yp, r, residual, out_dtype), r


class GroupedExpertFfn:
    """``y = down(silu(up(x)))`` per expert over routed rows (BASELINE MoE config).

    ``w_up`` is ``[experts, d, ff]`` and ``w_down`` ``[experts, ff, d]`` (the
    reference's ``[IN, OUT]`` orientation, read in place as MN-major B operands).
    """

    def __init__(self, gemm: Tcgen05Gemm, w_up, w_down):
        self.gemm, self.w_up, self.w_down = gemm, w_up, w_down

    def forward(self, x, scores, top_k: int, scores_are_logits: bool = False, residual=None,
                out_dtype=torch.float32):
        r = route(self.gemm, scores, top_k, scores_are_logits=scores_are_logits)
        xp = scatter(self.gemm, x, r)
        hidden = grouped_gemm(self.gemm, xp, self.w_up, r.offsets, transposed_b=True, silu=True)
        yp = grouped_gemm(self.gemm, hidden, self.w_down, r.offsets, transposed_b=True)
        return combine(self.gemm, yp, r, residual, out_dtype), r
