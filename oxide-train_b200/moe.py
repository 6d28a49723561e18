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


def grouped_gemm_silu(gemm: Tcgen05Gemm, a, b, offsets, out=None, before=None, want_before: bool = True,
                      transposed_b: bool = True, group_b_index=None):
    """``silu(a . W)`` per row group, keeping ``a . W`` (bf16) for the activation's backward.

    Returns ``(y, before)``; ``b`` as in :func:`grouped_gemm`."""
    rows, k = a.shape
    n = b.shape[2] if transposed_b else b.shape[1]
    groups = offsets.numel() - 1
    if out is None:
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=a.device)
    if before is None and want_before:
        before = torch.empty((rows, n), dtype=torch.bfloat16, device=a.device)
    L.check(gemm._lib.b200gemm_grouped_gemm_silu(
        gemm._h, _stream_ptr(), a.data_ptr(), a.stride(0), b.data_ptr(),
        L.MN_MAJOR if transposed_b else L.K_MAJOR, b.stride(1), b.stride(0), b.shape[0],
        None if group_b_index is None else group_b_index.data_ptr(), out.data_ptr(), out.stride(0),
        None if before is None else before.data_ptr(), 0 if before is None else before.stride(0),
        offsets.data_ptr(), groups, rows, n, k))
    return out, before


def grouped_wgrad(gemm: Tcgen05Gemm, a, b, offsets, out, accumulate: bool = True, group_c_index=None):
    """``out[g] (=|+=) a[rows_g]^T . b[rows_g]`` (fp32 ``[matrices, m, n]``): the weight gradients
    of the expert linears, the row groups being the reduction axis
    (gpu/model/src/lib.rs:2011-2055, over exact groups instead of capacity bins)."""
    rows, m = a.shape
    n = b.shape[1]
    if b.shape[0] != rows:
        raise ValueError("a and b must have the same rows")
    if out.dtype != torch.float32 or tuple(out.shape[1:]) != (m, n) or out.stride(2) != 1:
        raise TypeError("out must be fp32 [matrices, m, n]")
    groups = offsets.numel() - 1
    if group_c_index is None and out.shape[0] != groups:
        raise ValueError("one output matrix per group unless group_c_index is given")
    L.check(gemm._lib.b200gemm_grouped_wgrad(
        gemm._h, _stream_ptr(), a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(),
        out.stride(1), out.stride(0), out.shape[0],
        None if group_c_index is None else group_c_index.data_ptr(), offsets.data_ptr(), groups, rows, m, n,
        int(accumulate)))
    return out


def combine_backward(gemm: Tcgen05Gemm, dy, routing: MoeRouting, y_permuted=None, rows: int | None = None,
                     out=None):
    """Backward of :func:`combine`: ``(dy_permuted bf16 [rows, d], gate_grad fp32 [tokens * top_k] | None)``.

    ``y_permuted`` (the expert outputs the forward combined) is needed only for ``gate_grad``."""
    tokens, d = dy.shape
    rows = tokens * routing.top_k if rows is None else rows
    if out is None:
        out = torch.empty((rows, d), dtype=torch.bfloat16, device=dy.device)
    gate_grad = None
    if y_permuted is not None:
        gate_grad = torch.empty(tokens * routing.top_k, dtype=torch.float32, device=dy.device)
    L.check(gemm._lib.b200gemm_moe_combine_backward(
        gemm._h, _stream_ptr(), dy.data_ptr(), L.OUT_F32 if dy.dtype == torch.float32 else L.OUT_BF16,
        None if y_permuted is None else y_permuted.data_ptr(), routing.dest_row.data_ptr(),
        routing.gate_weights.data_ptr(), tokens, routing.top_k, d, out.data_ptr(),
        None if gate_grad is None else gate_grad.data_ptr()))
    return out, gate_grad


def scatter_backward(gemm: Tcgen05Gemm, dx_permuted, routing: MoeRouting, out_dtype=torch.float32):
    """Backward of :func:`scatter`: ``dx[token] = sum_rank dx_permuted[dest_row]``."""
    d = dx_permuted.shape[1]
    out = torch.empty((routing.tokens, d), dtype=out_dtype, device=dx_permuted.device)
    L.check(gemm._lib.b200gemm_moe_combine(
        gemm._h, _stream_ptr(), dx_permuted.data_ptr(), routing.dest_row.data_ptr(), None, None,
        routing.tokens, routing.top_k, d, out.data_ptr(),
        L.OUT_F32 if out_dtype == torch.float32 else L.OUT_BF16))
    return out


def activation_backward(gemm: Tcgen05Gemm, activation: str, saved, d_y, out=None):
    """``activation`` is ``"silu"`` (``saved`` = values before it, ``[rows, ff]``) or ``"swiglu"``
    (``saved`` = the ``[rows, 2, ff]`` gate/up panel); returns the gradient of ``saved``."""
    rows, ff = d_y.shape
    code = {"silu": 1, "swiglu": 2}[activation]
    if out is None:
        out = torch.empty_like(saved)
    L.check(gemm._lib.b200gemm_activation_backward(
        gemm._h, _stream_ptr(), code, saved.data_ptr(), saved.stride(0), d_y.data_ptr(), d_y.stride(0),
        rows, ff, out.data_ptr(), out.stride(0)))
    return out


def grouped_gemm_act_backward(gemm: Tcgen05Gemm, dy, w, offsets, activation: str, saved, out=None,
                              group_b_index=None):
    """``d_saved = act'(saved) * (dy . w^T)`` per row group in one launch: the input gradient of an
    expert's down projection with the activation's backward in its epilogue.

    ``w`` is ``[matrices, n, k]`` (the ``[IN, OUT]`` weight read K-major); ``saved`` / the result are
    ``[rows, n]`` (``"silu"``) or ``[rows, 2, n]`` (``"swiglu"``)."""
    rows, k = dy.shape
    n = w.shape[1]
    if w.shape[2] != k:
        raise ValueError("reduction extents differ")
    code = {"silu": 1, "swiglu": 2}[activation]
    groups = offsets.numel() - 1
    if out is None:
        out = torch.empty_like(saved)
    L.check(gemm._lib.b200gemm_grouped_gemm_act_backward(
        gemm._h, _stream_ptr(), dy.data_ptr(), dy.stride(0), w.data_ptr(), L.K_MAJOR, w.stride(1), w.stride(0),
        w.shape[0], None if group_b_index is None else group_b_index.data_ptr(), code, saved.data_ptr(),
        saved.stride(0), out.data_ptr(), out.stride(0), offsets.data_ptr(), groups, rows, n, k))
    return out


def route_backward(gemm: Tcgen05Gemm, probs, routing: MoeRouting, gate_grad, aux_coefficient: float = 0.0):
    """Gradient of the router's logits from the gradients of the combine weights (moe.rs:397-445)."""
    tokens, experts = probs.shape
    out = torch.empty_like(probs)
    L.check(gemm._lib.b200gemm_moe_route_backward(
        gemm._h, _stream_ptr(), probs.data_ptr(), routing.selected_experts.data_ptr(),
        routing.gate_weights.data_ptr(), gate_grad.data_ptr(), routing.assignment_counts.data_ptr(),
        float(aux_coefficient), tokens, experts, routing.top_k, out.data_ptr()))
    return out


def router_logits(gemm: Tcgen05Gemm, x, w_router):
    """``x [tokens, d] (bf16) . w_router [d, experts] (fp32)`` in the CPU router's own arithmetic."""
    tokens, d = x.shape
    experts = w_router.shape[1]
    if x.dtype != torch.bfloat16 or w_router.dtype != torch.float32 or not (x.is_contiguous() and w_router.is_contiguous()):
        raise TypeError("x must be dense bf16 and w_router dense fp32")
    out = torch.empty((tokens, experts), dtype=torch.float32, device=x.device)
    L.check(gemm._lib.b200gemm_router_logits(gemm._h, _stream_ptr(), x.data_ptr(), w_router.data_ptr(),
                                             tokens, d, experts, out.data_ptr()))
    return out


class _ExpertCtx:
    """What a forward keeps for its backward (the reference's ``GpuExpertActs``)."""

    def __init__(self, routing, x_permuted, saved, hidden, y_permuted):
        self.routing, self.x_permuted, self.saved = routing, x_permuted, saved
        self.hidden, self.y_permuted = hidden, y_permuted


class _ExpertFfnBase:
    activation = "silu"
    fuse_activation_backward = True

    def _up(self, xp, offsets, keep):
        raise NotImplementedError

    def forward(self, x, scores, top_k: int, scores_are_logits: bool = False, residual=None,
                out_dtype=torch.float32, keep_for_backward: bool = False, capacity: int | None = None):
        r = route(self.gemm, scores, top_k, capacity=capacity, scores_are_logits=scores_are_logits)
        xp = scatter(self.gemm, x, r)
        hidden, saved = self._up(xp, r.offsets, keep_for_backward)
        yp = grouped_gemm(self.gemm, hidden, self.w_down, r.offsets, transposed_b=True)
        self.ctx = _ExpertCtx(r, xp, saved, hidden, yp) if keep_for_backward else None
        return combine(self.gemm, yp, r, residual, out_dtype), r

    def backward(self, dy, d_w_up, d_w_down, want_gate_grad: bool = True, dx_dtype=torch.float32):
        """Backward of the last ``forward(..., keep_for_backward=True)``.

        Accumulates into the fp32 weight gradients (shapes of the weights) and returns
        ``(dx [tokens, d], gate_grad [tokens * top_k] | None)``.  Mirrors
        ``GpuExpertFfn::backward_profiled`` (gpu/model/src/lib.rs:2335-2425) between the
        backward of the combine and the backward of the dispatch (crates/nn/src/moe.rs:354-395)."""
        c = self.ctx
        if c is None:
            raise RuntimeError("forward was not asked to keep its activations")
        g, r = self.gemm, c.routing
        dyp, gate_grad = combine_backward(g, dy, r, c.y_permuted if want_gate_grad else None,
                                          rows=c.y_permuted.shape[0])
        # down projection: dW_down[e] += hidden_e^T dyp_e ; d_hidden = dyp . W_down^T
        grouped_wgrad(g, c.hidden, dyp, r.offsets, d_w_down, accumulate=True)
        ff = self.w_down.shape[1]
        if self.fuse_activation_backward and ff % (64 if self.activation == "swiglu" else 8) == 0:
            # d_hidden = dyp . W_down^T never leaves the SM: the activation's backward is the GEMM's epilogue
            d_saved = grouped_gemm_act_backward(g, dyp, self.w_down, r.offsets, self.activation, c.saved)
        else:
            d_hidden = grouped_gemm(g, dyp, self.w_down, r.offsets, transposed_b=False)
            d_saved = activation_backward(g, self.activation, c.saved, d_hidden)
        # up projection: dW_up[e] += x_e^T d_saved_e ; dx_permuted = d_saved . W_up^T
        flat = d_saved.reshape(d_saved.shape[0], -1)
        w_up = self.w_up.reshape(self.w_up.shape[0], self.w_up.shape[1], -1)
        grouped_wgrad(g, c.x_permuted, flat, r.offsets, d_w_up.reshape(w_up.shape), accumulate=True)
        dxp = grouped_gemm(g, flat, w_up, r.offsets, transposed_b=False)
        return scatter_backward(g, dxp, r, dx_dtype), gate_grad


class GatedExpertFfn(_ExpertFfnBase):
    """``y = down(silu(gate(x)) * up(x))`` per expert over routed rows -- the reference's
    own expert (crates/nn/src/moe.rs:76-90: SwiGLU over a fused gate/up projection).

    ``w_gate_up`` is ``[experts, d, 2, ff]``, ``w_down`` ``[experts, ff, d]``."""
    activation = "swiglu"

    def __init__(self, gemm: Tcgen05Gemm, w_gate_up, w_down):
        self.gemm, self.w_gate_up, self.w_down = gemm, w_gate_up, w_down
        self.w_up = w_gate_up
        self.gate_up = None

    def _up(self, xp, offsets, keep):
        res = grouped_gemm_swiglu(self.gemm, xp, self.w_gate_up, offsets, want_gate_up=keep)
        hidden, self.gate_up = res if keep else (res, None)
        return hidden, self.gate_up

    def forward(self, x, scores, top_k: int, scores_are_logits: bool = False, residual=None,
                out_dtype=torch.float32, keep_gate_up: bool = False, capacity: int | None = None):
        return super().forward(x, scores, top_k, scores_are_logits, residual, out_dtype,
                               keep_for_backward=keep_gate_up, capacity=capacity)


class GroupedExpertFfn(_ExpertFfnBase):
    """``y = down(silu(up(x)))`` per expert over routed rows (the 64-expert top-8 configuration).

    ``w_up`` is ``[experts, d, ff]`` and ``w_down`` ``[experts, ff, d]`` (the
    reference's ``[IN, OUT]`` orientation, read in place as MN-major B operands).
    """
    activation = "silu"

    def __init__(self, gemm: Tcgen05Gemm, w_up, w_down):
        self.gemm, self.w_up, self.w_down = gemm, w_up, w_down

    def _up(self, xp, offsets, keep):
        if keep:
            return grouped_gemm_silu(self.gemm, xp, self.w_up, offsets)
        return grouped_gemm(self.gemm, xp, self.w_up, offsets, transposed_b=True, silu=True), None
