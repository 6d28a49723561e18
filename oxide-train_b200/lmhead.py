"""Host mirror of the reference's lm-head + loss path, over the fused kernels.

Reference call sites: ``GpuBf16Head::{forward_into, backward_weight,
backward_input}`` (gpu/model/src/lib.rs:2987-3202) followed by
``cross_entropy_into`` / ``cross_entropy_backward_into`` (lib.rs:6977-7040).
There the ``[tokens, vocab]`` logits are written to HBM in bf16 and re-read by
the classifier kernels; here the GEMM's epilogue consumes them on chip.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from .gemm import Tcgen05Gemm, _stream_ptr


class FusedLmHead:
    """``loss = mean CE(hidden . W, targets)`` and its gradients.

    ``weight`` is ``[hidden, vocab_padded]`` (the reference's ``[IN, OUT]``
    master, ``w_layout="in_out"``) or ``[vocab_padded, hidden]``
    (``w_layout="out_in"``).  Columns at or beyond ``classes`` are padding.
    """

    def __init__(self, gemm: Tcgen05Gemm, classes: int, w_layout: str = "in_out"):
        self.gemm = gemm
        self.classes = int(classes)
        if w_layout not in ("in_out", "out_in"):
            raise ValueError("w_layout is 'in_out' or 'out_in'")
        self.w_layout = L.MN_MAJOR if w_layout == "in_out" else L.K_MAJOR
        self._ws = None

    def _dims(self, hidden, weight):
        m, k = hidden.shape
        if self.w_layout == L.MN_MAJOR:
            k2, v = weight.shape
        else:
            v, k2 = weight.shape
        if k != k2:
            raise ValueError(f"hidden width {k} does not match the weight's {k2}")
        for t in (hidden, weight):
            if t.dtype != torch.bfloat16 or not t.is_contiguous():
                raise TypeError("hidden and weight must be dense bf16")
        return m, k, v

    def workspace(self, m: int, device) -> torch.Tensor:
        need = self.gemm._lib.b200gemm_lmhead_ce_workspace_bytes(m)
        if self._ws is None or self._ws.numel() < need or self._ws.device != device:
            self._ws = torch.empty(need, dtype=torch.uint8, device=device)
        return self._ws

    def forward(self, hidden, weight, targets, workspace=None):
        """Returns ``(loss[1], lse[m], row_loss[m])`` as fp32 device tensors."""
        m, k, v = self._dims(hidden, weight)
        if targets.dtype != torch.int32 or targets.numel() != m:
            raise TypeError("targets must be int32 of length m")
        dev = hidden.device
        ws = self.workspace(m, dev) if workspace is None else workspace
        lse = torch.empty(m, dtype=torch.float32, device=dev)
        row_loss = torch.empty(m, dtype=torch.float32, device=dev)
        loss = torch.empty(1, dtype=torch.float32, device=dev)
        L.check(self.gemm._lib.b200gemm_lmhead_ce_forward(
            self.gemm._h, _stream_ptr(), hidden.data_ptr(), weight.data_ptr(), self.w_layout,
            targets.data_ptr(), m, k, v, self.classes, lse.data_ptr(), row_loss.data_ptr(),
            loss.data_ptr(), ws.data_ptr(), ws.numel()))
        return loss, lse, row_loss

    def backward(self, hidden, weight, targets, lse, dy: float = 1.0, dlogits=None, d_hidden=None,
                 d_weight=None, accumulate_dw: bool = False, want_d_hidden=True, want_d_weight=True):
        """Returns ``(dlogits bf16 [m, v], d_hidden fp32 [m, k], d_weight fp32 like weight)``."""
        m, k, v = self._dims(hidden, weight)
        dev = hidden.device
        if dlogits is None:
            dlogits = torch.empty((m, v), dtype=torch.bfloat16, device=dev)
        if d_hidden is None and want_d_hidden:
            d_hidden = torch.empty((m, k), dtype=torch.float32, device=dev)
        if d_weight is None and want_d_weight:
            d_weight = torch.zeros(weight.shape, dtype=torch.float32, device=dev)
        L.check(self.gemm._lib.b200gemm_lmhead_ce_backward(
            self.gemm._h, _stream_ptr(), hidden.data_ptr(), weight.data_ptr(), self.w_layout,
            targets.data_ptr(), lse.data_ptr(), float(dy), m, k, v, self.classes,
            dlogits.data_ptr(), d_hidden.data_ptr() if d_hidden is not None else None,
            d_weight.data_ptr() if d_weight is not None else None, int(accumulate_dw)))
        return dlogits, d_hidden, d_weight
