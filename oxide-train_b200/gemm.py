"""Host-side mirror of the reference's ``Tcgen05Gemm`` (gpu/gemm/src/host.rs:469-1098).

Same method names and argument meaning as the reference's Rust type, over the
C ABI.  PyTorch appears only as the owner of device memory and streams: every
method takes CUDA tensors, passes their raw pointers to the library and
launches asynchronously on the current stream.

Operand conventions (gpu/gemm/src/host.rs:112-125): a K-major operand is stored
``[rows, K]``; an MN-major ("transposed") operand is stored ``[K, rows]``.
``store*`` overwrite ``C``; ``accumulate*`` add into it.  Methods without the
``f32_`` prefix produce bf16 (round to nearest even), the others fp32.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


class Tcgen05Gemm:
    """One per device, like the reference's loaded module (host.rs:508-530)."""

    TC_TILE = 128          # host.rs:13
    TC_BK = 64             # host.rs:15
    TC_M_TILE = 256        # host.rs:17
    TC_N_TILE = 256        # host.rs:19

    def __init__(self, device: int | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("Tcgen05Gemm needs a CUDA device (B200, sm_100a); there is no CPU path")
        self.device = torch.cuda.current_device() if device is None else int(device)
        self._lib = L.load()
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            L.check(self._lib.b200gemm_create(self.device, C.byref(h)))
        self._h = h
        self.sm_limit = 0          # 0 = every SM; what set_sm_limit was last given

    @classmethod
    def load(cls, device: int | None = None) -> "Tcgen05Gemm":
        return cls(device)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.b200gemm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ core
    def _desc(self, a, b, c, *, transposed_a=False, transposed_b=False, accumulate=False,
              split_k=0, flags=0, m=None, n=None, k=None) -> L.GemmDesc:
        if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
            raise TypeError("operands must be bf16")
        if c.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("output must be fp32 or bf16")
        batched = a.dim() == 3
        if batched != (b.dim() == 3) or batched != (c.dim() == 3):
            raise ValueError("batched calls need 3-D a, b and c")
        for t in (a, b, c):
            if t.stride(-1) != 1:
                raise ValueError("innermost dimension must be contiguous")
        batch = a.shape[0] if batched else 1
        ar, ac = a.shape[-2], a.shape[-1]
        br, bc = b.shape[-2], b.shape[-1]
        M, K = (ac, ar) if transposed_a else (ar, ac)
        N, Kb = (bc, br) if transposed_b else (br, bc)
        if K != Kb:
            raise ValueError(f"reduction extents differ: {K} vs {Kb}")
        if tuple(c.shape[-2:]) != (M, N):
            raise ValueError(f"output is {tuple(c.shape[-2:])}, expected {(M, N)}")
        d = L.GemmDesc()
        d.a, d.b, d.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
        d.m, d.n, d.k = M, N, K
        d.lda, d.ldb, d.ldc = a.stride(-2), b.stride(-2), c.stride(-2)
        d.a_layout = L.MN_MAJOR if transposed_a else L.K_MAJOR
        d.b_layout = L.MN_MAJOR if transposed_b else L.K_MAJOR
        d.out_type = L.OUT_F32 if c.dtype == torch.float32 else L.OUT_BF16
        d.mode = L.ACCUMULATE if accumulate else L.STORE
        d.batch = batch
        d.split_k = split_k
        if batched:
            d.batch_stride_a, d.batch_stride_b, d.batch_stride_c = a.stride(0), b.stride(0), c.stride(0)
        d.flags = flags
        return d

    def gemm(self, a, b, c, **kw) -> None:
        """General form: ``c (=|+=) A . B^T`` with per-operand layouts."""
        d = self._desc(a, b, c, **kw)
        L.check(self._lib.b200gemm_gemm(self._h, _stream_ptr(), C.byref(d)))

    def f32_store_with_bf16_copy(self, a, b, out, out_bf16, **kw) -> None:
        """``out = A . B^T`` in fp32 and, from the same launch, ``out_bf16`` = the result
        rounded to bf16 (replaces ``f32_store`` + ``convert_f32_to_bf16_pairs``,
        gpu/model/src/lib.rs:1194-1199)."""
        if out.dtype != torch.float32 or out_bf16.dtype != torch.bfloat16:
            raise TypeError("outputs must be fp32 and bf16")
        if out_bf16.shape != out.shape or out_bf16.stride(-1) != 1:
            raise ValueError("the bf16 copy must have the output's shape and contiguous rows")
        d = self._desc(a, b, out, **kw)
        L.check(self._lib.b200gemm_gemm_dual(self._h, _stream_ptr(), C.byref(d), out_bf16.data_ptr(),
                                             out_bf16.stride(-2), out_bf16.stride(0) if out.dim() == 3 else 0))

    def launch_config(self, a, b, c, **kw) -> dict:
        d = self._desc(a, b, c, **kw)
        vals = [C.c_int32() for _ in range(4)]
        L.check(self._lib.b200gemm_launch_config(self._h, C.byref(d), *[C.byref(v) for v in vals]))
        return dict(zip(("grid", "cluster", "smem_bytes", "split_k"), (v.value for v in vals)))

    def set_sm_limit(self, sms: int = 0) -> None:
        """Keep the persistent kernels on at most ``sms`` SMs (0 = all of them)."""
        L.check(self._lib.b200gemm_set_sm_limit(self._h, int(sms)))
        self.sm_limit = int(sms)

    def set_exchange_ctas(self, ctas: int = 0, bulk: bool = False) -> None:
        """Thread blocks of the expert exchange's dispatch / combine kernels (0 = two per SM);
        ``bulk``: the forms that move rows by bulk asynchronous copies through shared memory."""
        L.check(self._lib.b200gemm_set_exchange_ctas(self._h, int(ctas), 1 if bulk else 0))

    def set_scheduler(self, dynamic: bool) -> None:
        """Tiles from a device-side counter (``True``) or the fixed round-robin walk (``False``)."""
        L.check(self._lib.b200gemm_set_scheduler(self._h, 1 if dynamic else 0))

    def device_status(self) -> int:
        """Synchronise and return the device status word (0 = ok); raises on a timeout."""
        code = C.c_int32()
        L.check(self._lib.b200gemm_device_status(self._h, _stream_ptr(), C.byref(code)))
        return code.value

    # ------------------------------------------------- reference method set
    # bf16 output (host.rs:616, 658, 695, 875)
    def store(self, a, b, out, **kw):
        """``C = A.B^T`` packed bf16 (host.rs:616)."""
        self.gemm(a, b, out, **kw)

    def store_batched(self, a, b, out, **kw):
        """``experts`` equal-shaped ``C = A.B^T`` in one launch (host.rs:658)."""
        self.gemm(a, b, out, **kw)

    def accumulate(self, a, b, out, **kw):
        """``C += A.B^T`` in bf16 (host.rs:695)."""
        self.gemm(a, b, out, accumulate=True, **kw)

    def accumulate_transposed(self, a, b, out, **kw):
        """``C += A^T.B`` with A ``[K, M]`` and B ``[K, N]`` read MN-major (host.rs:875)."""
        self.gemm(a, b, out, transposed_a=True, transposed_b=True, accumulate=True, **kw)

    # fp32 output, overwrite (host.rs:729, 766, 957, 1039)
    def f32_store(self, a, b, out, **kw):
        self.gemm(a, b, out, **kw)

    def f32_store_at(self, a, b, out, output_offset: int, output_elements: int, n: int, **kw):
        """Write into ``out[offset : offset + elements]`` viewed as ``[m, n]`` (host.rs:766)."""
        view = out.view(-1)[output_offset:output_offset + output_elements].view(-1, n)
        self.gemm(a, b, view, **kw)

    def f32_store_batched(self, a, b, out, **kw):
        self.gemm(a, b, out, **kw)

    def f32_store_transposed(self, a, b, out, **kw):
        self.gemm(a, b, out, transposed_a=True, transposed_b=True, **kw)

    # fp32 output, accumulate (host.rs:802, 837, 914, 997, 1074)
    def f32_accumulate(self, a, b, out, **kw):
        self.gemm(a, b, out, accumulate=True, **kw)

    def f32_accumulate_at(self, a, b, out, output_offset: int, output_elements: int, n: int, **kw):
        view = out.view(-1)[output_offset:output_offset + output_elements].view(-1, n)
        self.gemm(a, b, view, accumulate=True, **kw)

    def f32_accumulate_transposed(self, a, b, out, **kw):
        self.gemm(a, b, out, transposed_a=True, transposed_b=True, accumulate=True, **kw)

    def f32_accumulate_transposed_at(self, a, b, out, output_offset: int, output_elements: int,
                                     n: int, **kw):
        view = out.view(-1)[output_offset:output_offset + output_elements].view(-1, n)
        self.gemm(a, b, view, transposed_a=True, transposed_b=True, accumulate=True, **kw)

    def f32_accumulate_transposed_batched(self, a, b, out, **kw):
        self.gemm(a, b, out, transposed_a=True, transposed_b=True, accumulate=True, **kw)

    # --------------------------------------------- fp32 family and staging
    def sgemm(self, op: int, a, b, c, accumulate: bool = False) -> None:
        """fp32 CUDA-core GEMM (gpu/gemm/src/fp32.rs:141-191)."""
        for t in (a, b, c):
            if t.dtype != torch.float32 or not t.is_contiguous():
                raise TypeError("sgemm takes dense fp32 tensors")
        m, n = c.shape
        k = a.shape[0] if op == L.OP_TN else a.shape[1]
        L.check(self._lib.b200gemm_sgemm(self._h, _stream_ptr(), op, int(accumulate), a.data_ptr(),
                                         b.data_ptr(), c.data_ptr(), m, n, k))

    def matmul(self, a, b):
        """``GpuTensor::matmul`` (gpu/tensor-gpu/src/lib.rs:1754-1851): ``[M,K] x [K,N]``."""
        c = torch.empty(a.shape[0], b.shape[1], dtype=torch.float32, device=a.device)
        self.sgemm(L.OP_NN, a, b, c)
        return c

    def matmul_nt(self, a, b):
        c = torch.empty(a.shape[0], b.shape[0], dtype=torch.float32, device=a.device)
        self.sgemm(L.OP_NT, a, b, c)
        return c

    def matmul_tn(self, a, b):
        c = torch.empty(a.shape[1], b.shape[1], dtype=torch.float32, device=a.device)
        self.sgemm(L.OP_TN, a, b, c)
        return c

    def convert_f32_to_bf16(self, src, dst=None):
        dst = torch.empty_like(src, dtype=torch.bfloat16) if dst is None else dst
        L.check(self._lib.b200gemm_convert_f32_to_bf16(self._h, _stream_ptr(), src.data_ptr(),
                                                       dst.data_ptr(), src.numel()))
        return dst

    def convert_bf16_to_f32(self, src, dst=None):
        dst = torch.empty_like(src, dtype=torch.float32) if dst is None else dst
        L.check(self._lib.b200gemm_convert_bf16_to_f32(self._h, _stream_ptr(), src.data_ptr(),
                                                       dst.data_ptr(), src.numel()))
        return dst

    def transpose_bf16(self, src, dst=None):
        rows, cols = src.shape
        dst = torch.empty(cols, rows, dtype=torch.bfloat16, device=src.device) if dst is None else dst
        L.check(self._lib.b200gemm_transpose_bf16(self._h, _stream_ptr(), src.data_ptr(),
                                                  dst.data_ptr(), rows, cols))
        return dst
