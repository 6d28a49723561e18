"""The allocation-free head forward against the workspace-taking one.

Some hosts of this library cannot give it scratch memory: a trainer that has
already carved all of HBM into its own arena, or a step loop in which
cudaMalloc/cudaFree are banned because they stall the whole device.  For them
``b200gemm_lmhead_ce_forward_noalloc`` keeps its per-row softmax statistics in
an array built into the library.  This test calls it through the C ABI twice in
a row, with different shapes so that anything the first call left in the
shared array would show, and compares each result with the regular entry point
on the same inputs.

Kept in a file that sorts last so that a run stopping at the first failure has
already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run_pair(pkg, lib, handle, stream, m, k, v, classes, seed):
    import torch
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    hidden = torch.randn((m, k), generator=gen, device="cuda").to(torch.bfloat16)
    weight = (torch.randn((k, v), generator=gen, device="cuda") * 0.2).to(torch.bfloat16)
    targets = torch.randint(0, classes, (m,), generator=gen, device="cuda", dtype=torch.int32)
    L = pkg._lib

    def outputs():
        return (torch.empty(m, dtype=torch.float32, device="cuda"),
                torch.empty(m, dtype=torch.float32, device="cuda"),
                torch.empty(1, dtype=torch.float32, device="cuda"))

    # existing entry point, caller-provided workspace
    need = lib.b200gemm_lmhead_ce_workspace_bytes(m)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    lse0, row0, loss0 = outputs()
    L.check(lib.b200gemm_lmhead_ce_forward(handle, stream, hidden.data_ptr(), weight.data_ptr(),
                                           L.MN_MAJOR, targets.data_ptr(), m, k, v, classes,
                                           lse0.data_ptr(), row0.data_ptr(), loss0.data_ptr(),
                                           ws.data_ptr(), need))
    # new entry point: no workspace argument at all
    lse1, row1, loss1 = outputs()
    L.check(lib.b200gemm_lmhead_ce_forward_noalloc(handle, stream, hidden.data_ptr(), weight.data_ptr(),
                                                   L.MN_MAJOR, targets.data_ptr(), m, k, v, classes,
                                                   lse1.data_ptr(), row1.data_ptr(), loss1.data_ptr()))
    torch.cuda.synchronize()
    # Same kernels, same inputs: per-row results agree to fp32 rounding; the mean
    # is summed by atomics in f64, so allow its last bits to differ.
    assert np.allclose(lse1.cpu().numpy(), lse0.cpu().numpy(), rtol=1e-6, atol=1e-6)
    assert np.allclose(row1.cpu().numpy(), row0.cpu().numpy(), rtol=1e-6, atol=1e-6)
    assert abs(float(loss1.item()) - float(loss0.item())) <= 5e-5 * max(1.0, abs(float(loss0.item())))
    assert np.isfinite(float(loss1.item())) and float(loss1.item()) > 0.0


def test_noalloc_head_forward_matches_workspace_form_twice_in_a_row(pkg):
    import torch
    torch.cuda.set_device(0)
    gemm = pkg.Tcgen05Gemm(0)
    lib, handle = gemm._lib, gemm._h
    stream = torch.cuda.current_stream().cuda_stream
    try:
        _run_pair(pkg, lib, handle, stream, m=768, k=256, v=1024, classes=1000, seed=7)
        _run_pair(pkg, lib, handle, stream, m=300, k=128, v=520, classes=515, seed=8)
        assert gemm.device_status() == 0
        # beyond the built-in scratch: refused with a clear message, nothing launched
        dummy = torch.zeros(8, dtype=torch.float32, device="cuda")
        rc = lib.b200gemm_lmhead_ce_forward_noalloc(handle, stream, dummy.data_ptr(), dummy.data_ptr(),
                                                    pkg._lib.MN_MAJOR, dummy.data_ptr(), 32769, 64, 64, 64,
                                                    dummy.data_ptr(), None, None)
        assert rc == pkg._lib.ERR_SHAPE
        assert b"32768" in lib.b200gemm_last_error_string()
    finally:
        gemm.close()


def test_noalloc_head_forward_at_its_row_limit_allocates_nothing(pkg, oracle):
    """m = 32768, the largest row count the built-in array holds (the only size that uses all
    of it): sampled rows against the oracle, the whole result against the workspace form, and
    the entry point's one promise -- the device's free memory is the same before and after a call."""
    import torch
    from _util import THREADS
    torch.cuda.set_device(0)
    gemm = pkg.Tcgen05Gemm(0)
    lib, handle, L = gemm._lib, gemm._h, pkg._lib
    stream = torch.cuda.current_stream().cuda_stream
    m, k, v, classes = 32768, 256, 2048, 2000
    try:
        gen = torch.Generator(device="cuda")
        gen.manual_seed(9)
        hidden = torch.randn((m, k), generator=gen, device="cuda").to(torch.bfloat16)
        weight = (torch.randn((k, v), generator=gen, device="cuda") * 0.2).to(torch.bfloat16)
        targets = torch.randint(0, classes, (m,), generator=gen, device="cuda", dtype=torch.int32)
        lse, row, loss = (torch.empty(m, dtype=torch.float32, device="cuda"),
                          torch.empty(m, dtype=torch.float32, device="cuda"),
                          torch.empty(1, dtype=torch.float32, device="cuda"))
        args = (handle, stream, hidden.data_ptr(), weight.data_ptr(), L.MN_MAJOR, targets.data_ptr(), m, k, v,
                classes, lse.data_ptr(), row.data_ptr(), loss.data_ptr())
        L.check(lib.b200gemm_lmhead_ce_forward_noalloc(*args))          # first call: looks the array up
        torch.cuda.synchronize()
        first = (lse.clone(), row.clone(), float(loss.item()))
        free_before, _ = torch.cuda.mem_get_info()
        L.check(lib.b200gemm_lmhead_ce_forward_noalloc(*args))          # later calls only launch
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, "the call changed the device's free memory"
        assert torch.equal(lse, first[0]) and torch.equal(row, first[1])
        assert abs(float(loss.item()) - first[2]) <= 1e-6 * abs(first[2])
        assert gemm.device_status() == 0
        rows = np.array([0, 255, 256, 4097, 16383, 20000, 32767])
        logits = oracle.matmul(hidden[rows].float().cpu().numpy(), weight.float().cpu().numpy(), THREADS)
        _, _, rl = oracle.xent_forward(logits, targets.cpu().numpy()[rows], classes)
        assert np.allclose(row.cpu().numpy()[rows], rl, atol=5e-4, rtol=1e-5)
        # the whole result against the entry point that takes a workspace
        need = lib.b200gemm_lmhead_ce_workspace_bytes(m)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        lse0, row0, loss0 = torch.empty_like(lse), torch.empty_like(row), torch.empty_like(loss)
        L.check(lib.b200gemm_lmhead_ce_forward(handle, stream, hidden.data_ptr(), weight.data_ptr(), L.MN_MAJOR,
                                               targets.data_ptr(), m, k, v, classes, lse0.data_ptr(),
                                               row0.data_ptr(), loss0.data_ptr(), ws.data_ptr(), need))
        torch.cuda.synchronize()
        assert np.allclose(lse.cpu().numpy(), lse0.cpu().numpy(), rtol=1e-6, atol=1e-6)
        assert np.allclose(row.cpu().numpy(), row0.cpu().numpy(), rtol=1e-6, atol=1e-6)
        assert abs(float(loss.item()) - float(loss0.item())) <= 5e-5 * abs(float(loss0.item()))
    finally:
        gemm.close()
