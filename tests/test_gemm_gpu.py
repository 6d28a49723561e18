"""GPU parity of the tcgen05 GEMM against the CPU oracle, through the C ABI.

Shapes and checks follow the reference's own kernel gates
(gpu/gemm/src/main.rs:147-620): 256^3 in every mode against a CPU matmul on
bf16-rounded inputs, the MN-major weight-gradient orientation, and the
integer-periodic operands whose product is exact in fp32 so that bf16 outputs
can be compared with ``==``.
"""
import numpy as np
import pytest

from _util import THREADS, assert_gemm_close, bf16_operand, from_dev_bf16, to_dev_bf16

pytestmark = pytest.mark.gpu

CTA_GROUPS = [1, 2]


@pytest.fixture(scope="module")
def gemm(pkg):
    g = pkg.Tcgen05Gemm()
    yield g
    g.close()


def _flags(pkg, cg):
    return pkg._lib.FLAG_CTA_GROUP_1 if cg == 1 else pkg._lib.FLAG_CTA_GROUP_2


def _tight(out_dtype):
    # fp32 outputs differ from the oracle only by summation order; bf16 outputs
    # add one rounding of the result (relative 2^-9).
    import torch
    return dict(rel_fro=2e-5, elem=2e-4) if out_dtype == torch.float32 else dict(rel_fro=4e-3, elem=8e-3)


# ---- gpu/gemm/src/main.rs:515-620: 256^3, all four modes -------------------

@pytest.mark.parametrize("cg", CTA_GROUPS, ids=["cg1", "cg2"])
@pytest.mark.parametrize("out", ["f32", "bf16"])
def test_256_cubed_store_and_accumulate(pkg, oracle, gemm, cg, out):
    import torch
    M = N = K = 256
    a, av = bf16_operand(oracle, (M, K), 1, kind="uniform")
    b, bv = bf16_operand(oracle, (N, K), 2, kind="uniform")
    ref = oracle.matmul_nt(av, bv, THREADS)
    dt = torch.float32 if out == "f32" else torch.bfloat16
    c = torch.full((M, N), 7.0, dtype=dt, device="cuda")
    gemm.gemm(a, b, c, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    got = c.float().cpu().numpy()
    assert_gemm_close(got, ref, f"store cg{cg} {out}", **_tight(dt))
    # accumulate on top of a known C
    c0, c0v = bf16_operand(oracle, (M, N), 3, kind="uniform")
    c = c0.to(dt).clone()
    gemm.gemm(a, b, c, accumulate=True, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    assert_gemm_close(c.float().cpu().numpy(), ref + c0v, f"accumulate cg{cg} {out}", **_tight(dt))


# ---- gpu/gemm/src/main.rs:343-391: MN-major (weight-gradient) orientation ---

@pytest.mark.parametrize("cg", CTA_GROUPS, ids=["cg1", "cg2"])
@pytest.mark.parametrize("ta,tb", [(True, True), (False, True), (True, False)])
def test_mn_major_operands(pkg, oracle, gemm, cg, ta, tb):
    import torch
    M, N, K = 256, 512, 192
    a, av = bf16_operand(oracle, (K, M) if ta else (M, K), 4, kind="uniform")
    b, bv = bf16_operand(oracle, (K, N) if tb else (N, K), 5, kind="uniform")
    A = av.T if ta else av            # logical [M, K]
    Bt = bv if tb else bv.T           # logical [K, N]
    ref = oracle.matmul(np.ascontiguousarray(A), np.ascontiguousarray(Bt), THREADS)
    c = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    gemm.gemm(a, b, c, transposed_a=ta, transposed_b=tb, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    assert_gemm_close(c.cpu().numpy(), ref, f"mn-major ta={ta} tb={tb} cg{cg}", rel_fro=2e-5, elem=2e-4)


# ---- gpu/gemm/src/main.rs:180-335: many work items, exact equality ----------

def _periodic(lines, depth, mul_l, mul_d, mod, sub):
    i, d = np.meshgrid(np.arange(lines), np.arange(depth), indexing="ij")
    return (((i * mul_l + d * mul_d) % mod) - sub).astype(np.float32)


@pytest.mark.parametrize("cg", CTA_GROUPS, ids=["cg1", "cg2"])
@pytest.mark.parametrize("m,n", [(4096, 2560), (2816, 3584)])
def test_many_items_are_exact(pkg, oracle, gemm, cg, m, n):
    import torch
    K = 256
    av = _periodic(m, K, 5, 3, 7, 3)        # a_value, main.rs:266-268
    bv = _periodic(n, K, 4, 5, 21, 10)      # b_value, main.rs:272-274
    a = to_dev_bf16(oracle.bf16_bits(av))
    b = to_dev_bf16(oracle.bf16_bits(bv))
    table = av[:7].astype(np.int64) @ bv[:21].astype(np.int64).T          # exact 7x21 table
    want = oracle.bf16_round(table.astype(np.float32))
    full = np.tile(want, (m // 7 + 1, n // 21 + 1))[:m, :n]
    c = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    gemm.store(a, b, c, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    got = from_dev_bf16(c)
    assert np.array_equal(got, full), f"{int((got != full).sum())} of {m * n} elements wrong"
    # fp32 output is the exact integer table
    cf = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    gemm.f32_store(a, b, cf, flags=_flags(pkg, cg))
    exact = np.tile(table.astype(np.float32), (m // 7 + 1, n // 21 + 1))[:m, :n]
    assert np.array_equal(cf.cpu().numpy(), exact)
    # folding the same product into C doubles every element (fp32: exactly)
    gemm.f32_accumulate(a, b, cf, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    assert np.array_equal(cf.cpu().numpy(), 2 * exact)


# ---- split-K, batches, offsets, ragged edges --------------------------------

@pytest.mark.parametrize("cg", CTA_GROUPS, ids=["cg1", "cg2"])
@pytest.mark.parametrize("split", [2, 5])
def test_split_k_store_and_accumulate(pkg, oracle, gemm, cg, split):
    import torch
    M, N, K = 256, 256, 2048
    a, av = bf16_operand(oracle, (K, M), 6)           # weight-gradient layout
    b, bv = bf16_operand(oracle, (K, N), 7, std=0.01)
    ref = oracle.matmul_tn(av, bv, THREADS)
    c = torch.full((M, N), 3.0, dtype=torch.float32, device="cuda")
    gemm.f32_store_transposed(a, b, c, split_k=split, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    assert_gemm_close(c.cpu().numpy(), ref, f"split{split} store", rel_fro=2e-5, elem=2e-4)
    gemm.f32_accumulate_transposed(a, b, c, split_k=split, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    assert_gemm_close(c.cpu().numpy(), 2 * ref, f"split{split} accumulate", rel_fro=2e-5, elem=2e-4)


@pytest.mark.parametrize("cg", CTA_GROUPS, ids=["cg1", "cg2"])
def test_batched_experts(pkg, oracle, gemm, cg):
    import torch
    E, M, N, K = 3, 256, 256, 128
    a, av = bf16_operand(oracle, (E, M, K), 8, kind="uniform")
    b, bv = bf16_operand(oracle, (E, N, K), 9, kind="uniform")
    ref = np.stack([oracle.matmul_nt(av[e], bv[e], THREADS) for e in range(E)])
    c = torch.zeros((E, M, N), dtype=torch.float32, device="cuda")
    gemm.f32_store_batched(a, b, c, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    assert_gemm_close(c.cpu().numpy(), ref, "f32_store_batched", rel_fro=2e-5, elem=2e-4)
    cb = torch.zeros((E, M, N), dtype=torch.bfloat16, device="cuda")
    gemm.store_batched(a, b, cb, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    assert_gemm_close(from_dev_bf16(cb), ref, "store_batched", rel_fro=4e-3, elem=8e-3)


@pytest.mark.parametrize("cg", CTA_GROUPS, ids=["cg1", "cg2"])
def test_output_region_and_row_stride(pkg, oracle, gemm, cg):
    import torch
    M, N, K = 256, 256, 64
    a, av = bf16_operand(oracle, (M, K), 10, kind="uniform")
    b, bv = bf16_operand(oracle, (N, K), 11, kind="uniform")
    ref = oracle.matmul_nt(av, bv, THREADS)
    buf = torch.full((3 * M * N,), -1.0, dtype=torch.float32, device="cuda")
    gemm.f32_store_at(a, b, buf, M * N, M * N, N, flags=_flags(pkg, cg))     # middle third
    assert gemm.device_status() == 0
    host = buf.cpu().numpy()
    assert np.all(host[:M * N] == -1.0) and np.all(host[2 * M * N:] == -1.0)  # neighbours untouched
    assert_gemm_close(host[M * N:2 * M * N].reshape(M, N), ref, "f32_store_at", rel_fro=2e-5, elem=2e-4)
    # a column block of a wider matrix: ldc > n (the grouped QKV outputs, gpu/model/src/lib.rs:1379)
    wide = torch.full((M, 3 * N), -1.0, dtype=torch.float32, device="cuda")
    gemm.f32_store(a, b, wide[:, N:2 * N], flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    w = wide.cpu().numpy()
    assert np.all(w[:, :N] == -1.0) and np.all(w[:, 2 * N:] == -1.0)
    assert_gemm_close(w[:, N:2 * N], ref, "ldc > n", rel_fro=2e-5, elem=2e-4)


@pytest.mark.parametrize("cg", CTA_GROUPS, ids=["cg1", "cg2"])
@pytest.mark.parametrize("out", ["f32", "bf16"])
def test_ragged_edges_are_clipped(pkg, oracle, gemm, cg, out):
    import torch
    M, N, K = 200, 136, 72
    a, av = bf16_operand(oracle, (M, K), 12, kind="uniform")
    b, bv = bf16_operand(oracle, (N, K), 13, kind="uniform")
    ref = oracle.matmul_nt(av, bv, THREADS)
    dt = torch.float32 if out == "f32" else torch.bfloat16
    # canary rows after the matrix catch stores past the last row
    c = torch.full((M + 8, N), 5.0, dtype=dt, device="cuda")
    gemm.gemm(a, b, c[:M], flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    host = c.float().cpu().numpy()
    assert np.all(host[M:] == 5.0)
    assert_gemm_close(host[:M], ref, f"ragged {out}", **_tight(dt))
    if out == "bf16":
        c2 = c.clone()
        gemm.accumulate(a, b, c2[:M], flags=_flags(pkg, cg))
        assert gemm.device_status() == 0
        h2 = c2.float().cpu().numpy()
        assert np.all(h2[M:] == 5.0)
        assert_gemm_close(h2[:M], host[:M] + ref, "ragged bf16 accumulate", rel_fro=4e-3, elem=1.6e-2)


def test_contract_violations_return_status_codes(pkg, gemm):
    import torch
    L = pkg._lib
    a = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((64, 64), dtype=torch.float32, device="cuda")
    with pytest.raises(ValueError):
        gemm.gemm(a, a[:, :32].contiguous(), c)                      # K mismatch, caught on the host
    cb = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(pkg.B200GemmError) as e:
        gemm.gemm(a, a, cb, split_k=2)                               # split-K needs fp32 output
    assert e.value.code == L.ERR_UNSUPPORTED
    with pytest.raises(pkg.B200GemmError) as e:
        gemm.gemm(a[:, 1:], a[:, 1:], c)                             # base not 16-byte aligned
    assert e.value.code == L.ERR_SHAPE


def test_bounded_wait_reports_a_status_code_and_the_context_survives(pkg, oracle, gemm):
    """A wait that can never be satisfied gives up after its limit, the kernel
    returns, the host reads the code, and the next GEMM on the same handle is correct."""
    import torch
    from oxide_train_b200._lib import check
    stream = torch.cuda.current_stream().cuda_stream
    check(gemm._lib.b200gemm_wait_selftest(gemm._h, stream, 50))
    with pytest.raises(pkg.B200GemmError) as e:
        gemm.device_status()
    assert e.value.code == pkg._lib.ERR_DEVICE and "104" in str(e.value)
    assert gemm.device_status() == 0                      # reading the code cleared it
    a, av = bf16_operand(oracle, (256, 64), 61, kind="uniform")
    b, bv = bf16_operand(oracle, (256, 64), 62, kind="uniform")
    c = torch.zeros((256, 256), dtype=torch.float32, device="cuda")
    gemm.f32_store(a, b, c)
    assert gemm.device_status() == 0
    assert_gemm_close(c.cpu().numpy(), oracle.matmul_nt(av, bv, THREADS), "after timeout", rel_fro=2e-5, elem=2e-4)


def test_peer_barrier_passes_when_the_peer_arrived_and_gives_up_when_it_did_not(pkg, gemm):
    """The barrier between GPUs, both "ranks'" arrays on this GPU and the peer played by the
    host: with the peer's arrival word already written the kernel passes, delivers its integers
    into both tables (the half the epoch selects) and leaves status 0; with a word nothing
    writes it gives up after its limit with code 108 and the handle stays usable."""
    import ctypes as C
    import torch
    ops = pkg.parallel.DeviceOps(gemm)
    world, count = 2, 5
    words = [torch.zeros(world, dtype=torch.int64, device="cuda") for _ in range(world)]
    tables = [torch.full((2, world, count), -1, dtype=torch.int32, device="cuda") for _ in range(world)]
    pw, pt = (C.c_void_p * world)(), (C.c_void_p * world)()
    for r in range(world):
        pw[r], pt[r] = words[r].data_ptr(), tables[r].data_ptr()
    mine = torch.arange(10, 10 + count, dtype=torch.int32, device="cuda")
    for epoch in (1, 2):
        words[0][1] = epoch                                   # "rank 1" has arrived
        ops.peer_barrier(pw, world, 0, epoch, 200, mine + epoch, pt)
        assert gemm.device_status() == 0
        assert words[0].tolist() == [epoch, epoch] and words[1].tolist() == [epoch, 0]
        for t in tables:
            assert t[epoch & 1, 0].tolist() == (mine + epoch).tolist()
            assert t[epoch & 1, 1].tolist() == [-1] * count   # the peer's row is the peer's to write
    assert tables[0][1, 0].tolist() == (mine + 1).tolist()    # the other half kept the previous epoch's
    ops.peer_barrier(pw, world, 0, 3, 50)                     # nobody writes epoch 3 into words[0][1]
    with pytest.raises(pkg.B200GemmError) as e:
        gemm.device_status()
    assert e.value.code == pkg._lib.ERR_DEVICE and "108" in str(e.value)
    assert gemm.device_status() == 0
    ops.peer_barrier((C.c_void_p * 1)(words[0].data_ptr()), 1, 0, 4, 50)    # a world of one never waits
    assert gemm.device_status() == 0
    with pytest.raises(pkg.B200GemmError):
        ops.peer_barrier(pw, world, 0, 0, 50)                 # epochs start at 1
    with pytest.raises(pkg.B200GemmError):
        ops.peer_barrier(pw, world, 2, 1, 50)                 # rank outside the world


def test_host_buffer_form_copies_in_and_out(pkg, oracle, gemm):
    """b200gemm_gemm_host: A, B (and C when accumulating) live in host memory."""
    import ctypes as C
    L = pkg._lib
    M, N, K = 384, 256, 128
    av = oracle.bf16_round(oracle.uniform(M * K, 71)).reshape(M, K)
    bv = oracle.bf16_round(oracle.uniform(N * K, 72)).reshape(N, K)
    a_bits = np.ascontiguousarray(oracle.bf16_bits(av))
    b_bits = np.ascontiguousarray(oracle.bf16_bits(bv))
    c = np.full((M, N), 2.0, np.float32)
    d = L.GemmDesc()
    d.a, d.b, d.c = a_bits.ctypes.data, b_bits.ctypes.data, c.ctypes.data
    d.m, d.n, d.k = M, N, K
    d.out_type, d.mode, d.batch = L.OUT_F32, L.STORE, 1
    L.check(gemm._lib.b200gemm_gemm_host(gemm._h, None, C.byref(d)))
    ref = oracle.matmul_nt(av, bv, THREADS)
    assert_gemm_close(c, ref, "host store", rel_fro=2e-5, elem=2e-4)
    d.mode = L.ACCUMULATE
    L.check(gemm._lib.b200gemm_gemm_host(gemm._h, None, C.byref(d)))
    assert_gemm_close(c, 2 * ref, "host accumulate", rel_fro=2e-5, elem=2e-4)
    assert gemm.device_status() == 0


# ---- fp32 result + bf16 operand copy from one launch (replaces f32_store followed by
# ---- convert_f32_to_bf16_pairs, gpu/model/src/lib.rs:1194-1199) ------------------------

@pytest.mark.parametrize("cg", CTA_GROUPS, ids=["cg1", "cg2"])
@pytest.mark.parametrize("m,n,k,tb", [(512, 768, 256, True), (300, 200, 136, False), (2048, 1536, 512, True)])
def test_f32_store_with_bf16_copy(pkg, oracle, gemm, cg, m, n, k, tb):
    import torch
    a, av = bf16_operand(oracle, (m, k), 71)
    b, bv = bf16_operand(oracle, (k, n) if tb else (n, k), 72, std=0.1)
    plain = torch.empty((m, n), dtype=torch.float32, device="cuda")
    gemm.gemm(a, b, plain, transposed_b=tb, split_k=1, flags=_flags(pkg, cg))
    out = torch.full((m, n), 3.0, dtype=torch.float32, device="cuda")
    copy = torch.full((m + 8, n), 5.0, dtype=torch.bfloat16, device="cuda")     # canary rows at the end
    gemm.f32_store_with_bf16_copy(a, b, out, copy[:m], transposed_b=tb, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    assert torch.equal(out, plain)                               # the fp32 half is the plain store
    assert torch.equal(copy[:m], plain.to(torch.bfloat16))       # the copy is its nearest-even rounding
    assert torch.all(copy[m:] == 5.0).item()
    w = bv if tb else bv.T
    assert_gemm_close(out.cpu().numpy(), oracle.matmul(av, np.ascontiguousarray(w), THREADS), "dual fp32",
                      rel_fro=2e-5, elem=2e-4)
    with pytest.raises(pkg.B200GemmError):                       # an fp32 store only
        gemm.f32_store_with_bf16_copy(a, b, out, copy[:m], transposed_b=tb, accumulate=True)


def test_f32_store_with_bf16_copy_batched(pkg, oracle, gemm):
    """The dual form over a batch ("experts"): both outputs strided per matrix."""
    import torch
    e, m, n, k = 3, 320, 256, 192
    a, _ = bf16_operand(oracle, (e, m, k), 73)
    b, _ = bf16_operand(oracle, (e, n, k), 74, std=0.1)
    plain = torch.empty((e, m, n), dtype=torch.float32, device="cuda")
    gemm.f32_store_batched(a, b, plain, split_k=1)
    out = torch.zeros((e, m, n), dtype=torch.float32, device="cuda")
    copy = torch.zeros((e, m, n), dtype=torch.bfloat16, device="cuda")
    gemm.f32_store_with_bf16_copy(a, b, out, copy)
    assert gemm.device_status() == 0
    assert torch.equal(out, plain) and torch.equal(copy, plain.to(torch.bfloat16))


# ---- gpu/gemm/src/bin/transpose_probe.rs:123-171: the four operand encodings of the layout
# ---- sweep (128 x 64 x 64), in every storage order of A and B ---------------------------

def _probe_operands(oracle, encoding):
    M, N, K = 128, 64, 64
    if encoding == "random":
        return oracle.uniform(M * K, 71).reshape(M, K), oracle.uniform(N * K, 72).reshape(N, K)
    a = np.zeros((M, K), np.float32)
    b = np.zeros((N, K), np.float32)
    if encoding == "outer":                      # C[m, n] = (m + 1)(n + 1)
        a[:, 0] = np.arange(1, M + 1)
        b[:, 0] = np.arange(1, N + 1)
    elif encoding == "a_walk":                   # C[m, n] = (m mod K) + 1
        a[np.arange(M), np.arange(M) % K] = 1.0
        b[:] = np.arange(1, K + 1)
    else:                                        # b_walk: C[m, n] = n + 1
        a[:] = np.arange(1, K + 1)
        b[np.arange(N), np.arange(N)] = 1.0
    return a, b


@pytest.mark.parametrize("cg", CTA_GROUPS, ids=["cg1", "cg2"])
@pytest.mark.parametrize("encoding", ["outer", "a_walk", "b_walk", "random"])
def test_transpose_probe_encodings_in_every_storage_order(pkg, oracle, gemm, cg, encoding):
    import torch
    a, b = _probe_operands(oracle, encoding)
    a_bits, b_bits = oracle.bf16_bits(a.reshape(-1)).reshape(a.shape), oracle.bf16_bits(b.reshape(-1)).reshape(b.shape)
    av, bv = oracle.bf16_to_f32(a_bits).reshape(a.shape), oracle.bf16_to_f32(b_bits).reshape(b.shape)
    expected = oracle.matmul_nt(av, bv, THREADS)
    if encoding == "outer":
        assert np.array_equal(expected, np.outer(np.arange(1, 129), np.arange(1, 65)))
    # the reference's tolerances (transpose_probe.rs:125-130): integers admit no slack
    atol, rtol = (0.02, 0.01) if encoding == "random" else (1e-3, 0.0)
    for ta in (False, True):
        for tb in (False, True):
            a_dev = to_dev_bf16(np.ascontiguousarray(a_bits.T) if ta else a_bits)
            b_dev = to_dev_bf16(np.ascontiguousarray(b_bits.T) if tb else b_bits)
            c = torch.full((128, 64), -1.0, dtype=torch.float32, device="cuda")
            gemm.gemm(a_dev, b_dev, c, transposed_a=ta, transposed_b=tb, flags=_flags(pkg, cg))
            got = c.cpu().numpy()
            assert np.all(np.abs(got - expected) <= atol + rtol * np.abs(expected)), (encoding, ta, tb)
    assert gemm.device_status() == 0


# ---- the weight-gradient methods the reference gates at 256^3 (gpu/gemm/src/main.rs:343-391,
# ---- 515-620; gpu/gemm/src/host.rs:837-1026), plus one ragged shape each -----------------

@pytest.mark.parametrize("cg", CTA_GROUPS, ids=["cg1", "cg2"])
@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (200, 328, 456)])
def test_bf16_accumulate_transposed(pkg, oracle, gemm, cg, m, n, k):
    """``accumulate_transposed`` (host.rs:875-900): bf16 ``C += A^T.B``, both operands MN-major --
    the reference's lm-head weight-gradient form (gpu/model/src/lib.rs:3103-3123)."""
    a, av = bf16_operand(oracle, (k, m), 81)
    b, bv = bf16_operand(oracle, (k, n), 82, std=0.05)
    c0, c0v = bf16_operand(oracle, (m + 8, n), 83)                  # canary rows at the end
    ref = oracle.matmul_tn(av, bv, THREADS)
    gemm.accumulate_transposed(a, b, c0[:m], flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    got = from_dev_bf16(c0)
    assert np.array_equal(got[m:], c0v[m:])
    # one rounding of (old + product): half a bf16 ulp of the sum
    assert_gemm_close(got[:m], c0v[:m] + ref, "bf16 accumulate_transposed", rel_fro=4e-3, elem=8e-3)


@pytest.mark.parametrize("cg", CTA_GROUPS, ids=["cg1", "cg2"])
@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (192, 264, 328)])
def test_f32_accumulate_transposed_batched(pkg, oracle, gemm, cg, m, n, k):
    """``f32_accumulate_transposed_batched`` (host.rs:997-1026): the reference's expert
    weight-gradient form, one launch over the experts' capacity bins."""
    import torch
    E = 3
    a, av = bf16_operand(oracle, (E, k, m), 84)
    b, bv = bf16_operand(oracle, (E, k, n), 85, std=0.05)
    c0 = oracle.normal(E * m * n, 86).reshape(E, m, n)
    ref = np.stack([oracle.matmul_tn(av[e], bv[e], THREADS) for e in range(E)])
    c = torch.from_numpy(c0).cuda()
    gemm.f32_accumulate_transposed_batched(a, b, c, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    assert_gemm_close(c.cpu().numpy(), c0 + ref, "f32_accumulate_transposed_batched", rel_fro=2e-5, elem=2e-4)
    # dead capacity rows (zero-filled bins, gpu/model/src/lib.rs:1717-1748) add exactly nothing
    a2 = a.clone()
    a2[:, k // 2:] = 0
    c2 = torch.zeros((E, m, n), dtype=torch.float32, device="cuda")
    gemm.f32_accumulate_transposed_batched(a2, b, c2, flags=_flags(pkg, cg))
    half = np.stack([oracle.matmul_tn(av[e][:k // 2], bv[e][:k // 2], THREADS) for e in range(E)])
    assert_gemm_close(c2.cpu().numpy(), half, "dead bin rows", rel_fro=2e-5, elem=2e-4)


@pytest.mark.parametrize("cg", CTA_GROUPS, ids=["cg1", "cg2"])
def test_f32_accumulate_at_forms(pkg, oracle, gemm, cg):
    """``f32_accumulate_at`` (host.rs:837-864) and ``f32_accumulate_transposed_at`` (host.rs:914-941):
    add into a region of a larger buffer; the neighbours keep their values."""
    import torch
    M, N, K = 256, 256, 192
    a, av = bf16_operand(oracle, (M, K), 87)
    b, bv = bf16_operand(oracle, (N, K), 88, std=0.05)
    base = oracle.normal(3 * M * N, 89).astype(np.float32)
    buf = torch.from_numpy(base.copy()).cuda()
    gemm.f32_accumulate_at(a, b, buf, M * N, M * N, N, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    host = buf.cpu().numpy()
    assert np.array_equal(host[:M * N], base[:M * N]) and np.array_equal(host[2 * M * N:], base[2 * M * N:])
    ref = oracle.matmul_nt(av, bv, THREADS)
    assert_gemm_close(host[M * N:2 * M * N].reshape(M, N), base[M * N:2 * M * N].reshape(M, N) + ref,
                      "f32_accumulate_at", rel_fro=2e-5, elem=2e-4)
    at, atv = bf16_operand(oracle, (K, M), 90)
    bt, btv = bf16_operand(oracle, (K, N), 91, std=0.05)
    buf = torch.from_numpy(base.copy()).cuda()
    gemm.f32_accumulate_transposed_at(at, bt, buf, 2 * M * N, M * N, N, flags=_flags(pkg, cg))
    assert gemm.device_status() == 0
    host = buf.cpu().numpy()
    assert np.array_equal(host[:2 * M * N], base[:2 * M * N])
    assert_gemm_close(host[2 * M * N:].reshape(M, N), base[2 * M * N:].reshape(M, N) + oracle.matmul_tn(atv, btv, THREADS),
                      "f32_accumulate_transposed_at", rel_fro=2e-5, elem=2e-4)


def test_host_buffer_form_leaves_the_callers_padding_alone(pkg, oracle, gemm):
    """b200gemm_gemm_host with C a column slice of a wider host matrix (ldc > n) and A, B with
    padded rows: only the matrices' own elements are read or written; the canary columns of
    the caller's buffers survive, in store and in accumulate mode."""
    import ctypes as C
    L = pkg._lib
    M, N, K, LDA, LDB, LDC = 200, 136, 72, 96, 80, 3 * 136
    a_full = np.full((M, LDA), 0x7FC0, np.uint16)                       # NaN canaries in the padding
    b_full = np.full((N, LDB), 0x7FC0, np.uint16)
    av = oracle.bf16_round(oracle.uniform(M * K, 92)).reshape(M, K)
    bv = oracle.bf16_round(oracle.uniform(N * K, 93)).reshape(N, K)
    a_full[:, :K] = oracle.bf16_bits(av).reshape(M, K)
    b_full[:, :K] = oracle.bf16_bits(bv).reshape(N, K)
    # The last row is shortened to its K real elements: reading a whole padded row there would run off the buffer.
    a_buf = np.ascontiguousarray(a_full.reshape(-1)[: (M - 1) * LDA + K])
    b_buf = np.ascontiguousarray(b_full.reshape(-1)[: (N - 1) * LDB + K])
    wide = np.full((M, LDC), -7.0, np.float32)
    d = L.GemmDesc()
    d.a, d.b = a_buf.ctypes.data, b_buf.ctypes.data
    d.c = wide.ctypes.data + N * 4                                        # the middle column block
    d.m, d.n, d.k, d.lda, d.ldb, d.ldc = M, N, K, LDA, LDB, LDC
    d.out_type, d.mode, d.batch = L.OUT_F32, L.STORE, 1
    L.check(gemm._lib.b200gemm_gemm_host(gemm._h, None, C.byref(d)))
    ref = oracle.matmul_nt(av, bv, THREADS)
    assert np.all(wide[:, :N] == -7.0) and np.all(wide[:, 2 * N:] == -7.0)
    assert_gemm_close(wide[:, N:2 * N], ref, "host store into a column slice", rel_fro=2e-5, elem=2e-4)
    d.mode = L.ACCUMULATE
    L.check(gemm._lib.b200gemm_gemm_host(gemm._h, None, C.byref(d)))
    assert np.all(wide[:, :N] == -7.0) and np.all(wide[:, 2 * N:] == -7.0)
    assert_gemm_close(wide[:, N:2 * N], 2 * ref, "host accumulate into a column slice", rel_fro=2e-5, elem=2e-4)
    assert gemm.device_status() == 0


# ---- 256 x 512 tiles per CTA pair (one 512-column accumulator, two UMMAs per K step): chosen by
# ---- the planner for deep reductions, forced here on small shapes of every kind ------------

@pytest.mark.parametrize("ta,tb", [(False, False), (True, True), (False, True), (True, False)])
@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (512, 1024, 192), (200, 840, 328), (256, 264, 64)])
def test_wide_tiles_match_the_oracle(pkg, oracle, gemm, ta, tb, m, n, k):
    import torch
    wide = pkg._lib.FLAG_WIDE_TILE
    a, av = bf16_operand(oracle, (k, m) if ta else (m, k), 95, kind="uniform")
    b, bv = bf16_operand(oracle, (k, n) if tb else (n, k), 96, kind="uniform")
    A = np.ascontiguousarray(av.T if ta else av)
    Bt = np.ascontiguousarray(bv if tb else bv.T)
    ref = oracle.matmul(A, Bt, THREADS)
    c = torch.full((m + 8, n), 5.0, dtype=torch.float32, device="cuda")          # canary rows
    gemm.gemm(a, b, c[:m], transposed_a=ta, transposed_b=tb, flags=wide)
    assert gemm.device_status() == 0
    host = c.cpu().numpy()
    assert np.all(host[m:] == 5.0)
    assert_gemm_close(host[:m], ref, f"wide store ta={ta} tb={tb}", rel_fro=2e-5, elem=2e-4)
    narrow = torch.empty((m, n), dtype=torch.float32, device="cuda")
    gemm.gemm(a, b, narrow, transposed_a=ta, transposed_b=tb, flags=pkg._lib.FLAG_NARROW_TILE | pkg._lib.FLAG_CTA_GROUP_2, split_k=1)
    assert torch.equal(c[:m], narrow)            # the same products added in the same order: bit-identical
    gemm.gemm(a, b, c[:m], transposed_a=ta, transposed_b=tb, accumulate=True, flags=wide)
    assert_gemm_close(c[:m].cpu().numpy(), 2 * ref, "wide accumulate", rel_fro=2e-5, elem=2e-4)
    assert gemm.device_status() == 0


def test_wide_tiles_are_chosen_for_deep_reductions_and_split_k(pkg, oracle, gemm):
    """The planner picks wide tiles for the MLP's weight gradient over 32768 tokens (K slices deep
    enough that the unoverlapped drain does not matter) and keeps the 256-wide ones for a forward;
    wide tiles with K split four ways, many items per CTA pair, are exact on integer operands."""
    import torch
    L = pkg._lib
    x = torch.empty((32768, 4096), dtype=torch.bfloat16, device="cuda")
    dy = torch.empty((32768, 1536), dtype=torch.bfloat16, device="cuda")
    dw = torch.empty((4096, 1536), dtype=torch.float32, device="cuda")
    kw = dict(transposed_a=True, transposed_b=True, accumulate=True)
    chosen = gemm.launch_config(x, dy, dw, **kw)
    assert chosen == gemm.launch_config(x, dy, dw, flags=L.FLAG_WIDE_TILE, **kw)          # wide by itself
    assert chosen["smem_bytes"] != gemm.launch_config(x, dy, dw, flags=L.FLAG_NARROW_TILE, **kw)["smem_bytes"]
    y = torch.empty((32768, 1536), dtype=torch.float32, device="cuda")
    w = torch.empty((4096, 1536), dtype=torch.bfloat16, device="cuda")
    assert gemm.launch_config(x, w, y, transposed_b=True) == gemm.launch_config(x, w, y, transposed_b=True,
                                                                                 flags=L.FLAG_NARROW_TILE)
    del x, dy, dw, y, w
    m, n, k = 512, 1024, 16384
    i, j = np.meshgrid(np.arange(k), np.arange(m), indexing="ij")
    av = (((i * 5 + j * 3) % 7) - 3).astype(np.float32)
    i, j = np.meshgrid(np.arange(k), np.arange(n), indexing="ij")
    bv = (((i * 4 + j * 5) % 5) - 2).astype(np.float32)
    a, b = to_dev_bf16(oracle.bf16_bits(av)), to_dev_bf16(oracle.bf16_bits(bv))
    c = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    gemm.f32_accumulate_transposed(a, b, c, flags=L.FLAG_WIDE_TILE, split_k=4)
    assert gemm.device_status() == 0
    want = av.astype(np.int64).T @ bv.astype(np.int64)
    assert np.array_equal(c.cpu().numpy(), want.astype(np.float32))
    with pytest.raises(pkg.B200GemmError):                      # bf16 output has no wide form
        gemm.gemm(a, b, torch.zeros((m, n), dtype=torch.bfloat16, device="cuda"), transposed_a=True,
                  transposed_b=True, flags=L.FLAG_WIDE_TILE)
