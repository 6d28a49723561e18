"""Pins the CPU oracle to the reference's own known-answer tests.

Each test names the reference test it restates (path:line inside the reference
project).  Data that the reference derives from its RNG is derived here from
the restated RNG, which the splitmix tests below pin first.
"""
import numpy as np
import pytest


# ---- crates/tensor-core/src/rng.rs:67-87 -----------------------------------

def test_splitmix_stateless_mixer_is_the_generator_step(oracle):
    import ctypes as C
    gamma = 0x9E3779B97F4A7C15
    state = C.c_uint64(7)
    first = oracle.lib().orc_rng_next_u64(C.byref(state))
    assert first == oracle.splitmix64((7 + gamma) % 2**64)


def test_splitmix64_published_vector(oracle):
    # splitmix64 seeded with 0: the generator's widely published first outputs
    # (Vigna's reference implementation), which rng.rs:18-23,51-54 restates.
    import ctypes as C
    state = C.c_uint64(0)
    outs = [oracle.lib().orc_rng_next_u64(C.byref(state)) for _ in range(3)]
    assert outs == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]


def test_uniform_draws_are_24_bit_and_in_range(oracle):
    u = oracle.uniform(4096, 3)
    assert u.min() >= -1.0 and u.max() < 1.0
    # top-24-bit scheme: (u + 1) / 2 * 2^24 is an integer
    scaled = (u.astype(np.float64) + 1.0) * (1 << 23)
    assert np.all(scaled == np.round(scaled))
    assert np.array_equal(u, oracle.uniform(4096, 3))
    assert not np.array_equal(u, oracle.uniform(4096, 4))


# ---- crates/tensor-core/src/element.rs:72-81 -------------------------------

def test_bf16_round_to_nearest_even(oracle):
    L = oracle.lib()
    assert L.orc_bf16_from_f32(1.0) == 0x3F80
    assert oracle.bf16_round(np.array([-2.5], np.float32))[0] == -2.5
    halfway = np.array([0x3F808000], np.uint32).view(np.float32)
    assert oracle.bf16_bits(halfway)[0] == 0x3F80          # tie -> even (down)
    halfway_odd = np.array([0x3F818000], np.uint32).view(np.float32)
    assert oracle.bf16_bits(halfway_odd)[0] == 0x3F82      # tie -> even (up)
    above = np.array([0x3F808001], np.uint32).view(np.float32)
    assert oracle.bf16_bits(above)[0] == 0x3F81


def test_bf16_matches_torch_rounding(oracle):
    import torch
    x = oracle.normal(1 << 16, 11, 0.0, 3.0)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.bf16_bits(x), want)


def test_bf16_stochastic(oracle):
    # element.rs:15-17: add the low 16 entropy bits, truncate.
    L = oracle.lib()
    one = np.float32(1.0)
    assert L.orc_bf16_stochastic(one, 0) == 0x3F80
    assert L.orc_bf16_stochastic(np.float32(1.00390625 / 2 + 0.5), 0xFFFF) in (0x3F80, 0x3F81)
    v = np.array([0x3F808000], np.uint32).view(np.float32)[0]
    assert L.orc_bf16_stochastic(v, 0x7FFF) == 0x3F80
    assert L.orc_bf16_stochastic(v, 0x8000) == 0x3F81


# ---- crates/tensor-cpu/src/ops.rs:187-226 ----------------------------------

def test_matmul_known_values(oracle):
    a = np.array([[1, 2], [3, 4]], np.float32)
    b = np.array([[5, 6], [7, 8]], np.float32)
    assert np.array_equal(oracle.matmul(a, b), np.array([[19, 22], [43, 50]], np.float32))


def test_matmul_rectangular_shapes_compose(oracle):
    a = oracle.uniform(15, 1).reshape(3, 5)
    b = oracle.uniform(20, 2).reshape(5, 4)
    assert oracle.matmul(a, b).shape == (3, 4)


def test_fused_transposed_matmuls_match_explicit_transpose(oracle):
    a = oracle.uniform(12, 1).reshape(4, 3)
    b = oracle.uniform(20, 2).reshape(4, 5)
    fused = oracle.matmul_tn(a, b)
    explicit = oracle.matmul(oracle.transpose(a), b)
    assert np.all(np.abs(fused - explicit) < 1e-6)
    c = oracle.uniform(15, 3).reshape(5, 3)
    fused = oracle.matmul_nt(a, c)
    explicit = oracle.matmul(a, oracle.transpose(c))
    assert np.all(np.abs(fused - explicit) < 1e-6)


def test_matmul_accumulation_order_is_ascending_k_without_fma(oracle):
    # Values chosen so that (a) a fused multiply-add and (b) a different
    # summation order would each change the f32 result.
    rng = np.random.default_rng(0)
    a = (rng.standard_normal((5, 97)) * 1e3).astype(np.float32)
    b = rng.standard_normal((97, 7)).astype(np.float32)
    want = np.zeros((5, 7), np.float32)
    for k in range(97):
        want = (want + (a[:, k:k + 1] * b[k:k + 1, :]).astype(np.float32)).astype(np.float32)
    assert np.array_equal(oracle.matmul(a, b), want)
    assert np.array_equal(oracle.matmul_nt(a, np.ascontiguousarray(b.T)), want)
    assert np.array_equal(oracle.matmul_tn(np.ascontiguousarray(a.T), b), want)


@pytest.mark.parametrize("threads", [2, 5])
def test_threaded_matmuls_are_bit_identical(oracle, threads):
    a = oracle.uniform(37 * 53, 5).reshape(37, 53)
    b = oracle.uniform(53 * 29, 6).reshape(53, 29)
    assert np.array_equal(oracle.matmul(a, b, 1), oracle.matmul(a, b, threads))
    bt = np.ascontiguousarray(b.T)
    assert np.array_equal(oracle.matmul_nt(a, bt, 1), oracle.matmul_nt(a, bt, threads))
    d = oracle.uniform(37 * 11, 7).reshape(37, 11)
    assert np.array_equal(oracle.matmul_tn(a, d, 1), oracle.matmul_tn(a, d, threads))
    rows = np.array([0, 36, 5, 5])
    assert np.array_equal(oracle.matmul_rows(a, b, rows, threads), oracle.matmul(a, b)[rows])


def test_integer_periodic_operands_give_the_7x21_table(oracle):
    # gpu/gemm/src/main.rs:266-335: small integers make every partial sum exact
    # in f32, so C is a 7x21 table whatever order the products are added in.
    K, M, N = 256, 35, 63
    i, d = np.meshgrid(np.arange(M), np.arange(K), indexing="ij")
    a = (((i * 5 + d * 3) % 7) - 3).astype(np.float32)
    j, d = np.meshgrid(np.arange(N), np.arange(K), indexing="ij")
    b = (((j * 4 + d * 5) % 21) - 10).astype(np.float32)
    c = oracle.matmul_nt(a, b)
    exact = a.astype(np.int64) @ b.astype(np.int64).T
    assert np.array_equal(c, exact.astype(np.float32))
    for r in range(M):
        for col in range(N):
            assert c[r, col] == c[r % 7, col % 21]


# ---- crates/tensor-cpu/src/ops.rs:228-239, crates/nn/src/cross_entropy.rs ---

def test_softmax_rows_are_distributions(oracle):
    x = oracle.uniform(6 * 17, 7).reshape(6, 17)
    s = oracle.softmax_rows(x)
    assert np.all(np.abs(s.sum(axis=1) - 1.0) < 1e-5)
    assert np.all(s > 0)


def test_cross_entropy_matches_f64_definition_and_masks_padding(oracle):
    n, classes, ld = 9, 13, 16
    logits = oracle.uniform(n * ld, 21).reshape(n, ld) * 4
    targets = (np.arange(n) * 5) % classes
    loss, probs, row_loss = oracle.xent_forward(logits, targets, classes)
    z = logits[:, :classes].astype(np.float64)
    lse = np.log(np.exp(z - z.max(1, keepdims=True)).sum(1)) + z.max(1)
    want = (lse - z[np.arange(n), targets]).mean()
    assert abs(float(loss) - want) < 1e-6
    assert np.all(probs[:, classes:] == 0)
    d = oracle.xent_backward(probs, targets, classes)
    assert np.all(d[:, classes:] == 0)               # gpu/ops/src/main.rs:2103
    assert np.all(np.abs(d.sum(axis=1)) < 1e-6)       # rows of p - onehot sum to 0
    onehot = np.zeros((n, ld), np.float32)
    onehot[np.arange(n), targets] = 1
    assert np.allclose(d, (probs - onehot) / n, atol=1e-7)


def test_cross_entropy_is_stable_for_large_logits(oracle):
    logits = np.array([[1000.0, 999.0, -1000.0]], np.float32)
    loss, probs, _ = oracle.xent_forward(logits, np.array([0]))
    assert np.isfinite(loss) and abs(float(loss) - np.log1p(np.exp(-1.0))) < 1e-6


# ---- crates/nn/tests/moe.rs:182-197, gpu/ops/src/main.rs:1260-1283 ----------

def test_routing_ties_choose_lower_expert_indices(oracle):
    # MoeFfn<N=3, D=2, FF=3, E=3, K=2, C=2> with a zero router: all
    # probabilities are 1/3, so every token picks experts 0 and 1.
    probs = oracle.softmax_rows(np.zeros((3, 3), np.float32))
    r = oracle.moe_route(probs, top_k=2, capacity=2)
    assert r["selected"].tolist() == [0, 1, 0, 1, 0, 1]
    D = oracle.DROPPED
    assert r["slots"].tolist() == [0, 0, 1, 1, D, D]
    assert r["gates"].tolist() == [0.5] * 6
    assert r["assignment_counts"].tolist() == [3, 3, 0]
    assert r["accepted_counts"].tolist() == [2, 2, 0]
    assert r["offsets"].tolist() == [0, 2, 4, 4]
    assert r["dest_row"].tolist() == [0, 2, 1, 3, D, D]


def test_routing_matches_a_sort_based_restatement(oracle):
    N, E, K = 257, 16, 4
    probs = oracle.softmax_rows(oracle.normal(N * E, 5).reshape(N, E))
    probs[7] = probs[7, 0]                       # a full tie row
    probs[9, 3] = probs[9, 11]                   # a pair tie
    r = oracle.moe_route(probs, K, capacity=N * K)
    sel = r["selected"].reshape(N, K)
    for t in range(N):
        order = sorted(range(E), key=lambda e: (-float(probs[t, e]), e))
        assert sel[t].tolist() == order[:K]
    counts = np.bincount(sel.ravel(), minlength=E)
    assert r["assignment_counts"].tolist() == counts.tolist()
    assert r["accepted_counts"].tolist() == counts.tolist()
    # slot = arrival order within the expert in flattened (token, rank) order
    seen = np.zeros(E, np.int64)
    for p, e in enumerate(sel.ravel()):
        assert r["slots"][p] == seen[e]
        seen[e] += 1
    # destination rows are a permutation of 0..N*K-1 when nothing is dropped
    assert sorted(r["dest_row"].tolist()) == list(range(N * K))
    g = r["gates"].reshape(N, K)
    assert np.allclose(g.sum(axis=1), 1.0, atol=1e-6)


def test_routing_drops_beyond_capacity(oracle):
    # gpu/ops/src/main.rs:935-937 routes token t to experts (t % E, (t+1) % E);
    # with capacity below the load, late arrivals are dropped.
    N, E, K, Cap = 50, 5, 2, 7
    probs = np.full((N, E), 0.01, np.float32)
    for t in range(N):
        probs[t, t % E] = 0.6
        probs[t, (t + 1) % E] = 0.3
    r = oracle.moe_route(probs, K, Cap)
    assert r["assignment_counts"].tolist() == [20] * E
    assert r["accepted_counts"].tolist() == [Cap] * E
    assert int((r["slots"] == oracle.DROPPED).sum()) == N * K - E * Cap


def test_silu_matches_definition(oracle):
    g = oracle.uniform(64, 9) * 6
    want = g / (1 + np.exp(-g.astype(np.float64)))
    assert np.allclose(oracle.silu(g), want, atol=1e-6)
    assert np.allclose(oracle.swiglu(g, g), want * g, atol=1e-5)
