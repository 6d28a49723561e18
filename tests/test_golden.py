"""The committed golden vectors (tests/golden/reference_kats.json: known answers
transcribed from the reference's own tests) against the oracle on CPU and, on a
GPU, against the CUDA path through the C ABI."""
import json
import os

import numpy as np
import pytest

GOLD = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kats.json")))


def test_oracle_matches_matmul_golden(oracle):
    g = GOLD["matmul_known_values"]
    assert oracle.matmul(np.array(g["a"], np.float32), np.array(g["b"], np.float32)).tolist() == g["c"]


def test_oracle_matches_bf16_golden(oracle):
    for case in GOLD["bf16_round_to_nearest_even"]["cases"]:
        x = np.array([case["f32_bits"]], np.uint32).view(np.float32)
        assert int(oracle.bf16_bits(x)[0]) == case["bf16_bits"]


def test_oracle_matches_splitmix_golden(oracle):
    import ctypes as C
    g = GOLD["splitmix_step"]
    state = C.c_uint64(g["seed"])
    assert oracle.lib().orc_rng_next_u64(C.byref(state)) == oracle.splitmix64((g["seed"] + g["gamma"]) % 2**64)


def test_oracle_matches_routing_golden(oracle):
    g = GOLD["routing_ties"]
    probs = oracle.softmax_rows(np.zeros((g["tokens"], g["experts"]), np.float32))
    r = oracle.moe_route(probs, g["top_k"], g["capacity"])
    assert r["selected"].tolist() == g["selected_experts"]
    assert [None if s == oracle.DROPPED else int(s) for s in r["slots"]] == g["slots"]
    assert r["gates"].tolist() == g["gate_weights"]


def test_oracle_matches_periodic_table_golden(oracle):
    g = GOLD["periodic_gemm_table"]
    k = g["k"]
    i, d = np.meshgrid(np.arange(7), np.arange(k), indexing="ij")
    a = (((i * 5 + d * 3) % 7) - 3).astype(np.float32)
    j, d = np.meshgrid(np.arange(21), np.arange(k), indexing="ij")
    b = (((j * 4 + d * 5) % 21) - 10).astype(np.float32)
    assert oracle.matmul_nt(a, b).astype(np.int64).tolist() == g["table"]


@pytest.mark.gpu
def test_cuda_path_matches_goldens(pkg, oracle):
    import torch
    from _util import from_dev_bf16, to_dev_bf16
    gemm = pkg.Tcgen05Gemm()
    try:
        # periodic table on a shape that takes several work items per cluster
        g = GOLD["periodic_gemm_table"]
        m, n, k = 1792, 2688, g["k"]                     # multiples of 7*256 and 21*128
        i, d = np.meshgrid(np.arange(m), np.arange(k), indexing="ij")
        a = to_dev_bf16(oracle.bf16_bits((((i * 5 + d * 3) % 7) - 3).astype(np.float32)))
        j, d = np.meshgrid(np.arange(n), np.arange(k), indexing="ij")
        b = to_dev_bf16(oracle.bf16_bits((((j * 4 + d * 5) % 21) - 10).astype(np.float32)))
        c = torch.zeros((m, n), dtype=torch.float32, device="cuda")
        gemm.f32_store(a, b, c)
        table = np.array(g["table"], np.float32)
        want = np.tile(table, (m // 7, n // 21))
        assert np.array_equal(c.cpu().numpy(), want)
        # 2x2 known answer through the fp32 family
        kv = GOLD["matmul_known_values"]
        a2 = torch.tensor(kv["a"], dtype=torch.float32, device="cuda")
        b2 = torch.tensor(kv["b"], dtype=torch.float32, device="cuda")
        assert gemm.matmul(a2, b2).cpu().tolist() == kv["c"]
        # routing tie vector
        r = GOLD["routing_ties"]
        probs = torch.full((r["tokens"], r["experts"]), 1.0 / 3.0, dtype=torch.float32, device="cuda")
        probs = torch.from_numpy(oracle.softmax_rows(np.zeros((3, 3), np.float32))).cuda()
        routing = pkg.moe.route(gemm, probs, r["top_k"], r["capacity"])
        sel = routing.selected_experts.cpu().numpy().view(np.uint32).tolist()
        slots = routing.slots.cpu().numpy().view(np.uint32).tolist()
        assert sel == r["selected_experts"]
        assert [None if s == 0xFFFFFFFF else s for s in slots] == r["slots"]
        assert routing.gate_weights.cpu().tolist() == r["gate_weights"]
        # bf16 rounding of the staging convert
        for case in GOLD["bf16_round_to_nearest_even"]["cases"]:
            x = torch.from_numpy(np.array([case["f32_bits"]] * 8, np.uint32).view(np.float32).copy()).cuda()
            y = gemm.convert_f32_to_bf16(x)
            assert int(y.view(torch.int16).cpu().numpy().view(np.uint16)[0]) == case["bf16_bits"]
        assert gemm.device_status() == 0
    finally:
        gemm.close()
