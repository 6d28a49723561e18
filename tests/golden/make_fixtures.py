"""Writes ``reference_kats.json``: the known-answer vectors the reference's own
tests hold for the GEMM path, transcribed from its test sources (the reference
is Rust and cannot be run where this repository is built, so the values are
copied from the assertions, and the formula-defined operands are re-derived
from the formulas given there).  Each entry names the file:line it comes from.

    python tests/golden/make_fixtures.py
"""
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))


def periodic_table(k=256):
    # gpu/gemm/src/main.rs:266-274: a_value(row, depth) = ((row*5 + depth*3) % 7) - 3,
    # b_value(col, depth) = ((col*4 + depth*5) % 21) - 10; C is a 7 x 21 table of exact integers.
    a = [[((r * 5 + d * 3) % 7) - 3 for d in range(k)] for r in range(7)]
    b = [[((c * 4 + d * 5) % 21) - 10 for d in range(k)] for c in range(21)]
    return [[sum(a[r][d] * b[c][d] for d in range(k)) for c in range(21)] for r in range(7)]


def main():
    fixtures = {
        "matmul_known_values": {
            "source": "crates/tensor-cpu/src/ops.rs:194-199",
            "a": [[1, 2], [3, 4]], "b": [[5, 6], [7, 8]], "c": [[19, 22], [43, 50]],
        },
        "bf16_round_to_nearest_even": {
            "source": "crates/tensor-core/src/element.rs:72-81",
            "cases": [
                {"f32_bits": 0x3F800000, "bf16_bits": 0x3F80},   # 1.0
                {"f32_bits": 0xC0200000, "bf16_bits": 0xC020},   # -2.5 survives exactly
                {"f32_bits": 0x3F808000, "bf16_bits": 0x3F80},   # halfway, even mantissa: rounds down to 1.0
            ],
        },
        "splitmix_step": {
            "source": "crates/tensor-core/src/rng.rs:71-78",
            "seed": 7, "gamma": 0x9E3779B97F4A7C15,
            "statement": "SplitMix64::new(7).next_u64() == splitmix64(7 + gamma)",
        },
        "routing_ties": {
            "source": "crates/nn/tests/moe.rs:182-197; gpu/ops/src/main.rs:1260-1283",
            "tokens": 3, "experts": 3, "top_k": 2, "capacity": 2, "router": "all-zero weights",
            "selected_experts": [0, 1, 0, 1, 0, 1],
            "slots": [0, 0, 1, 1, None, None],
            "gate_weights": [0.5] * 6,
        },
        "periodic_gemm_table": {
            "source": "gpu/gemm/src/main.rs:180-335",
            "k": 256, "shapes": [[4096, 2560], [2816, 3584]],
            "statement": "C[row, col] == table[row % 7][col % 21], compared with == on bf16 words",
            "table": periodic_table(256),
        },
        "tolerances": {
            "tcgen05_vs_cpu": {"source": "gpu/gemm/src/main.rs:515-620", "atol": 0.03, "rtol": 0.01},
            "fp32_ladder": {"source": "gpu/gemm/src/main.rs:393-513", "tol": 2e-5, "shape": [73, 91, 47]},
            "classifier": {"source": "gpu/ops/src/main.rs:1984-2110", "loss": 5e-5, "dlogits_rel": 4e-3,
                           "padded_columns": "exactly zero"},
        },
    }
    with open(os.path.join(HERE, "reference_kats.json"), "w") as f:
        json.dump(fixtures, f, indent=1)
    print("wrote reference_kats.json")


if __name__ == "__main__":
    main()
