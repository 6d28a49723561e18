"""The benchmark driver's host side, without a GPU: the workload's arithmetic, the reference arm's
JSON line (the CPU restatement timed on a small sample), and the clock sampler's fall-back."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import bench
    return bench


def test_step_flops_is_the_sum_of_the_step_s_gemms():
    b = _bench()
    m, d, ff, layers, v = b.M_TOKENS, b.D_MODEL, b.D_FF, b.N_LAYERS, b.VOCAB_PAD
    per_layer = 2.0 * m * (d * 3 * d + d * d + d * ff + ff * d)          # the four projections, forward
    want = 3 * per_layer * layers + 3 * 2.0 * m * d * v                   # x3: forward, input and weight gradient
    assert b.step_flops() == want
    assert abs(b.step_flops() / 1e12 - 67.18) < 0.01                      # the figure the bench line is quoted on
    assert b.step_flops(m // 2) * 2 == b.step_flops()


def test_cpu_sample_counts_the_flops_it_times():
    b = _bench()
    secs, flops, text = b.cpu_sample(1, rows=4, k_tokens=8)
    want = sum(2.0 * 4 * i * o * 2 + 2.0 * 8 * i * o for _, i, o in b.PROJECTIONS)
    assert flops == want and secs > 0
    assert "4 token rows" in text and "8 tokens" in text


def test_reference_arm_prints_the_contract_s_line():
    """`bench.py --impl reference` on a reduced sample (the full one is ~10 s per step and core)."""
    code = ("import sys; sys.argv=['bench.py']; import bench, types\n"
            "orig = bench.cpu_sample\n"
            "bench.cpu_sample = lambda threads, rows=None, k_tokens=None: orig(threads, rows or 8, k_tokens or 16)\n"
            "bench.run_reference(types.SimpleNamespace(gpus=1, steps=2, warmup=1))\n")
    env = dict(os.environ, RANK="0")
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and line["metric"] == "bf16_gemm_tflops_full_step"
    assert line["unit"] == "TFLOP/s" and line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["value"] > 0 and line["steps"] == 2 and line["warmup"] == 1
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert "workload" in line["config"]
    # every other rank leaves without work and without output
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=dict(os.environ, RANK="1"),
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_clock_sampler_survives_a_box_without_a_gpu():
    b = _bench()
    s = b.ClockSampler(0)
    s.start()
    got = s.stop()
    assert set(got) >= {"sm_mhz", "sm_max_mhz", "reasons", "samples", "source"}
    assert got["source"] in ("NVML", "nvidia-smi")
    assert isinstance(got["reasons"], list)
