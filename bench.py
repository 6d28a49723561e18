#!/usr/bin/env python
"""Benchmark of the GEMM hot path: the full-step GEMM set of the ~183M dense model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (one "step"): every GEMM of one training step of the dense model
B=32, T=1024 (M=32768 tokens), D=1536, FF=4096, 12 layers, lm-head 1536->50432:
per layer the four forward projections (QKV, attention-out, MLP up, MLP down),
their four input gradients and their four weight gradients (K = 32768 tokens,
split-K), plus the lm-head fused with the softmax cross-entropy classifier (forward, and a
backward that recomputes the logits; the recompute is not credited as FLOPs).  Inputs are seeded synthetic tensors with the
shapes and value distributions the model has (activations ~N(0,1), weights
~N(0,0.02), upstream gradients ~N(0,1e-2)), bf16 operands, fp32 accumulation.

Prints ONE JSON line.  `value` is whole-job TFLOP/s with every operand resident
in HBM; `e2e` repeats the step with the token batch's activations copied from
pinned host memory and a result word read back inside the timed region.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# ---- the workload: the full-step GEMM set of the ~183M dense model --------------
M_TOKENS, D_MODEL, D_FF, N_LAYERS, VOCAB_PAD, VOCAB = 32768, 1536, 4096, 12, 50432, 50257
PROJECTIONS = [("qkv", D_MODEL, 3 * D_MODEL), ("attn_out", D_MODEL, D_MODEL),
               ("mlp_up", D_MODEL, D_FF), ("mlp_down", D_FF, D_MODEL)]


def step_flops(m=M_TOKENS) -> float:
    per_layer = sum(2.0 * m * i * o for _, i, o in PROJECTIONS) * 3
    return per_layer * N_LAYERS + 3 * 2.0 * m * D_MODEL * VOCAB_PAD


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"tflops": d.get("bf16_tflops_sustained"), "burst": d.get("bf16_tflops"),
                "hbm_gbs": d.get("hbm_gbs"), "source": "measured"}
    # Earlier measurement on the same pool, used only when the file is absent.
    return {"tflops": 1400.0, "burst": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


# ---- clocks ------------------------------------------------------------------

class ClockSampler(threading.Thread):
    """Polls the SM clock and the throttle reasons while the timed region runs.

    Reads them through NVML inside this process (initialised before the timed region starts)
    rather than by starting `nvidia-smi` every 100 ms, which attaches a new process to every
    GPU of the box each time.  `nvidia-smi` is the fallback when the NVML binding is missing."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    # nvmlClocksEventReason* bits
    REASONS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_flag = threading.Event()
        self._nvml, self._dev = None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            dev = None
            try:
                import torch
                uuid = str(torch.cuda.get_device_properties(index).uuid)
                dev = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(dev, pynvml.NVML_CLOCK_SM))
            self._nvml, self._dev = pynvml, dev
        except Exception:
            self._nvml = None

    def _read_nvml(self):
        n, dev = self._nvml, self._dev
        self.samples.append(float(n.nvmlDeviceGetClockInfo(dev, n.NVML_CLOCK_SM)))
        try:
            mask = n.nvmlDeviceGetCurrentClocksEventReasons(dev)
        except AttributeError:
            mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(dev)
        for name, bit in self.REASONS.items():
            if mask & bit:
                self.reasons.add(name)

    def _read_smi(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        out = subprocess.run(
            ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
             "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
        f = [x.strip() for x in out.strip().split(",")]
        self.samples.append(float(f[0]))
        self.max_mhz = float(f[1])
        for name, val in zip(names, f[2:6]):
            if val.lower().startswith("active"):
                self.reasons.add(name)

    def run(self):
        while not self._stop_flag.is_set():
            try:
                if self._nvml is not None:
                    self._read_nvml()
                else:
                    self._read_smi()
            except Exception:
                pass
            self._stop_flag.wait(0.02 if self._nvml is not None else 0.1)

    def stop(self):
        self._stop_flag.set()
        self.join(timeout=6)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s),
                "source": "NVML" if self._nvml is not None else "nvidia-smi"}


# ---- reference arm: the CPU restatement of the reference's matmul family ------

def cpu_sample(threads: int, rows: int | None = None, k_tokens: int | None = None):
    """Time the oracle's matmul family on a bounded sample of the workload.

    Forward and input-gradient shapes keep their full K and N but only `rows`
    token rows; weight-gradient shapes keep their full output but only
    `k_tokens` of the 32768-token reduction.  Returns (seconds, flops, text)."""
    from oracle import oracle as orc
    orc.build()
    # About 130 MFLOP per sampled row; measured at 4.8 GFLOP/s per host core of the GPU box, so
    # 384 rows per thread are about 10 s of scalar work.
    rows = min(8192, 384 * threads) if rows is None else rows
    k_tokens = rows if k_tokens is None else k_tokens
    flops, secs = 0.0, 0.0
    for _, i, o in PROJECTIONS:
        x = orc.bf16_round(orc.normal(rows * i, 1)).reshape(rows, i)
        w = orc.bf16_round(orc.normal(i * o, 2, 0.0, 0.02)).reshape(i, o)
        dy = orc.bf16_round(orc.normal(rows * o, 3, 0.0, 0.01)).reshape(rows, o)
        xs = orc.bf16_round(orc.normal(k_tokens * i, 4)).reshape(k_tokens, i)
        dys = orc.bf16_round(orc.normal(k_tokens * o, 5, 0.0, 0.01)).reshape(k_tokens, o)
        t0 = time.perf_counter()
        orc.matmul(x, w, threads)            # forward      y  = x W
        orc.matmul_nt(dy, w, threads)        # input grad   dx = dy W^T
        orc.matmul_tn(xs, dys, threads)      # weight grad  dW = x^T dy
        secs += time.perf_counter() - t0
        flops += 2.0 * rows * i * o * 2 + 2.0 * k_tokens * i * o
    text = (f"{rows} token rows of each forward/input-gradient GEMM (full K, N) and {k_tokens} "
            f"tokens of each weight-gradient reduction, all four projections")
    return secs, flops, text


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    for _ in range(args.warmup):
        cpu_sample(threads, rows=8, k_tokens=16)
    t, f = 0.0, 0.0
    text = ""
    for _ in range(args.steps):
        s, fl, text = cpu_sample(threads)
        t += s
        f += fl
    value = f / t / 1e12
    line = {
        "impl": "reference", "metric": "bf16_gemm_tflops_full_step", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_flops() / (value * 1e12) * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": text + "; ms_per_step is extrapolated from the sample's rate"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {"workload": "full-step GEMM set of the ~183M dense model (BASELINE configs[1]): "
                        "B=32 T=1024 M=32768 D=1536 FF=4096 L=12, lm-head 1536->50432; "
                        "forward + input-gradient + weight-gradient layouts",
            "m_tokens": M_TOKENS, "d_model": D_MODEL, "d_ff": D_FF, "layers": N_LAYERS,
            "vocab_padded": VOCAB_PAD,
            "parallelism": f"replicas x{n_gpus} (one token batch per GPU, no data-path collective); the paths "
                           "that do shard -- fused head, tensor-parallel MLP, expert-parallel MoE -- are "
                           "timed at this N in the line's `sharded` block",
            "l2": "no flush: one step touches about 8 GB of operands and outputs; the only operand shared by "
                  "successive launches (the 100.7 MB token activations, read by three of a layer's four forward "
                  "GEMMs) is followed by 201-604 MB of output writes that push most of it out of the 126 MB L2"}


# ---- the GPU arm ----------------------------------------------------------------

class StepBuffers:
    """All operands of one training step's GEMMs, resident in HBM."""

    def __init__(self, torch, device, seed=0):
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        bf, f32 = torch.bfloat16, torch.float32

        def rnd(shape, std):
            return (torch.randn(shape, generator=g, device=device, dtype=f32) * std).to(bf)

        self.layers = []
        for _ in range(N_LAYERS):
            layer = {}
            for name, i, o in PROJECTIONS:
                layer[name] = {
                    "w": rnd((i, o), 0.02),                                   # [IN, OUT], read in place
                    "dw": torch.zeros((i, o), device=device, dtype=f32),      # fp32 gradient accumulator
                }
            self.layers.append(layer)
        # Activations and gradients are workspaces shared by the layers, as in a
        # trainer; each is far larger than L2 on its own.
        self.x = {i: rnd((M_TOKENS, i), 1.0) for i in (D_MODEL, D_FF)}
        self.dy = {o: rnd((M_TOKENS, o), 0.01) for o in (D_MODEL, 3 * D_MODEL, D_FF)}
        self.y = {o: torch.empty((M_TOKENS, o), device=device, dtype=f32)
                  for o in (D_MODEL, 3 * D_MODEL, D_FF)}
        self.head_w = rnd((D_MODEL, VOCAB_PAD), 0.02)
        self.head_dw = torch.zeros((D_MODEL, VOCAB_PAD), device=device, dtype=f32)
        self.dlogits = torch.empty((M_TOKENS, VOCAB_PAD), device=device, dtype=bf)
        self.dh = torch.empty((M_TOKENS, D_MODEL), device=device, dtype=f32)
        self.targets = torch.randint(0, VOCAB, (M_TOKENS,), generator=g, device=device, dtype=torch.int32)
        self.loss = None


def run_step(gemm, head, buf):
    """One pass over the step's GEMMs.  Returns the number of kernel launches of this library."""
    n = 0
    for layer in buf.layers:                       # forward
        for name, i, o in PROJECTIONS:
            gemm.f32_store(buf.x[i], layer[name]["w"], buf.y[o], transposed_b=True)   # y = x W
            n += 1
    # lm-head fused with the classifier: the [tokens, vocab] logits never reach HBM.
    buf.loss, lse, _ = head.forward(buf.x[D_MODEL], buf.head_w, buf.targets)          # GEMM + merge kernel
    # backward: logits recomputed into bf16 dlogits, then dh = dlogits W^T and dW += h^T dlogits
    head.backward(buf.x[D_MODEL], buf.head_w, buf.targets, lse, dlogits=buf.dlogits, d_hidden=buf.dh,
                  d_weight=buf.head_dw, accumulate_dw=True)
    n += 5
    for layer in reversed(buf.layers):             # backward
        for name, i, o in reversed(PROJECTIONS):
            gemm.f32_accumulate_transposed(buf.x[i], buf.dy[o], layer[name]["dw"])   # dW += x^T dy
            gemm.f32_store(buf.dy[o], layer[name]["w"], buf.y[i])                     # dx = dy W^T
            n += 2
    return n


class CublasLtComparator:
    """cuBLASLt beside every row of the per-shape table, the way the reference builds its
    denominator (gpu/gemm/src/cublaslt.rs:55-61, 434-470; gpu/gemm/src/bin/model_shapes.rs:425-441):
    called directly, 32 MiB workspace, the heuristic's first algorithm, beta = 1 where the
    kernel adds into C, and its C compared with this library's before its time is believed.
    A separate shared library that only this column loads; never on the product path."""

    def __init__(self):
        path = os.path.join(ROOT, "oxide-train_b200", "comparator", "libcublaslt_compare.so")
        self.lib, self.session = None, C.c_void_p()
        if not os.path.exists(path):
            return
        lib = C.CDLL(path)
        lib.cmp_last_error.restype = C.c_char_p
        lib.cmp_create.argtypes = [C.POINTER(C.c_void_p)]
        lib.cmp_plan.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int,
                                 C.POINTER(C.c_void_p)]
        lib.cmp_run.argtypes = [C.c_void_p] * 6
        lib.cmp_plan_destroy.argtypes = [C.c_void_p]
        lib.cmp_destroy.argtypes = [C.c_void_p]
        if lib.cmp_create(C.byref(self.session)) == 0:
            self.lib = lib

    def plan(self, m, n, k, a_mn, b_mn, out_bf16, accumulate):
        plan = C.c_void_p()
        if self.lib is None or self.lib.cmp_plan(self.session, m, n, k, int(a_mn), int(b_mn), int(out_bf16),
                                                 int(accumulate), C.byref(plan)) != 0:
            return None
        return plan

    def run(self, plan, torch, a, b, c):
        rc = self.lib.cmp_run(self.session, plan, torch.cuda.current_stream().cuda_stream, a.data_ptr(),
                              b.data_ptr(), c.data_ptr())
        if rc != 0:
            raise RuntimeError(self.lib.cmp_last_error().decode())

    @staticmethod
    def agrees(torch, theirs, ours):
        """The reference's check (model_shapes.rs:485-510): |d| <= max(|theirs|, 1) / 32 for fp32
        results, 4/256 for bf16 ones -- loose, because the two sides add K in different orders;
        a transposed operand or a wrong stride is wrong by whole values."""
        tol = 1.0 / 32.0 if theirs.dtype == torch.float32 else 4.0 / 256.0
        t, o = theirs.float(), ours.float()
        return bool(((t - o).abs() <= tol * t.abs().clamp_min(1.0)).all().item())

    def close(self):
        if self.lib is not None:
            self.lib.cmp_destroy(self.session)
            self.lib = None


def per_shape_table(torch, gemm, head, buf, iters=3):
    """TFLOP/s of every distinct GEMM of the step, timed alone (reported, not the headline).

    The timed steps before it leave the GPU at its power-capped clock; a short pause lets the
    power controller recover, so that every row -- the first one too -- is a burst figure."""
    rows = []
    layer = buf.layers[0]
    torch.cuda.synchronize()
    time.sleep(1.0)

    def timed(fn, flops):
        fn()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / iters
        return ms, flops / ms / 1e9

    # Comparator column: the same products through cuBLASLt, same operands, same timing loop.
    f32 = torch.float32
    cmp = CublasLtComparator()

    def cublas(m, n, k, a, b, a_mn, b_mn, ours, flops, accumulate=False, out_dtype=f32):
        """TFLOP/s of cuBLASLt on one product, or None; `ours` = this library's C for the check
        (with `accumulate` the check runs on a zeroed C with beta = 1, which is the same sum)."""
        plan = cmp.plan(m, n, k, a_mn, b_mn, out_dtype != f32, accumulate)
        if plan is None:
            return None, None
        c = torch.zeros((m, n), device=a.device, dtype=out_dtype)
        cmp.run(plan, torch, a, b, c)
        ok = cmp.agrees(torch, c, ours) if ours is not None else None
        ms, tf = timed(lambda: cmp.run(plan, torch, a, b, c), flops)
        cmp.lib.cmp_plan_destroy(plan)
        del c
        return round(tf, 1), ok

    for name, i, o in PROJECTIONS:
        fl = 2.0 * M_TOKENS * i * o
        w, dw = layer[name]["w"], layer[name]["dw"]
        x, dy = buf.x[i], buf.dy[o]
        check = torch.zeros((i, o), device=x.device, dtype=f32)          # the weight gradient from zero, for the check
        gemm.f32_accumulate_transposed(x, dy, check)
        for kind, fn, ref in (
            ("forward", lambda: gemm.f32_store(x, w, buf.y[o], transposed_b=True),
             lambda: cublas(M_TOKENS, o, i, x, w, False, True, buf.y[o], fl)),
            ("input_grad", lambda: gemm.f32_store(dy, w, buf.y[i]),
             lambda: cublas(M_TOKENS, i, o, dy, w, False, False, buf.y[i], fl)),
            ("weight_grad", lambda: gemm.f32_accumulate_transposed(x, dy, dw),
             lambda: cublas(i, o, M_TOKENS, x, dy, True, True, check, fl, accumulate=True)),   # beta = 1, like the kernel
        ):
            ms, tf = timed(fn, fl)
            ctf, ok = ref()
            rows.append({"gemm": f"{name}.{kind}", "ms": round(ms, 4), "tflops": round(tf, 1),
                         "cublaslt_tflops": ctf, "cublaslt_agrees": ok})
        del check
    fl = 2.0 * M_TOKENS * D_MODEL * VOCAB_PAD
    lse = head.forward(buf.x[D_MODEL], buf.head_w, buf.targets)[1]
    h = buf.x[D_MODEL]

    ms, tf = timed(lambda: head.forward(h, buf.head_w, buf.targets), fl)
    # comparator: the logits product alone (bf16 logits written to HBM, no classifier)
    ctf, _ = cublas(M_TOKENS, VOCAB_PAD, D_MODEL, h, buf.head_w, False, True, None, fl, out_dtype=torch.bfloat16)
    rows.append({"gemm": "lm_head.fused_forward", "ms": round(ms, 4), "tflops": round(tf, 1),
                 "cublaslt_tflops": ctf, "cublaslt_agrees": None})
    # recompute + two gradient products; only the two products are credited.
    # comparator: the two products alone, on dlogits already in HBM (d_weight with beta = 1)
    ms, tf = timed(lambda: head.backward(h, buf.head_w, buf.targets, lse, dlogits=buf.dlogits, d_hidden=buf.dh,
                                         d_weight=buf.head_dw, accumulate_dw=True), 2 * fl)
    p1 = cmp.plan(M_TOKENS, D_MODEL, VOCAB_PAD, False, False, False, False)
    p2 = cmp.plan(D_MODEL, VOCAB_PAD, M_TOKENS, True, True, False, True)
    ctf = ok = None
    if p1 is not None and p2 is not None:
        cdh = torch.zeros_like(buf.dh)
        cdw = torch.zeros_like(buf.head_dw)

        def two_products():
            cmp.run(p1, torch, buf.dlogits, buf.head_w, cdh)
            cmp.run(p2, torch, h, buf.dlogits, cdw)

        two_products()
        ok = cmp.agrees(torch, cdh, buf.dh)
        ctf = round(timed(two_products, 2 * fl)[1], 1)
        del cdh, cdw
    rows.append({"gemm": "lm_head.fused_backward", "ms": round(ms, 4), "tflops": round(tf, 1),
                 "cublaslt_tflops": ctf, "cublaslt_agrees": ok})
    cmp.close()
    return rows



# ---- the sharded workloads: fused head, expert-parallel MoE, tensor-parallel MLP --------------

SHARDED = ("lmhead", "tp_mlp", "moe")
MLP_EXCHANGE = "copy"          # set from --mlp-exchange
HEAD_EXCHANGE = "copy"         # set from --head-exchange
MOE_PIECES = [6, 5, 3, 2]      # set from --moe-pieces: token slices of the expert-parallel step
MOE_RETURN = "pull"            # set from --moe-return
MOE_RESERVE = 24               # set from --moe-reserve-sms
MOE_CTAS = 48                  # set from --moe-exchange-ctas
MOE_BULK = True                # set from --moe-exchange-form
RANK_BARRIER = "kernel"        # set from --rank-barrier: how the copy / device exchanges order the ranks
MLP_PIECES = [1, 3, 4, 4, 3, 1]   # set from --mlp-pieces (several GPUs)


class Sharded:
    """One of the three configurations that shard over the GPUs of one box, ready to step."""


def build_sharded(workload, torch, pkg, gemm, ops, dev, rank, world):
    par = pkg.parallel
    gen = torch.Generator(device=dev)
    gen.manual_seed(1)                                    # replicated operands: same seed on every rank
    bf, f32 = torch.bfloat16, torch.float32
    w = Sharded()
    w.result, w.extra = {}, None

    def rnd(shape, std, g=gen):
        return (torch.randn(shape, generator=g, device=dev, dtype=f32) * std).to(bf)

    if workload == "lmhead":
        m, k, v, classes = M_TOKENS, D_MODEL, VOCAB_PAD, VOCAB
        # Several GPUs: the weight-gradient GEMM leaves 16-32 SMs to d_hidden's all-reduce, which
        # runs in a group limited to as many thread blocks, so the two overlap.
        # (the all-reduce takes about the same time whatever N is while the GEMM shrinks with N)
        if HEAD_EXCHANGE == "copy" or world == 1:
            # d_hidden's sum goes by copy-engine pushes into peer memory and a local sum: no SMs to
            # set aside for a collective's kernels; four stay free so that the sum kernel and the
            # barrier kernel start at once
            reserve = 0 if world == 1 else 4
            # each rank keeps its own m / N rows of the summed d_hidden (a reduce-scatter): what a
            # row-parallel layer below the head consumes; `d_hidden="all"` would gather them again
            head = par.VocabParallelHead(ops, classes, v, reserve_sms=reserve, exchange="copy",
                                         d_hidden="scatter" if world > 1 else "all", barrier=RANK_BARRIER)
        else:
            reserve = 32 if world >= 8 else 16
            head = par.VocabParallelHead(ops, classes, v, reserve_sms=reserve,
                                         group=par.nccl_group_with_cta_limit(reserve))
        hidden = rnd((m, k), 1.0)
        w_shard = rnd((k, head.c1 - head.c0), 0.02)
        targets = torch.randint(0, classes, (m,), generator=gen, device=dev, dtype=torch.int32)
        dw = torch.zeros((k, head.c1 - head.c0), device=dev, dtype=f32)

        def step():
            loss, lse, _ = head.forward(hidden, w_shard, targets)
            head.backward(hidden, w_shard, targets, lse, d_weight=dw, accumulate_dw=True)
            w.result["loss"] = loss
            return 8                     # forward GEMM + two merge kernels + mean; recompute, two products, widen

        w.flops = 3 * 2.0 * m * k * v
        w.title = ("fused lm-head + softmax cross-entropy: M=32768 K=1536 V=50432 (50257 classes), forward + "
                   "backward; the backward's logit recompute is not credited")
        w.par_text = (f"vocabulary split over {world} GPU(s); one all-gather of the shards' row max / sum-exp / "
                      f"target logit; d_hidden summed over the shards under the weight-gradient GEMM ({reserve} "
                      f"SMs left free), exchange: {HEAD_EXCHANGE if world > 1 else 'none'}"
                      + ("; every rank keeps its m / N rows of d_hidden (reduce-scatter)" if world > 1 else ""))
        w.host_in, w.scaling = hidden, "strong"
        w.compute_ops = ("head_forward_shard", "head_merge_shards", "head_dlogits", "head_dhidden_partial",
                         "head_dweight", "widen")
        w.exchange_ops = ("sum_parts", "peer_barrier")
    elif workload == "moe":
        # 32768 tokens PER GPU (weak scaling): expert parallelism serves data-parallel
        # token batches; the experts, not the tokens, are what is divided.
        n_tok, d, ff, experts, top_k = 32768 * world, 1536, 768, 64, 8
        n_local, e_local = n_tok // world, experts // world
        grank = torch.Generator(device=dev)
        grank.manual_seed(100 + rank)                     # each rank has its own tokens
        x = rnd((n_local, d), 1.0, grank)
        # Popularity rank r (Zipf bias 0.5*ln(1/r)) is dealt to the ranks in snake order, the
        # placement a deployment would choose: expert ids are arbitrary labels, and a
        # contiguous block of the hottest experts on one rank would triple its load.
        pop = torch.arange(experts)
        rnd_i, pos = pop // world, pop % world
        owner = torch.where(rnd_i % 2 == 0, pos, world - 1 - pos)
        expert_id = owner * e_local + rnd_i
        bias = torch.empty(experts, dtype=f32)
        bias[expert_id] = 0.5 * torch.log(1.0 / (pop.float() + 1.0))
        bias = bias.to(dev)
        logits = (torch.randn((n_local, experts), generator=grank, device=dev) + bias).contiguous()
        w_up = rnd((experts, d, ff), 0.02)[rank * e_local:(rank + 1) * e_local].contiguous()
        w_dn = rnd((experts, ff, d), 0.02)[rank * e_local:(rank + 1) * e_local].contiguous()
        ep = par.ExpertParallelMoe(ops, experts, top_k, w_up, w_dn, pieces=MOE_PIECES, exchange="device",
                                   return_path=MOE_RETURN, barrier=RANK_BARRIER)
        if MOE_RESERVE is not None:
            ep.reserve_sms = MOE_RESERVE
        ep.exchange_ctas, ep.exchange_bulk = MOE_CTAS, MOE_BULK

        def step():
            w.result["out"] = ep.forward(x, logits, scores_are_logits=True)
            return 9

        w.flops = 2.0 * n_tok * top_k * d * ff * 2
        w.title = ("MoE grouped expert GEMM: 32768 tokens per GPU, D=1536, E=64, top-8, expert FF=768, "
                   "up -> SiLU -> down, Zipf-skewed routing; routing, dispatch and combine included")
        how = ("bulk asynchronous copies through shared memory" if MOE_BULK and MOE_CTAS else "peer stores / peer loads")
        sync = ("this library's barrier kernel, which also gathers the counts" if RANK_BARRIER == "kernel"
                else "NCCL for the counts and the barriers")
        w.par_text = (f"experts split over {world} GPU(s), 32768 tokens on each; dispatch and combine by {how} over "
                      f"NVLink (symmetric memory, sizes never leave the device; {MOE_CTAS or 'two per SM'} blocks beside "
                      f"the GEMMs, which leave {ep.reserve_sms} SMs free), results returned by {MOE_RETURN}; {sync}; "
                      f"{MOE_PIECES} token slices as a pipeline")
        w.host_in, w.scaling, w.extra = x, "weak", ep
        w.compute_ops = ("route", "scatter", "combine", "combine_into", "grouped_indexed", "grouped_indexed_into",
                         "grouped_indexed_peer", "ep_plan", "ep_return_plan")
        w.exchange_ops = ("ep_push", "ep_pull_combine", "peer_barrier")
    else:
        m, d, ff = 65536, 4096, 16384
        cols = ff // world
        x = rnd((m, d), 1.0)
        w1 = rnd((d, cols), 0.015)
        w2 = rnd((cols, d), 0.015)
        # several GPUs: the row exchanges go by copy-engine pushes into peer memory (no SM taken
        # from the GEMMs), the parts are summed locally; `--mlp-exchange nccl` runs NCCL's instead
        how = MLP_EXCHANGE if world > 1 else "nccl"
        # rows go through in pieces; on several GPUs short pieces at both ends, because what no GEMM
        # covers is the exchange of the last piece (forward and backward) and the gather of the first
        pieces = 4 if world == 1 else MLP_PIECES
        mlp = par.TensorParallelMlp(ops, w1, w2, chunks=pieces, partial_dtype=bf, exchange=how, barrier=RANK_BARRIER)
        dy_local = rnd((m // world, d), 0.01)
        dw1 = torch.zeros((d, cols), device=dev, dtype=f32)
        dw2 = torch.zeros((cols, d), device=dev, dtype=f32)

        def step():
            w.result["out"] = mlp.forward(x)
            w.result["dx"] = mlp.backward(x, dy_local, dw1, dw2)
            return 6 * len(mlp.pieces(m))

        w.flops = 6 * 2.0 * m * d * ff
        w.title = ("tensor-parallel MLP block: M=65536 D=4096 FF=16384, column-parallel up, row-parallel down, "
                   "forward + input and weight gradients (K=65536 split-K)")
        w.par_text = (f"FF split over {world} GPU(s); reduce-scatter of the partial outputs, all-gather of dy and "
                      f"reduce-scatter of dx in the backward, each under the next row piece's GEMMs ({len(mlp.pieces(m))} pieces); "
                      f"exchange: {how}"
                      + (" (copy-engine pushes into peer memory + local sum)" if how == "copy" else ""))
        w.host_in, w.scaling = x, "strong"
        w.compute_ops = ("linear", "linear_weight_grad", "linear_input_grad", "linear_input_grad_into")
        w.exchange_ops = ("sum_parts", "peer_barrier")
    w.step = step
    if not hasattr(w, "exchange_ops"):
        w.exchange_ops = ()
    return w


def time_steps(torch, dist, step, steps, local, sample_clocks=True):
    """CUDA-event time of `steps` steps between barriers (ms per step, clocks)."""
    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    barrier()
    sampler = ClockSampler(local) if sample_clocks else None
    if sampler:
        sampler.start()
    s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    mallocs = torch.cuda.memory_stats().get("num_device_alloc", 0)
    s0.record()
    for _ in range(steps):
        step()
    e0.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    if clocks is not None:
        # a cudaMalloc inside the timed region (the caching allocator growing) would stall the stream
        clocks["cuda_mallocs_in_region"] = torch.cuda.memory_stats().get("num_device_alloc", 0) - mallocs
    return s0.elapsed_time(e0) / steps, clocks


def exchange_timeline(torch, dist, ops, w, spans_too=False):
    """More steps with CUDA events around every collective and every compute call (this rank),
    the middle one of three back-to-back steps analysed: how long each collective took and how
    much of that no GEMM of this rank covered.
    The events sit on whichever stream the call was issued on; an exposed millisecond is one
    during which a collective (or the expert exchange's push / pull kernels) ran and none of the
    compute calls did."""
    marks = []
    restore = []

    def wrap(obj, name, kind):
        fn = getattr(obj, name, None)
        if fn is None:
            return

        def wrapped(*a, **k):
            s, t = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            r = fn(*a, **k)
            t.record()
            nbytes = 0
            if kind == "collective":
                big = max((x for x in a if hasattr(x, "numel")), key=lambda x: x.numel(), default=None)
                nbytes = big.numel() * big.element_size() if big is not None else 0
            marks.append((name, kind, s, t, nbytes))
            return r

        restore.append((obj, name, fn))
        setattr(obj, name, wrapped)

    for name in w.compute_ops:
        wrap(ops, name, "compute")
    for name in w.exchange_ops:
        wrap(ops, name, "collective")
    for name in ("all_reduce", "reduce_scatter_tensor", "all_gather_into_tensor", "all_to_all_single"):
        wrap(dist, name, "collective")
    try:
        w.step()                      # once with the recorders in place, untimed (first-use costs of the events)
        torch.cuda.synchronize()
        dist.barrier()
        # three steps back to back, the middle one analysed: its neighbours keep the queues
        # full, as in the timed loop (a lone step after a synchronise also pays launch latency)
        marks.clear()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w.step()
        first = len(marks)
        t0.record()
        w.step()
        t1.record()
        last = len(marks)
        w.step()
        torch.cuda.synchronize()
        marks = marks[first:last]
    finally:
        for obj, name, fn in restore:
            setattr(obj, name, fn)
    spans = [(name, kind, t0.elapsed_time(s), t0.elapsed_time(t), nb) for name, kind, s, t, nb in marks]
    busy = sorted((a, b) for _, kind, a, b, _ in spans if kind == "compute")
    merged = []
    for a, b in busy:
        if merged and a <= merged[-1][1]:
            merged[-1][1] = max(merged[-1][1], b)
        else:
            merged.append([a, b])

    def covered(a, b):
        return sum(max(0.0, min(b, y) - max(a, x)) for x, y in merged)

    per_op = {}
    longest = None
    for name, kind, a, b, nb in spans:
        if kind != "collective":
            continue
        exposed = max(0.0, (b - a) - covered(a, b))
        d = per_op.setdefault(name, {"calls": 0, "ms": 0.0, "exposed_ms": 0.0, "bytes": 0})
        d["calls"] += 1
        d["ms"] += b - a
        d["exposed_ms"] += exposed
        d["bytes"] += nb
        if longest is None or exposed > longest["exposed_ms"]:
            longest = {"op": name, "ms": round(b - a, 4), "exposed_ms": round(exposed, 4), "bytes": nb}
    for d in per_op.values():
        d["ms"], d["exposed_ms"] = round(d["ms"], 4), round(d["exposed_ms"], 4)
    out = {"step_ms": round(t0.elapsed_time(t1), 4), "compute_busy_ms": round(sum(b - a for a, b in merged), 4),
           "collectives": per_op, "longest_exposed_collective": longest}
    if spans_too:
        out["spans"] = [[name, round(a, 4), round(b, 4)] for name, _, a, b, _ in sorted(spans, key=lambda t: t[2])]
    return out


def sharded_line(torch, dist, w, workload, world, ms, clocks, peaks, extra_e2e=None):
    value = w.flops / (ms * 1e-3) / 1e12
    out = {"ms_per_step": ms, "tflops": value, "tflops_per_gpu": value / world,
           "frac_of_sustained_peak": value / world / peaks["tflops"], "scaling": w.scaling,
           "algorithmic_flops_per_step": w.flops, "workload": w.title, "parallelism": w.par_text}
    if clocks is not None:
        out["clocks"] = clocks
    if workload == "moe":
        ep = w.extra
        dev = w.host_in.device
        recv = torch.tensor([float(ep.rows_received()), float(ep.last.get("rows_sent", 0)),
                             float(ep.rows_sent_remote())], device=dev)
        allr = [torch.zeros_like(recv) for _ in range(world)]
        dist.all_gather(allr, recv)
        rows = [float(t[0].item()) for t in allr]
        out["moe_rows_received_per_rank"] = rows
        out["moe_rows_routed_per_rank"] = [float(t[1].item()) for t in allr]
        out["moe_rows_sent_to_other_ranks"] = [float(t[2].item()) for t in allr]
        out["moe_return_path"] = ep.last.get("return_path")
        out["moe_load_imbalance_max_over_mean"] = max(rows) / (sum(rows) / len(rows))
    return out


def init_group(torch, dist, rank, world, dev):
    if not dist.is_initialized():
        if world == 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29517")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)


def run_sharded(args):
    """`--workload lmhead | moe | tp_mlp`: one of the paths that shard over the GPUs of one box,
    with the end-to-end leg.  Prints one JSON line (rank 0).  The default run reports all
    three, device-timed, inside its own line (`sharded`)."""
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    init_group(torch, dist, rank, world, dev)
    pkg = entry.load_package()
    gemm = pkg.Tcgen05Gemm(local)
    gemm.set_scheduler(args.scheduler == "dynamic")
    ops = pkg.parallel.DeviceOps(gemm)
    f32 = torch.float32
    w = build_sharded(args.workload, torch, pkg, gemm, ops, dev, rank, world)

    # The expert-parallel exchange sets up peer mappings, side streams and their scheduler
    # counters during its first steps; a few more untimed steps keep that out of the clock.
    # at least as many untimed steps as timed ones: see sharded_block
    warmup = max(args.warmup, args.steps, {"moe": 10, "tp_mlp": 6, "lmhead": 5}[args.workload])
    for _ in range(warmup):
        launches = w.step()
    ms, clocks = time_steps(torch, dist, w.step, args.steps, local)
    # end to end: this step's activations from pinned host memory, one result word back
    src = w.host_in
    host_x = torch.empty(src.shape, dtype=src.dtype).pin_memory()
    host_x.copy_(src.cpu())
    host_out = torch.empty(1, dtype=f32).pin_memory()

    def e2e_step():
        src.copy_(host_x, non_blocking=True)
        w.step()
        word = w.result.get("loss")
        if word is None:
            word = next(iter(w.result.values())).reshape(-1)[:1].float()
        host_out.copy_(word, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_step()
    e2e_ms, _ = time_steps(torch, dist, e2e_step, args.steps, local, sample_clocks=False)
    tt = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms, e2e_ms = tt.tolist()
    timeline = exchange_timeline(torch, dist, ops, w, spans_too=args.timeline_spans)
    status = gemm.device_status()
    peaks = measured_peaks()
    sub = sharded_line(torch, dist, w, args.workload, world, ms, None, peaks)
    value = sub["tflops"]
    line = {
        "metric": f"bf16_gemm_tflops_{args.workload}", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": w.scaling, "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": w.title, "parallelism": w.par_text,
                   "l2": "operands exceed the 126 MB L2"},
        "pct_of_nominal_dense_peak": 100.0 * value / world / 2250.0,
        "gpu_launches": launches * args.steps, "device_status": status, "clocks": clocks,
        "e2e": {"value": w.flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": host_x.numel() * host_x.element_size(), "d2h_bytes_per_step": 4},
        "roofline": {"bound": "tensor", "achieved": value / world, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": value / world / peaks["tflops"], "traffic": None,
                     "peak_source": f"{peaks['source']} cuBLAS bf16 sustained; burst {peaks['burst']}",
                     "algorithmic_flops_per_step": w.flops},
        "exchange_timeline": timeline,
    }
    for key in ("moe_rows_received_per_rank", "moe_rows_routed_per_rank", "moe_rows_sent_to_other_ranks",
                "moe_load_imbalance_max_over_mean", "moe_return_path"):
        if key in sub:
            line[key] = sub[key]
    if rank == 0:
        print(json.dumps(line), flush=True)
    gemm.close()
    dist.destroy_process_group()


def device_code(torch, gemm) -> int:
    """The handle's device status word (read and cleared), without raising."""
    import ctypes
    code = ctypes.c_int32(0)
    gemm._lib.b200gemm_device_status(gemm._h, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                     ctypes.byref(code))
    return int(code.value)


def sharded_block(args, torch, dist, pkg, gemm, dev, rank, world, local):
    """The three sharded configurations at this run's N, device-timed (10 steps each), each
    with its exchange timeline: what the default line carries as `sharded`."""
    ops = pkg.parallel.DeviceOps(gemm)
    peaks = measured_peaks()
    steps = max(3, min(args.steps, 10))
    block = {}
    global RANK_BARRIER
    chosen = RANK_BARRIER
    for workload in SHARDED:
        RANK_BARRIER = chosen
        w = build_sharded(workload, torch, pkg, gemm, ops, dev, rank, world)
        # the exchanges set up peer mappings, side streams and scheduler counters in their first
        # steps, and the first steps through freshly mapped peer memory are slow: keep them out
        for _ in range(2):
            w.step()
        # A bounded wait that ran out on any rank (the barrier kernel gives up after 2 s) must not
        # be repeated for twenty more steps: fall back to NCCL's barriers for this workload, once.
        fell_back = None
        code = torch.tensor([device_code(torch, gemm)], device=dev, dtype=torch.int32)
        dist.all_reduce(code, op=dist.ReduceOp.MAX)
        if int(code.item()) != 0:
            fell_back = int(code.item())
            if world == 1 or RANK_BARRIER != "kernel":
                block[workload] = {"error": f"device status {fell_back} in the first steps"}
                continue
            del w
            RANK_BARRIER = "nccl"
            w = build_sharded(workload, torch, pkg, gemm, ops, dev, rank, world)
            for _ in range(2):
                w.step()
        # ... and at least as many steps as will be timed, enqueued the same way (no host
        # synchronisation in between): the host runs several steps ahead of the GPU, every step in
        # flight holds its own output buffers, and the caching allocator must have grown to that
        # depth before the timed region, or it calls cudaMalloc inside it (reported per line as
        # clocks.cuda_mallocs_in_region).
        for _ in range(max({"moe": 8, "tp_mlp": 4, "lmhead": 3}[workload], steps)):
            w.step()
        ms, clocks = time_steps(torch, dist, w.step, steps, local)
        tt = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        sub = sharded_line(torch, dist, w, workload, world, float(tt.item()), clocks, peaks)
        sub["steps"] = steps
        sub["exchange_timeline"] = exchange_timeline(torch, dist, ops, w)
        sub["device_status"] = gemm.device_status()
        sub["rank_barrier"] = RANK_BARRIER if world > 1 else None
        if fell_back is not None:
            sub["rank_barrier_note"] = f"the barrier kernel left device status {fell_back}; NCCL's barriers were used instead"
        block[workload] = sub
        del w
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
    RANK_BARRIER = chosen
    return block


def run_only(args):
    """Profiling aid: launch ONE named GEMM of the step (e.g. qkv.forward) a few times.

    Holds under 2 GB on the device and launches `warmup + steps` kernels, so a
    profiler capture of it ends by itself.  Prints a short JSON line."""
    import torch
    import __graft_entry__ as entry
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pkg = entry.load_package()
    gemm = pkg.Tcgen05Gemm(0)
    gemm.set_scheduler(args.scheduler == "dynamic")
    name, kind = args.only.split(".")
    bf, f32 = torch.bfloat16, torch.float32
    if name == "lm_head" and kind.startswith("fused"):
        m = args.only_tokens
        head = pkg.FusedLmHead(gemm, VOCAB, "in_out")
        hid = torch.randn((m, D_MODEL), device=dev).to(bf)
        w = (torch.randn((D_MODEL, VOCAB_PAD), device=dev) * 0.02).to(bf)
        tg = torch.randint(0, VOCAB, (m,), device=dev, dtype=torch.int32)
        lse = head.forward(hid, w, tg)[1]
        if kind == "fused_forward":
            fn, fl = (lambda: head.forward(hid, w, tg)), 2.0 * m * D_MODEL * VOCAB_PAD
        else:
            dl = torch.empty((m, VOCAB_PAD), device=dev, dtype=bf)
            dh = torch.empty((m, D_MODEL), device=dev, dtype=f32)
            dw = torch.zeros((D_MODEL, VOCAB_PAD), device=dev, dtype=f32)
            fn = lambda: head.backward(hid, w, tg, lse, dlogits=dl, d_hidden=dh, d_weight=dw, accumulate_dw=True)
            fl = 4.0 * m * D_MODEL * VOCAB_PAD
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            fn()
        e0.record()
        torch.cuda.synchronize()
        ms = s0.elapsed_time(e0) / args.steps
        print(json.dumps({"only": args.only, "tokens": m, "ms": ms, "tflops": fl / ms / 1e9,
                          "device_status": gemm.device_status()}), flush=True)
        gemm.close()
        return
    if name == "moe" and kind.startswith("exchange"):
        # The expert exchange's dispatch and combine kernels alone, two ranks' buffers in this one
        # GPU's memory (every "peer" store and load is local: what is timed is the kernels' own
        # throughput, not the links).  moe.exchange: stores / loads from two blocks per SM;
        # moe.exchange_bulk: bulk asynchronous copies through shared memory from 48 blocks.
        import ctypes as C
        n_tok, d, experts, top_k, world = args.only_tokens, 1536, 64, 8, 2
        ops = pkg.parallel.DeviceOps(gemm)
        x = torch.randn((n_tok, d), device=dev).to(bf)
        bias = 0.5 * torch.log(1.0 / torch.arange(1, experts + 1, device=dev, dtype=f32))
        logits = (torch.randn((n_tok, experts), device=dev) + bias).contiguous()
        r = ops.route(logits, top_k, True)
        counts = torch.stack([r.accepted_counts.to(torch.int32), torch.zeros_like(r.accepted_counts, dtype=torch.int32)])
        dst_base, _, _ = ops.ep_plan(counts.contiguous(), world, 0, experts)
        cap = n_tok * top_k
        inbox = [torch.zeros((cap, d), dtype=bf, device=dev) for _ in range(world)]
        ptrs = (C.c_void_p * world)(*[t.data_ptr() for t in inbox])
        out = torch.empty((n_tok, d), dtype=f32, device=dev)
        gemm.set_exchange_ctas(48 if kind.endswith("bulk") else 0, kind.endswith("bulk"))

        def fn():
            ops.ep_push(x, r, dst_base, ptrs, cap, world, experts)
            ops.ep_pull_combine(ptrs, r, dst_base, None, cap, world, experts, d, out)
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            fn()
        e0.record()
        torch.cuda.synchronize()
        ms = s0.elapsed_time(e0) / args.steps
        moved = 2.0 * n_tok * top_k * d * 2 + n_tok * d * (2 + 4)       # rows written + read, x read, out written
        print(json.dumps({"only": args.only, "tokens": n_tok, "ms": ms, "gb_per_s": moved / ms / 1e6,
                          "bytes_per_step": moved, "device_status": gemm.device_status()}), flush=True)
        gemm.set_exchange_ctas(0)
        gemm.close()
        return
    if name == "moe":
        n_tok, d, ff, experts, top_k = args.only_tokens, 1536, 768, 64, 8
        x = torch.randn((n_tok, d), device=dev).to(bf)
        bias = 0.5 * torch.log(1.0 / torch.arange(1, experts + 1, device=dev, dtype=f32))
        logits = (torch.randn((n_tok, experts), device=dev) + bias).contiguous()
        gated = kind.startswith("gated")
        if gated:                          # the reference's own expert: SwiGLU over a fused gate/up projection
            ffn = pkg.GatedExpertFfn(gemm, (torch.randn((experts, d, 2, ff), device=dev) * 0.02).to(bf),
                                     (torch.randn((experts, ff, d), device=dev) * 0.02).to(bf))
            flops = 2.0 * n_tok * top_k * d * ff * 3
            d_up = torch.zeros((experts, d, 2, ff), device=dev, dtype=f32)
        else:
            ffn = pkg.GroupedExpertFfn(gemm, (torch.randn((experts, d, ff), device=dev) * 0.02).to(bf),
                                       (torch.randn((experts, ff, d), device=dev) * 0.02).to(bf))
            flops = 2.0 * n_tok * top_k * d * ff * 2
            d_up = torch.zeros((experts, d, ff), device=dev, dtype=f32)
        if kind.endswith("backward"):      # forward keeping its activations + the whole backward
            d_dn = torch.zeros((experts, ff, d), device=dev, dtype=f32)
            dy = (torch.randn((n_tok, d), device=dev) * 0.01).to(bf)
            keep = {"keep_gate_up": True} if gated else {"keep_for_backward": True}

            def fn():
                ffn.forward(x, logits, top_k, scores_are_logits=True, **keep)
                ffn.backward(dy, d_up, d_dn)
            flops *= 3
        else:
            fn = lambda: ffn.forward(x, logits, top_k, scores_are_logits=True)
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            fn()
        e0.record()
        torch.cuda.synchronize()
        ms = s0.elapsed_time(e0) / args.steps
        print(json.dumps({"only": args.only, "tokens": n_tok, "ms": ms,
                          "tflops": flops / ms / 1e9,
                          "device_status": gemm.device_status()}), flush=True)
        gemm.close()
        return
    if name == "mlp_gate_up":
        # Dense gated MLP, x [m, D] . W [D, 2, FF]: the fused launch (activation in the
        # epilogue, panel kept for the backward) against the same product as a plain
        # bf16 GEMM followed by a separate activation pass over the panel.
        m = args.only_tokens
        x = torch.randn((m, D_MODEL), device=dev).to(bf)
        w = (torch.randn((1, D_MODEL, 2, D_FF), device=dev) * 0.02).to(bf)
        offs = torch.tensor([0, m], dtype=torch.int32, device=dev)
        y = torch.empty((m, D_FF), device=dev, dtype=bf)
        panel = torch.empty((m, 2, D_FF), device=dev, dtype=bf)
        w2 = w.reshape(D_MODEL, 2 * D_FF)

        def unfused():
            gemm.gemm(x, w2, panel.view(m, 2 * D_FF), transposed_b=True)
            torch.mul(torch.nn.functional.silu(panel[:, 0].float()), panel[:, 1].float()).to(bf)

        variants = {"swiglu": lambda: pkg.moe.grouped_gemm_swiglu(gemm, x, w, offs, out=y, gate_up=panel),
                    "swiglu_no_panel": lambda: pkg.moe.grouped_gemm_swiglu(gemm, x, w, offs, out=y),
                    "plain_gemm_only": lambda: gemm.gemm(x, w2, panel.view(m, 2 * D_FF), transposed_b=True),
                    "unfused": unfused}
        fn = variants[kind]
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            fn()
        e0.record()
        torch.cuda.synchronize()
        ms = s0.elapsed_time(e0) / args.steps
        print(json.dumps({"only": args.only, "tokens": m, "ms": ms,
                          "tflops": 2.0 * m * D_MODEL * 2 * D_FF / ms / 1e9,
                          "device_status": gemm.device_status()}), flush=True)
        gemm.close()
        return
    if name == "lm_head":
        i, o = D_MODEL, VOCAB_PAD
    else:
        i, o = {n: (a, b) for n, a, b in PROJECTIONS}[name]
    m = args.only_tokens
    x = torch.randn((m, i), device=dev).to(bf)
    w = (torch.randn((i, o), device=dev) * 0.02).to(bf)
    dy = (torch.randn((m, o), device=dev) * 0.01).to(bf)
    tile = {"auto": 0, "wide": pkg._lib.FLAG_WIDE_TILE, "narrow": pkg._lib.FLAG_NARROW_TILE}[args.tile]
    if kind == "forward":
        out = torch.empty((m, o), device=dev, dtype=bf if name == "lm_head" else f32)
        fn = lambda: gemm.gemm(x, w, out, transposed_b=True, flags=0 if name == "lm_head" else tile)
    elif kind == "forward_dual":            # fp32 result + its bf16 copy from one launch
        out = torch.empty((m, o), device=dev, dtype=f32)
        out16 = torch.empty((m, o), device=dev, dtype=bf)
        fn = lambda: gemm.f32_store_with_bf16_copy(x, w, out, out16, transposed_b=True)
    elif kind == "forward_then_convert":    # the two passes the dual form replaces
        out = torch.empty((m, o), device=dev, dtype=f32)
        out16 = torch.empty((m, o), device=dev, dtype=bf)

        def fn():
            gemm.gemm(x, w, out, transposed_b=True)
            gemm.convert_f32_to_bf16(out, out16)
    elif kind == "input_grad":
        out = torch.empty((m, i), device=dev, dtype=f32)
        fn = lambda: gemm.f32_store(dy, w, out, flags=tile)
    else:
        out = torch.zeros((i, o), device=dev, dtype=f32)
        fn = lambda: gemm.f32_accumulate_transposed(x, dy, out, flags=tile)
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(args.steps):
        fn()
    e0.record()
    torch.cuda.synchronize()
    ms = s0.elapsed_time(e0) / args.steps
    print(json.dumps({"only": args.only, "tokens": m, "ms": ms, "tflops": 2.0 * m * i * o / ms / 1e9,
                      "device_status": gemm.device_status()}), flush=True)
    gemm.close()


def run_gpu(args):
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    init_group(torch, dist, rank, world, device)             # one rank too: the sharded block below needs a group
    pkg = entry.load_package()
    gemm = pkg.Tcgen05Gemm(local)
    gemm.set_scheduler(args.scheduler == "dynamic")
    head = pkg.FusedLmHead(gemm, VOCAB, "in_out")
    buf = StepBuffers(torch, device, seed=rank)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing -------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        launches = run_step(gemm, head, buf)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        run_step(gemm, head, buf)
    stop.record()
    barrier()
    clocks = sampler.stop()
    ms = start.elapsed_time(stop) / args.steps
    status = gemm.device_status()

    # ---- end to end: host token batch in, result word out ------------------------
    host_x = torch.empty((M_TOKENS, D_MODEL), dtype=torch.bfloat16).pin_memory()
    host_x.copy_(buf.x[D_MODEL].cpu())
    host_out = torch.empty(1, dtype=torch.float32).pin_memory()
    e2e_steps = args.steps                                       # as many as the device-timed region

    def e2e_step():
        buf.x[D_MODEL].copy_(host_x, non_blocking=True)         # this step's token activations
        run_step(gemm, head, buf)
        host_out.copy_(buf.loss, non_blocking=True)             # the step's loss
        torch.cuda.current_stream().synchronize()

    e2e_step()
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2.record()
    barrier()
    e2e_ms = s2.elapsed_time(e2) / e2e_steps

    t = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()

    traffic = {}
    tpath = os.path.join(ROOT, "profiles", "gemm_tcgen05_qkv_forward_ncu.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            traffic = json.load(f)
    flops = step_flops()
    value = flops * world / (ms * 1e-3) / 1e12
    e2e_value = flops * world / (e2e_ms * 1e-3) / 1e12
    peaks = measured_peaks()
    per_gpu = value / world
    line = {
        "metric": "bf16_gemm_tflops_full_step", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
        "full_step_gemm_ms": ms, "pct_of_nominal_dense_peak": 100.0 * per_gpu / 2250.0,
        "gpu_launches": launches * args.steps, "device_status": status, "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": host_x.numel() * 2, "d2h_bytes_per_step": 4,
                "api": "Tcgen05Gemm methods over the C ABI; token activations from pinned host memory"},
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": per_gpu / peaks["tflops"],
                     # dram__bytes_read + write of ONE launch of the dominant instantiation (the QKV
                     # forward, 718.8 MB algorithmic), as recorded beside the ncu summary under profiles/
                     "traffic": traffic.get("dram_bytes_per_launch"), "traffic_launch": traffic.get("launch"),
                     "traffic_source": traffic.get("source"),
                     "kernel": "gemm_tcgen05_kernel (every launch of the timed region)",
                     "peak_source": f"{peaks['source']} cuBLAS bf16 sustained; burst {peaks['burst']}",
                     "algorithmic_flops_per_step": flops},
    }
    if rank == 0 and not args.no_table:
        line["per_shape"] = per_shape_table(torch, gemm, head, buf)
    # ---- the configurations that shard over the box, at this N (every rank takes part)
    del buf, head
    torch.cuda.empty_cache()
    if not args.no_sharded:
        try:
            line["sharded"] = sharded_block(args, torch, dist, pkg, gemm, device, rank, world, local)
        except Exception as exc:                              # the headline stands on its own
            line["sharded"] = {"error": f"{type(exc).__name__}: {exc}"}
    if rank == 0:
        if world == 1 and not args.no_cpu:
            secs, fl, text = cpu_sample(1)
            line["cpu_baseline"] = {"value": fl / secs / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
                                    "sample": text + f"; {secs:.1f} s on one host core of {os.cpu_count()}"}
        print(json.dumps(line), flush=True)
    gemm.close()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-table", action="store_true", help="skip the per-shape table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sharded", action="store_true", help="skip the sharded configurations' block")
    ap.add_argument("--only", default=None,
                    help="profiling aid: run one piece, e.g. qkv.forward, mlp_up.weight_grad, lm_head.fused_forward, "
                         "lm_head.fused_backward, moe.forward, moe.gated_forward, moe.backward, moe.gated_backward, "
                         "moe.exchange, moe.exchange_bulk, "
                         "mlp_gate_up.{swiglu,swiglu_no_panel,plain_gemm_only,unfused}")
    ap.add_argument("--only-tokens", type=int, default=M_TOKENS)
    ap.add_argument("--tile", default="auto", choices=["auto", "wide", "narrow"],
                    help="with --only <gemm>.<kind>: 256x512 tiles per CTA pair, 256x256, or the planner's choice")
    ap.add_argument("--scheduler", default="dynamic", choices=["static", "dynamic"],
                    help="how the persistent kernels hand out tiles (see b200gemm_set_scheduler)")
    ap.add_argument("--workload", default="dense_step", choices=["dense_step", "lmhead", "moe", "tp_mlp"],
                    help="dense_step (default) is the headline; the others are the sharded configurations")
    ap.add_argument("--head-exchange", default="copy", choices=["copy", "nccl"],
                    help="vocabulary-parallel head on several GPUs: how d_hidden is summed over the shards")
    ap.add_argument("--moe-pieces", default="6,5,3,2",
                    help="expert-parallel MoE: token slices that go through dispatch, GEMMs and combine as a pipeline; "
                         "a count, or comma-separated weights (the default ends with short slices: what follows the "
                         "last dispatch -- that slice's GEMMs and combine -- overlaps nothing)")
    ap.add_argument("--moe-return", default="pull", choices=["pull", "push"],
                    help="expert-parallel MoE: results read by the token's rank while it combines (pull), or stored "
                         "into the token rank's buffer by the owner's down-projection GEMM (push)")
    ap.add_argument("--mlp-pieces", default="1,3,4,4,3,1",
                    help="tensor-parallel MLP on several GPUs: row pieces, a count or comma-separated weights")
    ap.add_argument("--mlp-exchange", default="copy", choices=["copy", "nccl"],
                    help="tensor-parallel MLP on several GPUs: copy-engine pushes + local sum, or NCCL collectives")
    ap.add_argument("--moe-reserve-sms", type=int, default=24,
                    help="expert-parallel MoE: SMs the expert GEMMs leave free for the exchange kernels")
    ap.add_argument("--moe-exchange-ctas", type=int, default=48,
                    help="expert-parallel MoE: thread blocks of the dispatch / combine kernels that run beside a GEMM "
                         "(0 = two per SM)")
    ap.add_argument("--moe-exchange-form", default="bulk", choices=["bulk", "plain"],
                    help="expert-parallel MoE: dispatch / combine by bulk asynchronous copies through shared memory, "
                         "or by plain stores / loads")
    ap.add_argument("--timeline-spans", action="store_true",
                    help="with --workload: add every timed call of the analysed step (name, start ms, end ms)")
    ap.add_argument("--rank-barrier", default="kernel", choices=["kernel", "nccl"],
                    help="how the copy-engine and device-driven exchanges order the ranks: this library's one-block "
                         "barrier kernel over peer memory, or one-element NCCL all-reduces")
    args = ap.parse_args()
    global MLP_EXCHANGE, HEAD_EXCHANGE, MOE_PIECES, MOE_RETURN, MLP_PIECES, RANK_BARRIER, MOE_RESERVE, MOE_CTAS, MOE_BULK
    MOE_RESERVE, MOE_CTAS, MOE_BULK = args.moe_reserve_sms, args.moe_exchange_ctas, args.moe_exchange_form == "bulk"
    RANK_BARRIER = args.rank_barrier
    MOE_RETURN = args.moe_return
    parts = [int(v) for v in str(args.mlp_pieces).split(",")]
    MLP_PIECES = parts[0] if len(parts) == 1 else parts
    MLP_EXCHANGE, HEAD_EXCHANGE = args.mlp_exchange, args.head_exchange
    parts = [int(v) for v in str(args.moe_pieces).split(",")]
    MOE_PIECES = parts[0] if len(parts) == 1 else parts
    if args.impl == "reference":
        run_reference(args)
    elif args.only:
        run_only(args)
    elif args.workload != "dense_step":
        run_sharded(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
