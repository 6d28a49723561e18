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

# ---- the workload: BASELINE "configs[1]" -----------------------------------
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
    """Polls nvidia-smi for SM clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_flag = threading.Event()

    def run(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop_flag.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                     "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                f = [x.strip() for x in out.strip().split(",")]
                self.samples.append(float(f[0]))
                self.max_mhz = float(f[1])
                for name, val in zip(names, f[2:6]):
                    if val.lower().startswith("active"):
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_flag.wait(0.1)

    def stop(self):
        self._stop_flag.set()
        self.join(timeout=6)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# ---- reference arm: the CPU restatement of the reference's matmul family ------

def cpu_sample(threads: int, rows: int | None = None, k_tokens: int | None = None):
    """Time the oracle's matmul family on a bounded sample of the workload.

    Forward and input-gradient shapes keep their full K and N but only `rows`
    token rows; weight-gradient shapes keep their full output but only
    `k_tokens` of the 32768-token reduction.  Returns (seconds, flops, text)."""
    from oracle import oracle as orc
    orc.build()
    # About 130 MFLOP per sampled row: 128 rows per thread is roughly 10 s of scalar work.
    rows = min(8192, 128 * threads) if rows is None else rows
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
            "vocab_padded": VOCAB_PAD, "parallelism": f"replicas x{n_gpus} (one token batch per GPU)",
            "l2": "operands of successive launches differ and exceed the 126 MB L2"}


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

    # Comparator column: the same products through cuBLASLt (torch.mm, fp32 output like the
    # rows they stand beside), timed the same way.  Reported only; not on the product path.
    f32 = torch.float32

    def cublas(fn, flops):
        try:
            return round(timed(fn, flops)[1], 1)
        except Exception:                                   # a torch build without out_dtype
            return None

    for name, i, o in PROJECTIONS:
        fl = 2.0 * M_TOKENS * i * o
        w, dw = layer[name]["w"], layer[name]["dw"]
        x, dy = buf.x[i], buf.dy[o]
        for kind, fn, ref in (
            ("forward", lambda: gemm.f32_store(x, w, buf.y[o], transposed_b=True),
             lambda: torch.mm(x, w, out_dtype=f32)),
            ("input_grad", lambda: gemm.f32_store(dy, w, buf.y[i]),
             lambda: torch.mm(dy, w.t(), out_dtype=f32)),
            ("weight_grad", lambda: gemm.f32_accumulate_transposed(x, dy, dw),
             lambda: torch.mm(x.t(), dy, out_dtype=f32)),     # overwrite: cuBLASLt's cheaper case
        ):
            ms, tf = timed(fn, fl)
            rows.append({"gemm": f"{name}.{kind}", "ms": round(ms, 4), "tflops": round(tf, 1),
                         "cublaslt_tflops": cublas(ref, fl)})
    fl = 2.0 * M_TOKENS * D_MODEL * VOCAB_PAD
    lse = head.forward(buf.x[D_MODEL], buf.head_w, buf.targets)[1]
    h = buf.x[D_MODEL]

    def two_products():
        torch.mm(buf.dlogits, buf.head_w.t(), out_dtype=f32)
        torch.mm(h.t(), buf.dlogits, out_dtype=f32)

    for kind, fn, credit, ref in (
        # comparator: the logits product alone (bf16 logits written to HBM, no classifier)
        ("fused_forward", lambda: head.forward(h, buf.head_w, buf.targets), fl,
         lambda: torch.mm(h, buf.head_w)),
        # recompute + two gradient products; only the two products are credited.
        # comparator: the two products alone, on dlogits already in HBM
        ("fused_backward", lambda: head.backward(h, buf.head_w, buf.targets, lse,
                                                 dlogits=buf.dlogits, d_hidden=buf.dh,
                                                 d_weight=buf.head_dw, accumulate_dw=True), 2 * fl,
         two_products),
    ):
        ms, tf = timed(fn, credit)
        rows.append({"gemm": f"lm_head.{kind}", "ms": round(ms, 4), "tflops": round(tf, 1),
                     "cublaslt_tflops": cublas(ref, credit)})
    return rows



# ---- the sharded workloads (BASELINE configs[2], [3], [4]) ------------------------

def run_sharded(args):
    """`--workload lmhead | moe | tp_mlp`: the paths that shard over the GPUs of one box.

    Strong scaling: the problem is the BASELINE configuration whatever N is; each
    rank holds its shard.  Prints one JSON line (rank 0)."""
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        if world == 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29517")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    pkg = entry.load_package()
    par = pkg.parallel
    gemm = pkg.Tcgen05Gemm(local)
    gemm.set_scheduler(args.scheduler == "dynamic")
    ops = par.DeviceOps(gemm)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1)                                    # replicated operands: same seed on every rank
    bf, f32 = torch.bfloat16, torch.float32

    def rnd(shape, std, g=gen):
        return (torch.randn(shape, generator=g, device=dev, dtype=f32) * std).to(bf)

    if args.workload == "lmhead":
        m, k, v, classes = M_TOKENS, D_MODEL, VOCAB_PAD, VOCAB
        # Several GPUs: the weight-gradient GEMM leaves 16-32 SMs to d_hidden's all-reduce, which
        # runs in a group limited to as many thread blocks, so the two overlap.
        # (the all-reduce takes about the same time whatever N is while the GEMM shrinks with N)
        reserve = 0 if world == 1 else (32 if world >= 8 else 16)
        head = par.VocabParallelHead(ops, classes, v, reserve_sms=reserve,
                                     group=par.nccl_group_with_cta_limit(reserve) if reserve else None)
        hidden = rnd((m, k), 1.0)
        w_shard = rnd((k, head.c1 - head.c0), 0.02)
        targets = torch.randint(0, classes, (m,), generator=gen, device=dev, dtype=torch.int32)
        dw = torch.zeros((k, head.c1 - head.c0), device=dev, dtype=f32)
        result = {}

        def step():
            loss, lse, _ = head.forward(hidden, w_shard, targets)
            head.backward(hidden, w_shard, targets, lse, d_weight=dw, accumulate_dw=True)
            result["loss"] = loss
            return 5

        flops = 3 * 2.0 * m * k * v
        name = ("fused lm-head + softmax cross-entropy (BASELINE configs[2]): M=32768 K=1536 V=50432 "
                "(50257 classes), forward + backward; the backward's logit recompute is not credited")
        par_text = (f"vocabulary split over {world} GPU(s); all-reduce of row max / sum-exp and of d_hidden "
                    f"(the latter under the weight-gradient GEMM, {reserve} SMs reserved for it)")
        host_in = (hidden, None)
    elif args.workload == "moe":
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
        ep = par.ExpertParallelMoe(ops, experts, top_k, w_up, w_dn, pieces=2, exchange="device")
        result = {}

        def step():
            result["out"] = ep.forward(x, logits, scores_are_logits=True)
            return 9


        flops = 2.0 * n_tok * top_k * d * ff * 2
        name = ("MoE grouped expert GEMM (BASELINE configs[3]): 32768 tokens per GPU, D=1536, E=64, top-8, "
                "expert FF=768, up -> SiLU -> down, Zipf-skewed routing; routing, dispatch and combine included")
        par_text = (f"experts split over {world} GPU(s), 32768 tokens on each; dispatch by peer stores and combine by "
                    "peer loads over NVLink (symmetric memory, sizes never leave the device), NCCL for the "
                    "counts and the two barriers; two token slices on two streams")
        host_in = (x, None)
    else:
        m, d, ff = 65536, 4096, 16384
        cols = ff // world
        x = rnd((m, d), 1.0)
        w1 = rnd((d, cols), 0.015)
        w2 = rnd((cols, d), 0.015)
        mlp = par.TensorParallelMlp(ops, w1, w2, chunks=4, partial_dtype=bf)
        dy_local = rnd((m // world, d), 0.01)
        dw1 = torch.zeros((d, cols), device=dev, dtype=f32)
        dw2 = torch.zeros((cols, d), device=dev, dtype=f32)
        result = {}

        def step():
            result["out"] = mlp.forward(x)
            result["dx"] = mlp.backward(x, dy_local, dw1, dw2)
            return 6 * 4

        flops = 6 * 2.0 * m * d * ff
        name = ("tensor-parallel MLP block (BASELINE configs[4]): M=65536 D=4096 FF=16384, column-parallel up, "
                "row-parallel down, forward + input and weight gradients (K=65536 split-K)")
        par_text = f"FF split over {world} GPU(s); reduce-scatter of the partial outputs, all-reduce of dx"
        host_in = (x, None)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    # The expert-parallel exchange sets up peer mappings, side streams and their scheduler
    # counters during its first steps; a few more untimed steps keep that out of the clock.
    warmup = max(args.warmup, 10 if args.workload == "moe" else 3)
    for _ in range(warmup):
        launches = step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    s0.record()
    for _ in range(args.steps):
        step()
    e0.record()
    barrier()
    clocks = sampler.stop()
    ms = s0.elapsed_time(e0) / args.steps
    # end to end: this step's activations from pinned host memory, one result word back
    src = host_in[0]
    host_x = torch.empty(src.shape, dtype=src.dtype).pin_memory()
    host_x.copy_(src.cpu())
    host_out = torch.empty(1, dtype=f32).pin_memory()

    def e2e_step():
        src.copy_(host_x, non_blocking=True)
        step()
        word = result.get("loss")
        if word is None:
            word = next(iter(result.values())).reshape(-1)[:1].float()
        host_out.copy_(word, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_step()
    barrier()
    s1, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s1.record()
    n_e2e = max(1, min(args.steps, 5))
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = s1.elapsed_time(e1) / n_e2e
    tt = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms, e2e_ms = tt.tolist()
    status = gemm.device_status()
    peaks = measured_peaks()
    value = flops / (ms * 1e-3) / 1e12
    line = {
        "metric": f"bf16_gemm_tflops_{args.workload}", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak" if args.workload == "moe" else "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": name, "parallelism": par_text,
                   "l2": "operands exceed the 126 MB L2"},
        "pct_of_nominal_dense_peak": 100.0 * value / world / 2250.0,
        "gpu_launches": launches * args.steps, "device_status": status, "clocks": clocks,
        "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": host_x.numel() * host_x.element_size(), "d2h_bytes_per_step": 4},
        "roofline": {"bound": "tensor", "achieved": value / world, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": value / world / peaks["tflops"], "traffic": None,
                     "peak_source": f"{peaks['source']} cuBLAS bf16 sustained; burst {peaks['burst']}",
                     "algorithmic_flops_per_step": flops},
    }
    if args.workload == "moe":
        recv = torch.tensor([float(ep.rows_received())], device=dev)
        allr = [torch.zeros_like(recv) for _ in range(world)]
        dist.all_gather(allr, recv)
        rows = [float(t.item()) for t in allr]
        line["moe_rows_received_per_rank"] = rows
        line["moe_load_imbalance_max_over_mean"] = max(rows) / (sum(rows) / len(rows))
    if rank == 0:
        print(json.dumps(line), flush=True)
    gemm.close()
    dist.destroy_process_group()

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
    if name == "moe":
        n_tok, d, ff, experts, top_k = args.only_tokens, 1536, 768, 64, 8
        x = torch.randn((n_tok, d), device=dev).to(bf)
        bias = 0.5 * torch.log(1.0 / torch.arange(1, experts + 1, device=dev, dtype=f32))
        logits = (torch.randn((n_tok, experts), device=dev) + bias).contiguous()
        if kind == "gated_forward":        # the reference's own expert: SwiGLU over a fused gate/up projection
            ffn = pkg.GatedExpertFfn(gemm, (torch.randn((experts, d, 2, ff), device=dev) * 0.02).to(bf),
                                     (torch.randn((experts, ff, d), device=dev) * 0.02).to(bf))
            flops = 2.0 * n_tok * top_k * d * ff * 3
        else:
            ffn = pkg.GroupedExpertFfn(gemm, (torch.randn((experts, d, ff), device=dev) * 0.02).to(bf),
                                       (torch.randn((experts, ff, d), device=dev) * 0.02).to(bf))
            flops = 2.0 * n_tok * top_k * d * ff * 2
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
    if kind == "forward":
        out = torch.empty((m, o), device=dev, dtype=bf if name == "lm_head" else f32)
        fn = lambda: gemm.gemm(x, w, out, transposed_b=True)
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
        fn = lambda: gemm.f32_store(dy, w, out)
    else:
        out = torch.zeros((i, o), device=dev, dtype=f32)
        fn = lambda: gemm.f32_accumulate_transposed(x, dy, out)
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
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    pkg = entry.load_package()
    gemm = pkg.Tcgen05Gemm(local)
    gemm.set_scheduler(args.scheduler == "dynamic")
    head = pkg.FusedLmHead(gemm, VOCAB, "in_out")
    buf = StepBuffers(torch, device, seed=rank)

    def barrier():
        if world > 1:
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
    e2e_steps = max(1, min(args.steps, 5))

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

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()

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
                     # forward, 718.8 MB algorithmic), from the ncu capture summarised under profiles/
                     "traffic": 706.7e6, "traffic_launch": "gemm_tcgen05_kernel<2,0,0> qkv.forward",
                     "kernel": "gemm_tcgen05_kernel (every launch of the timed region)",
                     "peak_source": f"{peaks['source']} cuBLAS bf16 sustained; burst {peaks['burst']}",
                     "algorithmic_flops_per_step": flops},
    }
    if rank == 0:
        if not args.no_table:
            line["per_shape"] = per_shape_table(torch, gemm, head, buf)
        if world == 1 and not args.no_cpu:
            secs, fl, text = cpu_sample(1)
            line["cpu_baseline"] = {"value": fl / secs / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
                                    "sample": text + f"; {secs:.1f} s on one host core of {os.cpu_count()}"}
        print(json.dumps(line), flush=True)
    gemm.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-table", action="store_true", help="skip the per-shape table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--only", default=None,
                    help="profiling aid: run one piece, e.g. qkv.forward, mlp_up.weight_grad, lm_head.fused_forward, "
                         "lm_head.fused_backward, moe.forward, moe.gated_forward, "
                         "mlp_gate_up.{swiglu,swiglu_no_panel,plain_gemm_only,unfused}")
    ap.add_argument("--only-tokens", type=int, default=M_TOKENS)
    ap.add_argument("--scheduler", default="dynamic", choices=["static", "dynamic"],
                    help="how the persistent kernels hand out tiles (see b200gemm_set_scheduler)")
    ap.add_argument("--workload", default="dense_step", choices=["dense_step", "lmhead", "moe", "tp_mlp"],
                    help="dense_step (default) is the headline; the others are the sharded configurations")
    args = ap.parse_args()
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
