"""Helpers shared by the GPU parity tests: seeded inputs, bf16 transport, tolerances."""
import os

import numpy as np

THREADS = max(1, min(32, os.cpu_count() or 1))

# Tolerance of the GEMM contract for bf16 inputs with fp32 accumulation:
# relative Frobenius error <= 1e-2 and per element |d| <= 2e-2 * (1 + |ref|).
REL_FRO = 1e-2
ELEM = 2e-2


def to_dev_bf16(bits: np.ndarray):
    """uint16 bf16 words -> CUDA bf16 tensor of the same shape."""
    import torch
    return torch.from_numpy(bits.view(np.int16).copy()).cuda().view(torch.bfloat16)


def from_dev_bf16(t) -> np.ndarray:
    """CUDA bf16 tensor -> f32 numpy array holding the same values."""
    import torch
    words = t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    return (words.astype(np.uint32) << 16).view(np.float32)


def bf16_operand(oracle, shape, seed, std=1.0, kind="normal"):
    """(device bf16 tensor, f32 numpy array of the values it holds)."""
    n = int(np.prod(shape))
    x = oracle.normal(n, seed, 0.0, std) if kind == "normal" else oracle.uniform(n, seed) * std
    bits = oracle.bf16_bits(x).reshape(shape)
    vals = oracle.bf16_to_f32(bits).reshape(shape)
    return to_dev_bf16(bits), vals


def assert_gemm_close(got: np.ndarray, ref: np.ndarray, what: str, rel_fro=REL_FRO, elem=ELEM):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    denom = np.linalg.norm(ref)
    fro = np.linalg.norm(got - ref) / (denom if denom > 0 else 1.0)
    worst = np.max(np.abs(got - ref) / (1.0 + np.abs(ref)))
    assert fro <= rel_fro, f"{what}: relative Frobenius error {fro:.3e} > {rel_fro}"
    assert worst <= elem, f"{what}: per-element error {worst:.3e} > {elem}"
    return fro, worst
