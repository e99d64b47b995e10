"""Helpers shared by the GPU parity tests: seeded synthetic inputs and bit-pattern views."""

from __future__ import annotations

import numpy as np
import torch

import fdk_oracle as O


def to_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def from_bits(bits: np.ndarray, dtype=torch.bfloat16, device="cuda") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).view(dtype).to(device)


def kmeans_like_codebook(bits: int, seed: int = 0) -> np.ndarray:
    """Sorted 2^bits centroids of N(0,1) samples (a few Lloyd iterations), as bf16 bits."""
    rng = np.random.default_rng(seed)
    x = np.sort(rng.standard_normal(20000).astype(np.float32))
    c = np.quantile(x, (np.arange(1 << bits) + 0.5) / (1 << bits)).astype(np.float32)
    for _ in range(8):
        edges = (c[1:] + c[:-1]) / 2
        idx = np.searchsorted(edges, x)
        c = np.array([x[idx == i].mean() if (idx == i).any() else c[i] for i in range(1 << bits)], dtype=np.float32)
    return O.f32_to_bf16(np.sort(c))


def random_problem(n: int, k: int, bits: int, m: int, seed: int, g: int = 64, codebook: str = "kmeans"):
    """Random packed weights the way the reference's kernel tests draw them (uniform random
    bytes, rand scales; kernels.py:185-196), with a k-means-like or linspace codebook.
    Returns numpy bit patterns: codes, lut (byte table or 8-entry codebook), scale, x."""
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 256, size=(n, k * bits // 8), dtype=np.uint8)
    if codebook == "kmeans":
        base = kmeans_like_codebook(bits, seed)
    else:
        base = O.f32_to_bf16(np.linspace(-1, 1, 1 << bits, dtype=np.float32))
    lut = base.reshape(-1, 1) if bits == 3 else O.byte_lut(base, bits)
    scale = O.f32_to_bf16(rng.random((n, k // g), dtype=np.float32) * np.float32(2.0 / np.sqrt(k)))
    x = O.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    return codes, lut, scale, x


def oracle_dense(codes, lut, scale, bits, k):
    if bits == 3:
        return O.dequantise_indices(O.unpack_indices(codes, 3, k), lut.reshape(-1), scale)
    return O.dequantise(codes, lut, scale)
