"""Seeded synthetic NVFP4 tensors shared by the tests (shapes and distributions of the benchmark configurations)."""
from __future__ import annotations

import numpy as np

from oracle import q35oracle as o


def make_weight(n: int, k: int, seed: int, std: float = 0.02, row_outlier_frac: float = 0.0):
    """fp32 N(0, std) [n, k], optionally with a fraction of rows scaled x8, quantised by the oracle.
    Returns (w_f32, codes, scales, s2)."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * std).astype(np.float32)
    if row_outlier_frac > 0:
        rows = rng.choice(n, size=max(1, int(np.ceil(row_outlier_frac * n))), replace=False)
        w[rows] *= 8.0
    codes, scales, s2 = o.quantize_nvfp4(w)
    return w, codes, scales, s2


def make_activations(m: int, k: int, seed: int, outlier_frac: float = 0.0):
    """BF16 N(0,1) [m, k] as uint16 bit patterns, optionally with a fraction of channels scaled x20."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k)).astype(np.float32)
    if outlier_frac > 0:
        ch = rng.choice(k, size=max(1, int(np.ceil(outlier_frac * k))), replace=False)
        x[:, ch] *= 20.0
    return o.bf16_round(x)


def to_torch_bf16(bits: np.ndarray, device="cuda"):
    import torch

    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(device)


def from_torch_bf16(t) -> np.ndarray:
    import torch

    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
