"""Seeded synthetic inputs shared by the tests (and mirrored by bench.py)."""

from __future__ import annotations

import numpy as np
import torch

from oracle import nvfp4 as onv


def make_weight(N: int, K: int, seed: int, std: float = 0.02):
    """bf16 N(0, std) weight quantized offline with the oracle quantizer.
    Returns (codes [N,K/2] u8, scales [N,K/16] u8, global_scale float)."""
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(N, K, generator=g, dtype=torch.float32) * std).to(torch.bfloat16).float().numpy()
    gs = onv.global_scale_for(w)
    codes, sf = onv.quantize_nvfp4(w, 1.0 / gs)
    return codes, sf, gs


def make_activation(M: int, K: int, seed: int, outlier_frac: float = 0.001, outlier_mult: float = 20.0):
    """bf16 N(0,1) tokens with a fraction of channels scaled up (outliers).
    Returns a torch bf16 tensor [M,K] on the CPU."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g, dtype=torch.float32)
    n_out = max(1, int(round(K * outlier_frac)))
    cols = torch.randperm(K, generator=g)[:n_out]
    x[:, cols] *= outlier_mult
    return x.to(torch.bfloat16)


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def cuda(t):
    if isinstance(t, np.ndarray):
        t = torch.from_numpy(np.ascontiguousarray(t))
    return t.cuda()
