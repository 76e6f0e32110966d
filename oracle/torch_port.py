"""Torch-on-CPU port of the reference's dequantise-then-matmul path, for TIMING.

TEST/BENCH INFRASTRUCTURE ONLY. The reference's CPU-runnable implementation
of the NVFP4 linear is a PyTorch gather-dequantise followed by an fp32
contraction (kernels/tests/conftest.py:23-55). ``bench.py`` times this port
on the host cores as the ``cpu_baseline`` / ``--impl reference`` leg; the
numpy oracle in ``oracle/nvfp4.py`` is the correctness checker. Same ops in
the same order as the reference (table gather per nibble, interleave, e4m3
view-cast, per-block multiply, einsum), so the timing is representative of
the reference's own CPU path.
"""

from __future__ import annotations

import torch

_MAGS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_TABLE = torch.tensor(_MAGS + tuple(-m for m in _MAGS), dtype=torch.float32)


def dequant_torch(packed: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """uint8 [..., K/2] + uint8 [..., K/16] -> float32 [..., K] (conftest.py:23-41)."""
    lo = _TABLE[(packed & 0xF).long()]
    hi = _TABLE[(packed >> 4).long()]
    vals = torch.stack((lo, hi), dim=-1).flatten(-2)
    s = scale.view(torch.float8_e4m3fn).to(torch.float32)
    out = vals.unflatten(-1, (-1, 16)) * s.unsqueeze(-1)
    return out.flatten(-2)


def linear_torch(w_codes, w_sf, x_codes, x_sf, alpha: float = 1.0) -> torch.Tensor:
    """[N,K/2],[N,K/16] x [M,K/2],[M,K/16] -> [M,N] float32: dequantise both
    operands, contract in fp32 (conftest.py:44-54), scale by alpha."""
    w = dequant_torch(w_codes, w_sf)
    a = dequant_torch(x_codes, x_sf)
    return torch.einsum("nk,mk->mn", w, a) * alpha


def quantize_torch(x: torch.Tensor, global_scale_inv: float):
    """bf16/fp32 [M,K] -> (codes uint8 [M,K/2], scales uint8 [M,K/16]) with torch
    CPU ops; same arithmetic as ``oracle.nvfp4.quantize_nvfp4`` (timing leg of
    the quantizer; checked against it in tests)."""
    xf = x.to(torch.float32)
    M, K = xf.shape
    gs = torch.tensor(global_scale_inv, dtype=torch.float32)
    xb = xf.view(M, K // 16, 16)
    amax = xb.abs().amax(dim=-1)
    s = (gs * (amax * torch.tensor(1.0 / 6.0, dtype=torch.float32))).clamp(-448.0, 448.0)
    sf8 = s.to(torch.float8_e4m3fn)
    sf = sf8.to(torch.float32)
    denom = sf * (1.0 / gs)
    r = torch.where(denom == 0, torch.zeros_like(denom), 1.0 / denom)
    y = (xb * r.unsqueeze(-1)).clamp(-6.0, 6.0).reshape(M, K)
    mag = y.abs()
    # round-to-nearest-even on the e2m1 grid, expressed as interval tests
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=torch.float32)
    ties_up = torch.tensor([False, True, False, True, False, True, False])
    code = torch.zeros_like(mag, dtype=torch.uint8)
    for b, up in zip(bounds.tolist(), ties_up.tolist()):
        code += ((mag >= b) if up else (mag > b)).to(torch.uint8)
    code = code | (torch.signbit(y).to(torch.uint8) << 3)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), sf8.view(torch.uint8).contiguous()
