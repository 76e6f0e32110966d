"""Small exhaustive and out-of-bounds checks of the decode paths (GPU).

The reference's own GEMV test draws random bytes (kernels/tests/conftest.py:58-83: codes
uniform in 0..255, scale bytes in [1, 0x38)); it never shows that EVERY code byte and EVERY
scale byte decodes right. Here every one of the 256 code bytes meets every non-negative
finite e4m3 scale byte (0x00..0x7E) in one product, through the CUDA-core GEMV (both
kernels), the packed tensor-core linear's operand path (`nvfp4r_gemm` on pre-quantized
operands) and the oracle. A second group of tests surrounds every output buffer with
sentinel values and checks that the kernels write inside it only.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import nvfp4 as onv
from helpers import cuda, make_activation, rel_l2

pytestmark = pytest.mark.gpu

SCALE_BYTES = 0x7F          # 0x00 .. 0x7E: zero, subnormals, every normal up to 448


@pytest.fixture(scope="module")
def capi():
    from reset_b200 import capi as c
    return c


def _all_bytes_weight(N=128, K=512):
    """Row r uses scale byte r (rows past 0x7E repeat it); every row holds each of the 256
    code bytes once (K/2 = 256 bytes), rotated by the row index so that the pairing with the
    activation codes differs from row to row."""
    assert K // 2 == 256
    w = np.stack([np.roll(np.arange(256, dtype=np.uint8), r) for r in range(N)])
    ws = np.stack([np.full(K // 16, min(r, SCALE_BYTES - 1), dtype=np.uint8) for r in range(N)])
    return w, ws


def _magnitude(w, ws, xc, xsf):
    """Sum of |w| * |x| per output (sign bits of all codes cleared): the yardstick for the error
    of a sum whose terms may cancel."""
    return onv.linear_f64(w & 0x77, ws, xc & 0x77, xsf, alpha=1.0)


def _check_rows(got, exact, mag):
    """Every output, not only the norm: rows with tiny scales must be right too. fp32
    accumulation over 32 exact block sums: a few 1e-7 of the magnitude sum at most."""
    assert np.isfinite(got).all()
    assert np.all(np.abs(got - exact) <= 2e-6 * mag)
    assert np.all(got[mag == 0] == 0)


@pytest.mark.parametrize("generic", [False, True, "rows"])
def test_gemv_decodes_every_code_and_scale_byte(capi, generic):
    """Through the ring kernel, the plain-load fallback and the register-resident kernel."""
    from reset_b200 import _lib
    rows_mode = 1 if generic == "rows" else -1
    generic = generic is True
    N, K = 128, 512
    w, ws = _all_bytes_weight(N, K)
    x = np.arange(256, dtype=np.uint8)[::-1].copy().reshape(1, 1, K // 2)      # every code byte as activation too
    xs = (np.arange(K // 16, dtype=np.uint8) * 3 % 0x50 + 1).reshape(1, 1, K // 16)  # varied, finite, non-zero
    exact = onv.linear_f64(w, ws, x[:, 0], xs[:, 0], alpha=1.0)
    out = torch.full((1, N), float("nan"), dtype=torch.float32, device="cuda")
    _lib.check(_lib.lib().nvfp4r_set_gemv_tuning(-1, -1, 1 if generic else 0), "tuning")
    _lib.check(_lib.lib().nvfp4r_set_gemv_rows_tuning(rows_mode, 0, 0), "rows tuning")
    try:
        capi.gemv_out(cuda(w).unsqueeze(0), cuda(ws).unsqueeze(0), cuda(x), cuda(xs), out, 1.0)
        torch.cuda.synchronize()
    finally:
        _lib.check(_lib.lib().nvfp4r_set_gemv_tuning(-1, -1, 0), "tuning")
        _lib.check(_lib.lib().nvfp4r_set_gemv_rows_tuning(0, 0, 0), "rows tuning")
    _check_rows(out.cpu().numpy(), exact, _magnitude(w, ws, x[:, 0], xs[:, 0]))


def test_tensor_core_operands_decode_every_code_and_scale_byte(capi):
    N, K, M = 128, 512, 3
    w, ws = _all_bytes_weight(N, K)
    xc = np.stack([np.roll(np.arange(256, dtype=np.uint8)[::-1], 7 * m) for m in range(M)])
    xsf = np.stack([(np.arange(K // 16, dtype=np.uint8) * (3 + m) % 0x50 + 1) for m in range(M)]).astype(np.uint8)
    exact = onv.linear_f64(w, ws, xc, xsf, alpha=1.0)
    C = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    wksp = capi.gemm_workspace(M, N, K, "cuda")
    capi.gemm(cuda(xc), cuda(w), cuda(onv.swizzle_blockscale(xsf)), cuda(onv.swizzle_blockscale(ws)), C, 1.0,
              wksp, n_major=False)
    torch.cuda.synchronize()
    _check_rows(C.cpu().numpy(), exact, _magnitude(w, ws, xc, xsf))


def test_packed_linear_decodes_every_code_and_scale_byte(capi):
    """The product path: the packed weight holds every code byte under every scale byte; the
    activations are bf16 and go through the fused quantizer."""
    from reset_b200 import _lib
    N, K, M = 128, 512, 2
    w, ws = _all_bytes_weight(N, K)
    x = make_activation(M, K, seed=4).cuda()
    gs = torch.tensor([40.0], dtype=torch.float32, device="cuda")
    packed = capi.pack_weight(cuda(w), cuda(ws))
    out = capi.linear_packed(x, gs, packed, N, 1.0, capi.packed_workspace(M, N, K, "cuda"),
                             out_dtype=torch.float32, rcp_mode=_lib.RCP_EXACT)
    torch.cuda.synchronize()
    xc, xsf = onv.quantize_nvfp4(x.float().cpu().numpy(), 40.0)
    exact = onv.linear_f64(w, ws, xc, xsf, alpha=1.0)
    _check_rows(out.cpu().numpy(), exact, _magnitude(w, ws, xc, xsf))


# ---------------------------------------------------------------------------------------
# Sentinels around every output
# ---------------------------------------------------------------------------------------

def _guarded(shape, dtype, pad=4096):
    """A tensor of `shape` cut out of the middle of a larger buffer filled with a sentinel."""
    n = int(np.prod(shape))
    raw = torch.empty(n + 2 * pad, dtype=dtype, device="cuda")
    sentinel = -1024.0 if dtype.is_floating_point else 77          # exactly representable in bf16
    raw.fill_(sentinel)
    view = raw[pad:pad + n].view(*shape)

    def intact():
        torch.cuda.synchronize()
        return bool((raw[:pad] == sentinel).all()) and bool((raw[pad + n:] == sentinel).all())

    return view, intact


@pytest.mark.parametrize("M,N,K", [(1, 1000, 320), (3, 4096, 1024), (8, 6144, 4096), (5, 1280, 5120)])
def test_outputs_stay_inside_their_buffers(capi, M, N, K):
    from reset_b200 import _lib
    w, ws = onv.random_nvfp4((N,), K, seed=N % 31)
    wd, wsd = cuda(w), cuda(ws)
    x = make_activation(M, K, seed=M).cuda()
    gs = torch.tensor([30.0], dtype=torch.float32, device="cuda")
    # stand-alone quantizer: codes and scales
    codes, codes_ok = _guarded((M, K // 2), torch.uint8)
    scales, scales_ok = _guarded((M, K // 16), torch.uint8)
    st = _lib.lib().nvfp4r_quant(x.data_ptr(), x.stride(0), M, K, gs.data_ptr(), codes.data_ptr(),
                                 scales.data_ptr(), 0, _lib.RCP_EXACT, torch.cuda.current_stream().cuda_stream)
    assert st == 0 and codes_ok() and scales_ok()
    xc, xsf = onv.quantize_nvfp4(x.float().cpu().numpy(), 30.0)
    assert np.array_equal(codes.cpu().numpy(), xc) and np.array_equal(scales.cpu().numpy(), xsf)
    exact = onv.linear_f64(w, ws, xc, xsf, alpha=0.25)
    # fused CUDA-core linear
    out, out_ok = _guarded((M, N), torch.bfloat16)
    capi.linear(x, gs, wd, wsd, 0.25, out=out, rcp_mode=_lib.RCP_EXACT)
    assert out_ok() and rel_l2(out.float().cpu().numpy(), exact) <= 6e-3
    # packed tensor-core linear (where the shape allows it)
    if N % 128 == 0 and K % 128 == 0:
        out2, out2_ok = _guarded((M, N), torch.bfloat16)
        wk, wk_ok = _guarded((int(_lib.lib().nvfp4r_linear_packed_workspace_bytes(M, N, K)) // 8 + 2,), torch.int64,
                             pad=512)
        wk.zero_()
        capi.linear_packed(x, gs, capi.pack_weight(wd, wsd), N, 0.25, wk, rcp_mode=_lib.RCP_EXACT, out=out2)
        assert out2_ok() and wk_ok() and rel_l2(out2.float().cpu().numpy(), exact) <= 6e-3
        assert bool((wk == 0).all())                     # the split-K scratch is left all zero
    assert _lib.lib().nvfp4r_check_device_status() == 0
