"""GPU parity of the fused quantize+GEMV (``nvfp4r_linear``)."""

from __future__ import annotations

import zlib

import numpy as np
import pytest
import torch

from oracle import nvfp4 as onv
from helpers import cuda, make_activation, make_weight, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from reset_b200 import capi as c
    return c


QWEN3_8B = {"qkv_proj": (6144, 4096), "o_proj": (4096, 4096),
            "gate_up_proj": (24576, 4096), "down_proj": (4096, 12288)}


@pytest.mark.parametrize("name", list(QWEN3_8B))
@pytest.mark.parametrize("M", [1, 2, 4, 8])
def test_linear_qwen3_8b_shapes(capi, name, M):
    """The Qwen3-8B decode linears incl. activation quantization.
    Row count is cut to 512 rows of the full N for the oracle's sake; the full-N
    case is covered by the property test below."""
    N, K = QWEN3_8B[name]
    Nt = 512
    wc, wsf, gs_w = make_weight(Nt, K, seed=zlib.crc32(f"{name}{M}w".encode()) % 1000)
    xb = make_activation(M, K, seed=zlib.crc32(f"{name}{M}x".encode()) % 1000)
    gs_x = onv.global_scale_for(xb.float().numpy())
    gs_inv = float(np.float32(1.0) / np.float32(gs_x))
    alpha = gs_w * gs_x
    gs = torch.tensor([gs_inv], dtype=torch.float32, device="cuda")
    out = capi.linear(xb.cuda(), gs, cuda(wc), cuda(wsf), alpha, out_dtype=torch.float32)
    torch.cuda.synchronize()
    xc, xsf = onv.quantize_nvfp4(xb.float().numpy(), gs_inv)
    exact = onv.linear_f64(wc, wsf, xc, xsf, alpha=alpha)
    assert rel_l2(out.cpu().numpy(), exact) <= 1e-3
    assert rel_l2(out.cpu().numpy(), exact) <= 1e-5
    out_bf = capi.linear(xb.cuda(), gs, cuda(wc), cuda(wsf), alpha)
    assert out_bf.dtype == torch.bfloat16
    ref_bf = torch.from_numpy(exact.astype(np.float32)).to(torch.bfloat16).float().numpy()
    diff = np.abs(out_bf.float().cpu().numpy() - ref_bf)
    ulp = np.abs(ref_bf) * 2.0 ** -7             # >= one bf16 ulp of the reference value
    rms = float(np.sqrt(np.mean(exact ** 2)))
    assert np.all(diff <= np.maximum(ulp, 1e-5 * rms))


@pytest.mark.parametrize("N,K,M", [(24576, 4096, 1), (4096, 12288, 8), (6144, 4096, 3), (5120, 3200, 2)])
def test_linear_equals_quant_then_gemv_full_size(capi, N, K, M):
    """Size-independent property at full size: the fused launch gives bit-identical
    output to nvfp4r_quant followed by nvfp4r_gemv on the same inputs."""
    w, ws = onv.random_nvfp4((N,), K, seed=3)
    xb = make_activation(M, K, seed=4).cuda()
    gs = torch.tensor([123.0], dtype=torch.float32, device="cuda")
    wd, wsd = cuda(w), cuda(ws)
    fused = capi.linear(xb, gs, wd, wsd, 0.5, out_dtype=torch.float32)
    xc, xsf = capi.quant(xb, gs)
    out = torch.empty((M, N), dtype=torch.float32, device="cuda")
    capi.gemv_out(wd.unsqueeze(0).expand(M, -1, -1), wsd.unsqueeze(0).expand(M, -1, -1),
                  xc.view(M, 1, -1), xsf.view(M, 1, -1), out, 0.5)
    torch.cuda.synchronize()
    assert torch.equal(fused, out)


def test_linear_m_above_eight_and_strided_x(capi):
    N, K, M = 256, 2048, 13
    w, ws = onv.random_nvfp4((N,), K, seed=5)
    big = make_activation(M, 2 * K, seed=6).cuda()
    xb = big[:, K:]
    gs = torch.tensor([77.0], dtype=torch.float32, device="cuda")
    out = capi.linear(xb, gs, cuda(w), cuda(ws), 1.0, out_dtype=torch.float32)
    torch.cuda.synchronize()
    xc, xsf = onv.quantize_nvfp4(xb.cpu().float().numpy(), 77.0)
    assert rel_l2(out.cpu().numpy(), onv.linear_f64(w, ws, xc, xsf)) <= 1e-5


def test_linear_rejects_m_above_limit(capi):
    from reset_b200 import _lib
    w, ws = onv.random_nvfp4((8,), 64, seed=1)
    xb = make_activation(17, 64, seed=2).cuda()
    gs = torch.tensor([1.0], dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.Nvfp4rError):
        capi.linear(xb, gs, cuda(w), cuda(ws), 1.0)


@pytest.mark.parametrize("N,K,M", [(4096, 1024, 1), (6144, 4096, 2), (1024, 4096, 8)])
def test_linear_auto_out_variant(N, K, M):
    """`linear_auto(..., out=buf)` writes the same bits into a caller-owned buffer as the
    allocating call returns, on both sides of the crossover."""
    from reset_b200 import nvfp4r
    w, ws = onv.random_nvfp4((N,), K, seed=31)
    wd, wsd = cuda(w), cuda(ws)
    packed = nvfp4r.pack_weight(wd, wsd)
    x = make_activation(M, K, seed=32).cuda()
    gs = torch.tensor([50.0], dtype=torch.float32, device="cuda")
    want = nvfp4r.linear_auto(x, gs, wd, wsd, packed, N, 0.75, torch.bfloat16)
    buf = torch.full((M + 1, N), 7.0, dtype=torch.bfloat16, device="cuda")
    got = nvfp4r.linear_auto(x, gs, wd, wsd, packed, N, 0.75, torch.bfloat16, out=buf[:M])
    torch.cuda.synchronize()
    assert got.data_ptr() == buf.data_ptr()
    assert torch.equal(buf[:M], want) and bool((buf[M] == 7.0).all())


@pytest.mark.parametrize("N,K,with_delta", [(1536, 5120, True), (1280, 5120, False), (300, 3200, True), (4096, 12288, True)])
def test_gemv_fused_add_rmsnorm_prologue(capi, N, K, with_delta):
    """``nvfp4r_linear_ex`` with the add + RMSNorm prologue on the CUDA-core GEMV (flat weight, one
    token): the residual stream is bit-identical to the separate add_rmsnorm kernel; the output
    agrees with the oracle and with the packed linear's fused prologue up to the bf16 roundings
    that a different summation order of the mean square can flip."""
    from reset_b200 import _lib
    w, ws = onv.random_nvfp4((N,), K, seed=31)
    g = torch.Generator(device="cuda").manual_seed(32)
    res = torch.randn(1, K, device="cuda", generator=g).to(torch.bfloat16)
    delta = torch.randn(1, K, device="cuda", generator=g).to(torch.bfloat16) if with_delta else None
    nw = (1 + 0.1 * torch.randn(K, device="cuda", generator=g)).to(torch.bfloat16)
    gs = torch.tensor([40.0], dtype=torch.float32, device="cuda")
    res_out = torch.zeros_like(res)
    out = torch.full((1, N), float("nan"), dtype=torch.float32, device="cuda")
    capi.linear_rmsnorm(delta, res, res_out, nw, 1e-6, gs, cuda(w), cuda(ws), 0.5, out, rcp_mode=_lib.RCP_EXACT)
    torch.cuda.synchronize()
    want_res = (res.float() + delta.float()).to(torch.bfloat16) if with_delta else res
    assert torch.equal(res_out, want_res)
    f = want_res.float()
    normed = (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()).to(torch.bfloat16)
    xc, xsf = onv.quantize_nvfp4(normed.float().cpu().numpy(), 40.0)
    assert rel_l2(out.cpu().numpy(), onv.linear_f64(w, ws, xc, xsf, alpha=0.5)) <= 5e-3
    # the separate operators of this library
    r2, normed2 = res.clone(), torch.empty_like(res)
    _lib.check(_lib.lib().nvfp4r_add_rmsnorm(None if delta is None else delta.data_ptr(), r2.data_ptr(),
                                             nw.data_ptr(), normed2.data_ptr(), 1, K, 1e-6,
                                             torch.cuda.current_stream().cuda_stream), "add_rmsnorm")
    unfused = capi.linear(normed2, gs, cuda(w), cuda(ws), 0.5, out_dtype=torch.float32, rcp_mode=_lib.RCP_EXACT)
    torch.cuda.synchronize()
    assert torch.equal(r2, res_out)
    assert rel_l2(out.cpu().numpy(), unfused.cpu().numpy()) <= 5e-3


@pytest.mark.parametrize("N,K", [(1024, 3072), (5120, 3200), (640, 25600)])
def test_gemv_fused_silu_mul_prologue(capi, N, K):
    """silu(gate) * up computed in the GEMV's prologue: same arithmetic and roundings as the
    separate silu_mul kernel, so the result is bit-identical to silu_mul + linear."""
    from reset_b200 import _lib
    w, ws = onv.random_nvfp4((N,), K, seed=33)
    g = torch.Generator(device="cuda").manual_seed(34)
    gu = torch.randn(1, 2 * K, device="cuda", generator=g).to(torch.bfloat16)
    gs = torch.tensor([30.0], dtype=torch.float32, device="cuda")
    out = torch.full((1, N), float("nan"), dtype=torch.float32, device="cuda")
    _lib.check(_lib.lib().nvfp4r_set_gemv_rows_tuning(1, 0, 0), "rows")      # the same kernel on both sides
    try:
        capi.linear_silu(gu, gs, cuda(w), cuda(ws), 1.0, out, rcp_mode=_lib.RCP_EXACT)
        act = torch.empty(1, K, dtype=torch.bfloat16, device="cuda")
        _lib.check(_lib.lib().nvfp4r_silu_mul(gu.data_ptr(), act.data_ptr(), 1, K,
                                              torch.cuda.current_stream().cuda_stream), "silu")
        unfused = capi.linear(act, gs, cuda(w), cuda(ws), 1.0, out_dtype=torch.float32, rcp_mode=_lib.RCP_EXACT)
        torch.cuda.synchronize()
    finally:
        _lib.check(_lib.lib().nvfp4r_set_gemv_rows_tuning(0, 0, 0), "rows")
    assert torch.equal(out, unfused)
    ref_act = (torch.nn.functional.silu(gu[:, :K].float()) * gu[:, K:].float()).to(torch.bfloat16)
    xc, xsf = onv.quantize_nvfp4(ref_act.float().cpu().numpy(), 30.0)
    assert rel_l2(out.cpu().numpy(), onv.linear_f64(w, ws, xc, xsf)) <= 5e-3


def test_gemv_fused_prologue_argument_checks(capi):
    from reset_b200 import _lib
    w, ws = onv.random_nvfp4((128,), 256, seed=1)
    res = torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda")
    res2 = torch.zeros(2, 256, dtype=torch.bfloat16, device="cuda")
    nw = torch.ones(256, dtype=torch.bfloat16, device="cuda")
    gs = torch.tensor([1.0], dtype=torch.float32, device="cuda")
    out = torch.zeros(1, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.Nvfp4rError):
        capi.linear_rmsnorm(None, res, res, nw, 1e-6, gs, cuda(w), cuda(ws), 1.0, out)          # aliasing
    with pytest.raises(_lib.Nvfp4rError):
        capi.linear_rmsnorm(None, res2, torch.zeros_like(res2), nw, 1e-6, gs, cuda(w), cuda(ws), 1.0,
                            torch.zeros(2, 128, dtype=torch.bfloat16, device="cuda"))          # two tokens
