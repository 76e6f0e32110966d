"""GPU parity of the packed-weight tensor-core linear (``nvfp4r_pack_weight`` +
``nvfp4r_linear_packed``), the adapter's product path, against the CPU oracle:
rel-L2 <= 1e-3 stated (fp32 output vs float64 dequantise-matmul), ~1e-7 measured."""

from __future__ import annotations

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


@pytest.fixture(autouse=True)
def _auto_tuning():
    from reset_b200 import _lib
    yield
    _lib.lib().nvfp4r_set_packed_tuning(0)


def _oracle_pack(w, ws):
    """Packed layout restated on the CPU: block (tile, kb) = 16 KB of 128B-swizzled codes
    followed by 4 chunks of 512 B scales in [row%32][row//32][4] order."""
    N, K2 = w.shape
    K = K2 * 2
    out = np.zeros((N // 128, K // 256, 18432), dtype=np.uint8)
    rows = np.arange(128)
    for t in range(N // 128):
        for kb in range(K // 256):
            blk = w[t * 128:(t + 1) * 128, kb * 128:(kb + 1) * 128]          # [128 rows, 128 B]
            for u in range(8):
                dst = (rows // 8) * 1024 + (rows % 8) * 128 + ((u ^ (rows % 8)) * 16)
                for b in range(16):
                    out[t, kb, dst + b] = blk[:, u * 16 + b]
            sf = ws[t * 128:(t + 1) * 128, kb * 16:(kb + 1) * 16]             # [128, 16]
            for ch in range(4):
                for j in range(4):
                    out[t, kb, 16384 + ch * 512 + (rows % 32) * 16 + (rows // 32) * 4 + j] = sf[:, ch * 4 + j]
    return out.reshape(-1)


def test_pack_weight_layout(capi):
    w, ws = onv.random_nvfp4((256,), 512, seed=1)
    got = capi.pack_weight(cuda(w), cuda(ws)).cpu().numpy()
    assert np.array_equal(got, _oracle_pack(w, ws))


@pytest.mark.parametrize("N,K", [(128, 256), (256, 768), (4096, 4096), (6144, 4096), (1280, 5120),
                                 (4096, 12288), (512, 25600), (24576, 4096), (896, 5120),
                                 # tensor-parallel shards of the bench's Qwen3-8B set (TP 4 / 8)
                                 (768, 4096), (4096, 512), (3072, 4096), (4096, 1536), (4096, 1024),
                                 (6144, 4096), (4096, 3072),
                                 # rows that end in the middle of a 256-element block: the row-parallel
                                 # shards of Qwen3-32B (TP 8: 3200) and Qwen3-14B (TP 8: 640, 2176)
                                 (128, 128), (256, 384), (5120, 3200), (5120, 640), (5120, 2176)])
@pytest.mark.parametrize("M", [1, 8])
def test_linear_packed_matches_oracle(capi, N, K, M):
    w, ws = onv.random_nvfp4((N,), K, seed=N % 89 + M)
    xb = make_activation(M, K, seed=K % 97 + M)
    gs_inv = 64.0
    gs = torch.tensor([gs_inv], dtype=torch.float32, device="cuda")
    packed = capi.pack_weight(cuda(w), cuda(ws))
    wksp = capi.packed_workspace(M, N, K, "cuda")
    out = capi.linear_packed(xb.cuda(), gs, packed, N, 0.25, wksp, out_dtype=torch.float32)
    out2 = capi.linear_packed(xb.cuda(), gs, packed, N, 0.25, wksp, out_dtype=torch.float32)
    torch.cuda.synchronize()
    xc, xsf = onv.quantize_nvfp4(xb.float().numpy(), gs_inv)
    err = rel_l2(out.cpu().numpy(), onv.linear_f64(w, ws, xc, xsf, alpha=0.25))
    assert err <= 1e-3 and err <= 1e-5, err
    assert torch.equal(out, out2)                       # scratch reusable, deterministic


@pytest.mark.parametrize("M", [2, 3, 5, 16, 17, 31, 32, 33, 70])
def test_linear_packed_token_counts(capi, M):
    N, K = 384, 2048
    w, ws = onv.random_nvfp4((N,), K, seed=3)
    xb = make_activation(M, K, seed=4)
    gs = torch.tensor([50.0], dtype=torch.float32, device="cuda")
    packed = capi.pack_weight(cuda(w), cuda(ws))
    wksp = capi.packed_workspace(M, N, K, "cuda")
    out = capi.linear_packed(xb.cuda(), gs, packed, N, 1.0, wksp, out_dtype=torch.float32)
    torch.cuda.synchronize()
    xc, xsf = onv.quantize_nvfp4(xb.float().numpy(), 50.0)
    assert rel_l2(out.cpu().numpy(), onv.linear_f64(w, ws, xc, xsf)) <= 1e-5


@pytest.mark.parametrize("splits", [2, 3, 5, 8, 16])
def test_linear_packed_every_split_agrees(capi, splits):
    from reset_b200 import _lib
    N, K, M = 1024, 4096, 4
    w, ws = onv.random_nvfp4((N,), K, seed=5)
    xb = make_activation(M, K, seed=6).cuda()
    gs = torch.tensor([80.0], dtype=torch.float32, device="cuda")
    packed = capi.pack_weight(cuda(w), cuda(ws))
    big = torch.zeros(8 << 20, dtype=torch.int64, device="cuda")
    ref = capi.linear_packed(xb, gs, packed, N, 1.0, big, out_dtype=torch.float32)
    _lib.check(_lib.lib().nvfp4r_set_packed_tuning(splits), "tuning")
    a = capi.linear_packed(xb, gs, packed, N, 1.0, big, out_dtype=torch.float32)
    b = capi.linear_packed(xb, gs, packed, N, 1.0, big, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    assert rel_l2(a.cpu().numpy(), ref.cpu().numpy()) <= 1e-6


def test_linear_packed_equals_cuda_core_linear_config1(capi):
    """The Qwen3-8B linear set at full size: tensor-core path vs CUDA-core path on the
    same quantized weights (bf16 N(0,0.02)) and activations (N(0,1) + outliers)."""
    for name, (N, K) in {"qkv": (6144, 4096), "down": (4096, 12288)}.items():
        wc, wsf, gs_w = make_weight(N, K, seed=7)
        for M in (1, 4):
            xb = make_activation(M, K, seed=8 + M)
            gs_x = onv.global_scale_for(xb.float().numpy())
            gs = torch.tensor([1.0 / gs_x], dtype=torch.float32, device="cuda")
            packed = capi.pack_weight(cuda(wc), cuda(wsf))
            wksp = capi.packed_workspace(M, N, K, "cuda")
            a = capi.linear_packed(xb.cuda(), gs, packed, N, gs_w * gs_x, wksp, out_dtype=torch.float32)
            b = capi.linear(xb.cuda(), gs, cuda(wc), cuda(wsf), gs_w * gs_x, out_dtype=torch.float32)
            torch.cuda.synchronize()
            assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) <= 1e-6, (name, M)


def test_linear_packed_bf16_and_approx_mode(capi):
    from reset_b200 import _lib
    N, K, M = 512, 2048, 3
    w, ws = onv.random_nvfp4((N,), K, seed=9)
    xb = make_activation(M, K, seed=10).cuda()
    gs = torch.tensor([44.0], dtype=torch.float32, device="cuda")
    packed = capi.pack_weight(cuda(w), cuda(ws))
    wksp = capi.packed_workspace(M, N, K, "cuda")
    out = capi.linear_packed(xb, gs, packed, N, 1.0, wksp, rcp_mode=_lib.RCP_APPROX)
    assert out.dtype == torch.bfloat16
    xc, xsf = capi.quant(xb, gs, rcp_mode=_lib.RCP_APPROX)
    exact = onv.linear_f64(w, ws, xc.cpu().numpy(), xsf.cpu().numpy())
    assert rel_l2(out.float().cpu().numpy(), exact) <= 4e-3           # bf16 output rounding


def test_packed_rejects_bad_shapes(capi):
    w, ws = onv.random_nvfp4((100,), 256, seed=1)
    with pytest.raises(ValueError):
        capi.pack_weight(cuda(w), cuda(ws))


@pytest.mark.parametrize("splits", [2, 3, 8])
@pytest.mark.parametrize("M", [1, 5, 16])
def test_linear_packed_forced_splits(capi, splits, M):
    """Split-K hand-over through the self-validating slots: any forced split count gives the
    unsplit result up to fp32 summation order, twice in a row bit-identically, and leaves the
    workspace all zero (the contract that lets linears share one workspace)."""
    from reset_b200 import _lib
    N, K = 1024, 4096
    w, ws = onv.random_nvfp4((N,), K, seed=15)
    xb = make_activation(M, K, seed=16).cuda()
    gs = torch.tensor([80.0], dtype=torch.float32, device="cuda")
    packed = capi.pack_weight(cuda(w), cuda(ws))
    big = torch.zeros(1 << 20, dtype=torch.int64, device="cuda")
    try:
        _lib.check(_lib.lib().nvfp4r_set_packed_tuning(2), "tuning")     # K = 4096 needs at least 2 parts
        ref = capi.linear_packed(xb, gs, packed, N, 1.0, big, out_dtype=torch.float32)
        _lib.check(_lib.lib().nvfp4r_set_packed_tuning(splits), "tuning")
        a = capi.linear_packed(xb, gs, packed, N, 1.0, big, out_dtype=torch.float32)
        b = capi.linear_packed(xb, gs, packed, N, 1.0, big, out_dtype=torch.float32)
        torch.cuda.synchronize()
    finally:
        _lib.check(_lib.lib().nvfp4r_set_packed_tuning(0), "tuning")
    assert torch.equal(a, b)
    assert rel_l2(a.cpu().numpy(), ref.cpu().numpy()) <= 1e-6
    assert int(big.count_nonzero().item()) == 0
    _lib.check(_lib.lib().nvfp4r_check_device_status(), "device status")


@pytest.mark.parametrize("M,with_delta", [(1, True), (1, False), (5, True)])
def test_fused_add_rmsnorm_prologue(capi, M, with_delta):
    """linear(RMSNorm(residual + delta) * w) in one launch vs the separate operators: the
    residual stream is bit-identical; the linear output agrees up to the bf16 roundings
    that a different summation order of the mean square can flip (a handful of codes)."""
    from reset_b200 import _lib
    N, K = 1536, 5120
    w, ws = onv.random_nvfp4((N,), K, seed=21)
    packed = capi.pack_weight(cuda(w), cuda(ws))
    g = torch.Generator(device="cuda").manual_seed(22)
    res = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    delta = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16) if with_delta else None
    nw = (1 + 0.1 * torch.randn(K, device="cuda", generator=g)).to(torch.bfloat16)
    gs = torch.tensor([40.0], dtype=torch.float32, device="cuda")
    wksp = capi.packed_workspace(M, N, K, "cuda")
    res_out = torch.zeros_like(res)
    fused = capi.linear_packed_rmsnorm(delta, res, res_out, nw, 1e-6, gs, packed, N, 0.5, wksp,
                                       out_dtype=torch.float32, rcp_mode=_lib.RCP_EXACT)
    torch.cuda.synchronize()
    want_res = (res.float() + delta.float()).to(torch.bfloat16) if with_delta else res
    assert torch.equal(res_out, want_res)
    f = want_res.float()
    normed = (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()).to(torch.bfloat16)
    xc, xsf = onv.quantize_nvfp4(normed.float().cpu().numpy(), 40.0)
    exact = onv.linear_f64(w, ws, xc, xsf, alpha=0.5)
    assert rel_l2(fused.cpu().numpy(), exact) <= 5e-3
    # and against the unfused kernels of this library
    normed2 = torch.empty_like(res)
    r2 = res.clone()
    lib = _lib.lib()
    _lib.check(lib.nvfp4r_add_rmsnorm(None if delta is None else delta.data_ptr(), r2.data_ptr(), nw.data_ptr(),
                                      normed2.data_ptr(), M, K, 1e-6, torch.cuda.current_stream().cuda_stream), "n")
    unfused = capi.linear_packed(normed2, gs, packed, N, 0.5, wksp, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(r2, res_out)
    assert rel_l2(fused.cpu().numpy(), unfused.cpu().numpy()) <= 5e-3


@pytest.mark.parametrize("M", [1, 4])
@pytest.mark.parametrize("N,K", [(1024, 3072), (5120, 3200)])          # 3200: ends inside a block
def test_fused_silu_mul_prologue(capi, M, N, K):
    from reset_b200 import _lib
    w, ws = onv.random_nvfp4((N,), K, seed=23)
    packed = capi.pack_weight(cuda(w), cuda(ws))
    g = torch.Generator(device="cuda").manual_seed(24)
    gu = torch.randn(M, 2 * K, device="cuda", generator=g).to(torch.bfloat16)
    gs = torch.tensor([30.0], dtype=torch.float32, device="cuda")
    wksp = capi.packed_workspace(M, N, K, "cuda")
    fused = capi.linear_packed_silu(gu, gs, packed, N, 1.0, wksp, out_dtype=torch.float32,
                                    rcp_mode=_lib.RCP_EXACT)
    act = torch.empty(M, K, dtype=torch.bfloat16, device="cuda")
    _lib.check(_lib.lib().nvfp4r_silu_mul(gu.data_ptr(), act.data_ptr(), M, K,
                                          torch.cuda.current_stream().cuda_stream), "silu")
    unfused = capi.linear_packed(act, gs, packed, N, 1.0, wksp, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(fused, unfused)          # same arithmetic, same roundings
    ref_act = (torch.nn.functional.silu(gu[:, :K].float()) * gu[:, K:].float()).to(torch.bfloat16)
    xc, xsf = onv.quantize_nvfp4(ref_act.float().cpu().numpy(), 30.0)
    assert rel_l2(fused.cpu().numpy(), onv.linear_f64(w, ws, xc, xsf)) <= 5e-3


def test_fused_prologue_argument_checks(capi):
    from reset_b200 import _lib
    w, ws = onv.random_nvfp4((128,), 256, seed=1)
    packed = capi.pack_weight(cuda(w), cuda(ws))
    res = torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda")
    nw = torch.ones(256, dtype=torch.bfloat16, device="cuda")
    gs = torch.tensor([1.0], dtype=torch.float32, device="cuda")
    wk = capi.packed_workspace(1, 128, 256, "cuda")
    with pytest.raises(_lib.Nvfp4rError):
        capi.linear_packed_rmsnorm(None, res, res, nw, 1e-6, gs, packed, 128, 1.0, wk)   # aliasing
