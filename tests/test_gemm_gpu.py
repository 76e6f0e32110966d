"""GPU parity of the tensor-core path (``nvfp4r_linear_tc`` / ``nvfp4r_gemm``) against
the CPU oracle. The tcgen05 block-scaled MMA multiplies e2m1 codes and ue4m3 scales
exactly and accumulates in fp32; results are compared with the float64
dequantise-matmul at rel-L2 <= 1e-3 (stated tolerance; measured ~1e-7)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import nvfp4 as onv
from helpers import cuda, make_activation, rel_l2

pytestmark = pytest.mark.gpu

TOL = 1e-3


@pytest.fixture(scope="module")
def capi():
    from reset_b200 import capi as c
    return c


@pytest.fixture(autouse=True)
def _auto_tuning():
    from reset_b200 import _lib
    yield
    _lib.lib().nvfp4r_set_gemm_tuning(0, 0)


def _weights(N, K, seed):
    w, ws = onv.random_nvfp4((N,), K, seed=seed)
    return w, ws, cuda(w), cuda(onv.swizzle_blockscale(ws))


@pytest.mark.parametrize("N,K", [(128, 256), (256, 1024), (4096, 4096), (6144, 4096), (1280, 5120),
                                 (4096, 12288), (512, 25600), (24576, 4096)])
@pytest.mark.parametrize("M", [1, 8])
def test_linear_tc_matches_oracle(capi, N, K, M):
    w, ws, wd, wsd = _weights(N, K, seed=N % 89 + M)
    xb = make_activation(M, K, seed=K % 97 + M)
    gs_inv = 64.0
    gs = torch.tensor([gs_inv], dtype=torch.float32, device="cuda")
    wksp = capi.gemm_workspace(M, N, K, "cuda")
    out = capi.linear_tc(xb.cuda(), gs, wd, wsd, 0.25, wksp, out_dtype=torch.float32)
    torch.cuda.synchronize()
    xc, xsf = onv.quantize_nvfp4(xb.float().numpy(), gs_inv)
    exact = onv.linear_f64(w, ws, xc, xsf, alpha=0.25)
    err = rel_l2(out.cpu().numpy(), exact)
    assert err <= TOL, err
    assert err <= 1e-5, err
    # the scratch is left ready for the next call: a second call gives the same bits
    out2 = capi.linear_tc(xb.cuda(), gs, wd, wsd, 0.25, wksp, out_dtype=torch.float32)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("M", [2, 3, 5, 16, 17, 31, 32, 33, 70])
def test_linear_tc_token_counts(capi, M):
    N, K = 384, 2048
    w, ws, wd, wsd = _weights(N, K, seed=3)
    xb = make_activation(M, K, seed=4)
    gs = torch.tensor([50.0], dtype=torch.float32, device="cuda")
    wksp = capi.gemm_workspace(M, N, K, "cuda")
    out = capi.linear_tc(xb.cuda(), gs, wd, wsd, 1.0, wksp, out_dtype=torch.float32)
    torch.cuda.synchronize()
    xc, xsf = onv.quantize_nvfp4(xb.float().numpy(), 50.0)
    assert rel_l2(out.cpu().numpy(), onv.linear_f64(w, ws, xc, xsf)) <= 1e-5


@pytest.mark.parametrize("splits", [1, 2, 3, 5, 8, 16])
def test_linear_tc_every_split_gives_same_answer(capi, splits):
    """Split-K parts are added in part order: any split gives a result within fp32
    re-association of the unsplit one, and repeated runs are bit-identical."""
    from reset_b200 import _lib
    N, K, M = 1024, 4096, 4
    w, ws, wd, wsd = _weights(N, K, seed=5)
    xb = make_activation(M, K, seed=6).cuda()
    gs = torch.tensor([80.0], dtype=torch.float32, device="cuda")
    wksp = capi.gemm_workspace(M, N, K, "cuda")
    _lib.check(_lib.lib().nvfp4r_set_gemm_tuning(1, 0), "tuning")
    ref = capi.linear_tc(xb, gs, wd, wsd, 1.0, wksp, out_dtype=torch.float32)
    _lib.check(_lib.lib().nvfp4r_set_gemm_tuning(splits, 0), "tuning")
    big = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda").view(torch.int64)  # room for any split
    a = capi.linear_tc(xb, gs, wd, wsd, 1.0, big, out_dtype=torch.float32)
    b = capi.linear_tc(xb, gs, wd, wsd, 1.0, big, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    assert rel_l2(a.cpu().numpy(), ref.cpu().numpy()) <= 1e-6


@pytest.mark.parametrize("stages", [1, 2, 3])
def test_linear_tc_shallow_ring(capi, stages):
    """Ring shallower than the K loop: every stage is reused many times."""
    from reset_b200 import _lib
    N, K, M = 256, 8192, 2
    w, ws, wd, wsd = _weights(N, K, seed=7)
    xb = make_activation(M, K, seed=8)
    gs = torch.tensor([30.0], dtype=torch.float32, device="cuda")
    _lib.check(_lib.lib().nvfp4r_set_gemm_tuning(1, stages), "tuning")
    wksp = capi.gemm_workspace(M, N, K, "cuda")
    out = capi.linear_tc(xb.cuda(), gs, wd, wsd, 1.0, wksp, out_dtype=torch.float32)
    torch.cuda.synchronize()
    xc, xsf = onv.quantize_nvfp4(xb.float().numpy(), 30.0)
    assert rel_l2(out.cpu().numpy(), onv.linear_f64(w, ws, xc, xsf)) <= 1e-5


@pytest.mark.parametrize("M,n_major", [(1, True), (8, True), (8, False), (40, True), (64, False), (130, True)])
def test_gemm_prequantized_matches_oracle(capi, M, n_major):
    """torch.ops.nvfp4r.gemm semantics: A activations, B weights, swizzled scales, C
    buffer written N-major (kernels/python/nvfp4r/ops.py:86-88) or M-major."""
    N, K = 512, 2048
    w, ws, wd, wsd = _weights(N, K, seed=9)
    xc, xsf = onv.random_nvfp4((M,), K, seed=10)
    C = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    wksp = capi.gemm_workspace(M, N, K, "cuda")
    capi.gemm(cuda(xc), wd, cuda(onv.swizzle_blockscale(xsf)), wsd, C, 0.5, wksp, n_major=n_major)
    torch.cuda.synchronize()
    got = C.cpu().numpy()
    got = got.reshape(N, M).T if n_major else got
    assert rel_l2(got, onv.linear_f64(w, ws, xc, xsf, alpha=0.5)) <= 1e-5


def test_fused_equals_quant_then_gemm(capi):
    N, K, M = 1024, 4096, 8
    w, ws, wd, wsd = _weights(N, K, seed=11)
    xb = make_activation(M, K, seed=12).cuda()
    gs = torch.tensor([90.0], dtype=torch.float32, device="cuda")
    wksp = capi.gemm_workspace(M, N, K, "cuda")
    fused = capi.linear_tc(xb, gs, wd, wsd, 1.0, wksp, out_dtype=torch.float32)
    xc, xsf = capi.quant(xb, gs, swizzled=True)
    C = torch.empty((M, N), dtype=torch.float32, device="cuda")
    capi.gemm(xc, wd, xsf, wsd, C, 1.0, wksp, n_major=False)
    torch.cuda.synchronize()
    assert torch.equal(fused, C)


def test_tc_and_cuda_core_paths_agree(capi):
    """Same inputs through the CUDA-core GEMV and the tensor-core kernel."""
    N, K, M = 2048, 4096, 4
    w, ws, wd, wsd = _weights(N, K, seed=13)
    xb = make_activation(M, K, seed=14).cuda()
    gs = torch.tensor([70.0], dtype=torch.float32, device="cuda")
    wksp = capi.gemm_workspace(M, N, K, "cuda")
    a = capi.linear_tc(xb, gs, wd, wsd, 1.0, wksp, out_dtype=torch.float32)
    b = capi.linear(xb, gs, wd, cuda(ws), 1.0, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) <= 1e-6


def test_tc_rejects_bad_shapes(capi):
    from reset_b200 import _lib
    xb = make_activation(1, 384, seed=1).cuda()
    gs = torch.tensor([1.0], dtype=torch.float32, device="cuda")
    w = torch.zeros((128, 192), dtype=torch.uint8, device="cuda")
    sf = torch.zeros((128, 24), dtype=torch.uint8, device="cuda")
    wk = torch.zeros(1024, dtype=torch.int64, device="cuda")
    with pytest.raises(_lib.Nvfp4rError):
        capi.linear_tc(xb, gs, w, sf, 1.0, wk)                # K % 256
    xb = make_activation(1, 256, seed=1).cuda()
    w = torch.zeros((100, 128), dtype=torch.uint8, device="cuda")
    with pytest.raises(_lib.Nvfp4rError):
        capi.linear_tc(xb, gs, w, sf, 1.0, wk)                # N % 128
