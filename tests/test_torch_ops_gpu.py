"""The reference's operator surface on the GPU: ``torch.ops.nvfp4r.gemv`` / ``gemm`` and the
``nvfp4r.gemv()`` / ``nvfp4r.gemm()`` wrappers (kernels/csrc/bindings.cpp:27-121,
kernels/python/nvfp4r/ops.py:23-88), called the way the reference's own tests call them
(kernels/tests/test_gemv.py:30-66) and compared with the CPU oracle.

Tolerances: float32 outputs rel-L2 <= 1e-5 against the float64 dequantise-matmul (stated bar
1e-3); float16 / bfloat16 outputs under the reference's criterion, max relative error
< 5e-2 or max absolute error < 1.0 (test_gemv.py:46-50)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import nvfp4 as onv
from helpers import cuda, rel_l2

pytestmark = pytest.mark.gpu

# (L, N, K) of the reference's own test (kernels/tests/test_gemv.py:14-28)
REFERENCE_SHAPES = [
    (1, 256, 4096), (1, 1024, 8192), (1, 2048, 16384), (4, 512, 2048), (8, 512, 7168),
    (2, 4096, 4096), (1, 4608, 3584), (1, 3584, 3584), (1, 3584, 18944), (1, 6144, 4096),
    (1, 4096, 4096), (1, 4096, 12288),
]


@pytest.fixture(scope="module")
def nvfp4r():
    from reset_b200 import nvfp4r as pkg
    return pkg


def _reference_criterion(got: np.ndarray, exact: np.ndarray) -> None:
    diff = np.abs(got.astype(np.float64) - exact)
    rel = diff / (np.abs(exact) + 1e-3)
    assert rel.max() < 5e-2 or diff.max() < 1.0, (diff.max(), rel.max())


@pytest.mark.parametrize("L,N,K", REFERENCE_SHAPES)
def test_gemv_op_broadcast_weight(nvfp4r, L, N, K):
    """One weight expanded over L tokens (stride 0), the layout the adapter passes
    (kernels/python/nvfp4r/vllm_integration.py:216-219)."""
    w, ws = onv.random_nvfp4((N,), K, seed=0)
    x, xs = onv.random_nvfp4((L, 1), K, seed=1)
    exact = onv.linear_f64(w, ws, x[:, 0], xs[:, 0], alpha=0.5)
    wd = cuda(w).unsqueeze(0).expand(L, -1, -1)
    wsd = cuda(ws).unsqueeze(0).expand(L, -1, -1)
    assert L == 1 or wd.stride(0) == 0
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        out = torch.full((L, N), float("nan"), dtype=dtype, device="cuda")
        ptr = out.data_ptr()
        ret = torch.ops.nvfp4r.gemv(wd, wsd, cuda(x), cuda(xs), out, 0.5)
        torch.cuda.synchronize()
        assert ret is None and out.data_ptr() == ptr
        got = out.float().cpu().numpy()
        if dtype == torch.float32:
            assert rel_l2(got, exact) <= 1e-5
        else:
            _reference_criterion(got, exact)


@pytest.mark.parametrize("L,N,K", [(4, 512, 2048), (2, 1024, 4096), (3, 96, 3584)])
def test_gemv_op_one_weight_per_token(nvfp4r, L, N, K):
    """Distinct weights along L, as the reference's test builds them
    (kernels/tests/test_gemv.py:35-38, ``random_nvfp4_tensor((L, M), K)``)."""
    w, ws = onv.random_nvfp4((L, N), K, seed=2)
    x, xs = onv.random_nvfp4((L, 1), K, seed=3)
    out = torch.full((L, N), float("nan"), dtype=torch.float32, device="cuda")
    torch.ops.nvfp4r.gemv(cuda(w), cuda(ws), cuda(x), cuda(xs), out, 1.0)
    torch.cuda.synchronize()
    for l in range(L):
        exact = onv.linear_f64(w[l], ws[l], x[l], xs[l])
        assert rel_l2(out[l].cpu().numpy(), exact[0]) <= 1e-5


def test_gemv_op_reads_row_zero_of_padded_x(nvfp4r):
    """x may carry padding rows along its middle dimension; only row 0 is read
    (kernels/csrc/bindings.cpp:77-81)."""
    L, N, K, P = 2, 384, 4096, 8
    w, ws = onv.random_nvfp4((N,), K, seed=4)
    x, xs = onv.random_nvfp4((L, P), K, seed=5)
    out = torch.empty((L, N), dtype=torch.float32, device="cuda")
    torch.ops.nvfp4r.gemv(cuda(w).unsqueeze(0).expand(L, -1, -1), cuda(ws).unsqueeze(0).expand(L, -1, -1),
                          cuda(x), cuda(xs), out, 1.0)
    torch.cuda.synchronize()
    assert rel_l2(out.cpu().numpy(), onv.linear_f64(w, ws, x[:, 0], xs[:, 0])) <= 1e-5


def test_gemv_writes_into_provided_out(nvfp4r):
    """The out-variant contract exactly as kernels/tests/test_gemv.py:56-66 states it."""
    L, N, K = 1, 256, 4096
    w, ws = onv.random_nvfp4((L, N), K, seed=2)
    x, xs = onv.random_nvfp4((L, 1), K, seed=3)
    out = torch.empty((L, N), dtype=torch.float16, device="cuda")
    before = out.data_ptr()
    ret = torch.ops.nvfp4r.gemv(cuda(w), cuda(ws), cuda(x), cuda(xs), out)
    assert ret is None
    assert out.data_ptr() == before
    assert torch.isfinite(out).all().item()


def test_gemv_wrapper_defaults(nvfp4r):
    """``nvfp4r.gemv``: 2-D operands gain L = 1, the default result is float16 [L, N]
    (kernels/python/nvfp4r/ops.py:23-58)."""
    N, K = 1024, 4096
    w, ws = onv.random_nvfp4((N,), K, seed=6)
    x, xs = onv.random_nvfp4((1,), K, seed=7)
    y = nvfp4r.gemv(cuda(w), cuda(ws), cuda(x), cuda(xs))
    torch.cuda.synchronize()
    assert y.shape == (1, N) and y.dtype == torch.float16
    _reference_criterion(y.float().cpu().numpy(), onv.linear_f64(w, ws, x, xs))
    out = torch.empty((1, N), dtype=torch.bfloat16, device="cuda")
    y2 = nvfp4r.gemv(cuda(w), cuda(ws), cuda(x), cuda(xs), out=out, alpha=2.0)
    assert y2.data_ptr() == out.data_ptr()
    _reference_criterion(y2.float().cpu().numpy(), onv.linear_f64(w, ws, x, xs, alpha=2.0))


def test_gemv_op_rejects_what_the_reference_rejects(nvfp4r):
    N, K = 256, 1024
    w, ws = onv.random_nvfp4((1, N), K, seed=8)
    x, xs = onv.random_nvfp4((1, 1), K, seed=9)
    out = torch.empty((1, N), dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):       # 2-D operands (bindings.cpp:45-48)
        torch.ops.nvfp4r.gemv(cuda(w)[0], cuda(ws)[0], cuda(x), cuda(xs), out, 1.0)
    with pytest.raises(RuntimeError):       # out of the wrong shape (bindings.cpp:69-72)
        torch.ops.nvfp4r.gemv(cuda(w), cuda(ws), cuda(x), cuda(xs), out[:, :128].contiguous(), 1.0)
    with pytest.raises(RuntimeError):       # integer out
        torch.ops.nvfp4r.gemv(cuda(w), cuda(ws), cuda(x), cuda(xs), out.to(torch.int32), 1.0)
    with pytest.raises(RuntimeError):       # scale / weight shape mismatch
        torch.ops.nvfp4r.gemv(cuda(w), cuda(ws)[:, :, :32].contiguous(), cuda(x), cuda(xs), out, 1.0)


@pytest.mark.parametrize("M,N,K", [(64, 512, 2048), (128, 1024, 4096), (64, 256, 5120), (8, 384, 1024)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_op_and_wrapper(nvfp4r, M, N, K, dtype):
    """``torch.ops.nvfp4r.gemm`` writes C's buffer N-major; ``nvfp4r.gemm`` returns the
    ``C.view(N, M).T`` view (kernels/python/nvfp4r/ops.py:62-88)."""
    w, ws = onv.random_nvfp4((N,), K, seed=10)
    a, a_s = onv.random_nvfp4((M,), K, seed=11)
    exact = onv.linear_f64(w, ws, a, a_s, alpha=0.25)
    A, B = cuda(a), cuda(w)
    SFA, SFB = cuda(onv.swizzle_blockscale(a_s)), cuda(onv.swizzle_blockscale(ws))
    C = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
    ptr = C.data_ptr()
    ret = torch.ops.nvfp4r.gemm(A, B, SFA, SFB, C, 0.25)
    torch.cuda.synchronize()
    assert ret is None and C.data_ptr() == ptr
    _reference_criterion(C.view(N, M).T.float().cpu().numpy(), exact)
    C2 = torch.empty((M, N), dtype=dtype, device="cuda")
    y = nvfp4r.gemm(A, B, SFA, SFB, C2, 0.25)
    torch.cuda.synchronize()
    assert y.shape == (M, N) and y.data_ptr() == C2.data_ptr() and y.stride() == (1, M)
    assert torch.equal(y.contiguous(), C.view(N, M).T.contiguous())
    assert rel_l2(y.float().cpu().numpy(), exact) <= 5e-3      # one rounding to 16 bits


def test_gemm_op_accepts_the_packed_dtypes(nvfp4r):
    """Codes as ``float4_e2m1fn_x2`` and scales as ``float8_e4m3fn`` views, as vLLM holds
    them (kernels/csrc/bindings.cpp:15-25)."""
    if not hasattr(torch, "float4_e2m1fn_x2"):
        pytest.skip("this torch has no float4_e2m1fn_x2")
    M, N, K = 64, 256, 1024
    w, ws = onv.random_nvfp4((N,), K, seed=12)
    a, a_s = onv.random_nvfp4((M,), K, seed=13)
    C = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    torch.ops.nvfp4r.gemm(cuda(a).view(torch.float4_e2m1fn_x2), cuda(w).view(torch.float4_e2m1fn_x2),
                          cuda(onv.swizzle_blockscale(a_s)).view(torch.float8_e4m3fn),
                          cuda(onv.swizzle_blockscale(ws)).view(torch.float8_e4m3fn), C, 1.0)
    torch.cuda.synchronize()
    _reference_criterion(C.view(N, M).T.float().cpu().numpy(), onv.linear_f64(w, ws, a, a_s))


def test_gemm_workspace_is_fixed_across_shapes(nvfp4r):
    """The operator's hidden split-K scratch never moves: a CUDA graph captured on a small
    shape still gives the right answer after a much larger shape has run."""
    def operands(M, N, K, seed):
        w, ws = onv.random_nvfp4((N,), K, seed=seed)
        a, a_s = onv.random_nvfp4((M,), K, seed=seed + 1)
        return (cuda(a), cuda(w), cuda(onv.swizzle_blockscale(a_s)), cuda(onv.swizzle_blockscale(ws)),
                onv.linear_f64(w, ws, a, a_s))

    A, B, SFA, SFB, exact = operands(8, 256, 1024, 20)
    C = torch.zeros((8, 256), dtype=torch.bfloat16, device="cuda")
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        torch.ops.nvfp4r.gemm(A, B, SFA, SFB, C, 1.0)        # warm-up outside capture
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            torch.ops.nvfp4r.gemm(A, B, SFA, SFB, C, 1.0)
    A2, B2, SFA2, SFB2, exact2 = operands(64, 8192, 8192, 22)
    C_big = torch.empty((64, 8192), dtype=torch.bfloat16, device="cuda")
    torch.ops.nvfp4r.gemm(A2, B2, SFA2, SFB2, C_big, 1.0)
    torch.cuda.synchronize()
    _reference_criterion(C_big.view(8192, 64).T.float().cpu().numpy(), exact2)
    C.zero_()
    g.replay()
    torch.cuda.synchronize()
    _reference_criterion(C.view(256, 8).T.float().cpu().numpy(), exact)
