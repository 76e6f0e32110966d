"""GPU parity of the GEMV through the C ABI (``nvfp4r_gemv``) against the CPU oracle.

Tolerances: outputs in float32 are compared with the float64 dequantise-matmul of the
oracle at rel-L2 <= 1e-3 (the stated bound; measured values are ~1e-7 because the
per-block sums are exact), and float16 outputs with the reference's own criterion
(kernels/tests/test_gemv.py:46-50: max_rel < 5e-2 or max_abs < 1.0)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import nvfp4 as onv
from helpers import cuda, make_activation, make_weight, rel_l2

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3

# (L, N, K) of the reference's own test (kernels/tests/test_gemv.py:14-28)
REFERENCE_SHAPES = [
    (1, 256, 4096), (1, 1024, 8192), (1, 2048, 16384), (4, 512, 2048), (8, 512, 7168),
    (2, 4096, 4096), (1, 4608, 3584), (1, 3584, 3584), (1, 3584, 18944), (1, 6144, 4096),
    (1, 4096, 4096), (1, 4096, 12288),
]


@pytest.fixture(scope="module")
def capi():
    from reset_b200 import capi as c
    return c


@pytest.fixture(params=["stream", "rows", "generic"])
def path(request):
    """The three GEMV kernels: the bulk-copy ring kernel (the register-resident one switched off),
    the register-resident single-token kernel wherever it can take the launch, the plain-load
    fallback."""
    from reset_b200 import _lib
    _lib.check(_lib.lib().nvfp4r_set_gemv_tuning(-1, -1, 1 if request.param == "generic" else 0), "tuning")
    _lib.check(_lib.lib().nvfp4r_set_gemv_rows_tuning({"stream": -1, "rows": 1, "generic": -1}[request.param], 0, 0),
               "rows tuning")
    yield request.param
    _lib.check(_lib.lib().nvfp4r_set_gemv_tuning(-1, -1, 0), "tuning")
    _lib.check(_lib.lib().nvfp4r_set_gemv_rows_tuning(0, 0, 0), "rows tuning")


def _run(capi, w, ws, x, xs, L, dtype, alpha=1.0):
    N = w.shape[0]
    wd, wsd = cuda(w), cuda(ws)
    out = torch.full((L, N), float("nan"), dtype=dtype, device="cuda")
    capi.gemv_out(wd.unsqueeze(0).expand(L, -1, -1), wsd.unsqueeze(0).expand(L, -1, -1),
                  cuda(x), cuda(xs), out, alpha)
    torch.cuda.synchronize()
    return out.cpu()


@pytest.mark.parametrize("L,N,K", REFERENCE_SHAPES)
def test_gemv_matches_oracle_on_reference_shapes(capi, path, L, N, K):
    w, ws = onv.random_nvfp4((N,), K, seed=0)
    x, xs = onv.random_nvfp4((L, 1), K, seed=1)
    exact = onv.linear_f64(w, ws, x[:, 0], xs[:, 0])
    got32 = _run(capi, w, ws, x, xs, L, torch.float32).numpy()
    assert rel_l2(got32, exact) <= REL_L2_TOL
    assert rel_l2(got32, exact) <= 1e-5          # what the exact block sums deliver
    got16 = _run(capi, w, ws, x, xs, L, torch.float16).float().numpy()
    ref16 = exact.astype(np.float16).astype(np.float32)
    diff = np.abs(got16 - ref16)
    assert (diff / (np.abs(ref16) + 1e-3)).max() < 5e-2 or diff.max() < 1.0
    # and to the rounding itself: within one fp16 ulp of the rounded exact value (elements
    # that cancel to nearly zero are held to 1e-5 of the output's rms instead)
    ulp = np.abs(np.spacing(ref16.astype(np.float16))).astype(np.float32)
    rms = float(np.sqrt(np.mean(exact ** 2)))
    assert np.all(diff <= np.maximum(ulp, 1e-5 * rms))


def test_gemv_writes_into_provided_out(capi):
    """Out-variant contract (kernels/tests/test_gemv.py:56-66)."""
    w, ws = onv.random_nvfp4((1, 256), 4096, seed=2)
    x, xs = onv.random_nvfp4((1, 1), 4096, seed=3)
    out = torch.empty((1, 256), dtype=torch.float16, device="cuda")
    before = out.data_ptr()
    ret = capi.gemv_out(cuda(w), cuda(ws), cuda(x), cuda(xs), out)
    assert ret is None and out.data_ptr() == before
    assert torch.isfinite(out).all().item()


@pytest.mark.parametrize("L", [1, 2, 3, 4, 5, 7, 8, 9, 16])
def test_gemv_token_counts(capi, path, L):
    N, K = 520, 1024                               # N not a multiple of 8
    w, ws = onv.random_nvfp4((N,), K, seed=4)
    x, xs = onv.random_nvfp4((L, 1), K, seed=5)
    got = _run(capi, w, ws, x, xs, L, torch.float32, alpha=0.37).numpy()
    assert not np.isnan(got).any()
    assert rel_l2(got, onv.linear_f64(w, ws, x[:, 0], xs[:, 0], alpha=0.37)) <= 1e-5


@pytest.mark.parametrize("N,K", [(4, 256), (6, 512), (1, 2560), (130, 3200), (64, 640),
                                 (48, 2176), (9, 32), (40, 25600), (5120, 3200)])
def test_gemv_ragged_and_shard_shapes(capi, N, K):
    """Row counts that do not fill a 4-row group, K with a partial chunk, and the
    TP-8 shard K values (3200, 640, 2176) that have K/2 % 128 == 64."""
    for L in (1, 3):
        w, ws = onv.random_nvfp4((N,), K, seed=6)
        x, xs = onv.random_nvfp4((L, 1), K, seed=7)
        got = _run(capi, w, ws, x, xs, L, torch.float32).numpy()
        assert rel_l2(got, onv.linear_f64(w, ws, x[:, 0], xs[:, 0])) <= 1e-5


def test_gemv_padded_activation_rows_and_distinct_weights(capi):
    """x carries P > 1 rows per token (only row 0 is read, bindings.cpp:63-68) and a
    weight that is NOT broadcast over L is honoured per l."""
    L, N, K, P = 3, 64, 512, 4
    w, ws = onv.random_nvfp4((L, N), K, seed=8)
    x, xs = onv.random_nvfp4((L, P), K, seed=9)
    out = torch.empty((L, N), dtype=torch.float32, device="cuda")
    capi.gemv_out(cuda(w), cuda(ws), cuda(x), cuda(xs), out)
    torch.cuda.synchronize()
    for l in range(L):
        exact = onv.linear_f64(w[l], ws[l], x[l, :1], xs[l, :1])[0]
        assert rel_l2(out[l].cpu().numpy(), exact) <= 1e-5


def test_gemv_large_scales_do_not_overflow(capi, path):
    """Both block scales at the e4m3 maximum (448*448 overflows f16, not f32)."""
    N, K = 64, 1024
    w, _ = onv.random_nvfp4((N,), K, seed=10)
    x, _ = onv.random_nvfp4((1, 1), K, seed=11)
    ws = np.full((N, K // 16), 0x7E, dtype=np.uint8)
    xs = np.full((1, 1, K // 16), 0x7E, dtype=np.uint8)
    got = _run(capi, w, ws, x, xs, 1, torch.float32).numpy()
    assert np.isfinite(got).all()
    assert rel_l2(got, onv.linear_f64(w, ws, x[:, 0], xs[:, 0])) <= 1e-5


def test_gemv_config0_quantized_weights(capi, path):
    """The 4096 x 4096 single-token case: M=1, K=N=4096, bf16 N(0,0.02) weights and N(0,1) activations
    with outlier channels, both quantized; result vs fp32 dequant-matmul."""
    N = K = 4096
    wc, wsf, gs_w = make_weight(N, K, seed=0)
    xb = make_activation(1, K, seed=1)
    gs_x = onv.global_scale_for(xb.float().numpy())
    xc, xsf = onv.quantize_nvfp4(xb.float().numpy(), 1.0 / gs_x)
    alpha = gs_w * gs_x
    got = _run(capi, wc, wsf, xc[:, None], xsf[:, None], 1, torch.float32, alpha=alpha).numpy()
    exact = onv.linear_f64(wc, wsf, xc, xsf, alpha=alpha)
    assert rel_l2(got, exact) <= REL_L2_TOL
    # the quantized product also tracks the unquantized one (sanity of the whole chain)
    g = torch.Generator().manual_seed(0)
    w_bf = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16).float()
    dense = (xb.float() @ w_bf.T).numpy()
    assert rel_l2(got, dense) < 0.2


def test_row_parallel_shards_sum_to_full(capi):
    """TP parity: the sum of the K-shard partial products equals the unsharded GEMV
    (fp32 re-association only)."""
    N, K, tp = 256, 4096, 4
    w, ws = onv.random_nvfp4((N,), K, seed=12)
    x, xs = onv.random_nvfp4((2, 1), K, seed=13)
    full = _run(capi, w, ws, x, xs, 2, torch.float32).numpy()
    acc = np.zeros_like(full)
    ks = K // tp
    for r in range(tp):
        sl2 = slice(r * ks // 2, (r + 1) * ks // 2)
        sl16 = slice(r * ks // 16, (r + 1) * ks // 16)
        acc += _run(capi, np.ascontiguousarray(w[:, sl2]), np.ascontiguousarray(ws[:, sl16]),
                    np.ascontiguousarray(x[:, :, sl2]), np.ascontiguousarray(xs[:, :, sl16]),
                    2, torch.float32).numpy()
    assert rel_l2(acc, full) <= 1e-6


def test_bad_arguments_are_rejected(capi):
    from reset_b200 import _lib
    w, ws = onv.random_nvfp4((1, 8), 64, seed=1)
    x, xs = onv.random_nvfp4((1, 1), 64, seed=2)
    out = torch.empty((1, 8), dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        capi.gemv_out(cuda(w)[0], cuda(ws), cuda(x), cuda(xs), out)          # 2-D weight
    with pytest.raises(ValueError):
        capi.gemv_out(cuda(w), cuda(ws), cuda(x), cuda(xs), out.double())    # out dtype
    st = _lib.lib().nvfp4r_gemv(None, None, None, None, None, 1, 8, 64, 0, 32, 0, 4, 32, 4, 1.0, 1, None)
    assert st == -1
    wd = cuda(w)
    st = _lib.lib().nvfp4r_gemv(wd.data_ptr(), wd.data_ptr(), wd.data_ptr(), wd.data_ptr(),
                                out.data_ptr(), 1, 8, 48, 0, 24, 0, 3, 24, 3, 1.0, 1, None)
    assert st == -2                                                           # K % 32
