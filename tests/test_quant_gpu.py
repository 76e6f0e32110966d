"""GPU parity of the activation quantizer (``nvfp4r_quant``) - codes and scales are
compared bit for bit with the CPU oracle."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import nvfp4 as onv
from helpers import cuda, make_activation

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from reset_b200 import capi as c
    return c


def _gs_inv(x_bf16: torch.Tensor) -> float:
    return float(np.float32(1.0) / np.float32(onv.global_scale_for(x_bf16.float().numpy())))


def _quant(capi, x, gs_inv, **kw):
    gs = torch.tensor([gs_inv], dtype=torch.float32, device="cuda")
    c, s = capi.quant(x.cuda(), gs, **kw)
    torch.cuda.synchronize()
    return c.cpu().numpy(), s.cpu().numpy()


@pytest.mark.parametrize("M,K", [(1, 4096), (2, 5120), (4, 12288), (8, 4096), (1, 25600),
                                 (3, 16), (5, 48), (7, 3200), (16, 8192), (1, 17408)])
def test_quant_bit_exact_vs_oracle(capi, M, K):
    x = make_activation(M, K, seed=100 + M + K)
    gs_inv = _gs_inv(x)
    codes, sf = _quant(capi, x, gs_inv)
    ocodes, osf = onv.quantize_nvfp4(x.float().numpy(), gs_inv)
    assert np.array_equal(sf, osf)
    assert np.array_equal(codes, ocodes)


def test_quant_edge_values(capi):
    K = 256
    x = make_activation(6, K, seed=5).float()
    x[0, :32] = 0.0                  # all-zero blocks -> scale 0, codes 0
    x[1, 32:48] = 1e-7               # scale underflows to 0 -> codes are signed zeros
    x[2, 64:80] = -0.0
    x[3, :] = 0.0
    x[4, 16:32] = -x[4, 16:32].abs() # all-negative block
    x[5, 0] = 3.0e38                 # huge outlier: scale saturates at 448
    xb = x.to(torch.bfloat16)
    for gs_inv in (_gs_inv(xb), 1.0, 2688.0, 1e-3):
        codes, sf = _quant(capi, xb, gs_inv)
        ocodes, osf = onv.quantize_nvfp4(xb.float().numpy(), gs_inv)
        assert np.array_equal(sf, osf)
        assert np.array_equal(codes, ocodes)


def test_quant_exact_ties(capi):
    """Values that land exactly on e2m1 rounding boundaries (scale 1, gs_inv 1...)."""
    K = 32
    ties = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0]
    x = torch.tensor([ties + ties[::-1]], dtype=torch.float32).to(torch.bfloat16)
    codes, sf = _quant(capi, x, 1.0)
    ocodes, osf = onv.quantize_nvfp4(x.float().numpy(), 1.0)
    assert np.array_equal(sf, osf) and np.array_equal(codes, ocodes)


def test_quant_golden_fixture(capi, golden_dir):
    g = np.load(golden_dir / "quant_vllm_emulation.npz")
    for i in range(int(g["n_cases"])):
        bits = g[f"q{i}_x_bf16"]
        x = torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16)
        codes, sf = _quant(capi, x, float(g[f"q{i}_gs_inv"]))
        assert np.array_equal(sf, g[f"q{i}_sf"])
        ours, ref = onv.unpack_codes(codes), onv.unpack_codes(g[f"q{i}_codes"])
        assert ((ours == ref) | (((ours & 7) == 0) & ((ref & 7) == 0))).all()


@pytest.mark.parametrize("M,K", [(1, 4096), (5, 512), (130, 320), (64, 1088)])
def test_quant_swizzled_layout(capi, M, K):
    x = make_activation(M, K, seed=7)
    gs_inv = _gs_inv(x)
    codes_f, sf_flat = _quant(capi, x, gs_inv)
    codes_s, sf_sw = _quant(capi, x, gs_inv, swizzled=True)
    assert np.array_equal(codes_f, codes_s)
    assert np.array_equal(sf_sw, onv.swizzle_blockscale(sf_flat))


def test_quant_strided_rows(capi):
    M, K = 4, 1024
    big = make_activation(M, 2 * K, seed=9).cuda()
    view = big[:, :K]
    gs_inv = _gs_inv(view.cpu())
    gs = torch.tensor([gs_inv], dtype=torch.float32, device="cuda")
    c, s = capi.quant(view, gs)
    oc, osf = onv.quantize_nvfp4(view.cpu().float().numpy(), gs_inv)
    assert np.array_equal(c.cpu().numpy(), oc) and np.array_equal(s.cpu().numpy(), osf)


def test_swizzle_roundtrip_kernels(capi, golden_dir):
    g = np.load(golden_dir / "swizzle.npz")
    for i in range(int(g["n_cases"])):
        M, K = (int(v) for v in g[f"s{i}_MK"])
        un = capi.unswizzle_blockscale(cuda(g[f"s{i}_sw_in"]), M, K).cpu().numpy()
        assert np.array_equal(un, g[f"s{i}_unswizzled"])
        flat = g[f"s{i}_flat"]
        sw = capi.swizzle_blockscale(cuda(flat)).cpu().numpy()
        assert np.array_equal(sw, onv.swizzle_blockscale(flat))


def test_quant_approx_mode_vs_exact_and_vllm(capi):
    """APPROX mode uses rcp.approx.ftz as the CUDA op the reference calls does; it may
    differ from the exact mode only in codes at rounding ties (never in scales).
    Where the installed vLLM's own CUDA op is usable it is the authority for this mode."""
    from reset_b200 import _lib
    M, K = 8, 8192
    x = make_activation(M, K, seed=11)
    gs_inv = _gs_inv(x)
    ce, se = _quant(capi, x, gs_inv)
    ca, sa = _quant(capi, x, gs_inv, rcp_mode=_lib.RCP_APPROX)
    assert np.array_equal(se, sa)
    mism = np.count_nonzero(onv.unpack_codes(ce) != onv.unpack_codes(ca))
    assert mism <= 1e-3 * M * K, f"{mism} code mismatches between exact and approx"
    try:
        import vllm._custom_ops as vops
        gs = torch.tensor([gs_inv], dtype=torch.float32, device="cuda")
        vc, vs = vops.scaled_fp4_quant(x.cuda(), gs, is_sf_swizzled_layout=False)
        torch.cuda.synchronize()
    except Exception as exc:  # vLLM's extension is optional on the box
        pytest.skip(f"vLLM CUDA quantizer not usable here: {exc!r}")
    vc = vc.view(torch.uint8).cpu().numpy()
    vs = vs.view(torch.uint8).cpu().numpy().reshape(M, -1)[:, : K // 16]
    n_sf = np.count_nonzero(vs != sa)
    n_code = np.count_nonzero(onv.unpack_codes(vc) != onv.unpack_codes(ca))
    print(f"vs vLLM CUDA op: {n_sf} scale and {n_code} code mismatches of {M * K}")
    assert n_sf == 0 and n_code == 0


@pytest.mark.parametrize("K", [4096, 12288, 5120, 8192, 17408, 25600, 3200, 640])
@pytest.mark.parametrize("M", [1, 2, 4, 8])
def test_quant_approx_mode_is_the_installed_vllm_op_on_every_decode_shape(capi, M, K):
    """APPROX is the mode the adapter and the fused linears run in. Codes and scales against
    the installed vLLM's CUDA ``scaled_fp4_quant`` (the op the reference calls,
    kernels/python/nvfp4r/vllm_integration.py:213), bit for bit, for every K of the Qwen3-8B /
    14B / 32B decode linears (and the TP-8 shards with K % 256 != 0) at M = 1, 2, 4, 8, in the
    flat and in the swizzled scale layout."""
    from reset_b200 import _lib
    try:
        import vllm._custom_ops as vops
    except Exception as exc:
        pytest.skip(f"vLLM is not importable here: {exc!r}")
    x = make_activation(M, K, seed=1000 + M + K)
    gs_inv = _gs_inv(x)
    gs = torch.tensor([gs_inv], dtype=torch.float32, device="cuda")
    ca, sa = _quant(capi, x, gs_inv, rcp_mode=_lib.RCP_APPROX)
    try:
        vc, vs = vops.scaled_fp4_quant(x.cuda(), gs, is_sf_swizzled_layout=False)
        vcs, vss = vops.scaled_fp4_quant(x.cuda(), gs, is_sf_swizzled_layout=True)
        torch.cuda.synchronize()
    except Exception as exc:
        pytest.skip(f"vLLM CUDA quantizer not usable here: {exc!r}")
    vc = vc.view(torch.uint8).cpu().numpy()
    vs = vs.view(torch.uint8).cpu().numpy().reshape(M, -1)[:, : K // 16]
    assert np.array_equal(vs, sa), "scales differ from vLLM's"
    assert np.array_equal(onv.unpack_codes(vc), onv.unpack_codes(ca)), "codes differ from vLLM's"
    # swizzled layout: same codes; the scale bytes of the M real rows sit where vLLM puts them
    cs, ss = capi.quant(x.cuda(), gs, swizzled=True, rcp_mode=_lib.RCP_APPROX)
    torch.cuda.synchronize()
    assert np.array_equal(cs.cpu().numpy(), vcs.view(torch.uint8).cpu().numpy())
    ours_flat = capi.unswizzle_blockscale(ss, M, K).cpu().numpy()
    vllm_flat = capi.unswizzle_blockscale(vss.view(torch.uint8).reshape(-1).contiguous(), M, K).cpu().numpy()
    assert np.array_equal(ours_flat, sa) and np.array_equal(vllm_flat, sa)
