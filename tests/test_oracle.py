"""The CPU oracle against the fixtures generated from the reference's own code
(tests/golden/make_golden.py). Everything here is bit-exact unless stated."""

from __future__ import annotations

import hashlib

import numpy as np
import pytest
import torch

from oracle import nvfp4 as onv
from oracle import reset_policy as orp
from oracle import torch_port as otp


@pytest.fixture(scope="module")
def g_decode(golden_dir):
    return np.load(golden_dir / "nvfp4_decode_gemv.npz")


def test_code_tables_match_reference(g_decode):
    assert np.array_equal(onv.E2M1_TABLE.view(np.uint32), g_decode["e2m1_table"].view(np.uint32))
    ours, ref = onv.E4M3_TABLE, g_decode["e4m3_table"]
    assert np.array_equal(np.isnan(ours), np.isnan(ref))
    ok = ~np.isnan(ref)
    assert np.array_equal(ours[ok].view(np.uint32), ref[ok].view(np.uint32))


def test_dequant_matches_reference(g_decode):
    for i in range(int(g_decode["n_cases"])):
        w, ws = g_decode[f"c{i}_w"], g_decode[f"c{i}_ws"]
        assert np.array_equal(onv.dequant_nvfp4(w[:4], ws[:4]), g_decode[f"c{i}_dq4"])
    dq = onv.dequant_nvfp4(g_decode["wide_w"], g_decode["wide_ws"])
    assert np.array_equal(dq.view(np.uint32), g_decode["wide_dq"].view(np.uint32))


def test_reference_gemv_matches_reference(g_decode):
    for i in range(int(g_decode["n_cases"])):
        w, ws = g_decode[f"c{i}_w"], g_decode[f"c{i}_ws"]
        x, xs, y = g_decode[f"c{i}_x"], g_decode[f"c{i}_xs"], g_decode[f"c{i}_y"]
        L = x.shape[0]
        wb = np.broadcast_to(w, (L,) + w.shape)
        wsb = np.broadcast_to(ws, (L,) + ws.shape)
        ours = onv.reference_gemv_f32(wb, wsb, x, xs)
        # fp32 summation order differs between einsum implementations: compare
        # before the fp16 cast with a float tolerance, after it to 1 fp16 ulp.
        exact = np.stack([onv.linear_f64(w, ws, x[l, :1], xs[l, :1])[0] for l in range(L)])
        assert np.allclose(ours, exact, rtol=1e-5, atol=1e-4)
        ulp = np.abs(ours.astype(np.float16).view(np.int16).astype(np.int32)
                     - y.view(np.int16).astype(np.int32))
        assert ulp.max() <= 1


def test_blockwise_model_equals_plain_dequant(g_decode):
    w, ws = g_decode["c1_w"], g_decode["c1_ws"]
    x, xs = g_decode["c1_x"][:, 0], g_decode["c1_xs"][:, 0]
    a = onv.gemv_blockwise_f32(w, ws, x, xs, alpha=0.5)
    b = onv.linear_f64(w, ws, x, xs, alpha=0.5)
    assert np.allclose(a, b, rtol=1e-12, atol=1e-12)


def test_e4m3_encode_roundtrip_and_ties():
    finite = [b for b in range(256) if (b & 0x7F) != 0x7F]
    vals = onv.E4M3_TABLE[finite]
    enc = onv.e4m3_encode(vals)
    assert np.array_equal(onv.E4M3_TABLE[enc], vals)
    # against torch's own cast on a dense sweep incl. exact midpoints
    pos = onv.E4M3_TABLE[:127].astype(np.float64)
    mids = (pos[1:] + pos[:-1]) / 2
    sweep = np.concatenate([mids, np.linspace(0, 448, 20001), -mids, [500.0, -1e9]])
    sweep32 = sweep.astype(np.float32)
    ref = torch.from_numpy(np.clip(sweep32, -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(onv.e4m3_encode(sweep32), ref)


def test_e2m1_encode_ties_to_even():
    x = np.array([0.0, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.01, 7.0, -0.25, -0.75, -9.0])
    want = np.array([0, 0, 1, 2, 2, 4, 4, 6, 6, 7, 7, 8, 10, 15], dtype=np.uint8)
    assert np.array_equal(onv.e2m1_encode(x), want)


def test_quantizer_matches_vllm_emulation(golden_dir):
    g = np.load(golden_dir / "quant_vllm_emulation.npz")
    for i in range(int(g["n_cases"])):
        x = onv.bf16_bits_to_f32(g[f"q{i}_x_bf16"])
        codes, sf = onv.quantize_nvfp4(x, float(g[f"q{i}_gs_inv"]))
        assert np.array_equal(sf, g[f"q{i}_sf"]), f"scales differ in case {i}"
        # -0 and +0 dequantise alike; the emulation loses the sign of zero codes
        ours, ref = onv.unpack_codes(codes), onv.unpack_codes(g[f"q{i}_codes"])
        same = (ours == ref) | (((ours & 7) == 0) & ((ref & 7) == 0))
        assert same.all(), f"codes differ in case {i}: {np.count_nonzero(~same)}"


def test_quantizer_torch_port_equals_numpy():
    for seed, (M, K) in enumerate([(1, 4096), (5, 256), (8, 1024)]):
        g = torch.Generator().manual_seed(seed)
        x = (torch.randn(M, K, generator=g) * 3).to(torch.bfloat16)
        gs_inv = 1.0 / onv.global_scale_for(x.float().numpy())
        c0, s0 = onv.quantize_nvfp4(x.float().numpy(), gs_inv)
        c1, s1 = otp.quantize_torch(x, gs_inv)
        assert np.array_equal(s0, s1.numpy()) and np.array_equal(c0, c1.numpy())


def test_torch_port_linear_equals_numpy():
    w, ws = onv.random_nvfp4((24,), 512, seed=1)
    x, xs = onv.random_nvfp4((3,), 512, seed=2)
    a = otp.linear_torch(*(torch.from_numpy(t) for t in (w, ws, x, xs)), alpha=0.25).numpy()
    b = onv.linear_f64(w, ws, x, xs, alpha=0.25)
    assert np.allclose(a, b, rtol=1e-5, atol=1e-4)


def test_swizzle_matches_reference(golden_dir):
    g = np.load(golden_dir / "swizzle.npz")
    for i in range(int(g["n_cases"])):
        M, K = (int(v) for v in g[f"s{i}_MK"])
        assert np.array_equal(onv.unswizzle_blockscale(g[f"s{i}_sw_in"], M, K),
                              g[f"s{i}_unswizzled"])
        flat = g[f"s{i}_flat"]
        assert np.array_equal(onv.unswizzle_blockscale(onv.swizzle_blockscale(flat), M, K), flat)


def test_reset_policy_matches_reference(golden_dir):
    g = np.load(golden_dir / "reset_policy.npz")
    for i in range(int(g["n_cases"])):
        V, steps, seed, th, tl, tau0, w, sigma, delim, nl = g[f"r{i}_cfg"]
        V, steps, seed, w, delim, nl = (int(v) for v in (V, steps, seed, w, delim, nl))
        logits = orp.synthetic_logits(steps, V, seed, sigma=float(sigma))
        sha = hashlib.sha256(logits.numpy().tobytes()).hexdigest()
        if sha != str(g[f"r{i}_logits_sha256"]):
            if f"r{i}_logits" not in g.files:
                pytest.skip("torch RNG stream differs from the fixture's")
            logits = torch.from_numpy(g[f"r{i}_logits"])
        ids = g[f"r{i}_ids"]
        pol = orp.ResetPolicy(th, tl, tau0, w, frozenset([nl]), frozenset([delim]))
        for t in range(steps):
            scaled, d = pol(ids[:t].tolist(), logits[t])
            assert d.entropy == g[f"r{i}_entropy"][t]
            assert (0.0 if d.temp <= 1e-6 else d.temp) == g[f"r{i}_temp"][t], (i, t)
            finite = torch.where(torch.isinf(scaled), torch.zeros_like(scaled), scaled)
            assert float(finite.double().sum()) == g[f"r{i}_scaled_sum"][t]
        if f"r{i}_scaled_last" in g.files:
            assert np.array_equal(scaled.numpy(), g[f"r{i}_scaled_last"])


def test_entropy_f64_close_to_reference_fp32():
    """The reference evaluates the entropy with float32 torch ops. On a CPU its
    softmax denominator is a long sequential float32 sum per SIMD lane, which at
    vocab 151936 leaves the entropy a few 1e-5 away from the exact value (the
    offset is rounding noise of that summation order, not part of the
    algorithm). The float64 form is the yardstick the 1e-5 tolerance of the GPU
    tests is stated against; the float32 form is compared at 1e-4."""
    x = orp.synthetic_logits(4, 151936, seed=3)
    for r in range(4):
        assert abs(orp.token_entropy(x[r]) - orp.token_entropy_f64(x[r].numpy())) < 1e-4
    y = orp.synthetic_logits(4, 4096, seed=4)
    for r in range(4):
        assert abs(orp.token_entropy(y[r]) - orp.token_entropy_f64(y[r].numpy())) < 1e-5


def test_boundary_rule():
    pol = orp.ResetPolicy(1.0, 0.1, 0.5, 32, frozenset([7]), frozenset([9]))
    assert not pol.is_boundary([])
    assert pol.is_boundary([1, 9])
    assert not pol.is_boundary([7])
    assert not pol.is_boundary([1, 7])
    assert pol.is_boundary([7, 7])
    assert not pol.is_boundary([7, 7, 1])
