"""The batch-1 decode-step operators around the linears, against plain PyTorch fp32
references of the same operations (tolerances are bf16 output rounding), and the whole
step: CUDA-graph replay equals eager execution bit for bit."""

from __future__ import annotations

import ctypes
import math

import numpy as np

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    from reset_b200 import _lib
    return _lib


def _s():
    return torch.cuda.current_stream().cuda_stream


def test_add_rmsnorm(lib):
    H = 5120
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(1, H, device="cuda", generator=g).to(torch.bfloat16)
    res = torch.randn(1, H, device="cuda", generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    out = torch.empty_like(x)
    r = res.clone()
    lib.check(lib.lib().nvfp4r_add_rmsnorm(x.data_ptr(), r.data_ptr(), w.data_ptr(), out.data_ptr(), 1, H,
                                           1e-6, _s()), "add_rmsnorm")
    want_res = (res.float() + x.float()).to(torch.bfloat16)
    assert torch.equal(r, want_res)
    f = want_res.float()
    want = f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert torch.allclose(out.float(), want, rtol=2e-2, atol=2e-2)
    # x == NULL: residual untouched
    r2 = res.clone()
    lib.check(lib.lib().nvfp4r_add_rmsnorm(None, r2.data_ptr(), w.data_ptr(), out.data_ptr(), 1, H, 1e-6, _s()), "n")
    assert torch.equal(r2, res)


def _rope_ref(v, pos, theta):
    D = v.shape[-1]
    half = D // 2
    freq = theta ** (-torch.arange(0, half, device=v.device, dtype=torch.float32) * 2 / D)
    ang = pos * freq
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = v[..., :half], v[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def test_qk_norm_rope_kv_and_attention(lib):
    lib.check(lib.lib().nvfp4r_set_rope_table(None, 0), "no table: angles computed in the kernel")
    Hq, Hkv, D, T = 16, 2, 128, 512
    pos = 300
    g = torch.Generator(device="cuda").manual_seed(1)
    qkv = torch.randn(1, (Hq + 2 * Hkv) * D, device="cuda", generator=g).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(torch.bfloat16)
    kw = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(torch.bfloat16)
    kc = (torch.randn(Hkv, T, D, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(Hkv, T, D, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    kc0, vc0 = kc.clone(), vc.clone()
    position = torch.tensor([pos], dtype=torch.int32, device="cuda")
    q = torch.empty(1, Hq * D, dtype=torch.bfloat16, device="cuda")
    lib.check(lib.lib().nvfp4r_qk_norm_rope_kv(qkv.data_ptr(), qw.data_ptr(), kw.data_ptr(), position.data_ptr(),
                                               kc.data_ptr(), vc.data_ptr(), q.data_ptr(), Hq, Hkv, D, T, 1e6,
                                               1e-6, _s()), "qk")
    heads = qkv.float().view(Hq + 2 * Hkv, D)

    def norm(h, w):
        return (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).to(torch.bfloat16).float()
    q_ref = _rope_ref(norm(heads[:Hq], qw), pos, 1e6)
    k_ref = _rope_ref(norm(heads[Hq:Hq + Hkv], kw), pos, 1e6)
    assert torch.allclose(q.float().view(Hq, D), q_ref, rtol=2e-2, atol=2e-2)
    assert torch.allclose(kc[:, pos].float(), k_ref, rtol=2e-2, atol=2e-2)
    assert torch.equal(vc[:, pos], heads[Hq + Hkv:].to(torch.bfloat16))
    mask = torch.ones(T, dtype=torch.bool, device="cuda")
    mask[pos] = False
    assert torch.equal(kc[:, mask], kc0[:, mask]) and torch.equal(vc[:, mask], vc0[:, mask])

    for seq in (pos + 1, 129, 128, 5, T):
        seq_len = torch.tensor([seq], dtype=torch.int32, device="cuda")
        n = lib.lib().nvfp4r_attn_decode_workspace_bytes(Hq, T)
        ws = torch.zeros(n // 4 + 1, dtype=torch.float32, device="cuda")
        out = torch.empty(1, Hq * D, dtype=torch.bfloat16, device="cuda")
        lib.check(lib.lib().nvfp4r_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), seq_len.data_ptr(),
                                               out.data_ptr(), Hq, Hkv, D, T, ws.data_ptr(), ws.numel() * 4, _s()),
                  "attn")
        qf = q.float().view(Hkv, Hq // Hkv, D)
        kf, vf = kc[:, :seq].float(), vc[:, :seq].float()
        sc = torch.einsum("hgd,htd->hgt", qf, kf) / math.sqrt(D)
        want = torch.einsum("hgt,htd->hgd", torch.softmax(sc, -1), vf).reshape(1, Hq * D)
        assert torch.allclose(out.float(), want, rtol=2e-2, atol=1e-2), seq
        # the arrival counters are back at zero: a second call on the same workspace agrees bit for bit
        out2 = torch.empty_like(out)
        lib.check(lib.lib().nvfp4r_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), seq_len.data_ptr(),
                                               out2.data_ptr(), Hq, Hkv, D, T, ws.data_ptr(), ws.numel() * 4, _s()),
                  "attn")
        assert torch.equal(out, out2)


@pytest.mark.parametrize("with_table", [False, True])
@pytest.mark.parametrize("pos", [0, 127, 128, 300, 511])
def test_attention_with_fused_rope_equals_two_launches(lib, pos, with_table):
    """nvfp4r_attn_decode_rope (head norms + rotary + cache append + attention in one launch)
    against nvfp4r_qk_norm_rope_kv followed by nvfp4r_attn_decode: same caches bit for bit, same
    attention output bit for bit (the same arithmetic runs in both)."""
    Hq, Hkv, D, T = 16, 2, 128, 512
    table = None
    if with_table:                                      # (cos, sin) pairs per position and frequency
        freq = 1e6 ** (-torch.arange(0, D // 2, device="cuda", dtype=torch.float32) * 2 / D)
        ang = torch.arange(T, device="cuda", dtype=torch.float32)[:, None] * freq[None, :]
        table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()
    lib.check(lib.lib().nvfp4r_set_rope_table(None if table is None else table.data_ptr(), T if with_table else 0),
              "rope table")
    g = torch.Generator(device="cuda").manual_seed(10 + pos)
    qkv = torch.randn(1, (Hq + 2 * Hkv) * D, device="cuda", generator=g).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(torch.bfloat16)
    kw = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(torch.bfloat16)
    kc = (torch.randn(Hkv, T, D, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(Hkv, T, D, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    kc2, vc2 = kc.clone(), vc.clone()
    position = torch.tensor([pos], dtype=torch.int32, device="cuda")
    seq_len = torch.tensor([pos + 1], dtype=torch.int32, device="cuda")
    n = lib.lib().nvfp4r_attn_decode_workspace_bytes(Hq, T)
    ws = torch.zeros(n // 4 + 1, dtype=torch.float32, device="cuda")
    q = torch.empty(1, Hq * D, dtype=torch.bfloat16, device="cuda")
    out_a = torch.empty(1, Hq * D, dtype=torch.bfloat16, device="cuda")
    out_b = torch.empty_like(out_a)
    lib.check(lib.lib().nvfp4r_qk_norm_rope_kv(qkv.data_ptr(), qw.data_ptr(), kw.data_ptr(), position.data_ptr(),
                                               kc.data_ptr(), vc.data_ptr(), q.data_ptr(), Hq, Hkv, D, T, 1e6,
                                               1e-6, _s()), "qk")
    lib.check(lib.lib().nvfp4r_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), seq_len.data_ptr(),
                                           out_a.data_ptr(), Hq, Hkv, D, T, ws.data_ptr(), ws.numel() * 4, _s()),
              "attn")
    lib.check(lib.lib().nvfp4r_attn_decode_rope(qkv.data_ptr(), qw.data_ptr(), kw.data_ptr(), kc2.data_ptr(),
                                                vc2.data_ptr(), seq_len.data_ptr(), out_b.data_ptr(), Hq, Hkv, D,
                                                T, 1e6, 1e-6, ws.data_ptr(), ws.numel() * 4, _s()), "attn_rope")
    torch.cuda.synchronize()
    lib.check(lib.lib().nvfp4r_set_rope_table(None, 0), "clear")
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)
    assert torch.equal(out_a, out_b)
    heads = qkv.float().view(Hq + 2 * Hkv, D)
    qn = (heads[:Hq] * torch.rsqrt(heads[:Hq].pow(2).mean(-1, keepdim=True) + 1e-6) * qw.float()).to(torch.bfloat16).float()
    assert torch.allclose(q.float().view(Hq, D), _rope_ref(qn, pos, 1e6), rtol=2e-2, atol=2e-2)


def test_silu_mul_lm_head_argmax(lib):
    g = torch.Generator(device="cuda").manual_seed(2)
    I = 3072
    gu = torch.randn(2, 2 * I, device="cuda", generator=g).to(torch.bfloat16)
    out = torch.empty(2, I, dtype=torch.bfloat16, device="cuda")
    lib.check(lib.lib().nvfp4r_silu_mul(gu.data_ptr(), out.data_ptr(), 2, I, _s()), "silu")
    want = torch.nn.functional.silu(gu[:, :I].float()) * gu[:, I:].float()
    assert torch.allclose(out.float(), want, rtol=2e-2, atol=2e-2)

    V, H = 5000, 1024
    x = torch.randn(1, H, device="cuda", generator=g).to(torch.bfloat16)
    W = (torch.randn(V, H, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    logits = torch.empty(1, V, dtype=torch.float32, device="cuda")
    lib.check(lib.lib().nvfp4r_lm_head(x.data_ptr(), W.data_ptr(), logits.data_ptr(), V, H, _s()), "lm_head")
    assert torch.allclose(logits, x.float() @ W.float().T, rtol=1e-4, atol=1e-4)

    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.check(lib.lib().nvfp4r_argmax(logits.data_ptr(), V, 1, V, tok.data_ptr(), _s()), "argmax")
    assert int(tok.item()) == int(torch.argmax(logits[0]).item())
    flat = torch.zeros(2, 64, device="cuda")
    flat[1, 7] = 1.0
    flat[1, 9] = 1.0
    toks = torch.zeros(2, dtype=torch.int32, device="cuda")
    lib.check(lib.lib().nvfp4r_argmax(flat.data_ptr(), 64, 2, 64, toks.data_ptr(), _s()), "argmax")
    assert toks.tolist() == [0, 7]                       # first index among equals


def test_decode_step_graph_equals_eager():
    from reset_b200.decode import DecodeConfig, DecodeStep
    cfg = DecodeConfig("tiny", layers=3, hidden=1024, q_heads=8, kv_heads=2, head_dim=128,
                       intermediate=2048, vocab=4096, context=256)
    m = DecodeStep(cfg, "cuda", seed=3)
    m.step()
    torch.cuda.synchronize()
    eager_logits, eager_tok = m.logits_local.clone(), int(m.token.item())
    assert torch.isfinite(eager_logits).all()
    m.capture()
    m.logits_local.zero_()
    m.replay()
    torch.cuda.synchronize()
    assert torch.equal(m.logits_local, eager_logits) and int(m.token.item()) == eager_tok
    assert m.bytes_per_step() > 0 and m.fused
    # the unfused step (separate RMSNorm / SiLU kernels) computes the same model
    u = DecodeStep(cfg, "cuda", seed=3, fused=False)
    u.step()
    torch.cuda.synchronize()
    a, b = eager_logits.float(), u.logits_local.float()
    assert (a - b).norm() / b.norm() < 5e-2


# ---------------------------------------------------------------------------------------
# Device-side sampling (Gumbel-max) and the decode step with the ReSET processor in its graph
# ---------------------------------------------------------------------------------------

_M64 = (1 << 64) - 1


def _mix64(z):
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def _gumbel_token(logits_row, seed, row, draw):
    """CPU restatement of the generator of nvfp4r_sample for one row (Python integers)."""
    key = _mix64((seed ^ _mix64(((row << 40) + draw) & _M64)) & _M64)
    best, arg = -np.inf, 0
    for i, v in enumerate(logits_row):
        r = _mix64((key + i * 0x9E3779B97F4A7C15) & _M64)
        u = np.float32((np.float32(r >> 41) + np.float32(0.5)) * np.float32(1.0 / 8388608.0))
        g = -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)
        s = np.float32(v) + g
        if s > best:
            best, arg = s, i
    return arg


def test_sample_follows_the_restated_generator_and_is_reproducible():
    from reset_b200 import capi
    B, V = 6, 700
    g = torch.Generator().manual_seed(3)
    logits = (torch.randn(B, V, generator=g) * 3).cuda()
    draws = torch.tensor([0, 1, 2, 3, 40, 1 << 33], dtype=torch.int64, device="cuda")
    start = draws.clone()
    last = torch.full((B, 2), -1, dtype=torch.int32, device="cuda")
    ids = capi.sample(logits, draws, seed=1234, last_ids=last)
    torch.cuda.synchronize()
    expect = [_gumbel_token(logits[b].cpu().numpy(), 1234, b, int(start[b])) for b in range(B)]
    assert ids.tolist() == expect
    assert torch.equal(draws, start + 1)
    assert last[:, 0].tolist() == [-1] * B and last[:, 1].tolist() == expect
    again = capi.sample(logits, start.clone(), seed=1234)
    other = capi.sample(logits, start.clone(), seed=1235)
    assert again.tolist() == expect and other.tolist() != expect
    ids2 = capi.sample(logits, draws, seed=1234, last_ids=last)       # next draw of the same request
    assert last[:, 0].tolist() == expect and last[:, 1].tolist() == ids2.tolist()
    # what ReSET writes for a temperature of (almost) zero: 0 at one id, -inf elsewhere
    row = torch.full((1, V), float("-inf"), device="cuda")
    row[0, 321] = 0.0
    assert capi.sample(row, torch.zeros(1, dtype=torch.int64, device="cuda"), seed=9).tolist() == [321]


def test_sample_frequencies_match_softmax():
    from reset_b200 import capi
    B, V, calls = 256, 50, 60
    g = torch.Generator().manual_seed(8)
    row = torch.randn(V, generator=g) * 1.5
    logits = row.repeat(B, 1).contiguous().cuda()
    draws = torch.zeros(B, dtype=torch.int64, device="cuda")
    counts = torch.zeros(V, dtype=torch.int64)
    for _ in range(calls):
        counts += torch.bincount(capi.sample(logits, draws, seed=77).cpu().long(), minlength=V)
    n = B * calls
    p = torch.softmax(row.double(), dim=0)
    sigma = torch.sqrt(p * (1 - p) / n)
    z = (counts.double() / n - p).abs() / sigma
    assert float(z.max()) < 5.0, (float(z.max()), int(z.argmax()))
    chi2 = float((((counts.double() - n * p) ** 2) / (n * p)).sum())
    assert chi2 < 2.2 * (V - 1)                          # mean V-1, sd sqrt(2(V-1)) ~ 9.9


def _truncated_distribution(row: torch.Tensor, top_k: int, top_p: float, slack: float = 1e-4):
    """vLLM's order: top-k first, then top-p on the distribution renormalised over the top-k set.
    Returns (probabilities over the vocabulary in float64, mask of the ids a draw may return).
    The mask is the exact set widened by the tokens that a nucleus of mass top_p + slack would
    add: the kernel sums fixed-point masses (2^-32 of the largest token's weight each), so with
    tens of thousands of members its boundary can sit a few tokens of ~1e-6 mass away from the
    float64 one."""
    V = row.numel()
    x = row.double()
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        kth = torch.topk(x, top_k).values[-1]
        keep &= x >= kth
    p = torch.softmax(torch.where(keep, x, torch.full_like(x, float("-inf"))), dim=0)
    allowed = keep.clone()
    if top_p < 1.0:
        order = torch.argsort(p, descending=True)
        cum = torch.cumsum(p[order], dim=0)
        n_keep = int((cum < top_p).sum().item()) + 1           # smallest prefix whose mass reaches top_p
        n_allowed = int((cum < top_p + slack).sum().item()) + 1
        mask = torch.zeros(V, dtype=torch.bool)
        mask[order[:n_keep]] = True
        allowed = torch.zeros(V, dtype=torch.bool)
        allowed[order[:min(V, n_allowed)]] = True
        p = torch.where(mask, p, torch.zeros_like(p))
        p = p / p.sum()
    return p, allowed


@pytest.mark.parametrize("V,top_k,top_p", [(1000, 0, 0.9), (1000, 20, 1.0), (1000, 50, 0.8), (151936, 0, 0.95),
                                           (151936, 64, 1.0), (4096, 5, 0.5), (333, 0, 0.3)])
def test_sample_top_k_top_p_support_and_frequencies(V, top_k, top_p):
    """The truncated draw: every drawn id lies in the exact top-k / top-p set, every member of
    the set is reachable, and the frequencies follow the renormalised softmax
    (torch.multinomial on the same truncated distribution gives the reference counts)."""
    from reset_b200 import capi
    B, calls = 256, 40
    g = torch.Generator().manual_seed(1000 + V + top_k)
    row = torch.randn(V, generator=g) * 2.0
    row[int(torch.randint(0, V, (1,), generator=g))] += 6.0
    p, allowed = _truncated_distribution(row, top_k, top_p)
    logits = row.repeat(B, 1).contiguous().cuda()
    draws = torch.zeros(B, dtype=torch.int64, device="cuda")
    ws = capi.sample_workspace(B, "cuda")
    counts = torch.zeros(V, dtype=torch.int64)
    for _ in range(calls):
        ids = capi.sample(logits, draws, seed=5, top_k=top_k, top_p=top_p, workspace=ws)
        counts += torch.bincount(ids.cpu().long(), minlength=V)
    torch.cuda.synchronize()
    n = B * calls
    assert int(counts[~allowed].sum()) == 0, "a draw fell outside the truncated set"
    assert int(ws.count_nonzero().item()) <= 8 * B          # histograms zeroed again (only the small per-row record is left)
    big = p > 20.0 / n                                      # members with enough expected draws
    sigma = torch.sqrt(p * (1 - p) / n)
    z = ((counts.double() / n - p).abs() / sigma.clamp_min(1e-12))[big]
    assert float(z.max()) < 5.5, (float(z.max()), int(z.argmax()))
    ref = torch.bincount(torch.multinomial(p, n, replacement=True, generator=g), minlength=V)
    # same test statistic for our counts and for torch.multinomial's: both are samples of p
    chi_ours = float((((counts.double() - n * p) ** 2)[big] / (n * p)[big]).sum())
    chi_ref = float((((ref.double() - n * p) ** 2)[big] / (n * p)[big]).sum())
    dof = int(big.sum())
    assert chi_ours < dof + 6 * (2 * dof) ** 0.5 + 10, (chi_ours, chi_ref, dof)


def test_sample_truncation_edge_rows():
    """One-hot rows (what ReSET writes for temperature 0), rows with fewer finite entries than k,
    top_p so small that one token remains, and the untruncated call through the same entry."""
    from reset_b200 import capi
    V = 2048
    logits = torch.full((4, V), float("-inf"))
    logits[0, 77] = 0.0                                   # one-hot
    logits[1, :3] = torch.tensor([1.0, 2.0, 3.0])         # three finite entries, k = 10
    logits[2] = torch.randn(V, generator=torch.Generator().manual_seed(3))
    logits[2, 500] = 30.0                                 # one dominant token: any top_p keeps only it
    logits[3] = torch.linspace(-4, 4, V)
    dev = logits.cuda()
    draws = torch.zeros(4, dtype=torch.int64, device="cuda")
    ws = capi.sample_workspace(4, "cuda")
    seen3 = set()
    for it in range(50):
        ids = capi.sample(dev, draws, seed=it, top_k=10, top_p=0.9, workspace=ws).tolist()
        assert ids[0] == 77 and ids[1] in (0, 1, 2) and ids[2] == 500
        assert ids[3] >= V - 10                            # the ten largest of an increasing row
        seen3.add(ids[3])
    assert len(seen3) > 1
    assert draws.tolist() == [50, 50, 50, 50]
    # top_k >= V and top_p = 1: no truncation, same ids as the plain call with the same counters
    d1 = torch.zeros(4, dtype=torch.int64, device="cuda")
    d2 = torch.zeros(4, dtype=torch.int64, device="cuda")
    a = capi.sample(dev, d1, seed=9, top_k=V, top_p=1.0, workspace=ws)
    b = capi.sample(dev, d2, seed=9)
    assert torch.equal(a, b)


def test_decode_step_with_reset_processor_and_sampling_in_the_graph():
    from reset_b200 import _lib
    from reset_b200.decode import DecodeConfig, DecodeStep
    cfg = DecodeConfig("tiny", layers=2, hidden=1024, q_heads=8, kv_heads=2, head_dim=128,
                       intermediate=2048, vocab=4096, context=256)
    plain = DecodeStep(cfg, "cuda", seed=5)
    plain.step()
    torch.cuda.synchronize()
    raw = plain.logits_local.clone()
    m = DecodeStep(cfg, "cuda", seed=5)
    m.enable_reset(t_high=1.0, t_low=0.1, tau0=0.5505, window=32, dnl_ids=[7], seed=42)
    m.step()
    torch.cuda.synchronize()
    dec = _lib.ResetDecision.from_buffer_copy(m.reset.decisions.cpu().numpy().tobytes()[:ctypes.sizeof(_lib.ResetDecision)])
    assert dec.temp in (0.1, 1.0) and dec.boundary == 0
    # same model, same input: the processor divided the raw logits by the temperature it chose
    want = raw / np.float32(dec.temp) if dec.temp != 1.0 else raw
    assert torch.allclose(m.logits_local, want, rtol=3e-7, atol=0)
    p = torch.softmax(raw.double()[0], dim=0)
    ent = float(-(p * torch.log(p.clamp_min(1e-10))).sum())
    assert abs(dec.entropy - ent) <= 1e-4 * max(1.0, ent)
    first = int(m.token.item())
    assert 0 <= first < cfg.vocab and m.draws.tolist() == [1] and m.last_ids.tolist() == [[-1, first]]
    # graph replays keep drawing: counters advance, the recent ids follow the tokens
    m.capture()
    torch.cuda.synchronize()
    base = int(m.draws.item())
    toks = []
    for _ in range(4):
        m.replay()
        torch.cuda.synchronize()
        toks.append(int(m.token.item()))
    assert int(m.draws.item()) == base + 4
    assert m.last_ids.tolist() == [[toks[-2], toks[-1]]]
    assert all(0 <= t < cfg.vocab for t in toks)
    assert _lib.lib().nvfp4r_check_device_status() == 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_decode_step_runs_with_every_tensor_parallel_shard_shape(world, monkeypatch):
    """Rank 0's shard of a Qwen3-32B-shaped step at TP = 2 / 4 / 8 on one GPU (the collectives
    are replaced by their single-rank effect): every per-rank linear shape goes through the
    kernel the crossover picks for it (at TP = 8 the down projection has K = 3200, which only
    the plain-load GEMV takes, so the step falls back to separate norm / activation launches),
    eager and graph replay agree bit for bit, and no kernel reports a failed wait."""
    import dataclasses
    from reset_b200 import _lib
    from reset_b200.decode import QWEN3_32B, DecodeStep
    import torch.distributed as dist

    monkeypatch.setattr(dist, "all_reduce", lambda t, group=None: None)
    monkeypatch.setattr(dist, "all_gather_into_tensor",
                        lambda out, inp, group=None: out[:inp.numel()].copy_(inp))
    cfg = dataclasses.replace(QWEN3_32B, layers=2, context=256)
    m = DecodeStep(cfg, "cuda", rank=0, world=world, seed=11, peer_allreduce=False)
    inter = cfg.intermediate // world
    assert m.fused == (inter % 128 == 0)
    assert m.layers[0]["down"].K == inter and m.layers[0]["o"].K == cfg.q_heads // world * cfg.head_dim
    m.step()
    torch.cuda.synchronize()
    eager = m.logits_local.clone()
    assert torch.isfinite(eager).all() and float(eager.abs().max()) > 0
    m.capture()
    m.logits_local.zero_()
    m.replay()
    torch.cuda.synchronize()
    assert torch.equal(m.logits_local, eager)
    assert _lib.lib().nvfp4r_check_device_status() == 0
