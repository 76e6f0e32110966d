"""GPU parity of ``nvfp4r_lm_head_reset_step``: lm_head and the ReSET step of one token in one
launch, against (a) ``nvfp4r_lm_head`` followed by ``nvfp4r_reset_step_per_request`` and (b) the
oracle policy fed with the lm_head logits.

Bars. Logits before the division: bit-exact with ``nvfp4r_lm_head``. Entropy: 1e-5 absolute
against the float64 evaluation, 1e-4 against the reference's float32 CPU value (see
tests/test_reset_gpu.py). Temperature: the oracle's whenever its entropy is further than
``TIE_BAND`` from the threshold. Scaled logits: bit-exact against ``logits / temp``."""

from __future__ import annotations

import ctypes as C

import numpy as np
import pytest
import torch

from oracle import reset_policy as orp

pytestmark = pytest.mark.gpu

TIE_BAND = 1e-4
DEC = np.dtype([("entropy", "f8"), ("h_step", "f8"), ("h_bar", "f8"), ("temp", "f8"),
                ("boundary", "i4"), ("high", "i4")])


@pytest.fixture(scope="module")
def capi():
    from reset_b200 import capi as c
    return c


def _bitmap(ids, V):
    bm = np.zeros((V + 31) // 32, dtype=np.uint32)
    for i in ids:
        bm[i >> 5] |= np.uint32(1) << np.uint32(i & 31)
    return torch.from_numpy(bm.view(np.int32)).cuda()


def _params_dev(*records):
    from reset_b200 import _lib
    raw = b"".join(bytes(_lib.ResetParams(*r)) for r in records)
    return torch.frombuffer(bytearray(raw), dtype=torch.uint8).cuda()


def _lm_head(x, W):
    from reset_b200 import _lib
    V, H = W.shape
    out = torch.empty(1, V, dtype=torch.float32, device="cuda")
    _lib.check(_lib.lib().nvfp4r_lm_head(x.data_ptr(), W.data_ptr(), out.data_ptr(), V, H,
                                         torch.cuda.current_stream().cuda_stream), "lm_head")
    return out


def _model(V, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    W = (torch.randn(V, H, generator=g, device="cuda") * (3.0 / H ** 0.5)).to(torch.bfloat16)
    return W, g


@pytest.mark.parametrize("V,H,steps", [(151936, 1024, 96), (4096, 256, 160), (1000, 512, 64), (50257, 768, 64),
                                       (33, 256, 8)])
def test_fused_launch_against_two_launches_and_oracle(capi, V, H, steps):
    from reset_b200 import _lib
    W, g = _model(V, H, seed=V % 89)
    delim, nl = V - 5, V - 9
    stream = orp.synthetic_token_stream(steps, delim, V, 5, 10, 30)
    stream[20:22] = nl
    # a threshold at the typical entropy of these logits, so that both temperatures occur
    x0 = torch.randn(1, H, generator=g, device="cuda").to(torch.bfloat16)
    tau0 = float(orp.token_entropy_f64(_lm_head(x0, W)[0].cpu().numpy()))
    t_high, t_low, window = 1.0, 0.3, 8
    pol = orp.ResetPolicy(t_high, t_low, tau0, window, frozenset([nl]), frozenset([delim]))
    prm = _params_dev((t_high, t_low, tau0, window, 0))
    nl_bm, dnl_bm = _bitmap([nl], V), _bitmap([delim], V)
    size = C.sizeof(_lib.ResetState)
    st_f = torch.zeros(size, dtype=torch.uint8, device="cuda")
    st_r = torch.zeros(size, dtype=torch.uint8, device="cuda")
    dec_f = torch.zeros(C.sizeof(_lib.ResetDecision), dtype=torch.uint8, device="cuda")
    dec_r = torch.zeros_like(dec_f)
    ws_f = capi.lm_head_reset_workspace("cuda")
    ws_r = capi.reset_workspace(1, "cuda")
    out_f = torch.empty(1, V, dtype=torch.float32, device="cuda")
    ties = mism = lows = 0
    for t in range(steps):
        x = torch.randn(1, H, generator=g, device="cuda").to(torch.bfloat16)
        last = torch.tensor([[stream[t - 2] if t >= 2 else -1, stream[t - 1] if t >= 1 else -1]],
                            dtype=torch.int32, device="cuda")
        raw = _lm_head(x, W)
        out_r = raw.clone()
        capi.reset_step_per_request(out_r, st_r, prm, last_ids=last, nl_bitmaps=nl_bm, dnl_bitmaps=dnl_bm,
                                    n_id_sets=1, decisions=dec_r, workspace=ws_r)
        out_f.fill_(float("nan"))
        capi.lm_head_reset_step(x, W, out_f, st_f, prm, last_ids=last, nl_bitmaps=nl_bm, dnl_bitmaps=dnl_bm,
                                n_id_sets=1, decisions=dec_f, workspace=ws_f)
        gf = np.frombuffer(dec_f.cpu().numpy().tobytes(), dtype=DEC)[0]
        gr = np.frombuffer(dec_r.cpu().numpy().tobytes(), dtype=DEC)[0]
        logits = raw[0].cpu()
        d = pol.decide(pol.is_boundary(stream[max(0, t - 2):t].tolist()), orp.token_entropy(logits))
        thr = d.h_step if d.high_step else tau0
        near_tie = abs(d.entropy - thr) < TIE_BAND or abs(d.h_step - d.h_bar) < TIE_BAND
        ties += near_tie
        lows += d.temp != 1.0
        # (a) the two-launch path
        assert gf["boundary"] == gr["boundary"]
        assert abs(gf["entropy"] - gr["entropy"]) <= 1e-5 and abs(gf["h_step"] - gr["h_step"]) <= 1e-5
        if gf["temp"] == gr["temp"]:
            assert torch.equal(out_f, out_r), t
        else:
            assert near_tie, (t, gf, gr)
        # (b) the oracle
        assert bool(gf["boundary"]) == d.boundary
        assert abs(gf["entropy"] - orp.token_entropy_f64(logits.numpy())) <= 1e-5
        assert abs(gf["entropy"] - d.entropy) <= 1e-4
        assert abs(gf["h_step"] - d.h_step) <= 1e-4 and abs(gf["h_bar"] - d.h_bar) <= 1e-4
        if gf["temp"] != d.temp:
            assert near_tie, (t, gf, d)
            mism += 1
        else:
            assert torch.equal(out_f[0].cpu(), orp.apply_temperature(logits, d.temp)), t
    assert mism <= ties
    if steps >= 64:
        assert 0 < lows < steps                     # both temperatures were taken
    assert _lib.lib().nvfp4r_check_device_status() == 0


def test_fused_launch_one_hot_and_inactive_request(capi):
    from reset_b200 import _lib
    V, H = 8192, 512
    W, g = _model(V, H, seed=3)
    x = torch.randn(1, H, generator=g, device="cuda").to(torch.bfloat16)
    raw = _lm_head(x, W)
    size = C.sizeof(_lib.ResetState)
    ws = capi.lm_head_reset_workspace("cuda")
    out = torch.empty(1, V, dtype=torch.float32, device="cuda")
    # t_low = 0 below a threshold no entropy reaches: one-hot at the arg-max
    states = torch.zeros(2 * size, dtype=torch.uint8, device="cuda")
    prm = _params_dev((1.0, 0.5, 0.0, 32, 0), (1.0, 0.0, 100.0, 32, 0))
    slot = torch.tensor([1], dtype=torch.int32, device="cuda")
    capi.lm_head_reset_step(x, W, out, states, prm, state_slots=slot, workspace=ws)
    want = torch.full((V,), float("-inf"))
    want[int(raw.argmax())] = 0.0
    assert torch.equal(out[0].cpu(), want)
    st = states.cpu().numpy().reshape(2, size)
    assert st[0].max() == 0 and st[1].max() > 0
    # slot -1: a request without ReSET gets the plain lm_head logits, no state is touched
    before = states.clone()
    slot.fill_(-1)
    capi.lm_head_reset_step(x, W, out, states, prm, state_slots=slot, workspace=ws)
    assert torch.equal(out, raw) and torch.equal(states, before)
    # slot 0 (t_high = 1 at a threshold of 0): the logits come out untouched, the state advances
    slot.fill_(0)
    capi.lm_head_reset_step(x, W, out, states, prm, state_slots=slot, workspace=ws)
    assert torch.equal(out, raw)
    assert states.cpu().numpy().reshape(2, size)[0].max() > 0
    assert _lib.lib().nvfp4r_check_device_status() == 0


def test_fused_launch_replays_in_a_cuda_graph(capi):
    """Captured once, replayed with new activations: the request state lives on the device and the
    epoch-tagged slots need no clearing, so every replay is a full step."""
    from reset_b200 import _lib
    V, H = 32000, 1024
    W, g = _model(V, H, seed=8)
    x = torch.zeros(1, H, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(1, V, dtype=torch.float32, device="cuda")
    states = torch.zeros(C.sizeof(_lib.ResetState), dtype=torch.uint8, device="cuda")
    dec = torch.zeros(C.sizeof(_lib.ResetDecision), dtype=torch.uint8, device="cuda")
    prm = _params_dev((1.0, 0.25, 100.0, 4, 0))
    ws = capi.lm_head_reset_workspace("cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        capi.lm_head_reset_step(x, W, out, states, prm, decisions=dec, workspace=ws)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            capi.lm_head_reset_step(x, W, out, states, prm, decisions=dec, workspace=ws)
    torch.cuda.current_stream().wait_stream(side)
    states.zero_()
    ents = []
    for t in range(6):
        x.copy_(torch.randn(1, H, generator=g, device="cuda").to(torch.bfloat16))
        graph.replay()
        torch.cuda.synchronize()
        raw = _lm_head(x, W)
        assert torch.equal(out, raw / 0.25)
        ents.append(float(np.frombuffer(dec.cpu().numpy().tobytes(), dtype=DEC)[0]["entropy"]))
    st = _lib.ResetState.from_buffer_copy(states.cpu().numpy().tobytes())
    assert st.total_count == 6 and abs(st.total_sum - sum(ents)) <= 1e-9
    assert _lib.lib().nvfp4r_check_device_status() == 0
