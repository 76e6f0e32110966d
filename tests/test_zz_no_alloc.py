"""``nvfp4r_reset_step_static``: the ReSET step for hosts that cannot allocate device
memory when they need it (a sampler plug-in inside an engine whose pool already owns the
GPU, a C host holding only fixed input/output buffers). Its scratch is a static array in
the library, so the call takes no workspace. Checked here through the C ABI against the
regular entry point, on two consecutive steps (the static array keeps the previous call's
contents, which must not leak into the next result), bit for bit: the regular entry point
takes the single-launch kernel, the static one the three-launch form of the same arithmetic,
and the two are required to agree exactly."""

from __future__ import annotations

import ctypes as C

import numpy as np
import pytest
import torch

from oracle import reset_policy as orp

pytestmark = pytest.mark.gpu


def _run_two_steps(static: bool, B: int, V: int):
    from reset_b200 import _lib, capi
    lib = _lib.lib()
    params = _lib.ResetParams(1.0, 0.3, 5.2, 8, 0)
    states = torch.zeros(B * C.sizeof(_lib.ResetState), dtype=torch.uint8, device="cuda")
    decisions = torch.zeros(B * C.sizeof(_lib.ResetDecision), dtype=torch.uint8, device="cuda")
    workspace = None if static else capi.reset_workspace(B, "cuda")
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for step in range(2):
        logits = orp.synthetic_logits(B, V, seed=40 + step, sigma=1.5).cuda()
        last = torch.full((B, 2), -1, dtype=torch.int32, device="cuda")
        if static:
            st = lib.nvfp4r_reset_step_static(logits.data_ptr(), logits.stride(0), B, V,
                                              states.data_ptr(), None, last.data_ptr(), None, None,
                                              C.byref(params), decisions.data_ptr(), stream)
        else:
            st = lib.nvfp4r_reset_step(logits.data_ptr(), logits.stride(0), B, V, states.data_ptr(),
                                       None, last.data_ptr(), None, None, C.byref(params),
                                       decisions.data_ptr(), workspace.data_ptr(),
                                       workspace.numel() * 8, stream)
        _lib.check(st, "reset step")
        torch.cuda.synchronize()
        outs.append((logits.cpu(), decisions.cpu().clone()))
    return outs, states.cpu()


@pytest.mark.parametrize("B,V", [(3, 4096), (8, 151936)])
def test_static_scratch_step_equals_workspace_step(B, V):
    got, got_state = _run_two_steps(True, B, V)
    want, want_state = _run_two_steps(False, B, V)
    for (lg, dg), (lw, dw) in zip(got, want):
        assert torch.equal(lg, lw)              # scaled logits, bit for bit
        assert torch.equal(dg, dw)              # entropy, thresholds, temperature
    assert torch.equal(got_state, want_state)
    # and the values are right, not merely equal: entropy of the second step vs the oracle
    ent = np.frombuffer(got[1][1].numpy().tobytes(), dtype="f8").reshape(B, -1)[:, 0]
    ref = orp.synthetic_logits(B, V, seed=41, sigma=1.5)
    for b in range(B):
        assert abs(ent[b] - orp.token_entropy_f64(ref[b].numpy())) <= 1e-5


def test_static_scratch_rejects_too_many_rows():
    from reset_b200 import _lib
    lib = _lib.lib()
    B = _lib.RESET_STATIC_MAX_ROWS + 1
    logits = torch.zeros((B, 64), dtype=torch.float32, device="cuda")
    states = torch.zeros(B * C.sizeof(_lib.ResetState), dtype=torch.uint8, device="cuda")
    params = _lib.ResetParams(1.0, 0.5, 1.0, 8, 0)
    st = lib.nvfp4r_reset_step_static(logits.data_ptr(), 64, B, 64, states.data_ptr(), None, None,
                                      None, None, C.byref(params), None, None)
    assert st == -2 and b"NVFP4R_RESET_STATIC_MAX_ROWS" in lib.nvfp4r_last_error()
