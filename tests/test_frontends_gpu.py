"""The reference-facing front ends on the GPU: `ReSETRequest` / `ReSETBatchProcessor`
(reset/reset/logits_processor.py:62-155 of the reference) against the CPU oracle policy, and
the vLLM adapter entry points `prime_nvfp4r_caches` / `apply_nvfp4r_linear`
(kernels/python/nvfp4r/vllm_integration.py:359-396,448-496) on a stand-in layer object."""

from __future__ import annotations

from collections import namedtuple
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from oracle import nvfp4 as onv
from oracle import reset_policy as orp
from helpers import cuda, make_activation, rel_l2

pytestmark = pytest.mark.gpu
TIE_BAND = 1e-4
try:      # vLLM's own batch-update record and move enum when vLLM is installed, stand-ins otherwise
    from vllm.v1.sample.logits_processor import BatchUpdate as _VllmBatchUpdate, MoveDirectionality

    def BatchUpdate(removed, added, moved):
        return _VllmBatchUpdate(batch_size=len(added), removed=removed, added=added, moved=moved)

    UNIDIRECTIONAL = MoveDirectionality.UNIDIRECTIONAL
except ImportError:
    BatchUpdate = namedtuple("BatchUpdate", "removed added moved")
    UNIDIRECTIONAL = SimpleNamespace(name="UNIDIRECTIONAL")


def _near_tie(d, tau0):
    thr = d.h_step if d.high_step else tau0
    return abs(d.entropy - thr) < TIE_BAND or abs(d.h_step - d.h_bar) < TIE_BAND


def test_reset_request_matches_oracle():
    from reset_b200.reset import ReSETRequest
    V, steps, nl, dnl = 4096, 90, 11, 13
    ids = orp.synthetic_token_stream(steps, dnl, V, seed=5, gap_lo=10, gap_hi=25)
    ids[30:32] = nl                                     # two single newlines in a row: a boundary too
    req = ReSETRequest(1.0, 0.3, 6.0, 8, [nl], [dnl])
    pol = orp.ResetPolicy(1.0, 0.3, 6.0, 8, frozenset([nl]), frozenset([dnl]))
    temps = set()
    for t in range(steps):
        logits = orp.synthetic_logits(1, V, 1000 + t, sigma=2.0)[0]
        got = req(ids[:t].tolist(), logits.cuda())
        want, d = pol(ids[:t].tolist(), logits)
        g = req.last_decision()
        assert bool(g["boundary"]) == d.boundary
        assert abs(g["entropy"] - d.entropy) <= 1e-4
        if g["temp"] == d.temp:
            assert torch.equal(got.cpu(), want)
        else:
            assert _near_tie(d, 6.0)
        temps.add(g["temp"])
    assert temps == {1.0, 0.3}                          # both regimes were exercised


def test_batch_processor_matches_per_request_oracle():
    """Three batch rows (one not opted in), a removal and a move in mid-stream, through the
    vLLM v1 LogitsProcessor interface."""
    from reset_b200.reset import ReSETBatchProcessor
    V, dnl = 4096, 17
    ea = {"reset": True, "t_high": 1.0, "t_low": 0.5, "tau_0": 6.0, "window": 4, "reset_nl_ids": [],
          "reset_dnl_ids": [dnl]}
    proc = ReSETBatchProcessor(device="cuda", max_num_reqs=4, vocab_size=V)
    assert proc.is_argmax_invariant() is False
    outs = {0: [], 1: [], 2: []}                        # live output-id lists, as vLLM hands them over
    pols = {0: orp.ResetPolicy(1.0, 0.5, 6.0, 4, frozenset(), frozenset([dnl])),
            2: orp.ResetPolicy(1.0, 0.5, 6.0, 4, frozenset(), frozenset([dnl]))}
    proc.update_state(BatchUpdate(removed=[], moved=[], added=[
        (0, SimpleNamespace(extra_args=dict(ea)), [1, 2], outs[0]),
        (1, SimpleNamespace(extra_args=None), [3], outs[1]),
        (2, SimpleNamespace(extra_args=dict(ea)), [4], outs[2])]))
    rng = np.random.default_rng(3)
    rows = {0: 0, 1: 1, 2: 2}                           # request -> batch row

    def step(t, batch):
        logits = orp.synthetic_logits(batch, V, 2000 + t, sigma=2.0)
        dev = logits.cuda()
        ret = proc.apply(dev)
        assert ret.data_ptr() == dev.data_ptr()          # in place, like vLLM expects
        res = dev.cpu()
        for rq, row in rows.items():
            if rq in pols:
                want, d = pols[rq](list(outs[rq]), logits[row])
                if not _near_tie(d, 6.0):
                    assert torch.equal(res[row], want), (t, rq)
            else:
                assert torch.equal(res[row], logits[row])          # not opted in: untouched
        for rq in rows:
            outs[rq].append(dnl if rng.random() < 0.15 else int(rng.integers(20, V)))

    for t in range(12):
        step(t, 3)
        proc.update_state(None)
    # request 0 finishes; request 2 moves from row 2 to row 0 (vLLM condenses the batch)
    del rows[0], pols[0]
    rows[2] = 0
    proc.update_state(BatchUpdate(removed=[0], added=[], moved=[(2, 0, UNIDIRECTIONAL)]))
    for t in range(12, 24):
        step(t, 2)
        proc.update_state(None)


def test_batch_processor_keeps_each_requests_own_parameters():
    """Three requests with three different (t_high, t_low, tau_0, window) and two different
    newline-id sets in one batch, each against its own oracle policy: the reference builds one
    ReSETRequest per request from that request's extra_args
    (reset/reset/logits_processor.py:144-155)."""
    from reset_b200.reset import ReSETBatchProcessor
    V = 4096
    cfgs = {0: dict(t_high=1.0, t_low=0.5, tau_0=6.0, window=4, nl=[], dnl=[17]),
            1: dict(t_high=0.9, t_low=0.2, tau_0=5.2, window=16, nl=[23], dnl=[29]),
            2: dict(t_high=1.0, t_low=0.1, tau_0=6.6, window=32, nl=[], dnl=[17])}
    proc = ReSETBatchProcessor(device="cuda", max_num_reqs=4, vocab_size=V)
    outs = {r: [] for r in cfgs}
    pols = {r: orp.ResetPolicy(c["t_high"], c["t_low"], c["tau_0"], c["window"], frozenset(c["nl"]),
                               frozenset(c["dnl"])) for r, c in cfgs.items()}
    proc.update_state(BatchUpdate(removed=[], moved=[], added=[
        (r, SimpleNamespace(extra_args={"reset": True, "t_high": c["t_high"], "t_low": c["t_low"],
                                        "tau_0": c["tau_0"], "window": c["window"],
                                        "reset_nl_ids": c["nl"], "reset_dnl_ids": c["dnl"]}), [1], outs[r])
        for r, c in cfgs.items()]))
    rng = np.random.default_rng(11)
    seen = {r: set() for r in cfgs}
    checked = 0
    for t in range(60):
        logits = orp.synthetic_logits(3, V, 5000 + t, sigma=2.0)
        dev = logits.cuda()
        proc.apply(dev)
        res = dev.cpu()
        for r, c in cfgs.items():
            want, d = pols[r](list(outs[r]), logits[r])
            seen[r].add(d.temp)
            if not _near_tie(d, c["tau_0"]):
                assert torch.equal(res[r], want), (t, r)
                checked += 1
        for r, c in cfgs.items():
            u = rng.random()
            nxt = c["dnl"][0] if u < 0.1 else (c["nl"][0] if c["nl"] and u < 0.4 else int(rng.integers(40, V)))
            outs[r].append(nxt)
        proc.update_state(None)
    assert checked >= 100
    for r, c in cfgs.items():                            # every request used both of ITS temperatures
        assert seen[r] == {c["t_high"], c["t_low"]}, (r, seen[r])


def _fake_layer(N, K, seed, alpha=0.37, gs_inv=55.0, swizzled=True):
    from reset_b200 import capi
    w, ws = onv.random_nvfp4((N,), K, seed=seed)
    layer = torch.nn.Module()
    layer.weight = torch.nn.Parameter(cuda(w), requires_grad=False)
    flat = cuda(ws)
    scale = capi.swizzle_blockscale(flat) if swizzled else flat
    layer.weight_scale = torch.nn.Parameter(scale.view(torch.float8_e4m3fn), requires_grad=False)
    layer._nvfp4r_weight_scale_is_flat = not swizzled
    layer.input_global_scale_inv = torch.tensor([gs_inv], dtype=torch.float32, device="cuda")
    layer.alpha = torch.tensor(alpha, dtype=torch.float32, device="cuda")
    layer.input_size_per_partition, layer.output_size_per_partition = K, N
    layer.weights_padding_cols = 0
    return layer, w, ws


@pytest.mark.parametrize("N,K,swizzled", [(4096, 1024, True), (6144, 4096, True), (1000, 320, False)])
def test_vllm_adapter_on_a_stand_in_layer(N, K, swizzled):
    from reset_b200 import _lib, capi
    from reset_b200.nvfp4r import vllm_integration as vi
    layer, w, ws = _fake_layer(N, K, seed=N % 97, swizzled=swizzled)
    vi.prime_nvfp4r_caches(layer)
    vi.prime_nvfp4r_caches(layer)                       # idempotent
    assert layer._nvfp4r_caches_primed and abs(layer._nvfp4r_alpha_host - 0.37) < 1e-7
    assert tuple(layer._nvfp4r_weight_scale_flat_3d.shape) == (1, N, K // 16)
    assert np.array_equal(layer._nvfp4r_weight_scale_flat_3d[0].cpu().numpy(), ws)
    assert (layer._nvfp4r_weight_packed is not None) == (N % 128 == 0 and K % 128 == 0)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    for M in (1, 2, 5, 40):
        x = make_activation(M, K, seed=M).cuda()
        y = vi.apply_nvfp4r_linear(layer, x.view(1, M, K), bias if M == 5 else None)
        assert tuple(y.shape) == (1, M, N) and y.dtype == torch.bfloat16
        # The adapter quantizes with the reciprocal arithmetic of the CUDA op the reference
        # calls (bit-identical to the installed vLLM's scaled_fp4_quant, see test_quant_gpu), which
        # breaks exact rounding ties differently from the IEEE-division oracle; so the codes come
        # from the stand-alone quantizer in that mode and the oracle checks the linear on them.
        codes, scales = capi.quant(x, layer.input_global_scale_inv, rcp_mode=_lib.RCP_APPROX)
        exact = onv.linear_f64(w, ws, codes.cpu().numpy(), scales.cpu().numpy(), alpha=0.37)
        exact_mode = onv.linear_f64(w, ws, *onv.quantize_nvfp4(x.float().cpu().numpy(), 55.0), alpha=0.37)
        assert rel_l2(exact, exact_mode) <= 5e-2          # the two tie-breaking rules stay close
        if M == 5:
            exact = exact + bias.float().cpu().numpy()
        assert rel_l2(y[0].float().cpu().numpy(), exact) <= 6e-3        # bf16 output rounding


def test_vllm_adapter_rejects_padded_weights():
    from reset_b200.nvfp4r import vllm_integration as vi
    layer, _, _ = _fake_layer(256, 512, seed=1)
    vi.prime_nvfp4r_caches(layer)
    layer.weights_padding_cols = 64
    with pytest.raises(RuntimeError):
        vi.apply_nvfp4r_linear(layer, torch.zeros(1, 512, dtype=torch.bfloat16, device="cuda"))


def _modelopt_style_layer(N, K, seed, alpha=0.4, gs_inv=48.0):
    """The attributes vLLM's ModelOpt NVFP4 linear method leaves on a layer before it calls
    ``kernel.process_weights_after_loading`` (flat e4m3 block scales)."""
    w, ws = onv.random_nvfp4((N,), K, seed=seed)
    layer = torch.nn.Module()
    layer.weight = torch.nn.Parameter(cuda(w), requires_grad=False)
    layer.weight_scale = torch.nn.Parameter(cuda(ws).view(torch.float8_e4m3fn), requires_grad=False)
    layer.input_global_scale_inv = torch.nn.Parameter(torch.tensor(gs_inv, dtype=torch.float32, device="cuda"),
                                                      requires_grad=False)
    layer.alpha = torch.nn.Parameter(torch.tensor(alpha, dtype=torch.float32, device="cuda"), requires_grad=False)
    layer.input_size_per_partition, layer.output_size_per_partition = K, N
    return layer, w, ws


@pytest.mark.parametrize("N,K", [(4096, 1024), (6144, 4096)])
def test_kernel_class_selected_by_the_installed_vllm_and_agrees_with_its_cutlass_kernel(N, K, monkeypatch):
    """`nvfp4r.enable()` makes the installed vLLM's own selection routine return this
    library's kernel class; on the same layer it agrees with vLLM's CUTLASS kernel class
    (the comparison the reference makes in kernels/tests/test_vllm_integration.py:61-95,
    there against a patched vLLM) and with the oracle."""
    vk = pytest.importorskip("vllm.model_executor.kernels.linear")
    if not hasattr(vk, "_POSSIBLE_NVFP4_KERNELS"):
        pytest.skip("this vLLM has no NVFP4 kernel registry")
    from vllm.model_executor.kernels.linear.nvfp4.base import NvFp4LinearLayerConfig
    from vllm.model_executor.kernels.linear.nvfp4.cutlass import CutlassNvFp4LinearKernel
    from reset_b200 import _lib, capi, nvfp4r
    monkeypatch.delenv("VLLM_NVFP4_GEMM_BACKEND", raising=False)
    nvfp4r.enable()
    try:
        kernel = vk.init_nvfp4_linear_kernel()
        assert type(kernel).__name__ == "Nvfp4rLinearKernel"
    finally:
        nvfp4r.disable()
    ours, w, ws = _modelopt_style_layer(N, K, seed=21)
    kernel.process_weights_after_loading(ours)
    assert ours._nvfp4r_caches_primed and ours.weights_padding_cols == 0
    stock = None
    if CutlassNvFp4LinearKernel.is_supported()[0]:
        stock_layer, _, _ = _modelopt_style_layer(N, K, seed=21)
        stock = CutlassNvFp4LinearKernel(NvFp4LinearLayerConfig())
        stock.process_weights_after_loading(stock_layer)
    for M in (1, 2, 8, 32):
        x = make_activation(M, K, seed=100 + M).cuda()
        y = kernel.apply_weights(ours, x.view(1, M, K))
        assert tuple(y.shape) == (1, M, N) and y.dtype == torch.bfloat16
        codes, scales = capi.quant(x, ours.input_global_scale_inv.reshape(1), rcp_mode=_lib.RCP_APPROX)
        exact = onv.linear_f64(w, ws, codes.cpu().numpy(), scales.cpu().numpy(), alpha=0.4)
        assert rel_l2(y[0].float().cpu().numpy(), exact) <= 6e-3            # bf16 output rounding
        if stock is not None:
            z = stock.apply_weights(stock_layer, x.view(1, M, K))
            # same codes and scales on both sides (the quantizers are bit-identical in this mode),
            # fp32 accumulation in different orders, one bf16 rounding each
            assert rel_l2(y.float().cpu().numpy(), z.float().cpu().numpy()) <= 8e-3


def test_dispatch_is_one_registered_operator_with_a_fake():
    """`torch.ops.vllm.nvfp4r_linear` exists with the reference's argument list
    (kernels/python/nvfp4r/vllm_integration.py:165-178,342-353) and traces on fake tensors."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    from reset_b200.nvfp4r import vllm_integration as vi  # noqa: F401  (registers the op)
    schema = str(torch.ops.vllm.nvfp4r_linear.default._schema)
    for name in ("x_2d", "weight", "weight_scale_swizzled", "weight_scale_flat_3d", "input_global_scale_inv",
                 "alpha", "alpha_host", "output_size", "weights_padding_cols", "gemv_max_m", "out_dtype_int",
                 "enable_gemm"):
        assert name in schema
    layer, _, _ = _fake_layer(512, 1024, seed=2)
    vi.prime_nvfp4r_caches(layer)
    with FakeTensorMode(allow_non_fake_inputs=True):
        x = torch.empty((7, 1024), dtype=torch.bfloat16, device="cuda")
        y = vi.apply_nvfp4r_linear(layer, x)
    assert tuple(y.shape) == (7, 512) and y.dtype == torch.bfloat16


@pytest.mark.parametrize("N,K", [(4096, 1024), (6144, 4096)])
def test_adapter_compiles_fullgraph_and_replays_in_a_cuda_graph(N, K):
    """`apply_nvfp4r_linear` under torch.compile(fullgraph=True) is one opaque node whose M
    branch is taken at run time: the same compiled function serves M = 1 and M = 8 (each on
    its own side of the crossover) and equals the eager call bit for bit; the compiled call
    then replays inside a CUDA graph."""
    from reset_b200.nvfp4r import vllm_integration as vi
    layer, w, ws = _fake_layer(N, K, seed=31)
    vi.prime_nvfp4r_caches(layer)

    def forward(x):
        return vi.apply_nvfp4r_linear(layer, x)

    compiled = torch.compile(forward, fullgraph=True, backend="aot_eager", dynamic=True)
    xs = {M: make_activation(M, K, seed=40 + M).cuda() for M in (1, 8, 3)}
    for M in (1, 8, 3):
        eager = forward(xs[M])
        got = compiled(xs[M])
        torch.cuda.synchronize()
        assert tuple(got.shape) == (M, N) and torch.equal(got, eager)
    static_x = xs[8].clone()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        compiled(static_x)
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            static_y = compiled(static_x)
    for seed in (50, 51):
        fresh = make_activation(8, K, seed=seed).cuda()
        static_x.copy_(fresh)
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(static_y, forward(fresh))


@pytest.mark.parametrize("fallback", ["vllm-cutlass", "none"])
def test_adapter_prefill_sized_batch(fallback):
    """M above gemm_pad_max_m: the installed vLLM's own NVFP4 GEMM when it is importable and
    not switched off (the reference's fallback branch, vllm_integration.py:299-318), else this
    library's kernels in launches of 32 rows. Both agree with the oracle."""
    from reset_b200 import _lib, capi, nvfp4r
    from reset_b200.nvfp4r import vllm_integration as vi
    N, K, M = 1024, 2048, 100
    layer, w, ws = _fake_layer(N, K, seed=61)
    vi.prime_nvfp4r_caches(layer)
    saved = nvfp4r.status()["fallback_backend"]
    nvfp4r.configure(fallback_backend=fallback)
    try:
        if fallback != "none" and not vi._fallback_available():
            pytest.skip("vLLM's NVFP4 ops are not importable here")
        x = make_activation(M, K, seed=62).cuda()
        y = vi.apply_nvfp4r_linear(layer, x)
    finally:
        nvfp4r.configure(fallback_backend=saved)
    codes, scales = capi.quant(x, layer.input_global_scale_inv, rcp_mode=_lib.RCP_APPROX)
    exact = onv.linear_f64(w, ws, codes.cpu().numpy(), scales.cpu().numpy(), alpha=0.37)
    assert tuple(y.shape) == (M, N)
    assert rel_l2(y.float().cpu().numpy(), exact) <= 8e-3               # bf16 output rounding
