"""Benchmark of the NVFP4 W4A4 decode linear path on B200.

Workload (``config.workload``): the Qwen3-8B decode linear set - qkv_proj 4096->6144,
o_proj 4096->4096, gate_up_proj 4096->24576, down_proj 12288->4096 - in NVFP4 W4A4 at
M in {1,2,4,8}, each call including the activation quantization (one fused launch per
linear). One *step* is one pass over the 4 x 4 = 16 (linear, M) pairs. Every launch
reads a different copy of its weight (``weight_copies`` copies per linear, > 1 GB in
total, cycled), so no launch finds its weight in L2.

Metric: HBM GB/s = algorithmic bytes of the step / step time, where the algorithmic
bytes of one linear are N*K/2 + N*K/16 (weight codes + scales, counted once whatever
M is) + M*K*2 (bf16 activations in) + M*N*2 (bf16 out).

``python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]``; under
torchrun (N > 1) the linears are tensor-parallel: qkv/gate_up column-sharded, o/down
row-sharded with a sum of the [M, hidden] partial results after each (this library's
exchange over NVLink peer memory, fused into the linear's launch where that wins;
``--allreduce nccl`` for NCCL). Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

LINEARS = [  # name, N, K, tensor-parallel style
    ("qkv_proj", 6144, 4096, "column"),
    ("o_proj", 4096, 4096, "row"),
    ("gate_up_proj", 24576, 4096, "column"),
    ("down_proj", 4096, 12288, "row"),
]
M_VALUES = (1, 2, 4, 8)
HIDDEN = 4096
WEIGHT_COPIES = 12
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch, averaged over the 16 launches of a
# single-GPU step (an ncu capture of this program's --case launches; algorithmic bytes per
# launch: 27.1 MB). Reported at N = 1 only: a tensor-parallel launch moves 1/N of the bytes
# and has not been captured.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 27.4e6


def linear_bytes(N: int, K: int, M: int) -> int:
    return N * K // 2 + N * K // 16 + M * K * 2 + M * N * 2


def step_bytes(tp: int = 1) -> int:
    return sum(linear_bytes(N, K, M) for _, N, K, _ in LINEARS for M in M_VALUES)


def measured_peak():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons during the timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(index), "-lms", "100"], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        rows = [r.strip().split(", ") for r in Path(self.tmp.name).read_text().splitlines() if r.strip()]
        os.unlink(self.tmp.name)
        sm = sorted(int(r[0]) for r in rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v == "Active"})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None,
                "sm_max_mhz": int(rows[0][1]) if rows and rows[0][1].isdigit() else None,
                "samples": len(sm), "reasons": reasons}


# The shapes the bandwidth target is stated on: Qwen3-32B decode linears at M = 1 (N, K).
QWEN3_32B_LINEARS = [("qkv_proj", 10240, 5120), ("o_proj", 5120, 8192),
                     ("gate_up_proj", 51200, 5120), ("down_proj", 5120, 25600)]


def qwen3_32b_m1_detail(device, nvfp4r, peak: float) -> dict:
    """us / GB/s / % of peak of each Qwen3-32B decode linear at M = 1, quantizer included, through
    the crossover's choice of kernel; every launch reads a weight copy that has left L2 (enough
    copies of each weight for > 600 MB between two reads of the same copy)."""
    out = {}
    gs = torch.tensor([100.0], dtype=torch.float32, device=device)
    g = torch.Generator(device=device).manual_seed(4321)
    gemv_max_m = nvfp4r.status()["gemv_max_m"]
    side = torch.cuda.Stream(device=device)
    for name, N, K in QWEN3_32B_LINEARS:
        wbytes = N * K * 9 // 16
        ncopies = max(3, -(-600_000_000 // wbytes))
        copies = []
        for _ in range(ncopies):
            w = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=device, generator=g)
            sc = torch.randint(1, 0x38, (N, K // 16), dtype=torch.uint8, device=device, generator=g)
            use_gemv = nvfp4r.ops.use_gemv(1, N, K, gemv_max_m)
            copies.append((w, sc, None) if use_gemv else (None, None, nvfp4r.pack_weight(w, sc)))
        x = torch.randn(1, K, device=device, generator=g).to(torch.bfloat16)
        outbuf = torch.empty((1, N), dtype=torch.bfloat16, device=device)
        # warm-up once per copy (also sizes the split-K scratch outside the capture)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for w, sc, packed in copies:
                nvfp4r.linear_auto(x, gs, w, sc, packed, N, 1.0, torch.bfloat16, out=outbuf)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(2):
                    for w, sc, packed in copies:
                        nvfp4r.linear_auto(x, gs, w, sc, packed, N, 1.0, torch.bfloat16, out=outbuf)
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / (2 * ncopies) * 1e3)
        us = sorted(ts)[2]
        gbs = linear_bytes(N, K, 1) / us / 1e3
        out[f"qwen3_32b_{name}_M1"] = {"us": round(us, 2), "kernel": "gemv" if copies[0][2] is None else "tcgen05",
                                       "gbs": round(gbs, 1), "pct_of_peak": round(100.0 * gbs / peak, 1),
                                       "N": N, "K": K, "weight_copies": ncopies}
        del copies, graph
        torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------- ours

def build_weights(rank: int, tp: int, device, nvfp4r):
    """Random NVFP4 codes + scale bytes (scales below 1.0, as the reference's own test
    generator bounds them) for this rank's shard of every linear, WEIGHT_COPIES copies."""
    g = torch.Generator(device=device).manual_seed(1234 + rank)
    shards = []
    for name, N, K, style in LINEARS:
        n = N // tp if style == "column" else N
        k = K // tp if style == "row" else K
        copies = []
        for _ in range(WEIGHT_COPIES):
            w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=device, generator=g)
            s = torch.randint(1, 0x38, (n, k // 16), dtype=torch.uint8, device=device, generator=g)
            # weight preparation (once per layer, not timed): the packed block format of the
            # tensor-core path next to the flat format of the CUDA-core GEMV
            packed = nvfp4r.pack_weight(w, s) if (n % 128 == 0 and k % 128 == 0) else None
            copies.append((w, s, packed))
        shards.append((name, n, k, style, copies))
    return shards


def make_inputs(shards, device, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    xs = {}
    for name, n, k, style, _ in shards:
        for M in M_VALUES:
            x = torch.randn(M, k, generator=g, dtype=torch.float32)
            cols = torch.randperm(k, generator=g)[: max(1, k // 1000)]
            x[:, cols] *= 20.0
            xs[(name, M)] = x.to(torch.bfloat16)
    return xs


_T0 = time.perf_counter()
# Libraries (NCCL's version banner) write to file descriptor 1; the JSON line must be alone on
# stdout, so keep a private handle on the real stdout and point descriptor 1 at stderr.
_STDOUT = os.fdopen(os.dup(1), "w")
os.dup2(2, 1)


def stage(rank: int, what: str) -> None:
    """Progress line on stderr (the JSON line on stdout stays alone)."""
    print(f"[bench rank {rank} +{time.perf_counter() - _T0:.1f}s] {what}", file=sys.stderr, flush=True)


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist

    from reset_b200 import nvfp4r  # registers torch.ops.nvfp4r.* (raises if not built)
    from reset_b200.nvfp4r import _config as nv_config

    if args.no_fused_gather:
        nv_config.FUSED_GATHER = "0"
    if args.packed_tuning:
        from reset_b200 import _lib
        _lib.check(_lib.lib().nvfp4r_set_packed_tuning(args.packed_tuning), "packed tuning")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    tp = world
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if args.decode_only:
        out = run_decode(args, rank, world, device)
        return {"decode": out} if rank == 0 else None
    stage(rank, "process group up" if world > 1 else "device ready")
    shards = build_weights(rank, tp, device, nvfp4r)
    stage(rank, "weights built")
    host_x = make_inputs(shards, device, seed=7)
    dev_x = {k: v.to(device) for k, v in host_x.items()}
    gs = torch.tensor([100.0], dtype=torch.float32, device=device)
    peer = None
    if world > 1 and args.allreduce == "peer":
        from reset_b200.comm import PeerAllReduce
        peer = PeerAllReduce(device, max(M_VALUES) * HIDDEN)
    counters = {name: 0 for name, *_ in shards}
    path_used = {}
    gemv_max_m = nvfp4r.status()["gemv_max_m"]

    def one_linear(name, n, k, style, copies, M, x):
        w, s, packed = copies[counters[name] % WEIGHT_COPIES]
        counters[name] += 1
        fused_reduce = peer if (world > 1 and style == "row") else None
        out = nvfp4r.linear_auto(x, gs, w, s, packed, n, 1.0, torch.bfloat16, reduce=fused_reduce)
        path_used[(name, M)] = "gemv" if (packed is None or nvfp4r.ops.use_gemv(M, n, k, gemv_max_m)) else "tcgen05"
        if world > 1 and style == "row" and peer is None:
            dist.all_reduce(out)
        return out

    def step_resident():
        for M in M_VALUES:
            for name, n, k, style, copies in shards:
                one_linear(name, n, k, style, copies, M, dev_x[(name, M)])

    # End-to-end step: the step's activations come from pinned host memory (one transfer) and all
    # its results go back to pinned host memory (one transfer) inside the timed region; the 16
    # launches write into one output buffer through the out= variant of the public call. Steps are
    # pipelined the way a serving loop would: three sets of device buffers (one per weight-copy
    # phase), the transfer of step i + 1's inputs on a copy stream while step i computes, the
    # transfer of step i's results on a second copy stream while step i + 1 computes; the launches
    # themselves stay in stream order on one stream (one CUDA graph per step, nothing but the
    # launches in it, so the programmatic launch chain is intact).
    in_off, out_off, o_in, o_out = {}, {}, 0, 0
    for name, n, k, style, _ in shards:
        for M in M_VALUES:
            in_off[(name, M)] = (o_in, M, k)
            out_off[(name, M)] = (o_out, M, n)
            o_in += M * k
            o_out += M * n
    E2E_SETS = WEIGHT_COPIES // len(M_VALUES)
    pin_in = torch.empty(o_in, dtype=torch.bfloat16).pin_memory()
    for key, (o, M, k) in in_off.items():
        pin_in[o:o + M * k].copy_(host_x[key].reshape(-1))
    dev_in = [torch.empty(o_in, dtype=torch.bfloat16, device=device) for _ in range(E2E_SETS)]
    dev_out = [torch.empty(o_out, dtype=torch.bfloat16, device=device) for _ in range(E2E_SETS)]
    pin_out = torch.empty(o_out, dtype=torch.bfloat16).pin_memory()
    copy_in, copy_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    e2e_calls = [0]

    def step_e2e_launches():
        """The 16 launches of one step on buffer set (call number % E2E_SETS)."""
        b = e2e_calls[0] % E2E_SETS
        e2e_calls[0] += 1
        for M in M_VALUES:
            for name, n, k, style, copies in shards:
                o, _, _ = in_off[(name, M)]
                x = dev_in[b][o:o + M * k].view(M, k)
                oo, _, _ = out_off[(name, M)]
                out = dev_out[b][oo:oo + M * n].view(M, n)
                w, s, packed = copies[counters[name] % WEIGHT_COPIES]
                counters[name] += 1
                fused_reduce = peer if (world > 1 and style == "row") else None
                nvfp4r.linear_auto(x, gs, w, s, packed, n, 1.0, torch.bfloat16, out=out, reduce=fused_reduce)
                if world > 1 and style == "row" and peer is None:
                    dist.all_reduce(out)

    def timed_e2e(graphs, steps, warmup):
        """Time `steps` pipelined end-to-end steps; every step's two transfers are inside."""
        assert len(graphs) == E2E_SETS
        main = torch.cuda.current_stream()
        in_ready = [torch.cuda.Event() for _ in range(E2E_SETS)]
        computed = [torch.cuda.Event() for _ in range(E2E_SETS)]
        drained = [torch.cuda.Event() for _ in range(E2E_SETS)]
        for ev in computed + drained:
            ev.record(main)

        def run(n):
            for i in range(n):
                b = i % E2E_SETS
                copy_in.wait_event(computed[b])            # the step that last read this input buffer
                with torch.cuda.stream(copy_in):
                    dev_in[b].copy_(pin_in, non_blocking=True)
                    in_ready[b].record(copy_in)
                main.wait_event(in_ready[b])
                main.wait_event(drained[b])                # the step that last wrote this output buffer
                graphs[b].replay()
                computed[b].record(main)
                copy_out.wait_event(computed[b])
                with torch.cuda.stream(copy_out):
                    pin_out.copy_(dev_out[b], non_blocking=True)
                    drained[b].record(copy_out)
            for ev in drained:
                main.wait_event(ev)                        # the last results have reached the host

        run(max(warmup, E2E_SETS))
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run(steps)
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def capture_phases(fn):
        """One CUDA graph per phase of the weight-copy cycle: a step launches each
        linear 4 times, so WEIGHT_COPIES / 4 consecutive steps walk through all
        copies; replaying the phases in order repeats exactly the eager sequence."""
        phases = WEIGHT_COPIES // len(M_VALUES)
        graphs = []
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for name in counters:
                counters[name] = 0
            for _ in range(phases):
                fn()                                   # eager warm-up of every copy
            for name in counters:
                counters[name] = 0
            for _ in range(phases):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    fn()
                graphs.append(g)
        torch.cuda.current_stream().wait_stream(side)
        return graphs

    def timed(graphs, steps, warmup):
        for i in range(warmup):
            graphs[i % len(graphs)].replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            graphs[i % len(graphs)].replay()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    if args.case:
        # one (linear, M) pair launched eagerly, for profiler captures on a small case
        cname, cm = args.case.split(":")
        cm = int(cm)
        name, n, k, style, copies = next(sh for sh in shards if sh[0] == cname)
        for _ in range(args.warmup):
            one_linear(name, n, k, style, copies, cm, dev_x[(name, cm)])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            one_linear(name, n, k, style, copies, cm, dev_x[(name, cm)])
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / args.steps * 1e3
        return {"case": args.case, "us_eager": round(us, 2), "launches": args.steps,
                "algorithmic_bytes": linear_bytes(n, k, cm)}

    tp_check = None
    if world > 1:
        # Untimed correctness check of the real multi-GPU exchange: every row-parallel linear at
        # every M through the path the timed region uses, against the rank-ordered fp32 sum of
        # the ranks' own bf16 partial results (gathered with NCCL), rounded once to bf16.
        worst = 0.0
        for name, n, k, style, copies in shards:
            if style != "row":
                continue
            for M in M_VALUES:
                x = dev_x[(name, M)]
                w, s, packed = copies[0]
                got = nvfp4r.linear_auto(x, gs, w, s, packed, n, 1.0, torch.bfloat16,
                                         reduce=peer) if peer is not None else None
                part = nvfp4r.linear_auto(x, gs, w, s, packed, n, 1.0, torch.bfloat16).contiguous()
                if got is None:
                    got = part.clone()
                    dist.all_reduce(got)
                parts = [torch.empty_like(part) for _ in range(world)]
                dist.all_gather(parts, part)
                want32 = torch.zeros_like(part, dtype=torch.float32)
                for r in range(world):
                    want32 += parts[r].float()
                want = want32.to(torch.bfloat16)
                torch.cuda.synchronize()
                if peer is not None and not torch.equal(got, want):
                    worst = float("inf")           # the one-shot kernel promises exactly these bits
                err = (got.float() - want32).abs().max().item()
                scale = want32.abs().max().item() + 1e-30
                worst = max(worst, err / scale)    # NCCL may round per hop: one bf16 ulp of the largest value
        flag = torch.tensor([worst], dtype=torch.float64, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        tp_check = "ok" if float(flag.item()) <= 2.0 ** -7 else f"FAILED (max relative error {float(flag.item()):.3e})"
        stage(rank, f"tp_check {tp_check}")
        if tp_check != "ok":
            if rank == 0:
                _STDOUT.write(json.dumps({"tp_check": tp_check, "n_gpus": world}) + "\n")
                _STDOUT.flush()
            dist.barrier()
            os._exit(3)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    g_res = capture_phases(step_resident)
    stage(rank, "resident graphs captured")
    # keep the GPU busy long enough before the timed region for clock samples to exist; a FIXED
    # number of replays, the same on every rank (the graphs contain the all-reduces)
    for _ in range(800):
        for g in g_res:
            g.replay()
    torch.cuda.synchronize()
    ms_total = timed(g_res, args.steps, args.warmup)
    timed_launches = args.steps * 16
    stage(rank, "resident timed")
    g_e2e = capture_phases(step_e2e_launches)
    ms_e2e = timed_e2e(g_e2e, args.steps, max(3, args.warmup))
    clocks = sampler.stop() if sampler else None
    stage(rank, "e2e timed")

    # per-(linear, M) latency table: each pair alone, CUDA-graph replay of two passes over
    # its weight copies (so every launch still reads a cold weight)
    detail = {}
    if world == 1:
        side = torch.cuda.Stream(device=device)
        for name, n, k, style, copies in shards:
            for M in M_VALUES:
                reps = 2 * WEIGHT_COPIES
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    for _ in range(WEIGHT_COPIES):
                        one_linear(name, n, k, style, copies, M, dev_x[(name, M)])
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        for _ in range(reps):
                            one_linear(name, n, k, style, copies, M, dev_x[(name, M)])
                torch.cuda.current_stream().wait_stream(side)
                g.replay()
                torch.cuda.synchronize()
                ts = []
                for _ in range(5):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    g.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1) / reps * 1e3)
                us = sorted(ts)[2]
                detail[f"{name}_M{M}"] = {"us": round(us, 2), "kernel": path_used[(name, M)],
                                          "gbs": round(linear_bytes(n, k, M) / us / 1e3, 1)}

    # free the linear-set weights before the model benchmark
    h2d_bytes = sum(M * k * 2 for _, n, k, _, _ in shards for M in M_VALUES)
    d2h_bytes = sum(M * n * 2 for _, n, k, _, _ in shards for M in M_VALUES)
    del g_res, g_e2e, shards
    torch.cuda.empty_cache()
    target_detail = qwen3_32b_m1_detail(device, nvfp4r, measured_peak()[0]) if world == 1 else {}
    stage(rank, "Qwen3-32B M=1 shapes timed")
    decode = None if args.no_decode else run_decode(args, rank, world, device)
    stage(rank, "decode done")

    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    bytes_step = step_bytes()
    ms_step = ms_total / args.steps
    gbs = bytes_step / (ms_step * 1e-3) / 1e9
    gbs_e2e = bytes_step / (ms_e2e / args.steps * 1e-3) / 1e9
    for v in detail.values():
        v["pct_of_peak"] = round(100.0 * v["gbs"] / peak, 1)
    line = {
        "metric": "HBM GB/s over the Qwen3-8B NVFP4 W4A4 decode linear set, M=1..8, incl. activation quantization",
        "value": round(gbs, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 5), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "e2m1 x e2m1 with ue4m3 block scales, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": "Qwen3-8B decode linears qkv/o/gate_up/down x M{1,2,4,8}, fused quant+GEMV",
                   "kernel_choice": {f"{k[0]}_M{k[1]}": v for k, v in sorted(path_used.items())},
                   "launches_per_step": 16, "weight_copies": WEIGHT_COPIES,
                   "l2": "every launch reads a weight copy not touched for >1 GB of traffic (inputs larger than L2)",
                   "launch": "CUDA-graph replay, one graph per step",
                   "parallelism": f"tp{world}",
                   "allreduce": "none" if world == 1 else
                                (("push + sum inside the row-parallel linear's own launch over NVLink peer memory"
                                  if nv_config.fused_gather(world) else
                                  "push in the linear epilogue + one-shot gather kernel over NVLink peer memory")
                                 if peer is not None else "NCCL")},
        "e2e": {"value": round(gbs_e2e, 1), "unit": "GB/s",
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                "copies": "per step one transfer from and one to pinned host memory, on two copy streams; steps "
                          "pipelined over three device buffer sets (the launches stay in stream order)"},
        "gpu_launches": timed_launches,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(gbs / world, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(gbs / world / peak, 4), "peak_kind": f"of {peak_kind}",
                     "kernel": f"linear_packed_kernel ({sum(v == 'tcgen05' for v in path_used.values())} launches) / "
                               f"CUDA-core GEMV ({sum(v == 'gemv' for v in path_used.values())}) by measured crossover "
                               "(16 launches per step)",
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None},
        "detail_us_gbs": {**detail, **target_detail},
        "decode": decode,
    }
    if tp_check is not None:
        line["tp_check"] = tp_check
    if world == 1:
        line["cpu_baseline"] = cpu_baseline(sample_repeats=4)
    return line


def run_decode(args, rank, world, device):
    """Qwen3-32B batch-1 decode step: random-init NVFP4 weights, bf16 KV
    cache at context 2048, one CUDA graph per token, tensor-parallel over `world` ranks with
    an NCCL all-reduce after o_proj and down_proj."""
    import torch.distributed as dist

    import dataclasses

    from reset_b200.decode import QWEN3_32B, DecodeStep

    cfg = QWEN3_32B
    if args.decode_layers:                     # fewer layers of the same geometry: profiler captures
        cfg = dataclasses.replace(cfg, layers=args.decode_layers, name=f"{cfg.name} ({args.decode_layers} layers)")
    shard_of = args.decode_shard_of
    if shard_of > 1 and world == 1:
        # rank 0's shard of a `shard_of`-way tensor-parallel model on this one GPU, exchanges
        # left out: what the launches of one rank cost before any communication
        model = DecodeStep(cfg, device, rank=0, world=shard_of, seed=11, skip_exchange=True)
    else:
        model = DecodeStep(cfg, device, rank=rank, world=world, seed=11, peer_allreduce=(args.allreduce == "peer"),
                           fused_gather=not args.no_fused_gather)
    if args.decode_eager:
        for _ in range(args.decode_steps):
            model.step()
        torch.cuda.synchronize()
        del model
        return {"model": cfg.name, "mode": "eager (profiling)", "steps": args.decode_steps}
    model.capture()
    for _ in range(3):
        model.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    steps = args.decode_steps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        model.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_tok = float(ms.item()) / steps
    peak, kind = measured_peak()
    bytes_rank = model.bytes_per_step()
    out = {"model": cfg.name, "batch": 1, "context": cfg.context, "tp": world,
           "tok_s": round(1e3 / ms_tok, 1), "ms_per_token": round(ms_tok, 4), "steps": steps,
           "hbm_bytes_per_token_per_gpu": bytes_rank,
           "roofline_tok_s": round(peak * 1e9 / bytes_rank, 1),
           "frac_of_hbm_roofline": round((bytes_rank / (ms_tok * 1e-3) / 1e9) / peak, 4),
           "launch": "one CUDA graph per token", "kernels_per_token": model.kernels_per_step(),
           "allreduce": "none" if world == 1 else ("peer one-shot" if model.peer is not None else "NCCL")}
    if world == 1:
        # the same token with the ReSET processor and a draw from the scaled logits inside the
        # graph instead of the arg-max (the reference's deployment: processor + vLLM sampler;
        # its README puts the processor at ~1.5 % of a decode step)
        model.enable_reset(t_high=1.0, t_low=0.1, tau0=0.5505, window=32, dnl_ids=[198], seed=1)
        model.capture()
        for _ in range(3):
            model.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            model.replay()
        e1.record()
        torch.cuda.synchronize()
        ms_reset = e0.elapsed_time(e1) / steps
        out["with_reset_processor"] = {"tok_s": round(1e3 / ms_reset, 1), "ms_per_token": round(ms_reset, 4),
                                       "added_us_per_token": round((ms_reset - ms_tok) * 1e3, 1),
                                       "added_pct": round(100.0 * (ms_reset - ms_tok) / ms_tok, 2),
                                       "kernels_per_token": model.kernels_per_step()}
    del model
    torch.cuda.empty_cache()
    return out



# ------------------------------------------------------- secondary measurements

def _graph_us(fn, reps: int, device, samples: int = 7) -> float:
    """Median microseconds per call of `fn`, `reps` calls per CUDA-graph replay."""
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(reps):
            fn()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for _ in range(reps):
                fn()
    torch.cuda.current_stream().wait_stream(side)
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(samples):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / reps * 1e3)
    return sorted(ts)[len(ts) // 2]


SWEEP_SHAPES = {   # name, N, K, tensor-parallel style
    "qwen3-14b": [("qkv_proj", 7168, 5120, "column"), ("o_proj", 5120, 5120, "row"),
                  ("gate_up_proj", 34816, 5120, "column"), ("down_proj", 5120, 17408, "row")],
    "qwen3-8b": list(LINEARS),
    "qwen3-32b": [("qkv_proj", 10240, 5120, "column"), ("o_proj", 5120, 8192, "row"),
                  ("gate_up_proj", 51200, 5120, "column"), ("down_proj", 5120, 25600, "row")],
}


def _jsonl_done(path: str) -> dict:
    """Rows already in a sweep's JSONL file, keyed (sweep, tp, shape, M): an interrupted sweep
    resumes where it stopped (the reference's benches do the same,
    kernels/benchmarks/bench_e2e.py:119-134)."""
    done = {}
    if path and os.path.exists(path):
        for ln in Path(path).read_text().splitlines():
            try:
                r = json.loads(ln)
                done[(r["sweep"], r["tp"], r["shape"], r["M"])] = r
            except (ValueError, KeyError):
                continue
    return done


def run_sweep(args):
    """M sweep 1..16 over one model's four linear shapes: the fused
    quantize + CUDA-core GEMV, the fused quantize + tcgen05 packed linear, and, when the
    installed vLLM's operators load, its `scaled_fp4_quant` + `cutlass_scaled_fp4_mm` pair.
    Every launch reads a weight copy that has left L2 (copies total > 1 GB). ``--sweep-tp T``
    times one rank's shard of every shape under T-way tensor parallelism (column-parallel: N / T,
    row-parallel: K / T) on this one GPU; ``--jsonl PATH`` appends one line per (shape, M) and
    skips the pairs the file already holds."""
    from reset_b200 import capi, nvfp4r

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    try:
        import vllm._custom_ops as vops
    except Exception:
        vops = None
    peak, _ = measured_peak()
    gen = torch.Generator(device=device).manual_seed(3)
    gs = torch.tensor([100.0], dtype=torch.float32, device=device)
    alpha_t = torch.tensor([1.0], dtype=torch.float32, device=device)
    Ms = [int(m) for m in args.sweep_m.split(",")]
    tp = max(1, args.sweep_tp)
    done = _jsonl_done(args.jsonl)
    out = {"sweep": args.sweep, "tp": tp, "unit": "us per linear incl. activation quantization", "peak_gbs": peak,
           "l2": "weight copies cycled, > 1 GB between reuses", "shapes": {}}
    for name, N, K, style in SWEEP_SHAPES[args.sweep]:
        N, K = (N // tp, K) if style == "column" else (N, K // tp)
        shape_key = f"{name} ({N}x{K})"
        if all((args.sweep, tp, shape_key, M) in done for M in Ms):
            out["shapes"][shape_key] = {str(M): done[(args.sweep, tp, shape_key, M)]["row"] for M in Ms}
            continue
        copies = min(64, int(1.1e9 // (N * K * 9 // 16)) + 1)
        packable = N % 128 == 0 and K % 128 == 0
        ws = []
        for _ in range(copies):
            w = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=device, generator=gen)
            s = torch.randint(1, 0x38, (N, K // 16), dtype=torch.uint8, device=device, generator=gen)
            ws.append((w, s, capi.pack_weight(w, s) if packable else None,
                       capi.swizzle_blockscale(s) if vops else None))
        wksp = capi.packed_workspace(16, N, K, device)
        rows = {}
        for M in Ms:
            if (args.sweep, tp, shape_key, M) in done:
                rows[str(M)] = done[(args.sweep, tp, shape_key, M)]["row"]
                continue
            x = torch.randn(M, K, device=device, generator=gen).to(torch.bfloat16)
            o = torch.empty(M, N, dtype=torch.bfloat16, device=device)
            st = {"i": 0}

            def nxt():
                st["i"] += 1
                return ws[st["i"] % copies]

            def f_gemv():
                w, s, _, _ = nxt()
                capi.linear(x, gs, w, s, 1.0, out=o, rcp_mode=1)

            def f_tc():
                _, _, p, _ = nxt()
                capi.linear_packed(x, gs, p, N, 1.0, wksp, rcp_mode=1, out=o)

            def f_vllm():
                w, _, _, ssw = nxt()
                c, sf = vops.scaled_fp4_quant(x, gs)
                vops.cutlass_scaled_fp4_mm(c, w, sf, ssw.view(torch.float8_e4m3fn), alpha_t, torch.bfloat16)

            r = {}
            if M <= 16:
                r["gemv_us"] = round(_graph_us(f_gemv, 2 * copies, device), 2)
            if packable:
                r["tcgen05_us"] = round(_graph_us(f_tc, 2 * copies, device), 2)
            if vops is not None and K % 32 == 0:
                try:
                    r["vllm_cutlass_us"] = round(_graph_us(f_vllm, 2 * copies, device), 2)
                except Exception as e:  # library kernel unavailable for this shape/build
                    r["vllm_cutlass_error"] = str(e).splitlines()[0][:160]
                    torch.cuda.synchronize()
            best = min(v for k, v in r.items() if k in ("gemv_us", "tcgen05_us"))
            r["best_pct_of_peak"] = round(100.0 * linear_bytes(N, K, M) / best / 1e3 / peak, 1)
            r["chosen"] = "gemv" if (not packable or nvfp4r.ops.use_gemv(M, N, K, nvfp4r.status()["gemv_max_m"])) else "tcgen05"
            rows[str(M)] = r
            if args.jsonl:
                with open(args.jsonl, "a") as fh:
                    fh.write(json.dumps({"sweep": args.sweep, "tp": tp, "shape": shape_key, "M": M, "row": r}) + "\n")
        out["shapes"][shape_key] = rows
        del ws
        torch.cuda.empty_cache()
    return out


# The reference's published M=1 kernel latencies on one B200 (docs/index.html:213-224 of the
# reference: model, layer, N, K, microseconds of its nvfp4r GEMV and of vLLM's CUTLASS path).
PUBLISHED_M1 = [
    ("Qwen3-8B", "qkv_proj", 6144, 4096, 4.28, 8.69), ("Qwen3-8B", "o_proj", 4096, 4096, 3.75, 7.69),
    ("Qwen3-8B", "gate/up_proj", 12288, 4096, 6.40, 11.45), ("Qwen3-8B", "down_proj", 4096, 12288, 6.66, 16.61),
    ("Qwen3-14B", "qkv_proj", 7168, 5120, 5.53, 10.79), ("Qwen3-14B", "o_proj", 5120, 5120, 4.64, 9.08),
    ("Qwen3-14B", "gate/up_proj", 17408, 5120, 9.49, 14.93), ("Qwen3-14B", "down_proj", 5120, 17408, 10.35, 23.77),
    ("Qwen3-32B", "qkv_proj", 10240, 5120, 6.62, 13.41), ("Qwen3-32B", "o_proj", 5120, 8192, 7.73, 12.40),
    ("Qwen3-32B", "gate/up_proj", 25600, 5120, 13.25, 25.89), ("Qwen3-32B", "down_proj", 5120, 25600, 15.00, 33.26),
]


def _eager_us(fn, warmup: int = 10, iters: int = 100) -> float:
    """The reference's timing method (kernels/benchmarks/common.py:20-57): eager calls, one
    pair of CUDA events around every call, median of `iters` after `warmup`; host launch
    overhead is inside the number whenever the host is slower than the GPU."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for s, e in ev:
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    return sorted(s.elapsed_time(e) for s, e in ev)[iters // 2] * 1e3


def run_published(args):
    """The twelve shapes of the reference's published M=1 table, measured the way the reference
    measured them: the SAME buffers every iteration (every one of these weights fits in L2, so
    the numbers are L2-resident, not HBM, figures), eager launches timed by per-call CUDA events,
    and, beside that, CUDA-graph replay (pure GPU time). Three legs per shape:
      gemv_prequant  the raw out-variant op on already quantized activations (what the published
                     nvfp4r column timed, kernels/benchmarks/bench_nvfp4_gemv.py:104-121)
      linear_fused   quantizer + product in one launch through the measured crossover (the path
                     the adapter runs; the published column leaves the quantizer out)
      cold           the same fused launch with weight copies cycled (> 1 GB between reuses)"""
    from reset_b200 import capi, nvfp4r

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    gen = torch.Generator(device=device).manual_seed(5)
    gs = torch.tensor([100.0], dtype=torch.float32, device=device)
    rows = []
    for model, layer, N, K, pub_us, pub_vllm_us in PUBLISHED_M1:
        copies = int(1.1e9 // (N * K * 9 // 16)) + 1
        ws = []
        for _ in range(copies):
            w = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=device, generator=gen)
            sc = torch.randint(1, 0x38, (N, K // 16), dtype=torch.uint8, device=device, generator=gen)
            ws.append((w, sc, capi.pack_weight(w, sc)))
        x = torch.randn(1, K, device=device, generator=gen).to(torch.bfloat16)
        codes, xsf = capi.quant(x, gs, rcp_mode=1)
        o = torch.empty(1, N, dtype=torch.bfloat16, device=device)
        o16 = torch.empty(1, N, dtype=torch.float16, device=device)
        w0, s0, p0 = ws[0]
        w3, s3, x3, xs3 = w0.unsqueeze(0), s0.unsqueeze(0), codes.unsqueeze(0), xsf.view(torch.uint8).unsqueeze(0)
        st = {"i": 0}

        def f_raw():
            capi.gemv_out(w3, s3, x3, xs3, o16, 1.0)

        def f_fused():
            nvfp4r.ops.linear_auto(x, gs, w0, s0, p0, N, 1.0, out=o)

        def f_cold():
            st["i"] += 1
            w, sc, pk = ws[st["i"] % copies]
            nvfp4r.ops.linear_auto(x, gs, w, sc, pk, N, 1.0, out=o)

        r = {"model": model, "layer": layer, "N": N, "K": K, "published_nvfp4r_us": pub_us,
             "published_vllm_cutlass_us": pub_vllm_us,
             "gemv_prequant_eager_us": round(_eager_us(f_raw), 2),
             "gemv_prequant_graph_us": round(_graph_us(f_raw, 20, device), 2),
             "linear_fused_eager_us": round(_eager_us(f_fused), 2),
             "linear_fused_graph_us": round(_graph_us(f_fused, 20, device), 2),
             "linear_fused_cold_graph_us": round(_graph_us(f_cold, 2 * copies, device), 2),
             "fused_kernel": "gemv" if nvfp4r.ops.use_gemv(1, N, K, nvfp4r.status()["gemv_max_m"]) else "tcgen05"}
        best = min(r["gemv_prequant_graph_us"], r["linear_fused_graph_us"])
        r["published_over_best_graph"] = round(pub_us / best, 2)
        rows.append(r)
        del ws
        torch.cuda.empty_cache()
    return {"published_method": rows, "unit": "us per M=1 linear",
            "note": "same buffers every iteration = L2-resident, as the reference measured; 'cold' cycles weight copies"}


def run_reset_loop(args):
    """ReSET decode loop: vocab 151936, batch 1..8, a delimiter every 40-120
    tokens, t_high 1.0 / t_low 0.1 / tau_0 0.5505 / w 32. GPU: one fused step per token for the
    whole batch (ONE launch), CUDA-graph replay over a pool of distinct logits buffers larger
    than L2, restored before every replay because the step divides in place. With these logits
    every step chooses T = t_high = 1 and nothing is written back (x / 1 = x), so the loop is timed
    a second time with tau_0 = 100, where every step chooses t_low and the scaled row is written
    (`gpu_us_t_low`). CPU: the oracle's per-request processor (the reference's algorithm) on the
    host cores, same logits; the temperatures the device chose on those steps are compared with
    the oracle's (`temps_equal`)."""
    import ctypes as C

    import numpy as np

    from oracle import reset_policy as orp
    from reset_b200 import _lib, capi

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    V, steps = 151936, args.reset_steps
    out = {"reset_loop": {"vocab": V, "steps": steps, "unit": "us per decode step (whole batch)"}}
    delim = V - 5
    for B in (1, 2, 4, 8):
        pool_n = max(8, int(300e6 // (B * V * 4)))
        pristine = torch.randn(pool_n, B, V, device=device, generator=torch.Generator(device=device).manual_seed(B)) * 3.0
        pristine[:, :, 17] += 12.0
        pool = pristine.clone()
        states = torch.zeros(B * C.sizeof(_lib.ResetState), dtype=torch.uint8, device=device)
        ws = capi.reset_workspace(B, device)
        bm = torch.zeros((V + 31) // 32, dtype=torch.int32, device=device)
        bm[delim // 32] = 1 << (delim % 32)
        nl = torch.zeros_like(bm)
        streams = np.stack([orp.synthetic_token_stream(pool_n + 2, delim, V, 7 + b) for b in range(B)])
        last = [torch.from_numpy(np.ascontiguousarray(streams[:, t:t + 2]).astype(np.int32)).to(device)
                for t in range(pool_n)]

        decisions = torch.zeros(pool_n * B * C.sizeof(_lib.ResetDecision), dtype=torch.uint8, device=device)
        dec_rows = decisions.view(pool_n, B * C.sizeof(_lib.ResetDecision))
        timed = {}
        for label, tau0 in (("t_high", 0.5505), ("t_low", 100.0)):
            params = _lib.ResetParams(1.0, 0.1, tau0, 32, 0)
            states.zero_()
            pool.copy_(pristine)

            def one_pass():
                for t in range(pool_n):
                    capi.reset_step(pool[t], states, params, last_ids=last[t], nl_bitmap=nl, dnl_bitmap=bm,
                                    decisions=dec_rows[t], workspace=ws)

            side = torch.cuda.Stream(device=device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                one_pass()
                pool.copy_(pristine)
                states.zero_()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    one_pass()
            torch.cuda.current_stream().wait_stream(side)
            ts = []
            for _ in range(max(3, steps // pool_n)):
                pool.copy_(pristine)
                states.zero_()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) / pool_n * 1e3)
            timed[label] = sorted(ts)[len(ts) // 2]
            if label == "t_high":
                dec_t_high = np.frombuffer(decisions.cpu().numpy().tobytes(), dtype="f8").reshape(pool_n, B, -1)[:, :, 3].copy()
            del g
        gpu_us = timed["t_high"]
        # CPU: the per-request processor, one call per row per step
        host = pristine[: min(pool_n, 24)].cpu()
        pols = [orp.ResetPolicy(1.0, 0.1, 0.5505, 32, frozenset(), frozenset([delim])) for _ in range(B)]
        temps_equal = True
        t0 = time.perf_counter()
        for t in range(host.shape[0]):
            for b in range(B):
                _, d = pols[b](streams[b][: t + 2].tolist(), host[t, b])
                temps_equal = temps_equal and d.temp == dec_t_high[t, b]
        cpu_us = (time.perf_counter() - t0) / host.shape[0] * 1e6
        out["reset_loop"][f"B{B}"] = {"gpu_us": round(gpu_us, 2), "gpu_us_t_low": round(timed["t_low"], 2),
                                      "cpu_oracle_us": round(cpu_us, 1),
                                      "speedup": round(cpu_us / gpu_us, 1),
                                      "gbs_read_only": round(B * V * 4 / gpu_us / 1e3, 1),
                                      "gbs_t_low_read_write": round(2 * B * V * 4 / timed["t_low"] / 1e3, 1),
                                      "temps_equal_to_oracle": bool(temps_equal),
                                      "logits_pool_mb": round(pool_n * B * V * 4 / 1e6)}
        del pool, pristine
        torch.cuda.empty_cache()
    out["reset_loop"]["cpu_threads"] = torch.get_num_threads()
    return out

# ---------------------------------------------------------------------- reference / CPU

def _cpu_step(weights, xs, gs_inv):
    """One STEP of the workload on the host: the four linears at M = 1, 2, 4, 8 (16 pairs), each
    with the activation quantizer, through the torch-CPU port of the reference's
    dequantise-then-matmul (the weight is dequantised again for every pair, as the reference's
    path does per call)."""
    from oracle import torch_port as otp
    for M in M_VALUES:
        for (w, s), x in zip(weights, xs):
            xc, xsf = otp.quantize_torch(x[:M], gs_inv)
            otp.linear_torch(w, s, xc, xsf, 1.0)


def _cpu_setup():
    g = torch.Generator().manual_seed(99)
    weights, xs = [], []
    for name, N, K, _ in LINEARS:
        weights.append((torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g),
                        torch.randint(1, 0x38, (N, K // 16), dtype=torch.uint8, generator=g)))
        xs.append(torch.randn(max(M_VALUES), K, generator=g).to(torch.bfloat16))
    return weights, xs, step_bytes()


def cpu_baseline(sample_repeats: int) -> dict:
    torch.set_num_threads(os.cpu_count() or 1)
    weights, xs, nbytes = _cpu_setup()
    _cpu_step(weights, xs, 100.0)
    ts = []
    for _ in range(sample_repeats):
        t0 = time.perf_counter()
        _cpu_step(weights, xs, 100.0)
        ts.append(time.perf_counter() - t0)
    t = sorted(ts)[len(ts) // 2]
    return {"value": round(nbytes / t / 1e9, 3), "unit": "GB/s", "cores": torch.get_num_threads(),
            "kind": "port",
            "sample": f"{sample_repeats + 1} whole steps (the same 16 (linear, M) pairs as the GPU step) on the host "
                      f"cores, median {t * 1e3:.0f} ms per step"}


def run_reference(args, rank, world):
    """The reference's CPU implementation of the path (PyTorch gather-dequantise +
    fp32 matmul, kernels/tests/conftest.py:23-55) timed on the host cores through its
    port in oracle/torch_port.py; the Python reference itself is not present on the
    GPU box. A step is the SAME step as the GPU arm's: the four Qwen3-8B linears at
    M = 1, 2, 4, 8 with the activation quantizer (about a second of host time)."""
    if rank != 0:
        return None
    torch.set_num_threads(os.cpu_count() or 1)
    weights, xs, nbytes = _cpu_setup()
    for _ in range(args.warmup):
        _cpu_step(weights, xs, 100.0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        _cpu_step(weights, xs, 100.0)
    t = (time.perf_counter() - t0) / args.steps
    gbs = nbytes / t / 1e9
    sample = "each step = the whole workload step: 16 (linear, M) pairs incl. activation quantization"
    return {
        "impl": "reference",
        "metric": "HBM GB/s over the Qwen3-8B NVFP4 W4A4 decode linear set, M=1..8, incl. activation quantization",
        "value": round(gbs, 3), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(t * 1e3, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 dequantise + f32 matmul on CPU", "data": "synthetic",
        "config": {"workload": "Qwen3-8B decode linears qkv/o/gate_up/down x M{1,2,4,8}, fused quant+GEMV",
                   "launches_per_step": 16, "sample": sample, "parallelism": "host cores"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=600)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-decode", action="store_true", help="skip the Qwen3-32B decode-step measurement")
    ap.add_argument("--decode-steps", type=int, default=30)
    ap.add_argument("--decode-only", action="store_true", help="only the decode-step measurement")
    ap.add_argument("--decode-layers", type=int, default=0, help="override the layer count (profiling)")
    ap.add_argument("--decode-eager", action="store_true", help="run the decode steps eagerly (profiling)")
    ap.add_argument("--case", default="", help="profile one pair, e.g. gate_up_proj:1 (eager launches)")
    ap.add_argument("--sweep", default="", choices=["", *SWEEP_SHAPES],
                    help="M sweep over one model's linear shapes: GEMV vs tcgen05 vs the installed vLLM pair")
    ap.add_argument("--sweep-m", default="1,2,3,4,6,8,12,16")
    ap.add_argument("--sweep-tp", type=int, default=1, help="time one rank's shard shapes under this tensor parallelism")
    ap.add_argument("--jsonl", default="", help="append sweep rows to this file and skip the ones it already holds")
    ap.add_argument("--published", action="store_true",
                    help="the reference's published M=1 shapes under its own timing method (L2-resident)")
    ap.add_argument("--reset-loop", action="store_true", help="ReSET decode-loop step time vs the CPU oracle")
    ap.add_argument("--reset-steps", type=int, default=256)
    ap.add_argument("--allreduce", default="peer", choices=["peer", "nccl"],
                    help="sum exchange after row-parallel linears at N > 1: this library's one-shot kernel or NCCL")
    ap.add_argument("--packed-tuning", type=int, default=0,
                    help="value for nvfp4r_set_packed_tuning (experiments: 512 = one CTA per SM)")
    ap.add_argument("--decode-shard-of", type=int, default=0,
                    help="single GPU: time rank 0's shard of this tensor-parallel degree without the exchanges")
    ap.add_argument("--no-fused-gather", action="store_true",
                    help="tensor-parallel runs: gather in a second launch instead of inside the linear's own")
    ap.add_argument("--watchdog", type=int, default=1200,
                    help="seconds after which every rank dumps its Python stacks to stderr and exits")
    args = ap.parse_args()
    if args.watchdog > 0:
        import faulthandler
        faulthandler.dump_traceback_later(args.watchdog, exit=True)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        line = run_reference(args, rank, world)
    elif args.sweep or args.reset_loop or args.published:
        if world > 1:
            raise SystemExit("bench.py: --sweep / --reset-loop / --published are single-GPU measurements")
        line = run_sweep(args) if args.sweep else (run_published(args) if args.published else run_reset_loop(args))
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device (there is no CPU fallback for the product path)")
        line = run_ours(args, rank, world, local_rank)
    if args.impl == "ours" and torch.cuda.is_available():
        from reset_b200 import _lib
        _lib.check(_lib.lib().nvfp4r_check_device_status(), "a bounded device-side wait expired during the run")
    if line is not None:
        _STDOUT.write(json.dumps(line) + "\n")
        _STDOUT.flush()
    if world > 1 and args.impl == "ours":
        # Leave without tearing the communicator down: NCCL's destroy waits for every CUDA
        # graph that captured a collective, and graph objects die in interpreter-defined
        # order. All ranks meet once more, then exit.
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
