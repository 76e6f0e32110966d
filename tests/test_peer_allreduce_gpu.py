"""One-shot peer-memory all-reduce (`nvfp4r_peer_allreduce_bf16`).

On one GPU the ranks are emulated without any kernel waiting for another: every rank's PUSH
half runs first, then every rank's GATHER half (all data is in place when a gather starts).
With two or more GPUs the real thing runs as one process per GPU (spawned children), checked
against the rank-ordered fp32 sum and against NCCL."""

import ctypes as C
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parents[1]


def _expected(parts):
    acc = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:                                   # rank order, fp32, one rounding
        acc += p.float()
    return acc.to(torch.bfloat16)


@pytest.mark.parametrize("world", [2, 3, 8])
def test_emulated_ranks_on_one_gpu(world):
    from reset_b200 import _lib as L
    lib = L.lib()
    max_elems = 5120 * 2
    nbytes = lib.nvfp4r_peer_buffer_bytes(world, max_elems)
    assert nbytes == 256 + 2 * world * (max_elems // 2) * 8
    ptrs = []
    for _ in range(world):
        p, h = C.c_void_p(), C.create_string_buffer(64)
        L.check(lib.nvfp4r_peer_alloc(nbytes, C.byref(p), h), "alloc")
        ptrs.append(p)
    try:
        comms = []
        for r in range(world):
            c = L.PeerComm()
            c.world, c.rank, c.max_elems = world, r, max_elems
            for k in range(world):
                c.base[k] = ptrs[k].value
            comms.append(c)
        g = torch.Generator(device="cuda").manual_seed(world)
        stream = torch.cuda.current_stream().cuda_stream
        for call, count in enumerate([5120, 2, max_elems, 5120, 4096]):        # parity flips every call
            parts = [torch.randn(count, device="cuda", generator=g).to(torch.bfloat16) for _ in range(world)]
            outs = [torch.empty_like(p) for p in parts]
            for r in range(world):
                L.check(lib.nvfp4r_peer_allreduce_bf16(C.byref(comms[r]), parts[r].data_ptr(), outs[r].data_ptr(),
                                                       count, L.PEER_PUSH, stream), "push")
            for r in range(world):
                L.check(lib.nvfp4r_peer_allreduce_bf16(C.byref(comms[r]), parts[r].data_ptr(), outs[r].data_ptr(),
                                                       count, L.PEER_GATHER, stream), "gather")
            torch.cuda.synchronize()
            want = _expected(parts)
            for r in range(world):
                assert torch.equal(outs[r], want), (call, r)
        L.check(lib.nvfp4r_check_device_status(), "device status")
        # argument checks
        x = torch.zeros(6, dtype=torch.bfloat16, device="cuda")
        assert lib.nvfp4r_peer_allreduce_bf16(C.byref(comms[0]), x.data_ptr(), x.data_ptr(), 5, 3, stream) != 0
        assert lib.nvfp4r_peer_allreduce_bf16(C.byref(comms[0]), x.data_ptr(), x.data_ptr(), max_elems + 2, 3, stream) != 0
        assert lib.nvfp4r_peer_allreduce_bf16(C.byref(comms[0]), x.data_ptr(), x.data_ptr(), 6, 0, stream) != 0
    finally:
        torch.cuda.synchronize()
        for p in ptrs:
            lib.nvfp4r_peer_free(p)


_CHILD = r"""
import os, sys
sys.path.insert(0, os.environ["REPO"])
import torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dev = torch.device("cuda", rank); torch.cuda.set_device(dev)
dist.init_process_group("nccl", device_id=dev)
from reset_b200.comm import PeerAllReduce
from reset_b200 import _lib as L
ar = PeerAllReduce(dev, 8 * 5120)
ok = True
for call, count in enumerate([5120, 2, 8 * 5120, 5120, 10240, 5120]):
    parts = [torch.randn(count, device=dev, generator=torch.Generator(device=dev).manual_seed(100 * call + r)).to(torch.bfloat16)
             for r in range(world)]
    acc = torch.zeros(count, device=dev)
    for p in parts: acc += p.float()
    want = acc.to(torch.bfloat16)
    mine = parts[rank].clone()
    ar.all_reduce_(mine)
    nccl = parts[rank].clone(); dist.all_reduce(nccl)
    torch.cuda.synchronize()
    ok = ok and torch.equal(mine, want) and torch.allclose(mine.float(), nccl.float(), rtol=1e-2, atol=1e-2)
# graph capture and replay (the call counter advances on the device)
x = torch.ones(5120, device=dev, dtype=torch.bfloat16) * (rank + 1)
buf = x.clone()
s = torch.cuda.Stream(); s.wait_stream(torch.cuda.current_stream())
with torch.cuda.stream(s):
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        buf.copy_(x); ar.all_reduce_(buf)
        buf.copy_(x); ar.all_reduce_(buf); ar.all_reduce_(buf)
torch.cuda.current_stream().wait_stream(s)
for _ in range(5): g.replay()
torch.cuda.synchronize()
tot = world * (world + 1) // 2
ok = ok and bool((buf.float() == tot * world).all())
L.check(L.lib().nvfp4r_check_device_status(), "status")
flag = torch.tensor([1 if ok else 0], device=dev); dist.all_reduce(flag, op=dist.ReduceOp.MIN)
dist.barrier(); torch.cuda.synchronize()
print("PEER_OK" if int(flag.item()) == 1 else "PEER_MISMATCH", flush=True)
os._exit(0 if int(flag.item()) == 1 else 1)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_two_gpus(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    env = dict(os.environ, REPO=str(REPO), NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.count("PEER_OK") == 2, (r.stdout[-2000:], r.stderr[-3000:])


_CHILD_FUSED = r"""
import os, sys
sys.path.insert(0, os.environ["REPO"])
import torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dev = torch.device("cuda", rank); torch.cuda.set_device(dev)
dist.init_process_group("nccl", device_id=dev)
from reset_b200.comm import PeerAllReduce
from reset_b200 import _lib as L, capi
from reset_b200 import nvfp4r
ar = PeerAllReduce(dev, 8 * 5120)
ok = True
gs = torch.tensor([60.0], device=dev)
gen = torch.Generator(device=dev).manual_seed(7 + rank)
# row-parallel shards of o_proj / down_proj at TP 2: every rank holds its own K slice
for N, K, M in [(5120, 4096, 1), (5120, 12800, 1), (5120, 4096, 8), (4096, 2048, 3), (5120, 12800, 2)]:
    w = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=gen)
    s = torch.randint(1, 0x38, (N, K // 16), dtype=torch.uint8, device=dev, generator=gen)
    packed = capi.pack_weight(w, s)
    x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
    wk = capi.packed_workspace(M, N, K, dev)
    part = capi.linear_packed(x, gs, packed, N, 0.01, wk, rcp_mode=1)            # this rank's bf16 partial
    parts = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    acc = torch.zeros_like(part, dtype=torch.float32)
    for p in parts: acc += p.float()
    want = acc.to(torch.bfloat16)
    for rep in range(3):                                                         # both halves of the double buffer
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        capi.linear_packed_push(x, gs, packed, N, 0.01, wk, ar.comm, out, rcp_mode=1, gather=True)
        torch.cuda.synchronize()
        ok = ok and torch.equal(out, want)
    ok = ok and int(wk.count_nonzero().item()) == 0
    # interleaved with the two-launch form and the stand-alone all-reduce: one call counter serves all
    out2 = torch.empty_like(out)
    capi.linear_packed_push(x, gs, packed, N, 0.01, wk, ar.comm, out2, rcp_mode=1)
    ar.gather_(out2)
    mine = part.clone(); ar.all_reduce_(mine)
    torch.cuda.synchronize()
    ok = ok and torch.equal(out2, want) and torch.equal(mine, want)
# shards small enough for the CUDA-core GEMV: push and sum inside the GEMV's own launch
for N, K in [(4096, 2048), (5120, 1024), (5120, 2048), (1536, 4096)]:
    w = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=gen)
    s = torch.randint(1, 0x38, (N, K // 16), dtype=torch.uint8, device=dev, generator=gen)
    x = torch.randn(1, K, device=dev, generator=gen).to(torch.bfloat16)
    part = capi.linear(x, gs, w, s, 0.01, rcp_mode=1)
    parts = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    acc = torch.zeros_like(part, dtype=torch.float32)
    for p in parts: acc += p.float()
    want = acc.to(torch.bfloat16)
    for rep in range(3):
        out = torch.full((1, N), float("nan"), dtype=torch.bfloat16, device=dev)
        capi.linear_push(x, gs, w, s, 0.01, ar.comm, out, rcp_mode=1)
        torch.cuda.synchronize()
        ok = ok and torch.equal(out, want)
    mine = part.clone(); ar.all_reduce_(mine)                                     # the same call counter serves both
    torch.cuda.synchronize()
    ok = ok and torch.equal(mine, want)
    if N == 4096:                                                                # the crossover sends this one to the GEMV
        packed = capi.pack_weight(w, s)
        out = torch.zeros((1, N), dtype=torch.bfloat16, device=dev)
        nvfp4r.linear_auto(x, gs, w, s, packed, N, 0.01, out=out, reduce=ar)
        side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(3):
                    nvfp4r.linear_auto(x, gs, w, s, packed, N, 0.01, out=out, reduce=ar)
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            out.zero_(); g.replay(); torch.cuda.synchronize()
            ok = ok and torch.equal(out, want)
# through the public call, captured and replayed
N, K, M = 5120, 4096, 1
w = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=gen)
s = torch.randint(1, 0x38, (N, K // 16), dtype=torch.uint8, device=dev, generator=gen)
packed = capi.pack_weight(w, s)
x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
part = nvfp4r.linear_auto(x, gs, None, None, packed, N, 0.01)
parts = [torch.empty_like(part) for _ in range(world)]
dist.all_gather(parts, part)
want = sum(p.float() for p in parts).to(torch.bfloat16)
out = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
nvfp4r.linear_auto(x, gs, None, None, packed, N, 0.01, out=out, reduce=ar)
side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
with torch.cuda.stream(side):
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for _ in range(3):
            nvfp4r.linear_auto(x, gs, None, None, packed, N, 0.01, out=out, reduce=ar)
torch.cuda.current_stream().wait_stream(side)
for _ in range(4):
    out.zero_(); g.replay(); torch.cuda.synchronize()
    ok = ok and torch.equal(out, want)
L.check(L.lib().nvfp4r_check_device_status(), "status")
flag = torch.tensor([1 if ok else 0], device=dev); dist.all_reduce(flag, op=dist.ReduceOp.MIN)
dist.barrier(); torch.cuda.synchronize()
print("FUSED_OK" if int(flag.item()) == 1 else "FUSED_MISMATCH", flush=True)
os._exit(0 if int(flag.item()) == 1 else 1)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_linear_completes_the_all_reduce_in_its_own_launch_two_gpus(tmp_path):
    """Row-parallel linear with push AND sum in one launch (``push_gather``) on two GPUs: equal,
    bit for bit, to the rank-ordered fp32 sum of the ranks' bf16 partial results, for both halves
    of the double-buffered receive memory, mixed with the two-launch form and the stand-alone
    all-reduce, and under CUDA-graph replay through ``nvfp4r.linear_auto(..., reduce=)``."""
    script = tmp_path / "child_fused.py"
    script.write_text(_CHILD_FUSED)
    env = dict(os.environ, REPO=str(REPO), NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29534", str(script)],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.count("FUSED_OK") == 2, (r.stdout[-2000:], r.stderr[-3000:])


@pytest.mark.parametrize("M", [1, 3, 8])
def test_linear_push_epilogue_emulated_ranks(M):
    """Row-parallel linear with the PUSH half of the all-reduce fused into its epilogue
    (`nvfp4r_linear_packed_ex`, `push_to`), two ranks emulated on one GPU: each rank's linear
    over its K shard pushes into both receive buffers, then each rank's GATHER half runs. The
    result equals the rank-ordered sum of the two unfused bf16 linear outputs bit for bit."""
    import numpy as np
    from oracle import nvfp4 as onv
    from reset_b200 import _lib as L
    from reset_b200 import capi
    lib = L.lib()
    world, N, K = 2, 1024, 4096
    max_elems = 8 * N
    nbytes = lib.nvfp4r_peer_buffer_bytes(world, max_elems)
    ptrs = []
    for _ in range(world):
        p, h = C.c_void_p(), C.create_string_buffer(64)
        L.check(lib.nvfp4r_peer_alloc(nbytes, C.byref(p), h), "alloc")
        ptrs.append(p)
    try:
        comms = []
        for r in range(world):
            c = L.PeerComm()
            c.world, c.rank, c.max_elems = world, r, max_elems
            for k in range(world):
                c.base[k] = ptrs[k].value
            comms.append(c)
        g = torch.Generator(device="cuda").manual_seed(40 + M)
        gs = torch.tensor([60.0], dtype=torch.float32, device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        for call in range(3):                                            # parity flips between calls
            x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
            shards, parts = [], []
            for r in range(world):
                w, ws = onv.random_nvfp4((N,), K // world, seed=50 + 10 * call + r)
                packed = capi.pack_weight(torch.from_numpy(w).cuda(), torch.from_numpy(ws).cuda())
                xs = x[:, r * (K // world):(r + 1) * (K // world)]
                wk = capi.packed_workspace(M, N, K // world, "cuda")
                shards.append((packed, xs, wk))
                parts.append(capi.linear_packed(xs, gs, packed, N, 0.5, wk, rcp_mode=L.RCP_APPROX))
            outs = [torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
            for r in range(world):
                packed, xs, wk = shards[r]
                capi.linear_packed_push(xs, gs, packed, N, 0.5, wk, comms[r], outs[r])
            for r in range(world):
                L.check(lib.nvfp4r_peer_allreduce_bf16(C.byref(comms[r]), outs[r].data_ptr(), outs[r].data_ptr(),
                                                       M * N, L.PEER_GATHER, stream), "gather")
            torch.cuda.synchronize()
            want = _expected(parts)
            for r in range(world):
                assert torch.equal(outs[r], want), (call, r)
        L.check(lib.nvfp4r_check_device_status(), "device status")
    finally:
        torch.cuda.synchronize()
        for p in ptrs:
            lib.nvfp4r_peer_free(p)


def test_missing_peer_is_reported_not_waited_for_forever():
    """Failure detection: a gather whose peer never pushed gives up after its poll limit (set
    short here), the launch finishes, and the host reads a time-out status; the device stays
    usable."""
    from reset_b200 import _lib as L
    lib = L.lib()
    world, max_elems = 2, 1024
    nbytes = lib.nvfp4r_peer_buffer_bytes(world, max_elems)
    ptrs = []
    for _ in range(world):
        p, h = C.c_void_p(), C.create_string_buffer(64)
        L.check(lib.nvfp4r_peer_alloc(nbytes, C.byref(p), h), "alloc")
        ptrs.append(p)
    try:
        c = L.PeerComm()
        c.world, c.rank, c.max_elems = world, 0, max_elems
        for k in range(world):
            c.base[k] = ptrs[k].value
        x = torch.ones(512, dtype=torch.bfloat16, device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        L.check(lib.nvfp4r_check_device_status(), "clean before")
        mirror = L.status_mirror()                                     # host-visible twin of the flag
        mirror[0] = 0
        L.check(lib.nvfp4r_set_peer_poll_limit(100000), "limit")       # a few tens of milliseconds
        # rank 0 pushes and gathers, "rank 1" never shows up
        L.check(lib.nvfp4r_peer_allreduce_bf16(C.byref(c), x.data_ptr(), x.data_ptr(), 512, L.PEER_ALLREDUCE, stream),
                "launch")
        # the host learns of it without synchronising the device: poll the pinned word
        import time
        t0 = time.time()
        while mirror[0] == 0 and time.time() - t0 < 20.0:
            time.sleep(0.001)
        assert mirror[0] == 4                                          # code of the peer all-reduce
        mirror[0] = 0
        torch.cuda.synchronize()
        assert lib.nvfp4r_check_device_status() == -5                  # NVFP4R_ERR_DEVICE_TIMEOUT, and cleared
        L.check(lib.nvfp4r_check_device_status(), "cleared")
        y = torch.arange(8, device="cuda").float().sum()                # the context is alive
        assert float(y) == 28.0
    finally:
        lib.nvfp4r_set_peer_poll_limit(0)
        torch.cuda.synchronize()
        for p in ptrs:
            lib.nvfp4r_peer_free(p)
