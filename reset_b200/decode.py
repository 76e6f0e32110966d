"""Batch-1 decode step of a Qwen3-shaped model with NVFP4 W4A4 linears, for measurement.

Builds random-initialised weights of the named geometry directly as NVFP4 codes + block
scales (no bf16 master copy), shards them tensor-parallel (column: qkv, gate_up; row: o,
down), and runs one token through all layers with this library's kernels only; the
all-reduce after the two row-parallel linears of every layer is NCCL. The whole step is
captured in one CUDA graph. This is benchmark scaffolding: the reference leaves the model
to vLLM and has no counterpart for this file.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib as L
from . import capi
from .nvfp4r import ops as nvops


@dataclass(frozen=True)
class DecodeConfig:
    name: str
    layers: int
    hidden: int
    q_heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    context: int = 2048
    rope_theta: float = 1.0e6
    eps: float = 1.0e-6


QWEN3_32B = DecodeConfig("Qwen3-32B", 64, 5120, 64, 8, 128, 25600, 151936)
QWEN3_8B = DecodeConfig("Qwen3-8B", 36, 4096, 32, 8, 128, 12288, 151936)


class _Linear:
    """One NVFP4 linear shard: packed weight for the tensor-core kernel, flat weight for the
    CUDA-core GEMV where the measured crossover can choose it."""

    def __init__(self, N: int, K: int, device, gen, max_m: int = 1):
        self.N, self.K = N, K
        w = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=device, generator=gen)
        s = torch.randint(0x20, 0x38, (N, K // 16), dtype=torch.uint8, device=device, generator=gen)
        self.packed = capi.pack_weight(w, s) if (N % 128 == 0 and K % 256 == 0) else None
        keep_flat = self.packed is None or any(nvops.use_gemv(m, N, K, 2) for m in range(1, max_m + 1))
        self.w, self.s = (w, s) if keep_flat else (None, None)
        self.gs_inv = torch.tensor([64.0], dtype=torch.float32, device=device)
        self.alpha = 1.0

    def calibrate(self, x: torch.Tensor) -> None:
        """Pick alpha so that the output has unit RMS on a sample input (keeps the random
        model's activations finite; done once, outside any timed region)."""
        y = self(x).float()
        rms = float(y.pow(2).mean().sqrt().item())
        if rms > 0 and rms == rms:
            self.alpha = 1.0 / rms

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return nvops.linear_auto(x, self.gs_inv, self.w, self.s, self.packed, self.N, self.alpha,
                                 torch.bfloat16, L.RCP_APPROX)

    def weight_bytes(self) -> int:
        return self.N * self.K * 9 // 16


class DecodeStep:
    def __init__(self, cfg: DecodeConfig, device, rank: int = 0, world: int = 1, seed: int = 0,
                 process_group=None):
        if cfg.q_heads % world or cfg.kv_heads % world or cfg.intermediate % world or cfg.vocab % world:
            raise ValueError("tensor-parallel degree must divide heads, intermediate and vocab")
        self.cfg, self.device, self.rank, self.world, self.pg = cfg, torch.device(device), rank, world, process_group
        gen = torch.Generator(device=self.device).manual_seed(seed + 1000 * rank)
        D, H = cfg.head_dim, cfg.hidden
        self.hq, self.hkv = cfg.q_heads // world, cfg.kv_heads // world
        inter = cfg.intermediate // world
        bf = dict(dtype=torch.bfloat16, device=self.device)
        self.layers = []
        for _ in range(cfg.layers):
            self.layers.append({
                "qkv": _Linear((self.hq + 2 * self.hkv) * D, H, self.device, gen),
                "o": _Linear(H, self.hq * D, self.device, gen),
                "gate_up": _Linear(2 * inter, H, self.device, gen),
                "down": _Linear(H, inter, self.device, gen),
                "ln1": torch.ones(H, **bf), "ln2": torch.ones(H, **bf),
                "qn": torch.ones(D, **bf), "kn": torch.ones(D, **bf),
                "k": (torch.randn(self.hkv, cfg.context, D, device=self.device, generator=gen) * 0.5).to(torch.bfloat16),
                "v": (torch.randn(self.hkv, cfg.context, D, device=self.device, generator=gen) * 0.5).to(torch.bfloat16),
            })
        self.final_ln = torch.ones(H, **bf)
        self.vocab_local = cfg.vocab // world
        self.lm_head = (torch.randn(self.vocab_local, H, device=self.device, generator=gen) * 0.02).to(torch.bfloat16)
        self.embed = (torch.randn(1024, H, device=self.device, generator=gen)).to(torch.bfloat16)
        # step state (device-resident so that the captured graph can be replayed)
        self.position = torch.tensor([cfg.context - 1], dtype=torch.int32, device=self.device)
        self.seq_len = torch.tensor([cfg.context], dtype=torch.int32, device=self.device)
        self.token = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.residual = torch.zeros(1, H, **bf)
        self.normed = torch.zeros(1, H, **bf)
        self.q = torch.zeros(1, self.hq * D, **bf)
        self.attn = torch.zeros(1, self.hq * D, **bf)
        self.act = torch.zeros(1, inter, **bf)
        self.logits_local = torch.zeros(1, self.vocab_local, dtype=torch.float32, device=self.device)
        self.logits = torch.zeros(1, cfg.vocab, dtype=torch.float32, device=self.device)
        n = L.lib().nvfp4r_attn_decode_workspace_bytes(self.hq, cfg.context)
        self.attn_ws = torch.zeros((n + 3) // 4, dtype=torch.float32, device=self.device)
        self.graph = None
        self._calibrate()

    # -- thin wrappers over the C ABI ------------------------------------------------
    def _stream(self) -> int:
        return torch.cuda.current_stream().cuda_stream

    def _add_rmsnorm(self, x, weight):
        L.check(L.lib().nvfp4r_add_rmsnorm(None if x is None else x.data_ptr(), self.residual.data_ptr(),
                                           weight.data_ptr(), self.normed.data_ptr(), 1, self.cfg.hidden,
                                           self.cfg.eps, self._stream()), "add_rmsnorm")

    def _attention(self, layer, qkv):
        c = self.cfg
        lib = L.lib()
        L.check(lib.nvfp4r_qk_norm_rope_kv(qkv.data_ptr(), layer["qn"].data_ptr(), layer["kn"].data_ptr(),
                                           self.position.data_ptr(), layer["k"].data_ptr(),
                                           layer["v"].data_ptr(), self.q.data_ptr(), self.hq, self.hkv,
                                           c.head_dim, c.context, c.rope_theta, c.eps, self._stream()),
                "qk_norm_rope_kv")
        L.check(lib.nvfp4r_attn_decode(self.q.data_ptr(), layer["k"].data_ptr(), layer["v"].data_ptr(),
                                       self.seq_len.data_ptr(), self.attn.data_ptr(), self.hq, self.hkv,
                                       c.head_dim, c.context, self.attn_ws.data_ptr(),
                                       self.attn_ws.numel() * 4, self._stream()), "attn_decode")

    def _all_reduce(self, t):
        if self.world > 1:
            torch.distributed.all_reduce(t, group=self.pg)

    # -- the step ---------------------------------------------------------------------
    def step(self) -> None:
        """One token: embedding row -> all layers -> logits -> arg-max into ``self.token``."""
        c = self.cfg
        lib = L.lib()
        self.residual.copy_(self.embed[:1])
        x = None
        for layer in self.layers:
            self._add_rmsnorm(x, layer["ln1"])
            qkv = layer["qkv"](self.normed)
            self._attention(layer, qkv)
            x = layer["o"](self.attn)
            self._all_reduce(x)
            self._add_rmsnorm(x, layer["ln2"])
            gu = layer["gate_up"](self.normed)
            L.check(lib.nvfp4r_silu_mul(gu.data_ptr(), self.act.data_ptr(), 1, self.act.shape[1], self._stream()),
                    "silu_mul")
            x = layer["down"](self.act)
            self._all_reduce(x)
        self._add_rmsnorm(x, self.final_ln)
        L.check(lib.nvfp4r_lm_head(self.normed.data_ptr(), self.lm_head.data_ptr(), self.logits_local.data_ptr(),
                                   self.vocab_local, c.hidden, self._stream()), "lm_head")
        if self.world > 1:
            torch.distributed.all_gather_into_tensor(self.logits.view(-1), self.logits_local.view(-1), group=self.pg)
            full = self.logits
        else:
            full = self.logits_local
        L.check(lib.nvfp4r_argmax(full.data_ptr(), full.stride(0), 1, c.vocab, self.token.data_ptr(),
                                  self._stream()), "argmax")

    def _calibrate(self) -> None:
        g = torch.Generator(device=self.device).manual_seed(7)
        for layer in self.layers[:1]:
            for name in ("qkv", "o", "gate_up", "down"):
                lin = layer[name]
                x = torch.randn(1, lin.K, device=self.device, generator=g).to(torch.bfloat16)
                lin.calibrate(x)
        for layer in self.layers[1:]:
            for name in ("qkv", "o", "gate_up", "down"):
                layer[name].alpha = self.layers[0][name].alpha
        torch.cuda.synchronize()

    def capture(self) -> None:
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.step()                       # warm-up (workspaces, NCCL)
            self.step()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self.step()
        torch.cuda.current_stream().wait_stream(side)

    def replay(self) -> None:
        self.graph.replay()

    # -- accounting -------------------------------------------------------------------
    def bytes_per_step(self) -> int:
        """Algorithmic HBM bytes one rank moves per token: NVFP4 linears, bf16 KV cache of the
        context, bf16 lm_head shard."""
        c = self.cfg
        lin = sum(l[n].weight_bytes() for l in self.layers for n in ("qkv", "o", "gate_up", "down"))
        kv = c.layers * 2 * self.hkv * c.context * c.head_dim * 2
        return lin + kv + self.vocab_local * c.hidden * 2

    def kernels_per_step(self) -> int:
        return self.cfg.layers * 10 + 4
