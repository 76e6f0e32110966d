"""Batch-1 decode step of a Qwen3-shaped model with NVFP4 W4A4 linears, for measurement.

Builds random-initialised weights of the named geometry directly as NVFP4 codes + block
scales (no bf16 master copy), shards them tensor-parallel (column: qkv, gate_up; row: o,
down), and runs one token through all layers with this library's kernels only; the
all-reduce after the two row-parallel linears of every layer is this library's one-shot
kernel over peer memory (`comm.PeerAllReduce`) or, on request, NCCL. The whole step is
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
    CUDA-core GEMV where the measured crossover can choose it. Calls go through the C ABI with
    caller-owned output buffers (nothing is allocated inside a step)."""

    def __init__(self, N: int, K: int, device, gen, workspace: "Workspace"):
        self.N, self.K, self.ws = N, K, workspace
        w = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=device, generator=gen)
        s = torch.randint(0x20, 0x38, (N, K // 16), dtype=torch.uint8, device=device, generator=gen)
        self.packed = capi.pack_weight(w, s) if (N % 128 == 0 and K % 128 == 0) else None
        self.use_gemv = self.packed is None or nvops.use_gemv(1, N, K, 2)
        self.w, self.s = (w, s) if self.use_gemv else (None, None)
        self.gs_inv = torch.tensor([64.0], dtype=torch.float32, device=device)
        self.alpha = 1.0
        if self.packed is not None:
            workspace.reserve(L.lib().nvfp4r_linear_packed_workspace_bytes(1, N, K))

    @classmethod
    def from_checkpoint(cls, lin, device, workspace: "Workspace") -> "_Linear":
        """A shard read from a ModelOpt NVFP4 checkpoint (``nvfp4r.checkpoint.Nvfp4Linear``):
        codes, flat block scales, ``1 / input_global_scale`` for the quantizer and
        ``alpha = input_global_scale * weight_global_scale`` for the output."""
        self = cls.__new__(cls)
        self.N, self.K, self.ws = lin.N, lin.K, workspace
        w = lin.weight.to(device).contiguous()
        s = lin.weight_scale.to(device).contiguous()
        self.packed = capi.pack_weight(w, s) if (self.N % 128 == 0 and self.K % 128 == 0) else None
        self.use_gemv = self.packed is None or nvops.use_gemv(1, self.N, self.K, 2)
        self.w, self.s = (w, s) if self.use_gemv else (None, None)
        self.gs_inv = torch.tensor([lin.input_global_scale_inv], dtype=torch.float32, device=device)
        self.alpha = lin.alpha
        if self.packed is not None:
            workspace.reserve(L.lib().nvfp4r_linear_packed_workspace_bytes(1, self.N, self.K))
        return self

    def calibrate(self, x: torch.Tensor) -> None:
        """Pick alpha so that the output has unit RMS on a sample input (keeps the random
        model's activations finite; done once, outside any timed region)."""
        out = torch.empty((x.shape[0], self.N), dtype=torch.bfloat16, device=x.device)
        self.plain(x, out)
        rms = float(out.float().pow(2).mean().sqrt().item())
        if rms > 0 and rms == rms:
            self.alpha = 1.0 / rms

    def plain(self, x: torch.Tensor, out: torch.Tensor, push=None, gather: bool = False) -> torch.Tensor:
        if push is not None and not self.use_gemv:
            return capi.linear_packed_push(x, self.gs_inv, self.packed, self.N, self.alpha, self.ws.buf, push, out,
                                           gather=gather)
        if self.use_gemv:
            if push is not None:
                # a shard small enough for the GEMV: push and sum inside the GEMV's own launch
                return capi.linear_push(x, self.gs_inv, self.w, self.s, self.alpha, push, out, rcp_mode=L.RCP_APPROX)
            return capi.linear(x, self.gs_inv, self.w, self.s, self.alpha, out=out, rcp_mode=L.RCP_APPROX)
        return capi.linear_packed(x, self.gs_inv, self.packed, self.N, self.alpha, self.ws.buf,
                                  rcp_mode=L.RCP_APPROX, out=out)

    def gemv_can_push(self) -> bool:
        """The streaming GEMV's in-launch all-reduce takes rows of K % 256 == 0 and an even N."""
        return self.use_gemv and self.K % 256 == 0 and self.N % 2 == 0

    def after_rmsnorm(self, delta, res_in, res_out, norm_w, eps, out):
        # The tensor-core kernel wherever the weight is packed, also where the stand-alone crossover
        # would pick the GEMV: inside a decode layer the GEMV with this prologue measured slower
        # (Qwen3-32B shards, one GPU, exchanges left out: 213.6 / 405 / 439 tok/s against 221 / 430 /
        # 469 at TP 1 / 4 / 8): its CTAs fill the register file, so the attention launch that follows
        # cannot start fetching its cache rows early. The GEMV form serves shapes that cannot be packed.
        if self.packed is None:
            return capi.linear_rmsnorm(delta, res_in, res_out, norm_w, eps, self.gs_inv, self.w, self.s,
                                       self.alpha, out, rcp_mode=L.RCP_APPROX)
        return capi.linear_packed_rmsnorm(delta, res_in, res_out, norm_w, eps, self.gs_inv, self.packed,
                                          self.N, self.alpha, self.ws.buf, rcp_mode=L.RCP_APPROX, out=out)

    def after_silu_mul(self, gate_up, out, push=None, gather: bool = False):
        if self.packed is None:
            return capi.linear_silu(gate_up, self.gs_inv, self.w, self.s, self.alpha, out, rcp_mode=L.RCP_APPROX)
        return capi.linear_packed_silu(gate_up, self.gs_inv, self.packed, self.N, self.alpha, self.ws.buf,
                                       rcp_mode=L.RCP_APPROX, out=out, push=push, gather=gather)

    def weight_bytes(self) -> int:
        return self.N * self.K * 9 // 16


class Workspace:
    """One zero-initialised split-K scratch shared by all linears of a step (their launches
    are ordered on one stream)."""

    def __init__(self, device):
        self.device, self.bytes, self.buf = device, 0, None

    def reserve(self, n: int) -> None:
        self.bytes = max(self.bytes, int(n))

    def allocate(self) -> None:
        self.buf = torch.zeros((self.bytes + 15) // 16 * 2 + 2, dtype=torch.int64, device=self.device)


class DecodeStep:
    def __init__(self, cfg: DecodeConfig, device, rank: int = 0, world: int = 1, seed: int = 0,
                 process_group=None, fused: bool = True, peer_allreduce: bool = True,
                 fused_gather: bool = True, skip_exchange: bool = False):
        if cfg.q_heads % world or cfg.kv_heads % world or cfg.intermediate % world or cfg.vocab % world:
            raise ValueError("tensor-parallel degree must divide heads, intermediate and vocab")
        self.cfg, self.device, self.rank, self.world, self.pg = cfg, torch.device(device), rank, world, process_group
        self.ws = Workspace(self.device)
        gen = torch.Generator(device=self.device).manual_seed(seed + 1000 * rank)
        D, H = cfg.head_dim, cfg.hidden
        self.hq, self.hkv = cfg.q_heads // world, cfg.kv_heads // world
        inter = cfg.intermediate // world
        bf = dict(dtype=torch.bfloat16, device=self.device)
        self.layers = []
        for _ in range(cfg.layers):
            self.layers.append({
                "qkv": _Linear((self.hq + 2 * self.hkv) * D, H, self.device, gen, self.ws),
                "o": _Linear(H, self.hq * D, self.device, gen, self.ws),
                "gate_up": _Linear(2 * inter, H, self.device, gen, self.ws),
                "down": _Linear(H, inter, self.device, gen, self.ws),
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
        self.feed_tokens = False          # random model: the embedding table is a 1024-row stand-in
        self.reset = None                 # set by enable_reset(): ReSET processor + sampling instead of arg-max
        self.head_ws = None               # workspace of the fused lm_head + ReSET launch (enable_reset)
        self.ws.allocate()
        self.res = [torch.zeros(1, H, **bf), torch.zeros(1, H, **bf)]     # ping-pong residual stream
        self.residual = self.res[0]
        self.normed = torch.zeros(1, H, **bf)
        self.qkv_out = torch.zeros(1, (self.hq + 2 * self.hkv) * D, **bf)
        self.o_out = torch.zeros(1, H, **bf)
        self.gu_out = torch.zeros(1, 2 * inter, **bf)
        self.down_out = torch.zeros(1, H, **bf)
        probe = self.layers[0]
        self.fused = bool(fused) and all(probe[n].packed is not None or probe[n].K % 32 == 0
                                         for n in ("qkv", "gate_up", "down"))
        self.q = torch.zeros(1, self.hq * D, **bf)
        self.attn = torch.zeros(1, self.hq * D, **bf)
        self.act = torch.zeros(1, inter, **bf)
        self.logits_local = torch.zeros(1, self.vocab_local, dtype=torch.float32, device=self.device)
        self.logits = torch.zeros(1, cfg.vocab, dtype=torch.float32, device=self.device)
        n = L.lib().nvfp4r_attn_decode_workspace_bytes(self.hq, cfg.context)
        self.attn_ws = torch.zeros((n + 3) // 4, dtype=torch.float32, device=self.device)
        self.graph = None
        # rotary table (cos, sin)(pos * theta^(-2d/D)) for every position of the context
        half = D // 2
        freq = cfg.rope_theta ** (-torch.arange(0, half, device=self.device, dtype=torch.float32) * 2 / D)
        ang = torch.arange(cfg.context, device=self.device, dtype=torch.float32)[:, None] * freq[None, :]
        self.rope_table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()
        L.check(L.lib().nvfp4r_set_rope_table(self.rope_table.data_ptr(), cfg.context), "set_rope_table")
        # the sum exchange after o_proj / down_proj: one-shot kernel over peer memory, or NCCL
        # fused_gather: the row-parallel linear's own launch completes the all-reduce (push in the
        # epilogue, then the pushing thread sums the ranks' contributions); off = push in the
        # epilogue + one gather launch per exchange
        self.fused_gather = bool(fused_gather)
        # skip_exchange: one rank's shard of a tensor-parallel model on a single GPU with the sum
        # exchanges and the logits gather left out (timing / profiling of the compute only; the
        # values are those of the rank's partial sums)
        self.skip_exchange = bool(skip_exchange)
        self.peer = None
        if world > 1 and peer_allreduce and not skip_exchange:
            from .comm import PeerAllReduce
            self.peer = PeerAllReduce(self.device, H, group=process_group)
        self._calibrate()

    def load_checkpoint(self, reader, embed_rows: int = 0) -> None:
        """Replace the random weights by those of a ModelOpt NVFP4 Qwen3 checkpoint
        (``nvfp4r.checkpoint.CheckpointReader``), sliced for this rank. Call before
        :meth:`capture`. ``embed_rows`` limits how many embedding rows are kept on the device
        (0 = all). The lm_head stays bf16, as ModelOpt leaves it (tied to the embedding when the
        checkpoint has no ``lm_head.weight``)."""
        from .nvfp4r import checkpoint as ck
        c = self.cfg
        bf = dict(dtype=torch.bfloat16, device=self.device)
        for i, layer in enumerate(self.layers):
            got = ck.qwen3_layer(reader, i, self.rank, self.world, head_dim=c.head_dim)
            shapes = {"qkv": ((self.hq + 2 * self.hkv) * c.head_dim, c.hidden), "o": (c.hidden, self.hq * c.head_dim),
                      "gate_up": (2 * c.intermediate // self.world, c.hidden),
                      "down": (c.hidden, c.intermediate // self.world)}
            for name, (n, k) in shapes.items():
                lin = got[name]
                if (lin.N, lin.K) != (n, k):
                    raise ValueError(f"layer {i} {name}: checkpoint shard is {lin.N}x{lin.K}, model wants {n}x{k}")
                layer[name] = _Linear.from_checkpoint(lin, self.device, self.ws)
            for key in ("ln1", "ln2", "qn", "kn"):
                if key in got:
                    layer[key] = got[key].to(**bf).contiguous()
        self.final_ln = reader.tensor("model.norm.weight").to(**bf).contiguous()
        embed = reader.tensor("model.embed_tokens.weight")
        head = reader.tensor("lm_head.weight") if reader.has("lm_head.weight") else embed
        lo = self.rank * self.vocab_local
        self.lm_head = head[lo:lo + self.vocab_local].to(**bf).contiguous()
        self.embed = (embed[:embed_rows] if embed_rows else embed).to(**bf).contiguous()
        self.feed_tokens = self.embed.shape[0] >= c.vocab
        self.ws.allocate()
        probe = self.layers[0]
        self.fused = self.fused and all(probe[n].packed is not None or probe[n].K % 32 == 0
                                        for n in ("qkv", "gate_up", "down"))
        self.graph = None

    # -- thin wrappers over the C ABI ------------------------------------------------
    def _stream(self) -> int:
        return torch.cuda.current_stream().cuda_stream

    def _add_rmsnorm(self, x, residual, weight):
        L.check(L.lib().nvfp4r_add_rmsnorm(None if x is None else x.data_ptr(), residual.data_ptr(),
                                           weight.data_ptr(), self.normed.data_ptr(), 1, self.cfg.hidden,
                                           self.cfg.eps, self._stream()), "add_rmsnorm")

    def _attention(self, layer, qkv):
        c = self.cfg
        lib = L.lib()
        if self.fused:
            # head norms + rotary + cache append + attention in one launch
            L.check(lib.nvfp4r_attn_decode_rope(qkv.data_ptr(), layer["qn"].data_ptr(), layer["kn"].data_ptr(),
                                                layer["k"].data_ptr(), layer["v"].data_ptr(),
                                                self.seq_len.data_ptr(), self.attn.data_ptr(), self.hq, self.hkv,
                                                c.head_dim, c.context, c.rope_theta, c.eps,
                                                self.attn_ws.data_ptr(), self.attn_ws.numel() * 4, self._stream()),
                    "attn_decode_rope")
            return
        L.check(lib.nvfp4r_qk_norm_rope_kv(qkv.data_ptr(), layer["qn"].data_ptr(), layer["kn"].data_ptr(),
                                           self.position.data_ptr(), layer["k"].data_ptr(),
                                           layer["v"].data_ptr(), self.q.data_ptr(), self.hq, self.hkv,
                                           c.head_dim, c.context, c.rope_theta, c.eps, self._stream()),
                "qk_norm_rope_kv")
        L.check(lib.nvfp4r_attn_decode(self.q.data_ptr(), layer["k"].data_ptr(), layer["v"].data_ptr(),
                                       self.seq_len.data_ptr(), self.attn.data_ptr(), self.hq, self.hkv,
                                       c.head_dim, c.context, self.attn_ws.data_ptr(),
                                       self.attn_ws.numel() * 4, self._stream()), "attn_decode")

    def _all_reduce(self, t, pushed: bool = False):
        if self.skip_exchange:
            return
        if self.peer is not None:
            if pushed and self.fused_gather:
                return                        # the linear's launch pushed AND summed: nothing left to do
            if pushed:
                self.peer.gather_(t)          # the linear's epilogue already pushed the contributions
            else:
                self.peer.all_reduce_(t)
        elif self.world > 1:
            torch.distributed.all_reduce(t, group=self.pg)

    def _push(self, lin, silu: bool = False):
        """The communicator to push into from this linear's epilogue, or None. A GEMV-sized shard
        pushes only in the form that also sums in its own launch: the streaming GEMV for a plain
        linear, the tensor-core kernel where the SiLU prologue rides along."""
        if self.peer is None:
            return None
        if not lin.use_gemv:
            return self.peer.comm
        if not self.fused_gather:
            return None
        from .nvfp4r import _config
        ok = (lin.packed is not None) if silu else (lin.gemv_can_push() and self.world <= _config.GEMV_PUSH_MAX_WORLD)
        return self.peer.comm if ok else None

    # -- the step ---------------------------------------------------------------------
    def step(self) -> None:
        """One token: embedding row -> all layers -> logits -> arg-max into ``self.token``.
        With ``fused`` the two RMSNorms and the SiLU*up of a layer run inside the prologue of
        the linear that consumes them and the head norms / rotary embedding / cache append inside
        the attention launch (5 launches per layer instead of 9)."""
        c = self.cfg
        lib = L.lib()
        cur = 0
        if self.feed_tokens:
            torch.index_select(self.embed, 0, self.token, out=self.res[0])   # the previous step's token
        else:
            self.res[0].copy_(self.embed[:1])
        x = None                                            # output of the previous row-parallel linear
        for layer in self.layers:
            if self.fused:
                layer["qkv"].after_rmsnorm(x, self.res[cur], self.res[1 - cur], layer["ln1"], c.eps, self.qkv_out)
                cur = 1 - cur
            else:
                self._add_rmsnorm(x, self.res[cur], layer["ln1"])
                layer["qkv"].plain(self.normed, self.qkv_out)
            self._attention(layer, self.qkv_out)
            push = self._push(layer["o"])
            layer["o"].plain(self.attn, self.o_out, push=push, gather=self.fused_gather)
            self._all_reduce(self.o_out, pushed=push is not None)
            if self.fused:
                layer["gate_up"].after_rmsnorm(self.o_out, self.res[cur], self.res[1 - cur], layer["ln2"], c.eps,
                                               self.gu_out)
                cur = 1 - cur
                push = self._push(layer["down"], silu=True)
                layer["down"].after_silu_mul(self.gu_out, self.down_out, push=push, gather=self.fused_gather)
            else:
                push = None
                self._add_rmsnorm(self.o_out, self.res[cur], layer["ln2"])
                layer["gate_up"].plain(self.normed, self.gu_out)
                L.check(lib.nvfp4r_silu_mul(self.gu_out.data_ptr(), self.act.data_ptr(), 1, self.act.shape[1],
                                            self._stream()), "silu_mul")
                layer["down"].plain(self.act, self.down_out)
            self._all_reduce(self.down_out, pushed=push is not None)
            x = self.down_out
        self._add_rmsnorm(x, self.res[cur], self.final_ln)
        if self.reset is not None and self.head_ws is not None:
            # one rank holds the whole vocabulary: lm_head and the ReSET step are one launch, the
            # logits reach memory once, already divided by the temperature
            d = self.reset
            capi.lm_head_reset_step(self.normed, self.lm_head, self.logits_local, d.states, d.params_dev,
                                    last_ids=self.last_ids, nl_bitmaps=d.nl_bitmaps, dnl_bitmaps=d.dnl_bitmaps,
                                    n_id_sets=d.n_id_sets, decisions=d.decisions, workspace=self.head_ws)
            capi.sample(self.logits_local, self.draws, seed=self.sample_seed, last_ids=self.last_ids,
                        out=self.token, top_k=self.top_k, top_p=self.top_p, workspace=self.sample_ws)
            return
        L.check(lib.nvfp4r_lm_head(self.normed.data_ptr(), self.lm_head.data_ptr(), self.logits_local.data_ptr(),
                                   self.vocab_local, c.hidden, self._stream()), "lm_head")
        if self.world > 1 and not self.skip_exchange:
            torch.distributed.all_gather_into_tensor(self.logits.view(-1), self.logits_local.view(-1), group=self.pg)
            full = self.logits
        else:
            full = self.logits_local
        if self.reset is not None:
            # ReSET temperature on the full-vocabulary logits, then one draw from their softmax:
            # processor and sampler stay on the device, nothing returns to the host per token
            d = self.reset
            capi.reset_step_per_request(full, d.states, d.params_dev, last_ids=self.last_ids,
                                        nl_bitmaps=d.nl_bitmaps, dnl_bitmaps=d.dnl_bitmaps,
                                        n_id_sets=d.n_id_sets, decisions=d.decisions, workspace=d.workspace)
            capi.sample(full, self.draws, seed=self.sample_seed, last_ids=self.last_ids, out=self.token,
                        top_k=self.top_k, top_p=self.top_p, workspace=self.sample_ws)
            return
        L.check(lib.nvfp4r_argmax(full.data_ptr(), full.stride(0), 1, full.shape[1], self.token.data_ptr(),
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

    def enable_reset(self, t_high: float = 1.0, t_low: float = 0.1, tau0: float = 0.5505, window: int = 32,
                     nl_ids=(), dnl_ids=(), seed: int = 0, top_k: int = 0, top_p: float = 1.0,
                     fused_head: bool = True) -> None:
        """End every step with the ReSET processor (reset/reset/logits_processor.py:62-134) and a
        draw from the softmax of the scaled logits instead of the arg-max, optionally restricted
        to the top-k / top-p set as vLLM's sampler would. Every rank holds the full logits after
        the gather and runs the same processor with the same seed, so all ranks draw the same
        token. Call before :meth:`capture`; call again to start a new request (state, counters
        and recent ids are cleared)."""
        from .reset.logits_processor import _DeviceReset
        self.reset = _DeviceReset(1, self.cfg.vocab, self.device)
        self.reset.set_slot(0, t_high, t_low, tau0, window, nl_ids, dnl_ids)
        self.last_ids = torch.full((1, 2), -1, dtype=torch.int32, device=self.device)
        self.draws = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.sample_seed = int(seed)
        self.top_k, self.top_p = int(top_k), float(top_p)
        self.sample_ws = capi.sample_workspace(1, self.device)
        # lm_head + ReSET in one launch when this rank has the whole vocabulary and a warp of the
        # one-CTA-per-SM grid holds at most 64 logits
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        fits = self.world == 1 and self.cfg.vocab <= 64 * 32 * min(sms, 256) and self.cfg.hidden % 256 == 0
        self.head_ws = capi.lm_head_reset_workspace(self.device) if (fits and fused_head) else None
        self.graph = None

    def set_position(self, pos: int) -> None:
        """The next step writes the cache row ``pos`` and attends to rows 0..pos (device-side
        state, so a captured graph follows it)."""
        if not 0 <= pos < self.cfg.context:
            raise ValueError(f"position {pos} outside the context of {self.cfg.context}")
        self.position.fill_(pos)
        self.seq_len.fill_(pos + 1)

    # -- accounting -------------------------------------------------------------------
    def bytes_per_step(self) -> int:
        """Algorithmic HBM bytes one rank moves per token: NVFP4 linears, bf16 KV cache of the
        context, bf16 lm_head shard."""
        c = self.cfg
        lin = sum(l[n].weight_bytes() for l in self.layers for n in ("qkv", "o", "gate_up", "down"))
        kv = c.layers * 2 * self.hkv * c.context * c.head_dim * 2
        return lin + kv + self.vocab_local * c.hidden * 2

    def kernels_per_step(self) -> int:
        """Launches of this library per token on this rank (the logits all-gather of a
        tensor-parallel run is NCCL's and not counted)."""
        from .nvfp4r import _config
        per_layer = 5 if self.fused else 9
        if self.world > 1:
            if self.peer is None:
                per_layer += 0                                   # two NCCL all-reduces, not ours
            else:
                # o_proj / down_proj each: nothing extra when the linear's launch completes the
                # all-reduce, one gather launch after a pushing linear, one all-reduce launch
                # after a GEMV-sized linear
                probe = self.layers[0]
                for name in ("o", "down"):
                    lin = probe[name]
                    pushed = (not lin.use_gemv and (self.fused or name == "o")) or \
                        (lin.use_gemv and self.fused_gather and
                         ((lin.gemv_can_push() and self.world <= _config.GEMV_PUSH_MAX_WORLD) if name == "o"
                          else (self.fused and lin.packed is not None)))
                    per_layer += 0 if (pushed and self.fused_gather) else 1
        return self.cfg.layers * per_layer + 5 + (1 if self.reset is not None and self.head_ws is None else 0)
