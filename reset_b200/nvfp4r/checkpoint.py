"""Ingest of ModelOpt NVFP4 Hugging Face checkpoints (safetensors) for the nvfp4r linears.

The reference never reads a checkpoint itself: its ``reset-quantize`` tool writes one with
``modelopt`` (reset/quantize.py:84-107) and vLLM loads it, handing the adapter finished
layer attributes (kernels/python/nvfp4r/vllm_integration.py:377-396,461-491). This module
is the stand-alone form of that loading step, so that the kernels can run on real weights
without vLLM. It follows the layout and the scale conventions of vLLM's ModelOpt NVFP4
linear method (``model_executor/layers/quantization/modelopt.py``, ``create_weights`` /
``process_weights_after_loading``):

per quantized linear ``<prefix>``
    ``<prefix>.weight``          uint8 ``[N, K/2]``   two e2m1 codes per byte, even element low
    ``<prefix>.weight_scale``    e4m3  ``[N, K/16]``  flat block scales
    ``<prefix>.weight_scale_2``  fp32 scalar          per-tensor weight scale
    ``<prefix>.input_scale``     fp32 scalar          calibrated activation scale

    ``input_global_scale = max(input_scale of the merged parts)``,
    ``weight_global_scale = max(weight_scale_2 of the merged parts)``,
    ``alpha = input_global_scale * weight_global_scale``,
    ``input_global_scale_inv = 1 / input_global_scale``.

Merged projections (q/k/v -> qkv_proj, gate/up -> gate_up_proj) are concatenated along the
output rows; tensor parallelism slices every part first (by heads / by rows) and then
merges, as vLLM's ``QKVParallelLinear`` and ``MergedColumnParallelLinear`` do; row-parallel
projections (o_proj, down_proj) are sliced along K (codes by bytes, scales by blocks).

Everything here is host-side tensor slicing; the only device work is the one-time weight
re-layout in :func:`as_layer` (``prime_nvfp4r_caches``).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, Iterable, List, Sequence

import torch

from .. import tp

GROUP_SIZE = 16
_SUFFIXES = ("weight", "weight_scale", "weight_scale_2", "input_scale")


@dataclass
class Nvfp4Linear:
    """One NVFP4 linear (or a merged / sharded one) as plain tensors."""

    weight: torch.Tensor                 # uint8 [N, K/2]
    weight_scale: torch.Tensor           # uint8 [N, K/16] (e4m3 bit patterns, flat)
    weight_scale_2: torch.Tensor         # fp32 [parts]
    input_scale: torch.Tensor            # fp32 [parts]
    name: str = ""
    part_rows: List[int] = field(default_factory=list)   # output rows of every merged part

    @property
    def N(self) -> int:
        return int(self.weight.shape[0])

    @property
    def K(self) -> int:
        return int(self.weight.shape[1]) * 2

    @property
    def input_global_scale(self) -> float:
        return float(self.input_scale.max())

    @property
    def weight_global_scale(self) -> float:
        return float(self.weight_scale_2.max())

    @property
    def alpha(self) -> float:
        return float(torch.tensor(self.input_global_scale, dtype=torch.float32) *
                     torch.tensor(self.weight_global_scale, dtype=torch.float32))

    @property
    def input_global_scale_inv(self) -> float:
        return float(1.0 / torch.tensor(self.input_global_scale, dtype=torch.float32))

    @property
    def uniform_scales(self) -> bool:
        """False when the merged parts were calibrated with different global scales: the
        maximum is used for all of them, as vLLM does (with a warning about accuracy)."""
        return bool(torch.unique(self.input_scale).numel() == 1 and
                    torch.unique(self.weight_scale_2).numel() == 1)

    def validate(self) -> None:
        N, K = self.N, self.K
        if self.weight.dtype != torch.uint8 or self.weight.dim() != 2:
            raise ValueError(f"{self.name}: weight must be uint8 [N, K/2]")
        if K % GROUP_SIZE:
            raise ValueError(f"{self.name}: K={K} is not a multiple of {GROUP_SIZE}")
        if self.weight_scale.dtype != torch.uint8 or tuple(self.weight_scale.shape) != (N, K // GROUP_SIZE):
            raise ValueError(f"{self.name}: weight_scale must be [N, K/16] = [{N}, {K // GROUP_SIZE}], "
                             f"got {tuple(self.weight_scale.shape)} {self.weight_scale.dtype}")
        for t, what in ((self.weight_scale_2, "weight_scale_2"), (self.input_scale, "input_scale")):
            if t.dtype != torch.float32 or t.dim() != 1 or t.numel() < 1:
                raise ValueError(f"{self.name}: {what} must be fp32 [parts]")
            if not bool(torch.isfinite(t).all()) or not bool((t > 0).all()):
                raise ValueError(f"{self.name}: {what} must be finite and positive")


class CheckpointReader:
    """Lazy access to the tensors of a checkpoint directory (``*.safetensors`` with or
    without ``model.safetensors.index.json``) or of a single safetensors file."""

    def __init__(self, path):
        from safetensors import safe_open          # host-side file format library
        self._open = safe_open
        self.path = Path(path)
        self._where: Dict[str, Path] = {}
        self._handles: Dict[Path, object] = {}
        if self.path.is_file():
            files = [self.path]
            self.root = self.path.parent
        elif self.path.is_dir():
            self.root = self.path
            index = self.path / "model.safetensors.index.json"
            if index.exists():
                weight_map = json.loads(index.read_text())["weight_map"]
                for name, fname in weight_map.items():
                    self._where[name] = self.path / fname
                files = []
            else:
                files = sorted(self.path.glob("*.safetensors"))
                if not files:
                    raise FileNotFoundError(f"no safetensors files under {self.path}")
        else:
            raise FileNotFoundError(str(self.path))
        for f in files:
            for name in self._handle(f).keys():
                self._where[name] = f
        self.quant_config = self._read_quant_config()

    def _handle(self, f: Path):
        h = self._handles.get(f)
        if h is None:
            if not f.exists():
                raise FileNotFoundError(f"checkpoint shard {f} is listed in the index but missing")
            h = self._open(str(f), framework="pt", device="cpu")
            self._handles[f] = h
        return h

    def _read_quant_config(self) -> dict:
        """``hf_quant_config.json`` (ModelOpt export) or ``quantization_config`` of
        ``config.json``; {} when neither exists. A checkpoint that declares another
        algorithm or group size is refused."""
        cfg: dict = {}
        hf = self.root / "hf_quant_config.json"
        if hf.exists():
            cfg = dict(json.loads(hf.read_text()).get("quantization", {}))
        elif (self.root / "config.json").exists():
            cfg = dict(json.loads((self.root / "config.json").read_text()).get("quantization_config", {}))
        algo = cfg.get("quant_algo")
        if algo is not None and str(algo).upper() != "NVFP4":
            raise ValueError(f"checkpoint is quantized with {algo!r}, not NVFP4")
        group = cfg.get("group_size")
        if group is not None and int(group) != GROUP_SIZE:
            raise ValueError(f"NVFP4 group size {group} is not supported (must be {GROUP_SIZE})")
        return cfg

    # -- tensors ----------------------------------------------------------------------
    def names(self) -> Iterable[str]:
        return self._where.keys()

    def has(self, name: str) -> bool:
        return name in self._where

    def tensor(self, name: str) -> torch.Tensor:
        f = self._where.get(name)
        if f is None:
            raise KeyError(f"tensor {name!r} is not in the checkpoint")
        return self._handle(f).get_tensor(name)

    def is_quantized(self, prefix: str) -> bool:
        return self.has(f"{prefix}.weight_scale") and self.has(f"{prefix}.weight_scale_2")

    def linear(self, prefix: str) -> Nvfp4Linear:
        """The four tensors of one quantized linear."""
        missing = [s for s in _SUFFIXES if not self.has(f"{prefix}.{s}")]
        if missing:
            raise KeyError(f"{prefix}: not an NVFP4 W4A4 linear (missing {', '.join(missing)})")
        w = self.tensor(f"{prefix}.weight")
        ws = self.tensor(f"{prefix}.weight_scale")
        if ws.dtype == torch.float8_e4m3fn:
            ws = ws.view(torch.uint8)
        lin = Nvfp4Linear(
            weight=w.contiguous(), weight_scale=ws.contiguous(),
            weight_scale_2=self.tensor(f"{prefix}.weight_scale_2").to(torch.float32).reshape(-1),
            input_scale=self.tensor(f"{prefix}.input_scale").to(torch.float32).reshape(-1),
            name=prefix)
        lin.part_rows = [lin.N]
        lin.validate()
        return lin


# -- merging and tensor-parallel slicing ------------------------------------------------

def merge_column(parts: Sequence[Nvfp4Linear], name: str = "") -> Nvfp4Linear:
    """Concatenate linears that share their input along the output rows (q|k|v, gate|up).
    The global scales are kept per part; the merged layer uses their maxima."""
    if not parts:
        raise ValueError("merge_column: no parts")
    K = parts[0].K
    for p in parts:
        if p.K != K:
            raise ValueError(f"merge_column: {p.name} has K={p.K}, expected {K}")
    out = Nvfp4Linear(
        weight=torch.cat([p.weight for p in parts], dim=0).contiguous(),
        weight_scale=torch.cat([p.weight_scale for p in parts], dim=0).contiguous(),
        weight_scale_2=torch.cat([p.weight_scale_2 for p in parts]),
        input_scale=torch.cat([p.input_scale for p in parts]),
        name=name or "|".join(p.name for p in parts),
        part_rows=[r for p in parts for r in p.part_rows])
    out.validate()
    return out


def shard(lin: Nvfp4Linear, style: str, rank: int, world: int) -> Nvfp4Linear:
    """The slice of an un-merged linear that ``rank`` of ``world`` owns: ``"column"`` splits
    the output rows, ``"row"`` splits K (so K / world must stay a multiple of 16)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    if len(lin.part_rows) > 1:
        raise ValueError("shard the parts before merging them (each part is split on its own)")
    w, s = tp.shard_weight(lin.weight, lin.weight_scale, style, rank, world)
    out = Nvfp4Linear(weight=w.contiguous(), weight_scale=s.contiguous(),
                      weight_scale_2=lin.weight_scale_2.clone(), input_scale=lin.input_scale.clone(),
                      name=f"{lin.name}[{style} {rank}/{world}]")
    out.part_rows = [out.N]
    out.validate()
    return out


def _replicated_heads(lin: Nvfp4Linear, head_dim: int, n_heads: int, rank: int, world: int) -> Nvfp4Linear:
    """k/v projection slice when there are fewer KV heads than ranks: every group of
    world / n_heads ranks reads the same head."""
    head = rank * n_heads // world
    rows = slice(head * head_dim, (head + 1) * head_dim)
    out = Nvfp4Linear(weight=lin.weight[rows].contiguous(), weight_scale=lin.weight_scale[rows].contiguous(),
                      weight_scale_2=lin.weight_scale_2.clone(), input_scale=lin.input_scale.clone(),
                      name=f"{lin.name}[head {head}]")
    out.part_rows = [out.N]
    return out


# -- Qwen3 decoder layer ------------------------------------------------------------------

def qwen3_layer(reader: CheckpointReader, index: int, rank: int = 0, world: int = 1,
                head_dim: int = 128, prefix: str = "model.layers") -> Dict[str, object]:
    """The four NVFP4 linears and the four norm weights of decoder layer ``index`` for one
    tensor-parallel rank: ``qkv`` and ``gate_up`` merged and column-parallel, ``o`` and ``down``
    row-parallel, norms replicated (bf16 as stored)."""
    base = f"{prefix}.{index}"
    attn, mlp = f"{base}.self_attn", f"{base}.mlp"
    q, k, v = (reader.linear(f"{attn}.{n}_proj") for n in ("q", "k", "v"))
    kv_heads = k.N // head_dim
    q_r = shard(q, "column", rank, world)
    if kv_heads % world == 0:
        k_r, v_r = shard(k, "column", rank, world), shard(v, "column", rank, world)
    elif world % kv_heads == 0:
        k_r = _replicated_heads(k, head_dim, kv_heads, rank, world)
        v_r = _replicated_heads(v, head_dim, kv_heads, rank, world)
    else:
        raise ValueError(f"{kv_heads} KV heads cannot be spread over {world} ranks")
    gate, up = reader.linear(f"{mlp}.gate_proj"), reader.linear(f"{mlp}.up_proj")
    out: Dict[str, object] = {
        "qkv": merge_column([q_r, k_r, v_r], f"{attn}.qkv_proj"),
        "o": shard(reader.linear(f"{attn}.o_proj"), "row", rank, world),
        "gate_up": merge_column([shard(gate, "column", rank, world), shard(up, "column", rank, world)],
                                f"{mlp}.gate_up_proj"),
        "down": shard(reader.linear(f"{mlp}.down_proj"), "row", rank, world),
        "ln1": reader.tensor(f"{base}.input_layernorm.weight"),
        "ln2": reader.tensor(f"{base}.post_attention_layernorm.weight"),
    }
    for key, name in (("qn", f"{attn}.q_norm.weight"), ("kn", f"{attn}.k_norm.weight")):
        if reader.has(name):
            out[key] = reader.tensor(name)
    return out


# -- hand-over to the adapter ---------------------------------------------------------------

def as_layer(lin: Nvfp4Linear, device, prime: bool = True) -> torch.nn.Module:
    """A module carrying exactly the attributes the adapter reads
    (``apply_nvfp4r_linear(layer, x)``): ``weight``, flat ``weight_scale``,
    ``input_global_scale_inv``, ``alpha``, the partition sizes, and (with ``prime``) the
    derived state of ``prime_nvfp4r_caches`` including the packed tensor-core weight."""
    from . import vllm_integration as vi
    layer = torch.nn.Module()
    dev = torch.device(device)
    layer.weight = torch.nn.Parameter(lin.weight.to(dev), requires_grad=False)
    layer.weight_scale = torch.nn.Parameter(lin.weight_scale.to(dev).view(torch.float8_e4m3fn), requires_grad=False)
    layer.input_global_scale_inv = torch.nn.Parameter(
        torch.tensor([lin.input_global_scale_inv], dtype=torch.float32, device=dev), requires_grad=False)
    layer.alpha = torch.nn.Parameter(torch.tensor(lin.alpha, dtype=torch.float32, device=dev), requires_grad=False)
    layer.input_size_per_partition = lin.K
    layer.output_size_per_partition = lin.N
    layer.weights_padding_cols = 0
    layer._nvfp4r_weight_scale_is_flat = True
    if prime:
        vi.prime_nvfp4r_caches(layer)
    return layer
