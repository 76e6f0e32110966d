"""ModelOpt NVFP4 checkpoint ingest (reset_b200/nvfp4r/checkpoint.py).

The reference leaves loading to vLLM (kernels/python/nvfp4r/vllm_integration.py:377-396
only consumes the finished layer attributes), so there is no reference loader to compare
with; these tests pin the conventions of vLLM's ModelOpt NVFP4 linear method on a small
synthetic checkpoint written with the safetensors library:

* CPU: file discovery (single file, directory, sharded index), scale merging (max over the
  merged parts, alpha, inverse), column/row tensor-parallel slices reassembling to the full
  weight, replicated KV heads, refusal of foreign quantization configs;
* GPU: a loaded shard through the adapter and through the decode step equals the oracle's
  linear on the same checkpoint tensors, and the K-sharded partial products of two ranks
  sum to the full product.
"""

import json

import numpy as np
import pytest
import torch

from reset_b200.nvfp4r import checkpoint as ck

H, QH, KVH, D, INTER, VOCAB, LAYERS = 512, 4, 2, 128, 1024, 1024, 2


def _linear_tensors(g, prefix, N, K, w2, in_s):
    return {
        f"{prefix}.weight": torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g),
        f"{prefix}.weight_scale": torch.randint(0x20, 0x38, (N, K // 16), dtype=torch.uint8,
                                                generator=g).view(torch.float8_e4m3fn),
        f"{prefix}.weight_scale_2": torch.tensor(w2, dtype=torch.float32),
        f"{prefix}.input_scale": torch.tensor(in_s, dtype=torch.float32),
    }


def make_checkpoint(root, seed=0, files=2, uniform=True, with_index=True, lm_head=True):
    """A two-layer Qwen3-shaped NVFP4 checkpoint in ModelOpt's Hugging Face layout."""
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for i in range(LAYERS):
        a, m = f"model.layers.{i}.self_attn", f"model.layers.{i}.mlp"
        s_in = 0.02 + 0.001 * i
        tensors.update(_linear_tensors(g, f"{a}.q_proj", QH * D, H, 2.0e-4, s_in))
        tensors.update(_linear_tensors(g, f"{a}.k_proj", KVH * D, H, 2.0e-4 if uniform else 3.0e-4, s_in))
        tensors.update(_linear_tensors(g, f"{a}.v_proj", KVH * D, H, 2.0e-4, s_in if uniform else 0.5 * s_in))
        tensors.update(_linear_tensors(g, f"{a}.o_proj", H, QH * D, 1.5e-4, 0.03))
        tensors.update(_linear_tensors(g, f"{m}.gate_proj", INTER, H, 1.0e-4, 0.025))
        tensors.update(_linear_tensors(g, f"{m}.up_proj", INTER, H, 1.0e-4, 0.025))
        tensors.update(_linear_tensors(g, f"{m}.down_proj", H, INTER, 2.5e-4, 0.04))
        for n in (f"model.layers.{i}.input_layernorm.weight", f"model.layers.{i}.post_attention_layernorm.weight"):
            tensors[n] = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
        for n in (f"{a}.q_norm.weight", f"{a}.k_norm.weight"):
            tensors[n] = (1.0 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16)
    tensors["model.norm.weight"] = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    tensors["model.embed_tokens.weight"] = torch.randn(VOCAB, H, generator=g).to(torch.bfloat16)
    if lm_head:
        tensors["lm_head.weight"] = (0.05 * torch.randn(VOCAB, H, generator=g)).to(torch.bfloat16)
    names = sorted(tensors)
    weight_map = {}
    for f in range(files):
        fname = f"model-{f + 1:05d}-of-{files:05d}.safetensors" if files > 1 else "model.safetensors"
        part = {n: tensors[n].contiguous() for n in names[f::files]}
        save_file(part, str(root / fname))
        weight_map.update({n: fname for n in part})
    if with_index and files > 1:
        (root / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    (root / "hf_quant_config.json").write_text(json.dumps(
        {"producer": {"name": "modelopt"}, "quantization": {"quant_algo": "NVFP4", "group_size": 16,
                                                            "exclude_modules": ["lm_head"]}}))
    return tensors


# ---------------------------------------------------------------------------------------
# CPU
# ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("files,with_index", [(1, False), (2, True), (3, False)])
def test_reader_finds_every_tensor(tmp_path, files, with_index):
    tensors = make_checkpoint(tmp_path, files=files, with_index=with_index)
    r = ck.CheckpointReader(tmp_path)
    assert set(r.names()) == set(tensors)
    assert r.quant_config["quant_algo"] == "NVFP4"
    lin = r.linear("model.layers.1.mlp.down_proj")
    assert (lin.N, lin.K) == (H, INTER)
    assert torch.equal(lin.weight, tensors["model.layers.1.mlp.down_proj.weight"])
    assert torch.equal(lin.weight_scale, tensors["model.layers.1.mlp.down_proj.weight_scale"].view(torch.uint8))
    assert r.is_quantized("model.layers.0.self_attn.q_proj") and not r.is_quantized("lm_head")
    if files == 1:
        single = ck.CheckpointReader(tmp_path / "model.safetensors")
        assert set(single.names()) == set(tensors)


def test_reader_errors(tmp_path):
    make_checkpoint(tmp_path, files=1)
    r = ck.CheckpointReader(tmp_path)
    with pytest.raises(KeyError, match="not an NVFP4 W4A4 linear"):
        r.linear("lm_head")
    with pytest.raises(KeyError):
        r.tensor("model.layers.9.mlp.up_proj.weight")
    with pytest.raises(FileNotFoundError):
        ck.CheckpointReader(tmp_path / "nowhere")
    (tmp_path / "hf_quant_config.json").write_text(json.dumps({"quantization": {"quant_algo": "FP8"}}))
    with pytest.raises(ValueError, match="not NVFP4"):
        ck.CheckpointReader(tmp_path)
    (tmp_path / "hf_quant_config.json").write_text(
        json.dumps({"quantization": {"quant_algo": "NVFP4", "group_size": 32}}))
    with pytest.raises(ValueError, match="group size"):
        ck.CheckpointReader(tmp_path)


def test_merged_scales_follow_the_maximum(tmp_path):
    make_checkpoint(tmp_path, uniform=False)
    r = ck.CheckpointReader(tmp_path)
    layer = ck.qwen3_layer(r, 1, head_dim=D)
    qkv = layer["qkv"]
    assert (qkv.N, qkv.K) == ((QH + 2 * KVH) * D, H) and qkv.part_rows == [QH * D, KVH * D, KVH * D]
    assert not qkv.uniform_scales
    s_in = np.float32(0.02 + 0.001)
    assert qkv.weight_global_scale == float(np.float32(3.0e-4))
    assert qkv.input_global_scale == float(s_in)
    assert qkv.alpha == float(np.float32(3.0e-4) * s_in)
    assert qkv.input_global_scale_inv == float(np.float32(1.0) / s_in)
    assert layer["gate_up"].uniform_scales and layer["gate_up"].N == 2 * INTER


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_slices_reassemble(tmp_path, world):
    tensors = make_checkpoint(tmp_path)
    r = ck.CheckpointReader(tmp_path)
    per_rank = [ck.qwen3_layer(r, 0, rank, world, head_dim=D) for rank in range(world)]
    a, m = "model.layers.0.self_attn", "model.layers.0.mlp"
    # row-parallel: K slices side by side give the full weight
    for key, name in (("o", f"{a}.o_proj"), ("down", f"{m}.down_proj")):
        assert torch.equal(torch.cat([p[key].weight for p in per_rank], dim=1), tensors[f"{name}.weight"])
        assert torch.equal(torch.cat([p[key].weight_scale for p in per_rank], dim=1),
                           tensors[f"{name}.weight_scale"].view(torch.uint8))
    # column-parallel merged: rank r holds [q_r | k_r | v_r]; with 2 KV heads and 4 ranks every
    # KV head is read by two ranks
    qh, kvh = QH // world, max(KVH // world, 1)
    for rank, p in enumerate(per_rank):
        qkv = p["qkv"]
        assert qkv.part_rows == [qh * D, kvh * D, kvh * D]
        q_full = tensors[f"{a}.q_proj.weight"]
        assert torch.equal(qkv.weight[:qh * D], q_full[rank * qh * D:(rank + 1) * qh * D])
        head = rank * KVH // world
        k_full = tensors[f"{a}.k_proj.weight"]
        assert torch.equal(qkv.weight[qh * D:(qh + kvh) * D], k_full[head * D:(head + kvh) * D])
        gu = p["gate_up"]
        n = INTER // world
        assert torch.equal(gu.weight[:n], tensors[f"{m}.gate_proj.weight"][rank * n:(rank + 1) * n])
        assert torch.equal(gu.weight[n:], tensors[f"{m}.up_proj.weight"][rank * n:(rank + 1) * n])
        assert torch.equal(p["ln1"], tensors["model.layers.0.input_layernorm.weight"])


def test_shard_refuses_bad_requests(tmp_path):
    make_checkpoint(tmp_path, files=1)
    r = ck.CheckpointReader(tmp_path)
    lin = r.linear("model.layers.0.self_attn.o_proj")
    with pytest.raises(ValueError):
        ck.shard(lin, "row", 2, 2)
    with pytest.raises(ValueError, match="not divisible"):
        ck.shard(lin, "row", 0, 3)
    merged = ck.merge_column([lin, lin])
    with pytest.raises(ValueError, match="before merging"):
        ck.shard(merged, "column", 0, 2)
    with pytest.raises(ValueError, match="K="):
        ck.merge_column([lin, r.linear("model.layers.0.mlp.down_proj")])


# ---------------------------------------------------------------------------------------
# GPU: loaded shards through the adapter and the decode step
# ---------------------------------------------------------------------------------------

def _oracle_linear(lin, x_bf16_cuda):
    """fp64 product of the checkpoint's own tensors with the activations quantized the way
    the adapter quantizes them (stand-alone quantizer, approximate-reciprocal mode)."""
    from oracle import nvfp4 as onv
    from reset_b200 import _lib, capi
    gs_inv = torch.tensor([lin.input_global_scale_inv], dtype=torch.float32, device="cuda")
    codes, scales = capi.quant(x_bf16_cuda, gs_inv, rcp_mode=_lib.RCP_APPROX)
    return onv.linear_f64(lin.weight.numpy(), lin.weight_scale.numpy(), codes.cpu().numpy(),
                          scales.cpu().numpy(), alpha=lin.alpha)


@pytest.mark.gpu
def test_loaded_layer_through_the_adapter(tmp_path):
    from helpers import make_activation, rel_l2
    from reset_b200.nvfp4r import vllm_integration as vi
    make_checkpoint(tmp_path)
    r = ck.CheckpointReader(tmp_path)
    got = ck.qwen3_layer(r, 0, head_dim=D)
    for key in ("qkv", "o", "gate_up", "down"):
        lin = got[key]
        layer = ck.as_layer(lin, "cuda")
        assert layer._nvfp4r_caches_primed and layer._nvfp4r_weight_packed is not None
        assert abs(layer._nvfp4r_alpha_host - lin.alpha) <= 1e-12
        for M in (1, 3):
            x = (make_activation(M, lin.K, seed=11 + M).float() * lin.input_global_scale * 300).to(torch.bfloat16).cuda()
            y = vi.apply_nvfp4r_linear(layer, x)
            ref = _oracle_linear(lin, x)
            assert rel_l2(y.float().cpu().numpy(), ref) <= 6e-3, key      # bf16 output rounding


@pytest.mark.gpu
def test_row_parallel_checkpoint_shards_sum_to_the_full_product(tmp_path):
    from helpers import make_activation, rel_l2
    from reset_b200.nvfp4r import vllm_integration as vi
    make_checkpoint(tmp_path)
    r = ck.CheckpointReader(tmp_path)
    full = r.linear("model.layers.1.mlp.down_proj")
    x = (make_activation(2, full.K, seed=5).float() * full.input_global_scale * 300).to(torch.bfloat16).cuda()
    ref = _oracle_linear(full, x)
    world = 2
    total = np.zeros_like(ref)
    for rank in range(world):
        part = ck.shard(full, "row", rank, world)
        layer = ck.as_layer(part, "cuda")
        k = full.K // world
        y = vi.apply_nvfp4r_linear(layer, x[:, rank * k:(rank + 1) * k].contiguous())
        total += y.float().cpu().numpy()
    assert rel_l2(total, ref) <= 8e-3                     # two bf16 roundings before the sum


@pytest.mark.gpu
def test_decode_step_runs_on_a_loaded_checkpoint(tmp_path):
    from helpers import rel_l2
    from reset_b200.decode import DecodeConfig, DecodeStep
    tensors = make_checkpoint(tmp_path)
    r = ck.CheckpointReader(tmp_path)
    cfg = DecodeConfig("tiny-loaded", LAYERS, H, QH, KVH, D, INTER, VOCAB, context=256)
    m = DecodeStep(cfg, "cuda", seed=1)
    m.load_checkpoint(r)
    assert m.feed_tokens and m.fused
    # wiring: every linear of the step equals the oracle on the checkpoint's tensors
    got = ck.qwen3_layer(r, 1, head_dim=D)
    for key in ("qkv", "o", "gate_up", "down"):
        lin = got[key]
        x = (torch.randn(1, lin.K, device="cuda") * lin.input_global_scale * 300).to(torch.bfloat16)
        out = torch.empty(1, lin.N, dtype=torch.bfloat16, device="cuda")
        m.layers[1][key].plain(x, out)
        torch.cuda.synchronize()
        assert rel_l2(out.float().cpu().numpy(), _oracle_linear(lin, x)) <= 6e-3, key
    assert torch.equal(m.final_ln.cpu(), tensors["model.norm.weight"])
    assert torch.equal(m.lm_head.cpu(), tensors["lm_head.weight"])
    assert torch.equal(m.layers[0]["qn"].cpu(), tensors["model.layers.0.self_attn.q_norm.weight"])
    # a few tokens: the captured graph follows the fed-back token and the position
    m.token.fill_(17)
    m.set_position(3)
    m.step()
    torch.cuda.synchronize()
    eager_logits = m.logits_local.clone()
    eager_token = int(m.token.item())
    assert torch.isfinite(eager_logits).all() and 0 <= eager_token < VOCAB
    assert eager_token == int(eager_logits.argmax().item())
    m.capture()
    m.token.fill_(17)
    m.set_position(3)
    m.replay()
    torch.cuda.synchronize()
    assert torch.equal(m.logits_local, eager_logits) and int(m.token.item()) == eager_token
    m.set_position(4)
    m.replay()                                          # next token from the one just produced
    torch.cuda.synchronize()
    assert torch.isfinite(m.logits_local).all()
    from reset_b200 import _lib
    assert _lib.lib().nvfp4r_check_device_status() == 0
