"""Tensor parallelism by KV head for the large-model configuration (not in the reference, which is single-GPU:
"tensor parallelism" is on its not-implemented list, README.md:252-254).

Sharding (rank r of W): query heads [r*NH/W, (r+1)*NH/W) and KV heads [r*NKV/W, (r+1)*NKV/W) with their biases; the
matching input columns of o_proj; rows [r*I/W, (r+1)*I/W) of gate and up; the matching input columns of down_proj.
Embedding, norms and LM head are replicated. Each rank's paged pool holds NKV/W heads, so block tables, slot
mappings and every scheduler decision are identical on all ranks: every rank runs the same deterministic scheduler on
the same requests (lock-step), and the only data-path collective is an NCCL all-reduce (sum) of the [tokens, hidden]
activations after o_proj and after down_proj (the two sites of nanoserve/model.py:256-257). The all-reduced values,
hence the logits and the greedy tokens, are bitwise identical on every rank.
"""
from __future__ import annotations

import dataclasses

import torch
import torch.distributed as dist

from nanoserve_b200.model import ModelConfig, Qwen2Model


def local_config(cfg: ModelConfig, world: int) -> ModelConfig:
    if cfg.n_kv_heads % world or cfg.n_heads % world or cfg.intermediate_size % world:
        raise ValueError(f"cannot split {cfg.n_heads} heads / {cfg.n_kv_heads} KV heads / MLP {cfg.intermediate_size} "
                         f"over {world} ranks")
    return dataclasses.replace(cfg, n_heads=cfg.n_heads // world, n_kv_heads=cfg.n_kv_heads // world,
                               intermediate_size=cfg.intermediate_size // world)


def shard_state_dict(sd: dict, cfg: ModelConfig, rank: int, world: int) -> dict:
    """This rank's slice of a full Hugging Face-named state dict (views where possible, contiguous copies where the
    slice is along columns)."""
    hd = cfg.head_dim
    q0, q1 = rank * cfg.n_heads // world * hd, (rank + 1) * cfg.n_heads // world * hd
    k0, k1 = rank * cfg.n_kv_heads // world * hd, (rank + 1) * cfg.n_kv_heads // world * hd
    i0, i1 = rank * cfg.intermediate_size // world, (rank + 1) * cfg.intermediate_size // world
    out = {}
    for name, t in sd.items():
        if name.endswith("q_proj.weight") or name.endswith("q_proj.bias"):
            out[name] = t[q0:q1]
        elif name.endswith(("k_proj.weight", "k_proj.bias", "v_proj.weight", "v_proj.bias")):
            out[name] = t[k0:k1]
        elif name.endswith("o_proj.weight"):
            out[name] = t[:, q0:q1].contiguous()
        elif name.endswith(("gate_proj.weight", "up_proj.weight")):
            out[name] = t[i0:i1]
        elif name.endswith("down_proj.weight"):
            out[name] = t[:, i0:i1].contiguous()
        else:
            out[name] = t
    return out


def build_tp_model(cfg: ModelConfig, full_state_dict: dict, group=None) -> Qwen2Model:
    """Qwen2Model holding this rank's shard; its forward all-reduces after o_proj and down_proj over `group`."""
    group = group if group is not None else dist.group.WORLD
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    model = Qwen2Model(local_config(cfg, world), shard_state_dict(full_state_dict, cfg, rank, world))
    model.tp_group = group if world > 1 else None
    return model


def random_tp_model(shape_name: str, group=None, dtype=torch.bfloat16, device="cuda", seed: int = 0,
                    n_layers: int | None = None) -> Qwen2Model:
    """Random-init shard generated directly on the device (benchmarks of the large shapes: building the full matrices
    on the host first would take minutes). Each rank draws its own shard from seed + rank."""
    from nanoserve_b200.synthetic import SHAPES
    group = group if group is not None else dist.group.WORLD
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    L, H, NH, NKV, HD, I, V, tied = SHAPES[shape_name]
    L = n_layers or L
    cfg = ModelConfig(vocab_size=V, hidden_size=H, n_layers=L, n_heads=NH, n_kv_heads=NKV, head_dim=HD,
                      intermediate_size=I, rope_theta=1_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=tied)
    loc = local_config(cfg, world)
    g = torch.Generator(device=device).manual_seed(seed + rank)
    shared = torch.Generator(device=device).manual_seed(seed + 7919)      # replicated tensors: same on every rank

    def mat(gen, *shape):
        return (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * 0.02).to(dtype)

    sd = {"model.embed_tokens.weight": mat(shared, V, H), "model.norm.weight": torch.ones(H, dtype=dtype, device=device)}
    if not tied:
        sd["lm_head.weight"] = mat(shared, V, H)
    for i in range(L):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"] = torch.ones(H, dtype=dtype, device=device)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(H, dtype=dtype, device=device)
        sd[p + "self_attn.q_proj.weight"], sd[p + "self_attn.q_proj.bias"] = mat(g, loc.n_heads * HD, H), mat(g, loc.n_heads * HD)
        sd[p + "self_attn.k_proj.weight"], sd[p + "self_attn.k_proj.bias"] = mat(g, loc.n_kv_heads * HD, H), mat(g, loc.n_kv_heads * HD)
        sd[p + "self_attn.v_proj.weight"], sd[p + "self_attn.v_proj.bias"] = mat(g, loc.n_kv_heads * HD, H), mat(g, loc.n_kv_heads * HD)
        sd[p + "self_attn.o_proj.weight"] = mat(g, H, loc.n_heads * HD)
        sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"] = mat(g, loc.intermediate_size, H), mat(g, loc.intermediate_size, H)
        sd[p + "mlp.down_proj.weight"] = mat(g, H, loc.intermediate_size)
    model = Qwen2Model(loc, sd)
    model.tp_group = group if world > 1 else None
    return model
