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


class _DeviceBlock:
    """A library-owned device allocation seen by torch without a copy (`__cuda_array_interface__`)."""

    def __init__(self, ptr: int, shape: tuple, typestr: str):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 3, "strides": None}


class PeerReduce:
    """Peer-mapped partial buffers and flags for `ns_tp_allreduce_add_rmsnorm`: the all-reduce of a tensor-parallel layer
    fused with the residual add and the RMSNorm that follow it, over NVLink peer loads instead of an NCCL collective.

    Every rank allocates two partial buffers [max_rows, hidden] bf16 (used in turn from call to call), a flag word per
    peer and two state words, exports them, and maps every peer's. A GEMM writes its partial straight into
    `partial(k)`; `reduce_add_rmsnorm(k, rows, residual, weight, eps)` returns (h, x). Every rank must make the same
    sequence of calls with k alternating 0, 1, 0, 1 ... (two all-reduce sites per layer keep that true by themselves).
    Steps with more than max_rows token rows keep NCCL."""

    def __init__(self, group, hidden: int, max_rows: int, device):
        from nanoserve_b200 import _lib
        import ctypes
        self._lib, self._ct = _lib, ctypes
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.hidden, self.max_rows, self.device = hidden, max_rows, torch.device(device)
        lib = _lib.load()
        self.n_calls = 0
        with torch.cuda.device(self.device):
            buf_bytes = 2 * max_rows * hidden * 2
            ctrl_bytes = 256                                   # flags [world] uint32 at 0, state [2] uint32 at 128
            self._own = []
            ptrs = []
            for nbytes in (buf_bytes, ctrl_bytes):
                p = ctypes.c_void_p()
                _lib.call("ns_peer_alloc", nbytes, ctypes.byref(p))
                self._own.append(p.value)
                ptrs.append(p.value)
            self._buf_ptr, self._ctrl_ptr = ptrs
            handles = []
            for p in ptrs:
                h = ctypes.create_string_buffer(64)
                _lib.call("ns_peer_export", p, h)
                handles.append(bytes(h.raw))
            gathered = [None] * self.world
            dist.all_gather_object(gathered, handles, group=group)
            self._opened = []
            self.peer_buf, self.peer_ctrl = [0] * self.world, [0] * self.world
            for w, (hb, hc) in enumerate(gathered):
                if w == self.rank:
                    self.peer_buf[w], self.peer_ctrl[w] = self._buf_ptr, self._ctrl_ptr
                    continue
                for which, h in ((self.peer_buf, hb), (self.peer_ctrl, hc)):
                    p = ctypes.c_void_p()
                    _lib.call("ns_peer_open", ctypes.create_string_buffer(h, 64), ctypes.byref(p))
                    which[w] = p.value
                    self._opened.append(p.value)
            # torch views of this rank's own partial buffers: what the GEMMs write into
            self._partials = torch.as_tensor(_DeviceBlock(self._buf_ptr, (2, max_rows, hidden), "<i2"), device=self.device).view(torch.bfloat16)
            dist.barrier(group=group)                           # every mapping exists before the first call
        P = ctypes.c_void_p
        self._flag_args = (P * self.world)(*self.peer_ctrl)
        self._partial_args = [[(P * self.world)(*[b + k * max_rows * hidden * 2 for b in self.peer_buf]) for k in (0, 1)]]
        self._state_ptr = self._ctrl_ptr + 128

    def partial(self, k: int, rows: int) -> torch.Tensor:
        """This rank's k-th partial buffer, [rows, hidden]: the output of the GEMM before the all-reduce."""
        return self._partials[k, :rows]

    def reduce_add_rmsnorm(self, k: int, rows: int, residual: torch.Tensor, weight: torch.Tensor, eps: float):
        """(h, x): x = residual + sum over ranks of partial(k), h = weight * rmsnorm(x)."""
        h = torch.empty(rows, self.hidden, dtype=torch.bfloat16, device=self.device)
        x = torch.empty_like(h)
        self._lib.call("ns_tp_allreduce_add_rmsnorm", self._partial_args[0][k], self._flag_args, self._state_ptr,
                       residual.data_ptr(), weight.data_ptr(), h.data_ptr(), x.data_ptr(), rows, self.hidden, float(eps),
                       self.rank, self.world, self._lib.stream_ptr())
        return h, x

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (after a barrier: nobody may still be reading them)."""
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for p in self._opened:
                self._lib.call("ns_peer_close", p)
            dist.barrier(group=self.group)
            self._partials = None
            for p in self._own:
                self._lib.call("ns_peer_free", p)
        self._own = None


def enable_fused_allreduce(model: Qwen2Model, max_rows: int = 256) -> PeerReduce | None:
    """Give a tensor-parallel model the fused all-reduce + add + RMSNorm path for steps of at most max_rows token rows
    (bf16 only). Returns the PeerReduce it now owns, or None when the model is not tensor parallel."""
    if model.tp_group is None or model.dtype != torch.bfloat16:
        return None
    model.tp_peer = PeerReduce(model.tp_group, model.cfg.hidden_size, max_rows, model.device)
    return model.tp_peer
