"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

They stand in for the reference's prompt set and Hugging Face checkpoints, which cannot be downloaded where
this code runs: weights are random-init N(0, 0.02) (RMSNorm scales 1.0), prompt token ids are uniform over the
vocabulary, lengths are drawn from the stated uniform ranges.
"""
from __future__ import annotations

import random
from dataclasses import dataclass

import torch

# (n_layers, hidden, n_heads, n_kv_heads, head_dim, intermediate, vocab, tied)
SHAPES = {
    "qwen2.5-0.5b": (24, 896, 14, 2, 64, 4864, 151936, True),
    "qwen2.5-1.5b": (28, 1536, 12, 2, 128, 8960, 151936, True),
    "qwen2.5-7b": (28, 3584, 28, 4, 128, 18944, 152064, False),
    # one rank's shard of the 7B shape under tensor parallelism by KV head (hidden size unchanged): for single-GPU
    # measurements of a shard's kernels, without the all-reduces
    "qwen2.5-7b-tp2": (28, 3584, 14, 2, 128, 9472, 152064, False),
    "qwen2.5-7b-tp4": (28, 3584, 7, 1, 128, 4736, 152064, False),
}


@dataclass
class AttentionWorkload:
    """One op-level step: a mixed batch over one layer's paged pool (all tensors on `device`)."""
    q: torch.Tensor              # [N, n_heads, hd]
    k_new: torch.Tensor          # [N, n_kv, hd]   this step's keys (to be written through slot_mapping)
    v_new: torch.Tensor
    k_pool: torch.Tensor         # [num_blocks, 16, n_kv, hd]
    v_pool: torch.Tensor
    block_tables: torch.Tensor   # int32 [S, W]
    seq_lens: torch.Tensor       # int32 [S]  context + new tokens
    cu_seqlens: torch.Tensor     # int32 [S+1]
    slot_mapping: torch.Tensor   # int64 [N]
    scale: float
    n_decode: int
    kv_tokens: int               # sum of seq_lens
    decode_kv_tokens: int        # sum of seq_lens over the decode rows

    def decode_bytes(self) -> int:
        """Algorithmic bytes of the decode rows for one layer: K+V of every context token, Q in, O out,
        the block-table entries and the lengths."""
        nkv, hd = self.k_pool.shape[2:]
        e = self.k_pool.element_size()
        nh = self.q.shape[1]
        bs = self.k_pool.shape[1]
        lens = self.seq_lens[:self.n_decode].tolist()
        return (self.decode_kv_tokens * 2 * nkv * hd * e + 2 * self.n_decode * nh * hd * e
                + sum(-(-L // bs) for L in lens) * 4 + self.n_decode * 4)

    def prefill_flops(self) -> float:
        """4 * n_heads * hd * sum over prefill queries of the keys each one sees."""
        nh, hd = self.q.shape[1:]
        cu, lens = self.cu_seqlens.tolist(), self.seq_lens.tolist()
        total = 0
        for s in range(self.n_decode, len(lens)):
            T = cu[s + 1] - cu[s]
            ctx = lens[s] - T
            total += T * ctx + T * (T + 1) // 2
        return 4.0 * nh * hd * total


def attention_workload(n_decode: int = 48, decode_range=(128, 8192), n_prefill: int = 4, chunk: int = 512,
                       prefill_ctx_range=(0, 2048), n_heads: int = 14, n_kv_heads: int = 2, head_dim: int = 64,
                       num_blocks: int = 65536, block_size: int = 16, dtype=torch.bfloat16, device="cuda",
                       seed: int = 0) -> AttentionWorkload:
    """benchmark configuration 1: decode rows with context lengths uniform in decode_range (the new token included) plus
    prefill chunks of `chunk` new tokens on top of a cached context uniform in prefill_ctx_range. Block tables
    are consecutive slices of a seeded random permutation of the pool; Q/K/V are N(0,1); scale 1/sqrt(hd)."""
    rng = random.Random(seed)
    dec_lens = [rng.randint(*decode_range) for _ in range(n_decode)]
    pre_ctx = [rng.randint(*prefill_ctx_range) for _ in range(n_prefill)]
    lens = dec_lens + [c + chunk for c in pre_ctx]
    q_lens = [1] * n_decode + [chunk] * n_prefill
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_blocks, generator=g)
    nbs = [-(-L // block_size) for L in lens]
    if sum(nbs) > num_blocks:
        raise ValueError("pool too small for the drawn lengths")
    W = max(nbs)
    tables = torch.zeros(len(lens), W, dtype=torch.int32)
    slots, used = [], 0
    for s, (L, T, nb) in enumerate(zip(lens, q_lens, nbs)):
        row = perm[used:used + nb]
        tables[s, :nb] = row.int()
        used += nb
        pos = torch.arange(L - T, L)
        slots.append(row[pos // block_size] * block_size + pos % block_size)
    slot_mapping = torch.cat(slots).to(torch.int64)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    N = int(cu[-1])
    dg = torch.Generator(device=device).manual_seed(seed)
    shape = (num_blocks, block_size, n_kv_heads, head_dim)
    k_pool = torch.randn(shape, generator=dg, device=device, dtype=torch.float32).to(dtype)
    v_pool = torch.randn(shape, generator=dg, device=device, dtype=torch.float32).to(dtype)
    q = torch.randn(N, n_heads, head_dim, generator=dg, device=device).to(dtype)
    k_new = torch.randn(N, n_kv_heads, head_dim, generator=dg, device=device).to(dtype)
    v_new = torch.randn(N, n_kv_heads, head_dim, generator=dg, device=device).to(dtype)
    return AttentionWorkload(q=q, k_new=k_new, v_new=v_new, k_pool=k_pool, v_pool=v_pool,
                             block_tables=tables.to(device), seq_lens=torch.tensor(lens, dtype=torch.int32, device=device),
                             cu_seqlens=cu.to(device), slot_mapping=slot_mapping.to(device), scale=head_dim ** -0.5,
                             n_decode=n_decode, kv_tokens=sum(lens), decode_kv_tokens=sum(dec_lens))


def random_state_dict(shape_name: str, dtype=torch.bfloat16, device="cpu", seed: int = 0, n_layers: int | None = None,
                      vocab: int | None = None) -> tuple[dict, dict]:
    """Random-init weights of a Qwen2.5 architecture in Hugging Face naming: every matrix and bias N(0, 0.02)
    drawn in fp32 from torch.Generator().manual_seed(seed) in state-dict order, RMSNorm scales 1.0; returned in
    `dtype` on `device`, together with the config dict. n_layers / vocab can shrink the model for tests."""
    L, H, NH, NKV, HD, I, V, tied = SHAPES[shape_name]
    L = n_layers or L
    V = vocab or V
    g = torch.Generator().manual_seed(seed)

    def mat(*shape):
        return (torch.randn(*shape, generator=g, dtype=torch.float32) * 0.02).to(dtype).to(device)

    sd = {"model.embed_tokens.weight": mat(V, H)}
    for i in range(L):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"] = torch.ones(H, dtype=dtype, device=device)
        sd[p + "self_attn.q_proj.weight"] = mat(NH * HD, H)
        sd[p + "self_attn.q_proj.bias"] = mat(NH * HD)
        sd[p + "self_attn.k_proj.weight"] = mat(NKV * HD, H)
        sd[p + "self_attn.k_proj.bias"] = mat(NKV * HD)
        sd[p + "self_attn.v_proj.weight"] = mat(NKV * HD, H)
        sd[p + "self_attn.v_proj.bias"] = mat(NKV * HD)
        sd[p + "self_attn.o_proj.weight"] = mat(H, NH * HD)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(H, dtype=dtype, device=device)
        sd[p + "mlp.gate_proj.weight"] = mat(I, H)
        sd[p + "mlp.up_proj.weight"] = mat(I, H)
        sd[p + "mlp.down_proj.weight"] = mat(H, I)
    sd["model.norm.weight"] = torch.ones(H, dtype=dtype, device=device)
    if not tied:
        sd["lm_head.weight"] = mat(V, H)
    cfg = dict(vocab_size=V, hidden_size=H, n_layers=L, n_heads=NH, n_kv_heads=NKV, head_dim=HD, intermediate_size=I,
               rope_theta=1_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=tied)
    return sd, cfg


def serving_requests(n: int, prompt_range=(64, 1024), output_range=(16, 256), vocab: int = 151936, seed: int = 0,
                     shared_prefix: int = 0):
    """[(prompt_ids, max_new_tokens)] with prompt lengths and output lengths from separate seeded streams
    (the reference's harness draws lengths from its own RNG: bench/prompts.py:49,58). shared_prefix > 0
    prepends one seeded common prefix of that many tokens to every prompt (prefix-caching workload)."""
    rp, ro = random.Random(seed), random.Random(seed + 1)
    rprefix = random.Random(424242)              # the shared prefix does not depend on `seed`: new suffixes, same prefix
    prefix = [rprefix.randrange(vocab) for _ in range(shared_prefix)]
    reqs = []
    for _ in range(n):
        plen = rp.randint(*prompt_range)
        reqs.append((prefix + [rp.randrange(vocab) for _ in range(plen)], ro.randint(*output_range)))
    return reqs
