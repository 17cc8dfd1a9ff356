"""Qwen2 forward pass over plain tensors, B200 path.

Same class and method names as the reference model (nanoserve/model.py:26-367): `ModelConfig`, `LayerWeights`,
`SeqInput`, `DecodeMeta`, `Qwen2Model` with `_pre` / `_attend` / `_post` / `forward_batch` / `lm_head_rows` /
`rope` / `final_norm` / `with_fused_ops`. What differs is below the method boundary:

  * the GEMMs stay `F.linear` (cuBLAS); every other device op is a kernel of libnanoserve_b200.so;
  * attention is ONE ragged call per layer for the whole mixed batch (decode rows and prefill chunks), reading
    K/V from the paged pool only, instead of one Triton launch plus a Python loop of SDPA calls
    (nanoserve/model.py:274-322);
  * `forward_step` is the engine's path: all metadata (token ids, positions, slot mapping, cu_seqlens, seq_lens,
    block-table rows) already sits in device buffers built by a kernel, so a whole mixed step is graph-capturable;
  * the residual add after the MLP is fused into the next layer's RMSNorm (same rounding: the sum is rounded to
    the dtype, then normalised).

There is no CPU path: weights must be CUDA tensors.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class ModelConfig:
    vocab_size: int
    hidden_size: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    intermediate_size: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool

    @classmethod
    def from_hf_config(cls, d: dict) -> "ModelConfig":
        theta = d.get("rope_theta") or (d.get("rope_parameters") or {}).get("rope_theta")
        return cls(vocab_size=d["vocab_size"], hidden_size=d["hidden_size"], n_layers=d["num_hidden_layers"],
                   n_heads=d["num_attention_heads"], n_kv_heads=d["num_key_value_heads"],
                   head_dim=d.get("head_dim") or d["hidden_size"] // d["num_attention_heads"],
                   intermediate_size=d["intermediate_size"], rope_theta=float(theta),
                   rms_norm_eps=d["rms_norm_eps"], tie_word_embeddings=d.get("tie_word_embeddings", False))

    def kv_bytes_per_token(self, dtype: torch.dtype) -> int:
        return self.n_layers * 2 * self.n_kv_heads * self.head_dim * torch.finfo(dtype).bits // 8


_HF_LAYER_NAMES = {
    "ln1": "input_layernorm.weight",
    "q_w": "self_attn.q_proj.weight", "q_b": "self_attn.q_proj.bias",
    "k_w": "self_attn.k_proj.weight", "k_b": "self_attn.k_proj.bias",
    "v_w": "self_attn.v_proj.weight", "v_b": "self_attn.v_proj.bias",
    "o_w": "self_attn.o_proj.weight",
    "ln2": "post_attention_layernorm.weight",
    "gate_w": "mlp.gate_proj.weight", "up_w": "mlp.up_proj.weight", "down_w": "mlp.down_proj.weight",
}


@dataclass
class LayerWeights:
    ln1: torch.Tensor
    q_w: torch.Tensor
    q_b: torch.Tensor
    k_w: torch.Tensor
    k_b: torch.Tensor
    v_w: torch.Tensor
    v_b: torch.Tensor
    o_w: torch.Tensor
    ln2: torch.Tensor
    gate_w: torch.Tensor
    up_w: torch.Tensor
    down_w: torch.Tensor
    qkv_w: torch.Tensor | None = None       # merged [q; k; v] rows (one GEMM); the fields above become views
    qkv_b: torch.Tensor | None = None
    gate_up_w: torch.Tensor | None = None   # merged [gate; up] rows

    HF_NAMES = _HF_LAYER_NAMES

    @classmethod
    def from_state_dict(cls, sd: dict, i: int) -> "LayerWeights":
        return cls(**{name: sd[f"model.layers.{i}.{hf}"] for name, hf in _HF_LAYER_NAMES.items()})

    def merge(self) -> None:
        """Concatenate Q/K/V and gate/up once and re-point the per-matrix fields at row views of the result, so
        nothing is stored twice (nanoserve/model.py:101-114)."""
        if self.qkv_w is not None:
            return
        nq, nk, ng = self.q_w.shape[0], self.k_w.shape[0], self.gate_w.shape[0]
        self.qkv_w = torch.cat((self.q_w, self.k_w, self.v_w))
        self.qkv_b = torch.cat((self.q_b, self.k_b, self.v_b))
        self.gate_up_w = torch.cat((self.gate_w, self.up_w))
        self.q_w, self.k_w, self.v_w = self.qkv_w[:nq], self.qkv_w[nq:nq + nk], self.qkv_w[nq + nk:]
        self.q_b, self.k_b, self.v_b = self.qkv_b[:nq], self.qkv_b[nq:nq + nk], self.qkv_b[nq + nk:]
        self.gate_w, self.up_w = self.gate_up_w[:ng], self.gate_up_w[ng:]


@dataclass
class SeqInput:
    """One sequence's slice of a batched step (nanoserve/model.py:117-129). block_table may be a list of ints or
    an int tensor."""
    n_tokens: int
    cache: object | None = None
    block_table: object | None = None
    ctx_len: int = 0
    use_kernel: bool = False


@dataclass
class DecodeMeta:
    """Kernel inputs of the one-token decodes of a step (nanoserve/model.py:132-137)."""
    token_idx: torch.Tensor
    block_tables: torch.Tensor
    context_lens: torch.Tensor


@dataclass
class StepMeta:
    """Device-resident description of one step, as the metadata kernel leaves it (views into static buffers)."""
    tokens: torch.Tensor          # int64 [T]
    positions: torch.Tensor       # int64 [T]
    slot_mapping: torch.Tensor    # int64 [T]
    cu_seqlens: torch.Tensor      # int32 [S+1]
    seq_lens: torch.Tensor        # int32 [S]
    table_rows: torch.Tensor | None   # int32 [S] rows of block_tables (None: row s)
    block_tables: torch.Tensor    # int32 [rows, W]
    last_rows: torch.Tensor       # int64 [S] flattened row of each sequence's last token
    n_seqs: int
    workspace: object             # AttnWorkspace
    decode_only: bool = False     # every sequence has exactly one token


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Unfused RMSNorm in framework ops (nanoserve/model.py:140-146); the fused path uses kernels.fused.rms_norm."""
    xf = x.to(torch.float32)
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return weight * xf.to(x.dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


class Qwen2Model:
    """Weights + forward over plain tensors. `fused` (set by with_fused_ops) selects the kernel path for the
    token-wise ops; attention always runs on the ragged paged kernel."""

    fused = False
    skinny_gemms = True      # decode-sized steps: narrow GEMMs through the weight-streaming kernel (False = library GEMMs)
    tp_group = None          # torch.distributed process group when the model is one tensor-parallel shard
    _plan_streams: dict = {}  # one side stream per device for the attention plan (shared by every model)
    tp_size = 1
    tp_peer = None           # tensor_parallel.PeerReduce: fused all-reduce + add + RMSNorm over peer memory (small steps)

    def __init__(self, cfg: ModelConfig, state_dict: dict[str, torch.Tensor]):
        self.cfg = cfg
        self.embed = state_dict["model.embed_tokens.weight"]
        if not self.embed.is_cuda:
            raise ValueError("nanoserve_b200 runs on CUDA tensors only: move the weights to a GPU "
                             "(the CPU restatement used for parity checks lives in oracle/)")
        self.norm = state_dict["model.norm.weight"]
        self.lm_head = self.embed if cfg.tie_word_embeddings else state_dict["lm_head.weight"]
        self.layers = [LayerWeights.from_state_dict(state_dict, i) for i in range(cfg.n_layers)]
        self.device = self.embed.device
        self.dtype = self.embed.dtype
        # RoPE inverse frequencies in fp32, computed on the CPU like the reference (nanoserve/model.py:168)
        inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float) / cfg.head_dim))
        self.inv_freq = inv_freq.to(self.device)

    # ---- variants -----------------------------------------------------------------------------------------------
    def with_fused_ops(self) -> "Qwen2Model":
        """The same weights (merged in place, per-matrix names become views) behind the fused-kernel path."""
        for layer in self.layers:
            layer.merge()
        m = copy.copy(self)
        m.fused = True
        return m

    def named_weights(self) -> dict[str, torch.Tensor]:
        out = {"model.embed_tokens.weight": self.embed, "model.norm.weight": self.norm}
        if not self.cfg.tie_word_embeddings:
            out["lm_head.weight"] = self.lm_head
        for i, layer in enumerate(self.layers):
            for name, hf in _HF_LAYER_NAMES.items():
                out[f"model.layers.{i}.{hf}"] = getattr(layer, name)
        return out

    def _all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.tp_group is not None:
            torch.distributed.all_reduce(t, group=self.tp_group)
        return t

    # ---- token-wise pieces ------------------------------------------------------------------------------------
    def rope(self, positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """cos/sin [1, T, head_dim] in the model dtype for int64 positions [T]."""
        if self.fused:
            from nanoserve_b200.kernels.fused import rope_cos_sin
            cos, sin = rope_cos_sin(positions.contiguous(), self.inv_freq, self.cfg.head_dim, self.dtype)
            return cos[None], sin[None]
        freqs = positions[None, :, None].float() * self.inv_freq
        emb = torch.cat((freqs, freqs), dim=-1)
        return emb.cos().to(self.dtype), emb.sin().to(self.dtype)

    def final_norm(self, x: torch.Tensor) -> torch.Tensor:
        if self.fused:
            from nanoserve_b200.kernels.fused import rms_norm as fused_rms_norm
            return fused_rms_norm(x, self.norm, self.cfg.rms_norm_eps)
        return rms_norm(x, self.norm, self.cfg.rms_norm_eps)

    def _pre(self, i: int, x: torch.Tensor, cos, sin, paged=None, slot_mapping=None, dense_kv: bool = True):
        """RMSNorm, Q/K/V projection, RoPE, KV write of layer i. x: [1, N, hidden] -> q [1, N, n_heads, hd] and
        k, v [1, N, n_kv_heads, hd] (None when dense_kv is off)."""
        layer, cfg = self.layers[i], self.cfg
        if self.fused:
            from nanoserve_b200.kernels.fused import rms_norm as fused_rms_norm
            return self._qkv_rope(i, fused_rms_norm(x, layer.ln1, cfg.rms_norm_eps), cos, sin, paged, slot_mapping,
                                  dense_kv)
        h = rms_norm(x, layer.ln1, cfg.rms_norm_eps)
        N, hd = h.shape[1], cfg.head_dim
        q = F.linear(h, layer.q_w, layer.q_b).view(1, N, -1, hd)
        k = F.linear(h, layer.k_w, layer.k_b).view(1, N, -1, hd)
        v = F.linear(h, layer.v_w, layer.v_b).view(1, N, -1, hd)
        c, s = cos.unsqueeze(2), sin.unsqueeze(2)
        q = q * c + rotate_half(q) * s
        k = k * c + rotate_half(k) * s
        if paged is not None:
            paged.write(i, k[0], v[0], slot_mapping)
        return q, k, v

    def _qkv_rope(self, i: int, h: torch.Tensor, cos, sin, paged, slot_mapping, dense_kv: bool):
        from nanoserve_b200.kernels.fused import rope_qkv
        layer, cfg = self.layers[i], self.cfg
        qkv = F.linear(h, layer.qkv_w, layer.qkv_b)[0]
        q, k, v = rope_qkv(qkv, cos[0], sin[0], cfg.n_heads // self.tp_size, cfg.n_kv_heads // self.tp_size,
                           cfg.head_dim, paged.k[i] if paged is not None else None,
                           paged.v[i] if paged is not None else None, slot_mapping, dense_kv=dense_kv)
        return q[None], (k[None] if k is not None else None), (v[None] if v is not None else None)

    def _post(self, i: int, x: torch.Tensor, o: torch.Tensor) -> torch.Tensor:
        """Output projection + residual, RMSNorm, SwiGLU MLP + residual of layer i."""
        layer, eps = self.layers[i], self.cfg.rms_norm_eps
        if self.fused:
            from nanoserve_b200.kernels.fused import rms_norm as fused_rms_norm, silu_mul
            h, x = fused_rms_norm(self._all_reduce(F.linear(o, layer.o_w)), layer.ln2, eps, residual=x)
            return x + self._all_reduce(F.linear(silu_mul(F.linear(h, layer.gate_up_w)), layer.down_w))
        x = x + self._all_reduce(F.linear(o, layer.o_w))
        h = rms_norm(x, layer.ln2, eps)
        return x + self._all_reduce(F.linear(F.silu(F.linear(h, layer.gate_w)) * F.linear(h, layer.up_w), layer.down_w))

    # ---- attention ----------------------------------------------------------------------------------------------
    def _ragged_meta(self, seqs: list[SeqInput], paged, decode_meta: DecodeMeta | None):
        """Varlen metadata for the reference-style call (host SeqInput list): cu_seqlens, seq_lens and a padded
        block-table tensor. Decode rows may carry their tables in decode_meta instead of in SeqInput."""
        dev = self.device
        q_lens = [s.n_tokens for s in seqs]
        lens = [s.ctx_len + s.n_tokens for s in seqs]
        tables: list = []
        d = 0
        for s in seqs:
            bt = s.block_table
            if bt is None and s.use_kernel and decode_meta is not None:
                bt = decode_meta.block_tables[d]
                d += 1
            elif s.use_kernel and decode_meta is not None:
                d += 1
            tables.append(bt)
        bs = paged.block_size
        width = max(-(-L // bs) for L in lens)
        rows = torch.zeros(len(seqs), width, dtype=torch.int32, device=dev)
        for r, (bt, L) in enumerate(zip(tables, lens)):
            nb = -(-L // bs)
            if bt is None:
                raise ValueError("a sequence with cached context needs its block table")
            bt = torch.as_tensor(bt, device=dev)[:nb]
            rows[r, :bt.shape[0]] = bt.to(torch.int32)
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
        return rows, torch.tensor(lens, dtype=torch.int32, device=dev), cu

    def _attend(self, i: int, q, k, v, seqs: list[SeqInput], paged=None, decode_meta=None,
                out: torch.Tensor | None = None, _meta=None) -> torch.Tensor:
        """Attention of layer i for every sequence of the step in one ragged kernel call. q: [1, N, heads, hd];
        K/V are read from the paged pool (already written by _pre), so k and v are unused. Returns
        [1, N, n_heads*hd] (written into `out` if given)."""
        if paged is None:
            raise NotImplementedError("attention reads K/V from the paged pool: pass paged= (no contiguous cache)")
        from nanoserve_b200.kernels.paged_attention import ragged_paged_attention
        tables, lens, cu = _meta if _meta is not None else self._ragged_meta(seqs, paged, decode_meta)
        N, nh, hd = q.shape[1], q.shape[2], q.shape[3]
        o = None if out is None else out[0].view(N, nh, hd)
        o = ragged_paged_attention(q[0], paged.k[i], paged.v[i], tables, lens, cu, hd ** -0.5, out=o)
        return o.view(1, N, nh * hd)

    @torch.inference_mode()
    def forward_batch(self, token_ids: torch.Tensor, positions: torch.Tensor, seqs: list[SeqInput],
                      logits="last", paged=None, slot_mapping: torch.Tensor | None = None,
                      decode_meta: DecodeMeta | None = None) -> torch.Tensor:
        """Reference-style entry (nanoserve/model.py:325-349): metadata comes as host objects. Returns logits
        [len(seqs), vocab] ("last"), [N, vocab] ("all") or the rows of an index tensor."""
        if paged is None:
            raise NotImplementedError("forward_batch needs the paged KV pool (paged=, slot_mapping=)")
        assert sum(s.n_tokens for s in seqs) == token_ids.shape[0], "seqs must cover token_ids exactly"
        meta = self._ragged_meta(seqs, paged, decode_meta)
        x = F.embedding(token_ids, self.embed)[None]
        cos, sin = self.rope(positions)
        for i in range(self.cfg.n_layers):
            q, k, v = self._pre(i, x, cos, sin, paged, slot_mapping)
            x = self._post(i, x, self._attend(i, q, k, v, seqs, paged, decode_meta, _meta=meta))
        return self.lm_head_rows(self.final_norm(x), seqs, logits)

    def lm_head_rows(self, x: torch.Tensor, seqs: list[SeqInput], logits="last") -> torch.Tensor:
        if isinstance(logits, torch.Tensor):
            x = x[:, logits, :]
        elif logits == "last":
            if len(seqs) == 1:
                x = x[:, -1:, :]
            else:
                ends = torch.tensor([s.n_tokens for s in seqs], device=x.device).cumsum(0) - 1
                x = x[:, ends, :]
        return F.linear(x, self.lm_head)[0]

    # ---- the engine's path: metadata already on the device -------------------------------------------------------
    @torch.inference_mode()
    def forward_step(self, meta: StepMeta, paged, plan: bool = True) -> torch.Tensor:
        """One step over device-resident metadata (graph-capturable). Returns logits [n_seqs, vocab] of each
        sequence's last token. Fused path only."""
        if not self.fused:
            raise NotImplementedError("forward_step is the fused-kernel path: use model.with_fused_ops()")
        from nanoserve_b200.kernels.fused import (EPI_ROPE_KV, EPI_SILU_MUL, SKINNY_MAX_ROWS, rms_norm as norm, rope_cos_sin, skinny_gemm_fits,
                                                  rope_qkv, silu_mul, skinny_gemm, stream_gemm, stream_gemm_supported, swiglu_gemm,
                                                  sm_count, swiglu_gemm_supported, thin_gemm, thin_gemm_ctas, thin_gemm_supported, thin_swiglu_gemm,
                                                  thin_swiglu_gemm_supported, thin_gemm_residual, thin_swiglu_gemm_norm,
                                                  thin_swiglu_gemm_norm_supported)
        from nanoserve_b200.kernels.paged_attention import ragged_paged_attention
        cfg, eps = self.cfg, self.cfg.rms_norm_eps
        nh, nkv, hd = cfg.n_heads // self.tp_size, cfg.n_kv_heads // self.tp_size, cfg.head_dim
        T = meta.tokens.shape[0]
        cu = None if meta.decode_only else meta.cu_seqlens
        # Decode-sized steps (at most SKINNY_MAX_ROWS token rows, bf16): a GEMM is a weight read behind a dependency, and
        # this library's own kernels can request their weights while the preceding kernel still runs (programmatic
        # dependent launch). Larger steps keep F.linear everywhere.
        inter = self.layers[0].down_w.shape[1]
        skinny = self.dtype == torch.bfloat16 and T <= SKINNY_MAX_ROWS and self.skinny_gemms
        # down_proj on the split-K cluster kernel where its K slice fits shared memory; slices above 1024 columns (1.5B shape:
        # 1120) only up to 16 rows - at 32 rows the library GEMM is faster there (28-layer decode step 1,661 vs 1,739 us;
        # at 16 rows 1,491 vs 1,462)
        skinny_down = skinny and inter % 128 == 0 and skinny_gemm_fits(T, inter) and (inter // 8 <= 1024 or T <= 16)
        hidden = cfg.hidden_size
        import os
        # Which kernel serves which GEMM is a bit mask (NS_SKINNY_MASK; NS_SKINNY_MASK_SMALL for steps of at most 16 rows):
        #   bit 0 down_proj, 1 QKV (+RoPE, KV write), 2 o_proj on the split-K cluster kernel (ns_skinny_gemm);
        #   bit 3 gate/up + SiLU*mul, 4 o_proj on the persistent streaming kernel (ns_stream_gemm);
        #   bit 5 gate/up + SiLU*mul on the tcgen05 + TMA kernel (ns_swiglu_gemm; measured slower, never a default);
        #   bit 6 QKV (+RoPE, KV write), 7 o_proj on the 8-row-tile kernel without split-K (ns_thin_gemm; wins over bits
        #         1, 2 and 4), bit 8 gate/up + SiLU*mul on the same construction (ns_thin_swiglu_gemm, up to 32 rows).
        #   bit 9 (with bits 7 and 8): the residual add in o_proj's epilogue and the RMSNorm in gate/up's prologue
        #         (ns_thin_gemm_residual + ns_thin_swiglu_gemm_norm) instead of the add + RMSNorm kernel between them.
        # Defaults from measurements of whole decode steps: up to 4 rows the streaming kernel for gate/up and o_proj's
        # 8-row-tile kernel (219); 5..16 rows the 8-row-tile kernels everywhere with the norm folded in, the streaming kernel
        # where a shape does not fit them (987); 17..32 rows
        # the same without the fold, which gains nothing there (451); down_proj on the split-K kernel throughout; a GEMM
        # whose kernel does not take the step's shape falls back to the next choice and finally to F.linear.
        # (decode steps of 24 layers at 1 / 4 / 8 / 16 / 32 rows: 664 / 670 / 687 / 735 / - us with 219, 675 / 679 / 681 / 711 / 785
        # with 451, 703 at 16 and 784 at 32 rows with 963)
        if T <= 4:
            mask = int(os.environ.get("NS_SKINNY_MASK_SMALL", os.environ.get("NS_SKINNY_MASK", "219")))
        elif T <= 16:
            mask = int(os.environ.get("NS_SKINNY_MASK_SMALL", os.environ.get("NS_SKINNY_MASK", "987")))
        else:
            mask = int(os.environ.get("NS_SKINNY_MASK", "451"))
        skinny_down = skinny_down and bool(mask & 1)
        skinny_qkv = skinny and hd == 64 and hidden % 128 == 0 and bool(mask & 2)
        skinny_o = skinny and (nh * hd) % 128 == 0 and bool(mask & 4)
        # gate/up (+SiLU*mul) and o_proj through the persistent weight-streaming kernel: its weights are in flight while
        # the norm / attention kernel before it still runs
        stream_gu = skinny and bool(mask & 8) and stream_gemm_supported(T, 2 * inter, hidden)
        stream_o = skinny and bool(mask & 16) and stream_gemm_supported(T, hidden, nh * hd)
        umma_gu = skinny and bool(mask & 32) and swiglu_gemm_supported(T, inter, hidden)     # tcgen05 + TMA (off: slower)
        # (only where its CTAs - one per 8 weight rows, or per 16 - are one wave of the SMs)
        thin_qkv = (skinny and hd in (64, 128) and bool(mask & 64) and thin_gemm_ctas((nh + 2 * nkv) * hd) <= sm_count() and
                    thin_gemm_supported(T, (nh + 2 * nkv) * hd, hidden))
        thin_o = (skinny and bool(mask & 128) and thin_gemm_ctas(hidden) <= sm_count() and (nh * hd) % 128 == 0 and
                  thin_gemm_supported(T, hidden, nh * hd))
        thin_gu = skinny and bool(mask & 256) and thin_swiglu_gemm_supported(T, inter, hidden)      # bit 8: gate/up + SiLU*mul
        # bit 9: where both o_proj and gate/up run on the 8-row-tile kernels, the residual add moves into o_proj's epilogue
        # and the RMSNorm into gate/up's prologue (one kernel and one launch boundary less per layer); not with tensor
        # parallelism, whose all-reduce sits between the two
        fold_norm = (thin_o and thin_gu and bool(mask & 512) and self.tp_group is None and
                     thin_swiglu_gemm_norm_supported(T, inter, hidden))
        # The attention plan (one CTA, ~14 us) depends only on the step metadata and is first needed by layer 0's
        # attention: it runs on a second stream next to the RoPE tables, the embedding, the first norm and the first QKV
        # GEMM (inside a capture this becomes a fork and a join in the graph).
        # tensor parallel, small steps: the two all-reduces of a layer are fused with the add + RMSNorm after them and
        # read the peers' partials over NVLink (tensor_parallel.PeerReduce); larger steps use the NCCL all-reduce
        peer = self.tp_peer if (self.tp_peer is not None and self.tp_group is not None and T <= self.tp_peer.max_rows) else None
        plan_stream = None
        if plan:
            main = torch.cuda.current_stream()
            plan_stream = Qwen2Model._plan_streams.get(self.device)
            if plan_stream is None:
                plan_stream = Qwen2Model._plan_streams[self.device] = torch.cuda.Stream(device=self.device)
            plan_stream.wait_stream(main)
            with torch.cuda.stream(plan_stream):
                meta.workspace.plan(meta.seq_lens, cu, meta.n_seqs, paged.block_size, meta.table_rows)
        cos, sin = rope_cos_sin(meta.positions, self.inv_freq, hd, self.dtype)
        x = F.embedding(meta.tokens, self.embed)
        h = norm(x, self.layers[0].ln1, eps)
        scale = hd ** -0.5
        for i, layer in enumerate(self.layers):
            if thin_qkv:
                q = thin_gemm(h, layer.qkv_w, layer.qkv_b, epilogue=EPI_ROPE_KV, cos=cos, sin=sin, k_cache=paged.k[i],
                              v_cache=paged.v[i], slots=meta.slot_mapping, n_heads=nh, n_kv_heads=nkv)
            elif skinny_qkv:
                q = skinny_gemm(h, layer.qkv_w, layer.qkv_b, split_k=8, epilogue=EPI_ROPE_KV, cos=cos, sin=sin,
                                k_cache=paged.k[i], v_cache=paged.v[i], slots=meta.slot_mapping, n_heads=nh, n_kv_heads=nkv)
            else:
                qkv = F.linear(h, layer.qkv_w, layer.qkv_b)
                q, _, _ = rope_qkv(qkv, cos, sin, nh, nkv, hd, paged.k[i], paged.v[i], meta.slot_mapping, dense_kv=False)
            if plan_stream is not None:
                torch.cuda.current_stream().wait_stream(plan_stream)          # join: the plan is complete from here on
                plan_stream = None
            o = ragged_paged_attention(q, paged.k[i], paged.v[i], meta.block_tables, meta.seq_lens, cu, scale,
                                       n_seqs=meta.n_seqs, table_rows=meta.table_rows, workspace=meta.workspace,
                                       planned=True)
            o2 = o.view(T, nh * hd)
            if fold_norm:
                x, ss = thin_gemm_residual(o2, layer.o_w, x)
                m = thin_swiglu_gemm_norm(x, ss, layer.ln2, eps, layer.gate_up_w)
            elif thin_o:
                a = thin_gemm(o2, layer.o_w)
            elif stream_o:
                a = stream_gemm(o2, layer.o_w)
            elif skinny_o:
                a = skinny_gemm(o2, layer.o_w, split_k=8)
            elif peer is not None:
                a = None                                    # the library GEMM writes its partial where the peers read it
                torch.matmul(o2, layer.o_w.t(), out=peer.partial(0, T))
                h, x = peer.reduce_add_rmsnorm(0, T, x, layer.ln2, eps)
            else:
                a = F.linear(o2, layer.o_w)
            if fold_norm or (peer is not None and a is None):
                pass
            elif peer is not None:
                peer.partial(0, T).copy_(a)                 # (a GEMM kernel of this library: its output is copied over)
                h, x = peer.reduce_add_rmsnorm(0, T, x, layer.ln2, eps)
            else:
                a = self._all_reduce(a)
                h, x = norm(a, layer.ln2, eps, residual=x)
            if fold_norm:
                pass
            elif thin_gu:
                m = thin_swiglu_gemm(h, layer.gate_up_w)
            elif umma_gu:
                m = swiglu_gemm(h, layer.gate_up_w)
            elif stream_gu:
                m = stream_gemm(h, layer.gate_up_w, epilogue=EPI_SILU_MUL)
            else:
                m = silu_mul(F.linear(h, layer.gate_up_w))
            nxt = self.layers[i + 1].ln1 if i + 1 < len(self.layers) else self.norm
            if peer is not None:
                if skinny_down:
                    peer.partial(1, T).copy_(skinny_gemm(m, layer.down_w, split_k=8))
                else:
                    torch.matmul(m, layer.down_w.t(), out=peer.partial(1, T))
                h, x = peer.reduce_add_rmsnorm(1, T, x, nxt, eps)
            else:
                d = self._all_reduce(skinny_gemm(m, layer.down_w, split_k=8) if skinny_down else F.linear(m, layer.down_w))
                h, x = norm(d, nxt, eps, residual=x)      # x + mlp, then the next layer's (or the final) norm
        return F.linear(h.index_select(0, meta.last_rows), self.lm_head)
