"""Ragged paged attention on sm_100a.

`paged_attention_decode` keeps the name and signature of the reference's Triton wrapper
(nanoserve/kernels/paged_attention.py:85-105). `ragged_paged_attention` is the single call that replaces the
whole of nanoserve/model.py:262-323 (`Qwen2Model._attend`): decode rows and prefill chunks of a mixed step in
one pass over the paged pool, driven by block_tables / seq_lens / cu_seqlens that live on the device.

The tensor-core kernels need a small caller-owned workspace (`AttnWorkspace`): it holds the per-step plan
(built once per step by `plan`, reused by every layer) and the split-KV partials. Convenience calls without
an explicit workspace use a cached one per device.
"""
from __future__ import annotations

import torch

from nanoserve_b200 import _lib


class AttnWorkspace:
    """Zero-initialised device buffer sized for up to max_seqs sequences / max_tokens query tokens."""

    def __init__(self, max_seqs: int, max_tokens: int, n_heads: int, head_dim: int, device="cuda"):
        self.max_seqs, self.max_tokens = int(max_seqs), int(max(max_tokens, max_seqs))
        self.n_heads, self.head_dim = n_heads, head_dim
        nbytes = _lib.load().ns_attn_workspace_bytes(self.max_seqs, self.max_tokens, n_heads, head_dim)
        if nbytes <= 0:
            raise _lib.NanoserveB200Error("ns_attn_workspace_bytes rejected the sizes")
        self.nbytes = int(nbytes)
        # +256 so the used part can start on a 256-byte boundary whatever the allocator returns
        self._raw = torch.zeros(self.nbytes + 256, dtype=torch.uint8, device=device)
        off = (-self._raw.data_ptr()) % 256
        self.buf = self._raw[off:off + self.nbytes]

    def fits(self, n_seqs: int, n_tokens: int, n_heads: int, head_dim: int) -> bool:
        return (n_seqs <= self.max_seqs and n_tokens <= self.max_tokens and n_heads == self.n_heads
                and head_dim == self.head_dim)

    def plan(self, seq_lens: torch.Tensor, cu_seqlens: torch.Tensor | None, n_seqs: int, block_size: int,
             table_rows: torch.Tensor | None = None) -> None:
        """Build this step's plan (call once per step, before the first layer's attention)."""
        _lib.call("ns_attn_plan", seq_lens.data_ptr(), _lib.ptr(cu_seqlens), _lib.ptr(table_rows), n_seqs, block_size,
                  self.n_heads,
                  self.head_dim, self.buf.data_ptr(), self.nbytes, self.max_seqs, self.max_tokens, _lib.stream_ptr())


_cached: dict[tuple, AttnWorkspace] = {}


def _workspace_for(device, n_seqs: int, n_tokens: int, n_heads: int, head_dim: int) -> AttnWorkspace:
    key = (device.index if device.index is not None else torch.cuda.current_device(), n_heads, head_dim)
    ws = _cached.get(key)
    if ws is None or not ws.fits(n_seqs, n_tokens, n_heads, head_dim):
        cap_s = max(256, 1 << (max(n_seqs, 1) - 1).bit_length())
        cap_t = max(4096, 1 << (max(n_tokens, 1) - 1).bit_length())
        ws = _cached[key] = AttnWorkspace(cap_s, cap_t, n_heads, head_dim, device)
    return ws


def _check_pool(q, k_pool, v_pool):
    assert k_pool.dim() == 4 and q.dim() == 3
    assert q.stride(-1) == 1 and k_pool.stride(-1) == 1 and v_pool.stride() == k_pool.stride()
    assert q.stride(1) == q.shape[2], "query heads must be adjacent (head stride == head_dim)"
    assert k_pool.dtype == q.dtype and v_pool.dtype == q.dtype


def paged_attention_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor,
                           context_lens: torch.Tensor, scale: float, workspace: AttnWorkspace | None = None) -> torch.Tensor:
    """q: [B, n_heads, head_dim]; k_pool/v_pool: ONE layer's pool [num_blocks, block_size, n_kv_heads, head_dim];
    block_tables: int32 [B, max_blocks]; context_lens: int32 [B] (includes the new token, whose K/V must already
    be written). Returns [B, n_heads, head_dim]."""
    _lib.require_cuda(q, k_pool, v_pool, block_tables, context_lens)
    _check_pool(q, k_pool, v_pool)
    assert block_tables.dtype == torch.int32 and context_lens.dtype == torch.int32
    assert block_tables.stride(-1) == 1 and context_lens.is_contiguous()
    B, n_heads, head_dim = q.shape
    _, block_size, n_kv_heads, _ = k_pool.shape
    out = torch.empty(B, n_heads, head_dim, device=q.device, dtype=q.dtype)
    ws = workspace or _workspace_for(q.device, B, B, n_heads, head_dim)
    _lib.call("ns_paged_attn_decode", q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), block_tables.data_ptr(),
              context_lens.data_ptr(), out.data_ptr(), B, n_heads, n_kv_heads, head_dim, block_size,
              block_tables.stride(0), q.stride(0), out.stride(0), k_pool.stride(0), k_pool.stride(1), k_pool.stride(2),
              float(scale), _lib.dtype_code(q.dtype), ws.buf.data_ptr(), ws.nbytes, ws.max_seqs, ws.max_tokens,
              _lib.stream_ptr())
    return out


def paged_attention_decode_static(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                                  block_tables: torch.Tensor, context_lens: torch.Tensor, scale: float,
                                  out: torch.Tensor) -> torch.Tensor:
    """paged_attention_decode for callers that may not allocate on the device: `out` is supplied by the caller and
    the kernels' scratch is a fixed array inside the library (no workspace tensor, no torch allocation here).
    Limits: at most 64 rows, 32 query heads, head_dim 64 or 128, bf16, block size 16; larger inputs raise. All
    calls on a GPU share that scratch, so keep them on one stream; make the first call on each device outside any
    CUDA-graph capture (it resolves the scratch address)."""
    _lib.require_cuda(q, k_pool, v_pool, block_tables, context_lens, out)
    _check_pool(q, k_pool, v_pool)
    assert block_tables.dtype == torch.int32 and context_lens.dtype == torch.int32
    assert block_tables.stride(-1) == 1 and context_lens.is_contiguous()
    assert out.shape == q.shape and out.dtype == q.dtype and out.stride(-1) == 1 and out.stride(1) == q.shape[2]
    B, n_heads, head_dim = q.shape
    _, block_size, n_kv_heads, _ = k_pool.shape
    _lib.call("ns_paged_attn_decode_static", q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), block_tables.data_ptr(),
              context_lens.data_ptr(), out.data_ptr(), B, n_heads, n_kv_heads, head_dim, block_size,
              block_tables.stride(0), q.stride(0), out.stride(0), k_pool.stride(0), k_pool.stride(1), k_pool.stride(2),
              float(scale), _lib.dtype_code(q.dtype), _lib.stream_ptr())
    return out


def ragged_paged_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor,
                           seq_lens: torch.Tensor, cu_seqlens: torch.Tensor | None, scale: float, *,
                           n_seqs: int | None = None, table_rows: torch.Tensor | None = None,
                           workspace: AttnWorkspace | None = None, planned: bool = False,
                           out: torch.Tensor | None = None, simple: bool = False) -> torch.Tensor:
    """Attention for a mixed step. q: [N, n_heads, head_dim] = the flattened query tokens of S sequences;
    sequence s owns rows cu_seqlens[s]..cu_seqlens[s+1]-1 and seq_lens[s] keys (context + its new tokens,
    already in the pool), reached through block_tables[table_rows[s] if given else s]. cu_seqlens=None means
    one token per sequence. `planned=True` says workspace.plan(...) was already called for this step (the
    per-layer fast path); otherwise the plan is built here. `simple=True` forces the scalar fp32-accumulating
    kernel. Returns [N, n_heads, head_dim]."""
    _lib.require_cuda(q, k_pool, v_pool, block_tables, seq_lens, cu_seqlens, table_rows)
    _check_pool(q, k_pool, v_pool)
    assert block_tables.dtype == torch.int32 and seq_lens.dtype == torch.int32 and block_tables.stride(-1) == 1
    assert cu_seqlens is None or (cu_seqlens.dtype == torch.int32 and cu_seqlens.is_contiguous())
    assert table_rows is None or (table_rows.dtype == torch.int32 and table_rows.is_contiguous())
    N, n_heads, head_dim = q.shape
    S = int(n_seqs) if n_seqs is not None else seq_lens.shape[0]
    _, block_size, n_kv_heads, _ = k_pool.shape
    if out is None:
        out = torch.empty(N, n_heads, head_dim, device=q.device, dtype=q.dtype)
    else:
        assert out.shape == q.shape and out.stride(-1) == 1 and out.stride(1) == head_dim and out.dtype == q.dtype
    code = _lib.dtype_code(q.dtype)
    common = (q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), block_tables.data_ptr(), _lib.ptr(table_rows),
              seq_lens.data_ptr(), _lib.ptr(cu_seqlens), out.data_ptr(), S, N, n_heads, n_kv_heads, head_dim, block_size,
              block_tables.stride(0), q.stride(0), out.stride(0), k_pool.stride(0), k_pool.stride(1), k_pool.stride(2),
              float(scale), code)
    if simple or code != _lib.NS_BF16:
        _lib.call("ns_ragged_paged_attn_simple", *common, _lib.stream_ptr())
        return out
    ws = workspace or _workspace_for(q.device, S, N, n_heads, head_dim)
    if not planned:
        ws.plan(seq_lens, cu_seqlens, S, block_size, table_rows)
    _lib.call("ns_ragged_paged_attn", *common, ws.buf.data_ptr(), ws.nbytes, ws.max_seqs, ws.max_tokens,
              _lib.stream_ptr())
    if cu_seqlens is not None and N > S:
        _lib.note_launches(1)          # the prefill-tile kernel is launched next to the decode kernel
    return out
