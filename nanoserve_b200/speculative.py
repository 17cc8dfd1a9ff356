"""Greedy speculative decoding with a small draft model, on the ragged paged-attention kernel.

Same algorithm, constructor keywords, methods and counters as the reference's engine (nanoserve/speculative.py:64-305):
a DRAFT model guesses k tokens with k cheap steps, the TARGET checks them in ONE forward over [newest token, d1..dk],
the longest matching prefix is accepted plus the target's own token at the first mismatch, and both KV tables are
rewound to the accepted length. Every emitted token is the target's greedy choice given the tokens before it, so the
text equals plain greedy decoding with the target.

What differs underneath:
  * a verification is ONE ragged sequence with k+1 query tokens: `ns_ragged_paged_attn` applies causality inside the
    row (query j sees keys 0..ctx+j). The reference had to split it into k+1 decode rows that each carry a copy of the
    request's block table, because its decode kernel takes one query per row (speculative.py:193-210);
  * new requests' prefills ride in the same forward as the running requests' draft / verify rows (one mixed ragged
    step per model) instead of a separate eager pass;
  * the draft's k-1 follow-up steps read their input token from the device (the token the previous step's argmax left in
    `last_tokens[seat]`) and replay a decode graph: the host sees the drafts once, after the k-th step, and the target's
    choices once - two device->host reads per engine step instead of k+1.
Shortcuts kept from the reference: blocks for prompt + max_new + k + 1 tokens are reserved at admission (no
preemption), fixed k, greedy requests only.
"""
from __future__ import annotations

import math
import time
from collections import deque
from dataclasses import dataclass, field

import torch

from nanoserve_b200 import _lib
from nanoserve_b200.cuda_graphs import BUCKETS, DecodeGraphRunner, StepBuffers
from nanoserve_b200.engine import StepOutput
from nanoserve_b200.kv_cache import BlockTable, PagedKVCache
from nanoserve_b200.model import Qwen2Model


@dataclass(eq=False)
class SpecSeq:
    seq_id: int
    prompt_ids: list[int]
    max_new_tokens: int
    ignore_eos: bool
    arrival_time: float
    output_ids: list[int] = field(default_factory=list)
    t_table: BlockTable | None = None
    d_table: BlockTable | None = None
    seat: int = -1

    @property
    def tokens(self) -> list[int]:
        return self.prompt_ids + self.output_ids


class _Lane:
    """One model with its pool, its step buffers (block-table mirror, metadata kernel inputs) and a decode graph runner."""

    def __init__(self, model: Qwen2Model, pool: PagedKVCache, max_seqs: int, max_tokens: int, span: int, graphs: bool):
        self.model = model if model.fused else model.with_fused_ops()
        self.pool = pool
        self.garbage = pool.allocator.allocate()                      # padding rows of the graphs touch only this block
        seq_cap = next((b for b in BUCKETS if b >= max_seqs), max_seqs)
        self.buf = StepBuffers(self.model, pool, max_seqs=seq_cap, max_tokens=max_tokens + seq_cap, max_seq_len=span,
                               garbage_block=self.garbage, max_seats=max_seqs)
        self.runner = DecodeGraphRunner(self.model, pool, span, max_batch=seq_cap, buffers=self.buf) if graphs else None
        self.synced = [0] * max_seqs                                   # block-table entries already mirrored, per seat
        dev = model.device
        self.rows_dev = torch.zeros(self.buf.max_tokens, dtype=torch.int64, device=dev)
        self.rows_host = torch.zeros(self.buf.max_tokens, dtype=torch.int64, pin_memory=True)
        self.row_tokens = torch.zeros(self.buf.max_tokens, dtype=torch.int64, device=dev)

    def appends(self, seat: int, table: BlockTable) -> list[int]:
        out: list[int] = []
        for j in range(self.synced[seat], len(table.blocks)):
            out += (seat, j, table.blocks[j])
        self.synced[seat] = len(table.blocks)
        return out

    def forward(self, items, rows: list[int] | None = None):
        """items: [(seat, table, new token ids or None)]; None = one token, the one the previous step's argmax left on
        the device. Feeds the tokens on top of each table's stored context, writes their K/V and commits the tables.
        rows None: greedy token of every item's LAST row -> buf.sampled[:len(items)] (and last_tokens[seat]);
        rows given (flattened row indices): greedy token of each of those rows -> row_tokens[:len(rows)]."""
        records: list[int] = []
        appends: list[int] = []
        token_ids: list[int] = []
        n_tokens = 0
        for seat, table, toks in items:
            appends += self.appends(seat, table)
            if toks is None:
                records += (seat, table.num_tokens, 1, -1)
                n_tokens += 1
            else:
                records += (seat, table.num_tokens, len(toks), len(token_ids))
                token_ids += toks
                n_tokens += len(toks)
        n_seqs = len(items)
        buf = self.buf
        if rows is None and n_tokens == n_seqs and self.runner is not None and n_seqs <= self.runner.max_bucket:
            self.runner.run_packed(records, appends, token_ids)
            graph = True
        else:
            buf.upload(records, appends, token_ids, pad_seqs=n_seqs, pad_tokens=n_tokens)
            buf.build()
            meta = buf.meta(n_tokens, n_seqs, decode_only=False)
            if rows is not None:
                self.rows_host[:len(rows)] = torch.tensor(rows, dtype=torch.int64)
                self.rows_dev[:len(rows)].copy_(self.rows_host[:len(rows)], non_blocking=True)
                meta.last_rows = self.rows_dev[:len(rows)]
            logits = self.model.forward_step(meta, self.pool)
            if rows is None:
                buf.sample(logits, n_seqs)
            else:
                _lib.call("ns_argmax_rows", logits.data_ptr(), logits.stride(0), len(rows), logits.shape[1],
                          self.row_tokens.data_ptr(), None, None, _lib.dtype_code(logits.dtype), _lib.stream_ptr())
            graph = False
        for _, table, toks in items:
            table.commit(1 if toks is None else len(toks))
        return graph


class SpeculativeEngine:
    def __init__(self, target: Qwen2Model, draft: Qwen2Model, eos_token_ids: list[int], num_speculative_tokens: int = 4,
                 max_seq_len: int = 2048, max_num_seqs: int = 8, max_num_batched_tokens: int = 4096,
                 target_kv_tokens: int | None = None, draft_kv_tokens: int | None = None, block_size: int = 16,
                 cuda_graphs: bool | None = None):
        if target.cfg.vocab_size != draft.cfg.vocab_size:
            raise ValueError("draft and target must share a vocabulary")
        if target.device.type != "cuda":
            raise ValueError("nanoserve_b200 engines run on a CUDA device only")
        if num_speculative_tokens < 1:
            raise ValueError("num_speculative_tokens must be >= 1")
        self.k = num_speculative_tokens
        self.eos_token_ids = list(eos_token_ids)
        self._eos = set(eos_token_ids)
        self.max_seq_len = max_seq_len
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max(max_num_batched_tokens, max_seq_len)
        self.block_size = block_size
        span = max_seq_len + self.k + 1
        t_tokens = target_kv_tokens or 8 * span
        d_tokens = draft_kv_tokens or t_tokens
        self.tpool = PagedKVCache.from_token_budget(target.cfg, t_tokens + block_size, block_size, target.device, target.dtype)
        self.dpool = PagedKVCache.from_token_budget(draft.cfg, d_tokens + block_size, block_size, draft.device, draft.dtype)
        graphs = True if cuda_graphs is None else bool(cuda_graphs)
        step_tokens = self.max_num_batched_tokens + max_num_seqs * (self.k + 1)
        self._t = _Lane(target, self.tpool, max_num_seqs, step_tokens, span, graphs)
        self._d = _Lane(draft, self.dpool, max_num_seqs, step_tokens, span, graphs)
        self.target, self.draft = self._t.model, self._d.model
        self.t_graph, self.d_graph = self._t.runner, self._d.runner
        dev = target.device
        self._drafts_dev = torch.zeros(self.k, max_num_seqs, dtype=torch.int64, device=dev)
        self._free_seats = list(range(max_num_seqs - 1, -1, -1))
        self.waiting: deque[SpecSeq] = deque()
        self.running: list[SpecSeq] = []
        self.sequences: dict[int, SpecSeq] = {}
        self._next_id = 0
        self.reset_stats()

    # ---- bookkeeping --------------------------------------------------------------------------------------------------
    def reset_stats(self) -> None:
        self._stats = {"steps": 0, "target_forwards": 0, "draft_forwards": 0, "proposed": 0, "accepted": 0,
                       "emitted_by_verification": 0, "peak_running": 0, "graph_draft_steps": 0, "graph_verify_steps": 0,
                       "host_syncs": 0}

    @property
    def stats(self) -> dict:
        s = dict(self._stats)
        s["acceptance_rate"] = s["accepted"] / s["proposed"] if s["proposed"] else None
        s["tokens_per_target_forward"] = (s["emitted_by_verification"] / s["target_forwards"]
                                          if s["target_forwards"] else None)
        s["num_speculative_tokens"] = self.k
        s["cuda_graphs"] = self.t_graph is not None
        return s

    def _reserve_tokens(self, seq: SpecSeq) -> int:
        return len(seq.prompt_ids) + seq.max_new_tokens + self.k + 1

    def add_request(self, prompt_ids: list[int], max_new_tokens: int, ignore_eos: bool = False,
                    arrival_time: float | None = None, sampling=None) -> int:
        if sampling is not None and not sampling.greedy:
            # greedy verification accepts a draft token iff it equals the target's argmax; sampling would need
            # rejection sampling, which the reference does not build either (nanoserve/speculative.py:118-122)
            raise ValueError("speculative decoding is greedy-only (temperature must be 0)")
        if len(prompt_ids) + max_new_tokens > self.max_seq_len:
            raise ValueError(f"prompt + max_new_tokens exceeds max_seq_len ({self.max_seq_len})")
        seq = SpecSeq(self._next_id, list(prompt_ids), max_new_tokens, ignore_eos,
                      time.perf_counter() if arrival_time is None else arrival_time)
        need = math.ceil(self._reserve_tokens(seq) / self.block_size)
        if need > min(self.tpool.num_blocks, self.dpool.num_blocks) - 1:
            raise ValueError("request can never fit in the KV pools")
        self.waiting.append(seq)
        self.sequences[seq.seq_id] = seq
        self._next_id += 1
        return seq.seq_id

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def _release(self, seq: SpecSeq) -> None:
        if seq.t_table is not None:
            seq.t_table.release(self.tpool.allocator)
            seq.d_table.release(self.dpool.allocator)
            seq.t_table = seq.d_table = None
        if seq.seat >= 0:
            self._t.synced[seq.seat] = self._d.synced[seq.seat] = 0
            self._free_seats.append(seq.seat)
            seq.seat = -1
        self.sequences.pop(seq.seq_id, None)

    def abort(self, seq_id: int) -> None:
        seq = self.sequences.get(seq_id)
        if seq is None:
            return
        if seq in self.running:
            self.running.remove(seq)
        elif seq in self.waiting:
            self.waiting.remove(seq)
        self._release(seq)

    def _admit(self) -> list[SpecSeq]:
        admitted, budget = [], self.max_num_batched_tokens
        while self.waiting and len(self.running) + len(admitted) < self.max_num_seqs:
            seq = self.waiting[0]
            need = math.ceil(self._reserve_tokens(seq) / self.block_size)
            if (len(seq.prompt_ids) > budget or need > self.tpool.allocator.num_free
                    or need > self.dpool.allocator.num_free):
                break
            self.waiting.popleft()
            seq.t_table, seq.d_table = BlockTable(self.block_size), BlockTable(self.block_size)
            seq.t_table.reserve(self._reserve_tokens(seq), self.tpool.allocator)
            seq.d_table.reserve(self._reserve_tokens(seq), self.dpool.allocator)
            seq.seat = self._free_seats.pop()
            budget -= len(seq.prompt_ids)
            admitted.append(seq)
        self.running.extend(admitted)
        return admitted

    # ---- one engine step ------------------------------------------------------------------------------------------------
    @torch.inference_mode()
    def step(self) -> list[StepOutput]:
        admitted = self._admit()
        decoding = [s for s in self.running if s not in admitted]
        if not admitted and not decoding:
            return []
        st = self._stats
        st["steps"] += 1
        st["peak_running"] = max(st["peak_running"], len(self.running))
        k, D = self.k, len(decoding)

        # 1) DRAFT. One mixed ragged step: running requests catch up on the tokens their draft cache has not seen (one, or
        #    two after a fully accepted round) and propose d1; new requests prefill their prompt. Then k-1 one-token
        #    steps whose input is the previous step's token, read on the device.
        items = [(s.seat, s.d_table, s.tokens[s.d_table.num_tokens:]) for s in decoding]
        items += [(s.seat, s.d_table, s.prompt_ids) for s in admitted]
        self._d.forward(items)
        st["draft_forwards"] += 1
        drafts: list[list[int]] = [[] for _ in decoding]
        if decoding:
            self._drafts_dev[0, :D].copy_(self._d.buf.sampled[:D])
            for j in range(1, k):
                if self._d.forward([(s.seat, s.d_table, None) for s in decoding]):
                    st["graph_draft_steps"] += 1
                st["draft_forwards"] += 1
                self._drafts_dev[j, :D].copy_(self._d.buf.sampled[:D])
            got = self._drafts_dev[:, :D].t().tolist()                     # the drafts' only trip to the host
            st["host_syncs"] += 1
            drafts = got

        # 2) TARGET. One mixed ragged step: a verification row per running request - [newest token, d1..dk] on top of its
        #    context, the target's greedy choice wanted at all k+1 positions - and the prompt of every new request (its
        #    last position only).
        items, rows, off = [], [], 0
        for s, d in zip(decoding, drafts):
            toks = s.tokens[s.t_table.num_tokens:] + d
            items.append((s.seat, s.t_table, toks))
            rows += range(off + len(toks) - (k + 1), off + len(toks))
            off += len(toks)
        for s in admitted:
            items.append((s.seat, s.t_table, s.prompt_ids))
            off += len(s.prompt_ids)
            rows.append(off - 1)
        self._t.forward(items, rows)
        st["target_forwards"] += 1
        choices = self._t.row_tokens[:len(rows)].tolist()
        st["host_syncs"] += 1

        # 3) ACCEPT and emit (new requests first, as the reference orders a step's outputs).
        outputs = []
        for i, s in enumerate(admitted):
            outputs += self._emit(s, [choices[D * (k + 1) + i]])
        for i, (s, d) in enumerate(zip(decoding, drafts)):
            t = choices[i * (k + 1):(i + 1) * (k + 1)]
            n = 0
            while n < k and d[n] == t[n]:
                n += 1
            st["proposed"] += k
            st["accepted"] += n
            new_tokens = d[:n] + [t[n]]
            st["emitted_by_verification"] += len(new_tokens)
            outputs += self._emit(s, new_tokens)
        return outputs

    def _emit(self, s: SpecSeq, new_tokens: list[int]) -> list[StepOutput]:
        out, finished = [], False
        for tok in new_tokens:
            s.output_ids.append(tok)
            finished = (tok in self._eos and not s.ignore_eos) or len(s.output_ids) >= s.max_new_tokens
            out.append(StepOutput(s.seq_id, tok, finished))
            if finished:
                break
        if finished:
            self.running.remove(s)
            self._release(s)
            return out
        # Rewind: K/V is valid only for tokens that were accepted. Every token except the newest must be cached; what
        # is cached beyond that belongs to rejected drafts (it is overwritten by the next round).
        keep = len(s.tokens) - 1
        s.t_table.rewind(min(s.t_table.num_tokens, keep))
        s.d_table.rewind(min(s.d_table.num_tokens, keep))
        return out
