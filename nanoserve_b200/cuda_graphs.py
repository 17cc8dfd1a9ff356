"""CUDA-graph runners for engine steps, and the device-side step buffers they replay over.

Class names, buckets, padding rules and the garbage-block convention follow the reference
(nanoserve/cuda_graphs.py:28-259): `BUCKETS`, `PIECEWISE_CAP`, `piecewise_buckets`, `DecodeGraphRunner`,
`PiecewiseGraphRunner`, `captured_buckets`, `garbage_block`, `run(...)`.

What changed underneath:
  * the reference copies five host-built tensors into static buffers before every replay
    (cuda_graphs.py:112-117). Here ONE packed int32 buffer goes up (a few hundred bytes for a decode step) and the
    graph itself starts with the metadata kernel that expands it into token ids, positions, slot mapping,
    cu_seqlens, seq_lens and table rows, padded to the bucket with rows that only touch the garbage block;
  * attention is ragged and graph-safe, so a MIXED step (prefill chunks + decodes) is one full graph per token
    bucket. The reference had to cut such a step into L+1 graph pieces with eager attention in between
    (cuda_graphs.py:130-147); `PiecewiseGraphRunner` keeps its name and `run` signature for drop-in use;
  * LM head and greedy argmax are inside the graph; the sampled token also stays on the device for the next step.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from nanoserve_b200 import _lib
from nanoserve_b200.kernels.paged_attention import AttnWorkspace
from nanoserve_b200.model import StepMeta

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
PIECEWISE_CAP = 512
_HEADER_INTS = 8

_SIDE_STREAM = None


class DeviceStatusError(_lib.NanoserveB200Error):
    """A kernel of an engine step gave up on a bounded wait, or the step's bounds check found a violation (the library's
    status word grew)."""


def _capture_stream() -> torch.cuda.Stream:
    """One warm-up stream for every capture in the process (a fresh stream per capture keeps a cuBLAS workspace
    alive each, cuda_graphs.py:33-39)."""
    global _SIDE_STREAM
    if _SIDE_STREAM is None:
        _SIDE_STREAM = torch.cuda.Stream()
    return _SIDE_STREAM


def piecewise_buckets(max_tokens: int, cap: int = PIECEWISE_CAP) -> list[int]:
    """Token-count buckets for mixed steps: every 16 up to 256, then every 32; the budget itself (or the cap) is
    the last bucket. Steps above it run without a graph."""
    top = min(max_tokens, cap)
    grid = [b for b in range(16, 256, 16)] + [b for b in range(256, cap + 1, 32)]
    return [b for b in grid if b < top] + [top]


def step_buckets(max_tokens: int, coarse: int = 128) -> list[int]:
    """The engine's token buckets for mixed steps: the reference's grid up to its cap, then every `coarse` tokens up to
    the step budget itself. The reference ran larger steps without a graph (cuda_graphs.py:154-160: its L+1 graph
    pieces paid off only for small steps); here a mixed step is ONE graph of ~200 launches, and running a
    1300-token step eagerly was measured at 3.9 ms of host-bound launching against ~1.5 ms on the device."""
    fine = piecewise_buckets(max_tokens)
    if max_tokens <= PIECEWISE_CAP:
        return fine
    return fine + [b for b in range(PIECEWISE_CAP + coarse, max_tokens, coarse)] + [max_tokens]


class StepBuffers:
    """Static device buffers of one engine: the block-table mirror (one row per seat), the last sampled token per
    seat, and the per-step arrays the metadata kernel fills. One instance is shared by both runners."""

    def __init__(self, model, pool, max_seqs: int, max_tokens: int, max_seq_len: int, garbage_block: int,
                 max_seats: int = 256):
        cfg, dev = model.cfg, model.device
        self.model, self.pool = model, pool
        self.max_seqs, self.max_tokens = int(max_seqs), int(max(max_tokens, max_seqs))
        self.block_size = pool.block_size
        self.table_width = -(-max_seq_len // pool.block_size)
        self.garbage_block = garbage_block
        self.max_seats = max_seats
        self.pad_seat = max_seats                                   # mirror row of every padding sequence
        self.mirror = torch.zeros(max_seats + 1, self.table_width, dtype=torch.int32, device=dev)
        self.mirror[self.pad_seat, 0] = garbage_block
        self.last_tokens = torch.zeros(max_seats + 1, dtype=torch.int64, device=dev)
        i64 = dict(dtype=torch.int64, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        self.tokens = torch.zeros(self.max_tokens, **i64)
        self.positions = torch.zeros(self.max_tokens, **i64)
        self.slots = torch.zeros(self.max_tokens, **i64)
        self.cu_seqlens = torch.zeros(self.max_seqs + 1, **i32)
        self.seq_lens = torch.ones(self.max_seqs, **i32)
        self.seat_of = torch.full((self.max_seqs,), self.pad_seat, **i32)
        self.last_rows = torch.zeros(self.max_seqs, **i64)
        # word 0: the library's status word of the step (ns_collect_status); words 1..: the sampled tokens. One
        # device->host copy per step brings back both.
        self.fetched = torch.zeros(1 + self.max_seqs, **i64)
        self.sampled = self.fetched[1:]
        self.status_seen = 0              # status word of the newest step that was read back (process-wide, cumulative)
        # per-row sampling parameters read by the sampling kernel inside the graphs (8 words per row, all zero = every
        # row greedy); uploaded only on steps that sample and on the first all-greedy step after one
        self.sample_params = torch.zeros(8 * self.max_seqs, **i32)
        self._sample_staging = [torch.zeros(8 * self.max_seqs, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._sample_np = [(t.numpy(), t.numpy().view(np.float32)) for t in self._sample_staging]
        self._sample_turn = 0
        self._sample_done = [torch.cuda.Event() for _ in range(2)]
        self._sample_live = False         # the device copy holds an enabled row
        # two pinned landing buffers for sampled tokens and two pinned staging buffers for packed steps, used in
        # turn: with one step in flight the host may fill step t+1's staging buffer while step t's copy is pending
        self._sampled_host = [torch.zeros(1 + self.max_seqs, dtype=torch.int64, pin_memory=True) for _ in range(2)]
        self._fetch_events = [torch.cuda.Event() for _ in range(2)]
        self._fetch_turn = 0
        self.capacity = _HEADER_INTS + 4 * self.max_seqs + 3 * self.max_seqs * self.table_width + self.max_tokens
        self._staging = [torch.zeros(self.capacity, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._staging_np = [t.numpy() for t in self._staging]
        self._staging_turn = 0
        self._staging_done = [torch.cuda.Event() for _ in range(2)]
        self.host_packed = self._staging[0]          # the staging buffer of the latest upload
        self.dev_packed = torch.zeros(self.capacity, **i32)
        nh = cfg.n_heads // getattr(model, "tp_size", 1)
        self.workspace = AttnWorkspace(self.max_seqs, self.max_tokens, nh, cfg.head_dim, dev)
        # the library's counters are process-wide and cumulative: this engine reports what is counted from now on
        _lib.call("ns_collect_status", self.workspace.buf.data_ptr(), self.fetched.data_ptr(), _lib.stream_ptr())
        self.status_base = self.status_seen = self._status_ok = int(self.fetched[0].item())

    def upload(self, records: list[int], appends: list[int], token_ids: list[int], pad_seqs: int, pad_tokens: int) -> None:
        """Fill the pinned staging buffer and start its copy to the device (stream-ordered before the graph)."""
        n_seqs, n_app = len(records) // 4, len(appends) // 3
        n_tokens = self._count_tokens(records)
        if pad_seqs > self.max_seqs or pad_tokens > self.max_tokens:
            raise ValueError(f"step of {pad_seqs} sequences / {pad_tokens} tokens exceeds the buffers "
                             f"({self.max_seqs} / {self.max_tokens})")
        self._staging_turn ^= 1
        self.host_packed = self._staging[self._staging_turn]
        # the copy that last read this pinned buffer must have run before the host writes it again (a caller that issues
        # several steps without reading anything back, like a chain of draft steps, gets here with copies still queued)
        self._staging_done[self._staging_turn].synchronize()
        a = self._staging_np[self._staging_turn]
        a[:_HEADER_INTS] = (n_seqs, n_tokens, pad_seqs, pad_tokens, n_app, self.garbage_block, self.block_size,
                            self.table_width)
        o = _HEADER_INTS
        n = o + len(records) + len(appends) + len(token_ids)
        if n > self.capacity:
            raise ValueError("packed step does not fit the staging buffer")
        a[o:o + len(records)] = records
        o += len(records)
        if appends:
            a[o:o + len(appends)] = appends
            o += len(appends)
        if token_ids:
            a[o:o + len(token_ids)] = token_ids
        self.packed_ints = n
        self.dev_packed[:n].copy_(self.host_packed[:n], non_blocking=True)
        self._staging_done[self._staging_turn].record()

    def set_sampling(self, rows: list[tuple]) -> None:
        """rows: (row, temperature, top_p, top_k, 63-bit draw seed) for every sequence row of the coming step that
        samples with temperature > 0; every other row stays greedy. Stream-ordered before the step."""
        if not rows and not self._sample_live:
            return
        self._sample_turn ^= 1
        self._sample_done[self._sample_turn].synchronize()
        ints, floats = self._sample_np[self._sample_turn]
        ints[:] = 0
        for row, temperature, top_p, top_k, seed in rows:
            o = 8 * row
            floats[o], floats[o + 1] = temperature, top_p
            ints[o + 2], ints[o + 3] = top_k, 1
            ints[o + 4:o + 6] = np.array([seed & 0xFFFFFFFF, seed >> 32], dtype=np.uint32).view(np.int32)
        self.sample_params.copy_(self._sample_staging[self._sample_turn], non_blocking=True)
        self._sample_done[self._sample_turn].record()
        self._sample_live = bool(rows)

    @staticmethod
    def _count_tokens(records: list[int]) -> int:
        return sum(records[2::4])

    def build(self) -> None:
        """Launch the metadata kernel over the uploaded packed buffer (graph-capturable: sizes are read on the
        device from the packed header)."""
        _lib.call("ns_build_step_metadata", self.dev_packed.data_ptr(), self.capacity, self.mirror.data_ptr(),
                  self.last_tokens.data_ptr(), self.pad_seat, self.tokens.data_ptr(), self.positions.data_ptr(),
                  self.slots.data_ptr(), self.cu_seqlens.data_ptr(), self.seq_lens.data_ptr(), self.seat_of.data_ptr(),
                  self.last_rows.data_ptr(), self.max_seqs, self.max_tokens, _lib.stream_ptr())

    # NS_BOUNDS_CHECK=1 adds ns_check_step_metadata to every step (and to every captured graph): block ids, slots,
    # positions, cu_seqlens and token ids are verified on the device and violations arrive with the step's status word
    bounds_check = os.environ.get("NS_BOUNDS_CHECK", "0") not in ("", "0")

    def check(self, n_tokens: int, n_seqs: int) -> None:
        _lib.call("ns_check_step_metadata", self.mirror.data_ptr(), self.seat_of.data_ptr(), self.mirror.stride(0),
                  self.seq_lens.data_ptr(), self.cu_seqlens.data_ptr(), self.slots.data_ptr(), self.positions.data_ptr(),
                  self.tokens.data_ptr(), n_seqs, n_tokens, self.pool.num_blocks, self.block_size,
                  self.model.cfg.vocab_size, _lib.stream_ptr())

    def meta(self, n_tokens: int, n_seqs: int, decode_only: bool) -> StepMeta:
        return StepMeta(tokens=self.tokens[:n_tokens], positions=self.positions[:n_tokens],
                        slot_mapping=self.slots[:n_tokens], cu_seqlens=self.cu_seqlens[:n_seqs + 1],
                        seq_lens=self.seq_lens[:n_seqs], table_rows=self.seat_of[:n_seqs], block_tables=self.mirror,
                        last_rows=self.last_rows[:n_seqs], n_seqs=n_seqs, workspace=self.workspace,
                        decode_only=decode_only)

    def sample(self, logits: torch.Tensor, n_seqs: int) -> None:
        """Greedy token per row into `sampled`, and into last_tokens[seat] for the next step; rows whose request samples
        (set_sampling) are then redrawn with temperature / top-k / top-p; then the library's status word (bounded waits that ran out in any of its kernels) next to the tokens."""
        _lib.call("ns_argmax_rows", logits.data_ptr(), logits.stride(0), n_seqs, logits.shape[1], self.sampled.data_ptr(),
                  self.seat_of.data_ptr(), self.last_tokens.data_ptr(), _lib.dtype_code(logits.dtype), _lib.stream_ptr())
        _lib.call("ns_sample_rows", logits.data_ptr(), logits.stride(0), n_seqs, logits.shape[1], self.sample_params.data_ptr(),
                  self.sampled.data_ptr(), self.seat_of.data_ptr(), self.last_tokens.data_ptr(), None, None,
                  _lib.dtype_code(logits.dtype), _lib.stream_ptr())
        _lib.call("ns_collect_status", self.workspace.buf.data_ptr(), self.fetched.data_ptr(), _lib.stream_ptr())

    def step(self, n_tokens: int, n_seqs: int, decode_only: bool) -> torch.Tensor:
        """metadata kernel -> forward -> argmax over the first n_tokens / n_seqs rows; returns the logits."""
        self.build()
        if self.bounds_check:
            self.check(n_tokens, n_seqs)
        logits = self.model.forward_step(self.meta(n_tokens, n_seqs, decode_only), self.pool)
        self.sample(logits, n_seqs)
        return logits

    def queue_fetch(self, n: int):
        """Start the copy of the step's n sampled token ids to pinned host memory (stream-ordered after the step) and
        record an event behind it. Returns a handle for wait_fetch. At most two fetches may be outstanding."""
        turn = self._fetch_turn
        self._fetch_turn ^= 1
        self._sampled_host[turn][:n + 1].copy_(self.fetched[:n + 1], non_blocking=True)
        self._fetch_events[turn].record()
        return turn, n

    def wait_fetch(self, handle) -> list[int]:
        """Block until the fetch behind `handle` has landed: the step's only device->host sync. Raises
        DeviceStatusError if the status word that came back with the tokens has grown since the last fetch: a bounded
        wait ran out inside one of the step's kernels and the step's results are undefined."""
        turn, n = handle
        self._fetch_events[turn].synchronize()
        words = self._sampled_host[turn][:n + 1].tolist()
        status, self.status_seen = words[0], max(self.status_seen, words[0])
        if status > self._status_ok:
            grown, self._status_ok = status - self._status_ok, status
            raise DeviceStatusError(f"{grown} device-side error(s) in this step's kernels - bounded waits that ran out, or "
                                    f"bounds-check violations (status word {status}): its tokens are undefined")
        return words[1:]

    @property
    def device_errors(self) -> int:
        """Failed bounded waits / bounds-check violations counted since this object was built."""
        return self.status_seen - self.status_base

    def fetch_sampled(self, n: int) -> list[int]:
        return self.wait_fetch(self.queue_fetch(n))


class _GraphRunner:
    """Capture / replay of StepBuffers.step for fixed (token rows, sequences) shapes."""

    def __init__(self, buffers: StepBuffers):
        self.buffers = buffers
        self.graphs: dict = {}
        self.outputs: dict = {}
        self.launches: dict = {}         # kernels of this library inside each captured graph
        self.mempool = None

    def _capture(self, key, n_tokens: int, n_seqs: int, decode_only: bool) -> None:
        """Warm up and capture one step shape. A capture that the runtime invalidates (an unrelated call elsewhere in the
        process while the stream was capturing) is repeated once from the warm-up; a second failure is raised."""
        for attempt in (0, 1):
            try:
                self._capture_once(key, n_tokens, n_seqs, decode_only)
                return
            except (RuntimeError, _lib.NanoserveB200Error) as e:
                if attempt or "capture" not in str(e):
                    raise
                self.capture_retries += 1
                torch.cuda.synchronize()

    capture_retries = 0

    def _capture_once(self, key, n_tokens: int, n_seqs: int, decode_only: bool) -> None:
        buf = self.buffers
        # warm-up and capture run on an all-padding step: nothing but the garbage block is written
        buf.upload([], [], [], pad_seqs=n_seqs, pad_tokens=n_tokens)
        side = _capture_stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                buf.step(n_tokens, n_seqs, decode_only)
        torch.cuda.current_stream().wait_stream(side)
        if self.mempool is None:
            self.mempool = torch.cuda.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        before = _lib.launch_count
        try:
            with torch.cuda.graph(graph, pool=self.mempool):
                out = buf.step(n_tokens, n_seqs, decode_only)
        finally:
            captured = _lib.launch_count - before
            _lib.note_launches(-captured)             # captured, not executed
        self.launches[key] = captured
        self.graphs[key], self.outputs[key] = graph, out

    def replay(self, key) -> None:
        self.graphs[key].replay()
        _lib.note_launches(self.launches[key])


class DecodeGraphRunner(_GraphRunner):
    """One full-step graph per decode batch bucket (every sequence feeds exactly one token)."""

    def __init__(self, model, pool, max_seq_len: int, max_batch: int = BUCKETS[-1], buffers: StepBuffers | None = None):
        self.model, self.pool = model, pool
        self.buckets = [b for b in BUCKETS if b <= max_batch] or [max_batch]
        self.max_bucket = self.buckets[-1]
        self.max_blocks = -(-max_seq_len // pool.block_size)
        if buffers is None:
            garbage = pool.allocator.allocate()              # padding rows read / write only this block
            buffers = StepBuffers(model, pool, self.max_bucket, self.max_bucket, max_seq_len, garbage,
                                  max_seats=max(self.max_bucket, 1))
        self.garbage_block = buffers.garbage_block
        super().__init__(buffers)

    @property
    def captured_buckets(self) -> list[int]:
        return sorted(self.graphs)

    def bucket_for(self, n: int) -> int | None:
        return next((b for b in self.buckets if b >= n), None)

    def capture_all(self, max_batch: int) -> None:
        top = self.bucket_for(min(max_batch, self.max_bucket))
        for b in self.buckets:
            if b <= top and b not in self.graphs:
                self._capture(b, b, b, True)

    def run_packed(self, records: list[int], appends: list[int], token_ids: list[int]) -> torch.Tensor:
        """Engine entry: one decode step from packed records. Returns logits [n, vocab] (a view of the graph's
        output, valid until the next replay of that bucket); the sampled tokens are in buffers.sampled."""
        n = len(records) // 4
        B = self.bucket_for(n)
        if B is None:
            raise ValueError(f"batch of {n} exceeds the largest graph bucket ({self.max_bucket})")
        if B not in self.graphs:
            self._capture(B, B, B, True)
        self.buffers.upload(records, appends, token_ids, pad_seqs=B, pad_tokens=B)
        self.replay(B)
        self.last_key = B
        return self.outputs[B][:n]

    def run(self, tokens: list[int], positions: list[int], slots: list[int], block_tables: list[list[int]],
            context_lens: list[int]) -> torch.Tensor:
        """Reference signature (cuda_graphs.py:99-119): host lists in, logits [n, vocab] out. Row i uses seat i;
        positions and slots are implied by context_lens and the tables (the device recomputes them)."""
        records, appends = [], []
        for i, (table, length) in enumerate(zip(block_tables, context_lens)):
            records += (i, length - 1, 1, i)
            for j, b in enumerate(table):
                appends += (i, j, b)
        return self.run_packed(records, appends, list(tokens))


class PiecewiseGraphRunner(_GraphRunner):
    """Graphs for MIXED steps, one per token bucket. The name is the reference's: there a mixed step was L+1 graph
    pieces around eager attention; here the ragged kernel makes the whole step one graph."""

    def __init__(self, model, pool, garbage_block: int, max_tokens: int = PIECEWISE_CAP,
                 buckets: list[int] | None = None, buffers: StepBuffers | None = None, max_seqs: int | None = None,
                 max_seq_len: int = 2048):
        self.model, self.pool, self.garbage_block = model, pool, garbage_block
        self.buckets = sorted(buckets) if buckets else piecewise_buckets(max_tokens)
        self.max_tokens = self.buckets[-1]
        if buffers is None:
            seqs = max_seqs or min(self.max_tokens, BUCKETS[-1])
            buffers = StepBuffers(model, pool, seqs, self.max_tokens, max_seq_len, garbage_block, max_seats=seqs)
        # every mixed graph carries the same number of sequence rows: padding sequences are one-token decodes on
        # the garbage block, so a fixed count costs next to nothing and keeps one graph per token bucket
        self.seq_rows = max_seqs or buffers.max_seqs
        self.gslot = garbage_block * pool.block_size
        super().__init__(buffers)

    @property
    def captured_buckets(self) -> list[int]:
        return sorted(self.graphs)

    def bucket_for(self, n: int) -> int | None:
        return next((b for b in self.buckets if b >= n), None)

    def fits(self, n_tokens: int, n_seqs: int) -> bool:
        return n_seqs <= self.seq_rows and n_tokens + (self.seq_rows - n_seqs) <= self.max_tokens

    @torch.inference_mode()
    def capture_all(self) -> None:
        for b in reversed(self.buckets):          # largest first: its temporaries carve the pool once
            if b >= self.seq_rows and b not in self.graphs:
                self._capture(b, b, self.seq_rows, False)

    @torch.inference_mode()
    def run_packed(self, records: list[int], appends: list[int], token_ids: list[int]) -> torch.Tensor:
        n_seqs = len(records) // 4
        n_tokens = StepBuffers._count_tokens(records)
        need = n_tokens + (self.seq_rows - n_seqs)       # padding sequences bring one token row each
        B = self.bucket_for(need)
        if B is None or n_seqs > self.seq_rows:
            raise ValueError(f"step of {n_tokens} tokens / {n_seqs} sequences exceeds the largest bucket "
                             f"({self.max_tokens} / {self.seq_rows})")
        if B not in self.graphs:
            self._capture(B, B, self.seq_rows, False)
        self.buffers.upload(records, appends, token_ids, pad_seqs=self.seq_rows, pad_tokens=B)
        self.replay(B)
        self.last_key = B
        return self.outputs[B][:n_seqs]

    @torch.inference_mode()
    def run(self, tokens: list[int], positions: list[int], slots: list[int], seqs, decode_meta, rows=None) -> torch.Tensor:
        """Reference signature (cuda_graphs.py:239-259). Sequence i uses seat i; block tables come from the
        SeqInput objects (decode rows: from decode_meta). Returns logits of each sequence's last token."""
        records, appends, off, d = [], [], 0, 0
        for i, s in enumerate(seqs):
            table = s.block_table
            if s.use_kernel and decode_meta is not None:
                if table is None:
                    table = decode_meta.block_tables[d]
                d += 1
            if table is None:
                # a fresh prefill: its slots are its only blocks
                bs = self.pool.block_size
                table = [slots[off + j] // bs for j in range(0, s.n_tokens, 1) if (s.ctx_len + j) % bs == 0 or j == 0]
            table = [int(b) for b in (table.tolist() if hasattr(table, "tolist") else table)]
            need = -(-(s.ctx_len + s.n_tokens) // self.pool.block_size)
            for j, b in enumerate(table[:need]):
                appends += (i, j, b)
            records += (i, s.ctx_len, s.n_tokens, off)
            off += s.n_tokens
        if rows is not None:
            ends = np.cumsum([s.n_tokens for s in seqs]) - 1
            if rows.tolist() != ends.tolist():
                raise NotImplementedError("the graphs score each sequence's last token only")
        return self.run_packed(records, appends, list(tokens))
