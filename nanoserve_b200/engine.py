"""Inference engine: scheduler + one batched forward per step + sampling (greedy argmax, or temperature / top-k / top-p per
request) on the device.

`LLMEngine` keeps the reference's constructor keywords, methods and counters (nanoserve/engine.py:46-298):
`add_request`, `abort`, `has_unfinished`, `step() -> list[StepOutput]`, `capture_graphs`, `stats`, `last_step`,
`timing`, `reset_stats`. One step is still schedule -> forward -> sample (one device->host sync) -> commit, but
the forward's inputs are no longer Python lists turned into tensors: the scheduler's decision is packed into a
small int32 record buffer, uploaded once, and expanded on the device, so pure-decode AND mixed steps replay a
single CUDA graph that already contains the LM head and the argmax.

`lookahead=True` (not in the reference) keeps one step in flight: after launching step t the host does step t's
bookkeeping with the sampled tokens still unknown, and the next call schedules and launches step t+1 BEFORE it
waits for step t's tokens, so scheduling and launching overlap the device. The scheduler only ever needs a token's
VALUE for the end-of-sequence test, so this is done only for steps whose sampling sequences all have
ignore_eos=True; any other step is waited for before the host goes on, exactly as without the option. Scheduling
decisions, and therefore tokens, are the same as without lookahead; `step()` returns a step's outputs one call
later and `has_unfinished()` stays true until they have been returned.
"""
from __future__ import annotations

import random
import time
from dataclasses import dataclass

import torch

from nanoserve_b200.cuda_graphs import (BUCKETS, DecodeGraphRunner, DeviceStatusError, PiecewiseGraphRunner, StepBuffers,
                                        step_buckets)
from nanoserve_b200.kv_manager import PagedKVManager
from nanoserve_b200.model import Qwen2Model
from nanoserve_b200.sampling import mix_seed
from nanoserve_b200.scheduler import Scheduler, Sequence


@dataclass
class StepOutput:
    seq_id: int
    token: int
    finished: bool


@dataclass
class StepStats:
    n_prefill: int
    n_decode: int
    n_tokens: int


class LLMEngine:
    def __init__(self, model: Qwen2Model, eos_token_ids: list[int], max_seq_len: int = 2048,
                 policy: str = "continuous", max_num_seqs: int = 8, max_num_batched_tokens: int = 2048,
                 batch_wait_s: float = 0.02, kv_cache: str = "paged", kv_cache_tokens: int | None = None,
                 block_size: int = 16, attn_backend: str | None = None, cuda_graphs: bool | None = None,
                 chunked_prefill: bool | None = None, piecewise_graphs: bool | None = None,
                 fused_ops: bool | None = None, prefix_caching: bool = False, lookahead: bool = False):
        if model.device.type != "cuda":
            raise ValueError("nanoserve_b200 engines run on a CUDA device only")
        if kv_cache != "paged":
            raise ValueError(f"kv_cache={kv_cache!r}: this engine has the paged KV cache only")
        if attn_backend not in (None, "native", "triton"):     # "triton" = the reference's name for its fast path
            raise ValueError(f"attn_backend={attn_backend!r}: the ragged paged-attention kernel is the only backend "
                             "(the SDPA restatement used for parity lives in oracle/)")
        if fused_ops is False:
            raise ValueError("fused_ops=False: the engine path always runs the fused kernels "
                             "(Qwen2Model.forward_batch still offers the unfused ops for comparisons)")
        self.attn_backend = "native"
        self.lookahead = bool(lookahead)
        self._pending = None        # lookahead: (fetch handle, [(seq, index into output_ids, row, finished)])
        self.eos_token_ids = list(eos_token_ids)
        self._eos = set(self.eos_token_ids)
        self.max_seq_len = max_seq_len
        budget = kv_cache_tokens if kv_cache_tokens is not None else 32 * max_seq_len
        self.model = model if model.fused else model.with_fused_ops()
        max_seats = max(max_num_seqs, 1)
        self.kv = PagedKVManager(model.cfg, budget, block_size, device=model.device, dtype=model.dtype,
                                 attn_backend="native", prefix_caching=prefix_caching, max_seats=max_seats)
        if chunked_prefill is None:
            chunked_prefill = True
        if not chunked_prefill:
            # a preempted request re-prefills prompt + outputs in one step (nanoserve/engine.py:90-93)
            max_num_batched_tokens = max(max_num_batched_tokens, max_seq_len)
        self.chunked_prefill = bool(chunked_prefill)
        self.scheduler = Scheduler(policy, max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens,
                                   batch_wait_s=batch_wait_s, kv=self.kv, chunked_prefill=self.chunked_prefill)
        if cuda_graphs is None:
            cuda_graphs = True
        if piecewise_graphs is None:
            piecewise_graphs = bool(cuda_graphs)
        # the garbage block is the first allocation, as in the reference (nanoserve/cuda_graphs.py:48)
        self._garbage_block = self.kv.pool.allocator.allocate() if (cuda_graphs or piecewise_graphs) else 0
        # sequence rows of the static buffers: max_num_seqs rounded up to a decode bucket
        seq_cap = next((b for b in BUCKETS if b >= max_num_seqs), max_num_seqs)
        step_tokens = max_num_batched_tokens + seq_cap
        self.buffers = StepBuffers(self.model, self.kv.pool, max_seqs=seq_cap, max_tokens=step_tokens,
                                   max_seq_len=max_seq_len, garbage_block=self._garbage_block, max_seats=max_seats)
        self.graph_runner = None
        if cuda_graphs:
            self.graph_runner = DecodeGraphRunner(self.model, self.kv.pool, max_seq_len, max_batch=seq_cap,
                                                  buffers=self.buffers)
            if seq_cap not in self.graph_runner.buckets:          # more than the largest default bucket
                self.graph_runner.buckets.append(seq_cap)
                self.graph_runner.max_bucket = seq_cap
        self.piecewise_runner = None
        if piecewise_graphs:
            self.piecewise_runner = PiecewiseGraphRunner(self.model, self.kv.pool, self._garbage_block,
                                                         max_tokens=step_tokens, buffers=self.buffers,
                                                         buckets=step_buckets(step_tokens), max_seqs=seq_cap,
                                                         max_seq_len=max_seq_len)
        self.sequences: dict[int, Sequence] = {}
        self.last_step: StepStats | None = None
        # logits [sequences, vocab] of the newest step, rows in scheduling order: a view of a static graph output,
        # valid until that graph is replayed again
        self.last_logits: torch.Tensor | None = None
        self._next_id = 0
        self._stats = {"steps": 0, "graph_steps": 0, "piecewise_steps": 0, "prefill_chunks": 0, "peak_running": 0,
                       "kv_used_tokens_peak": 0, "kv_reserved_tokens_peak": 0, "kv_util_sum": 0.0,
                       "kv_util_samples": 0}

    # ---- bookkeeping --------------------------------------------------------------------------------------------
    def reset_stats(self) -> None:
        for k, v in self._stats.items():
            self._stats[k] = 0.0 if isinstance(v, float) else 0
        self.scheduler.num_preemptions = 0
        self.kv.reset_stats()

    @property
    def stats(self) -> dict:
        s = dict(self._stats)
        s["num_preemptions"] = self.scheduler.num_preemptions
        s["kv_util_mean"] = s["kv_util_sum"] / s["kv_util_samples"] if s["kv_util_samples"] else None
        s["kv_cache"] = self.kv.kind
        s["attn_backend"] = self.attn_backend
        s["cuda_graphs"] = self.graph_runner is not None
        s["graph_buckets"] = self.graph_runner.captured_buckets if self.graph_runner else []
        s["piecewise_graphs"] = self.piecewise_runner is not None
        s["fused_ops"] = self.model.fused
        s["prefix_caching"] = self.kv.prefix_caching
        s["prefix_query_tokens"] = self.kv.prefix_query_tokens
        s["prefix_hit_tokens"] = self.kv.prefix_hit_tokens
        s["piecewise_buckets"] = self.piecewise_runner.captured_buckets if self.piecewise_runner else []
        return s

    def capture_graphs(self) -> float:
        """Capture every graph this engine can use now, so no request pays for a capture mid-run."""
        t0 = time.perf_counter()
        if self.graph_runner is not None:
            self.graph_runner.capture_all(self.scheduler.max_num_seqs)
        if self.piecewise_runner is not None:
            self.piecewise_runner.capture_all()
        torch.cuda.synchronize()
        return time.perf_counter() - t0

    def add_request(self, prompt_ids: list[int], max_new_tokens: int, ignore_eos: bool = False,
                    arrival_time: float | None = None, sampling=None) -> int:
        if len(prompt_ids) + max_new_tokens > self.max_seq_len:
            raise ValueError(f"prompt ({len(prompt_ids)}) + max_new_tokens ({max_new_tokens}) "
                             f"exceeds max_seq_len ({self.max_seq_len})")
        seed = sampling.seed if (sampling is not None and getattr(sampling, "seed", None) is not None) \
            else random.getrandbits(62)
        seq = Sequence(seq_id=self._next_id, prompt_ids=list(prompt_ids), max_new_tokens=max_new_tokens,
                       ignore_eos=ignore_eos,
                       arrival_time=time.perf_counter() if arrival_time is None else arrival_time,
                       sampling=sampling, seed=seed)
        self.scheduler.add(seq)
        self.sequences[seq.seq_id] = seq
        self._next_id += 1
        return seq.seq_id

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._pending is not None

    def abort(self, seq_id: int) -> None:
        seq = self.sequences.pop(seq_id, None)
        if seq is not None:
            self.scheduler.abort(seq)

    # ---- one step -----------------------------------------------------------------------------------------------
    _UNKNOWN = -1                  # stands in output_ids for a token that was sampled but not yet read back

    def step(self) -> list[StepOutput]:
        if self.timing is not None:
            self.timing["_step_start"] = time.perf_counter()
        outputs: list[StepOutput] = []
        plan = self.scheduler.schedule(now=time.perf_counter())
        scheduled, chunks = plan.scheduled, plan.chunks
        if not scheduled:
            self.last_step = None
            return self._resolve_pending(outputs)
        self._mark("schedule")
        if self._pending is not None and self._needs_unknown_token(scheduled, chunks):
            self._resolve_pending(outputs)             # a re-prefill is about to read a token id from the host lists
        records, appends, token_ids = self.kv.step_records(scheduled, chunks)
        n_seqs, n_tokens = len(scheduled), sum(chunks)
        n_prefill = sum(1 for s in scheduled if s.is_prefill)
        self.last_step = StepStats(n_prefill=n_prefill, n_decode=n_seqs - n_prefill, n_tokens=n_tokens)
        self._mark("prepare", gpu_start=True)

        runner, pw, buf = self.graph_runner, self.piecewise_runner, self.buffers
        # draw n of request r is keyed by mix_seed(seed_r, n), n = tokens generated so far: the same text whatever the
        # batch, and across a preemption + recompute (nanoserve/engine.py:233-237)
        buf.set_sampling([(row, s.sampling.temperature, s.sampling.top_p, s.sampling.top_k, mix_seed(s.seed, len(s.output_ids)))
                          for row, (s, n) in enumerate(zip(scheduled, chunks))
                          if s.sampling is not None and not s.sampling.greedy and s.num_cached + n >= s.num_tokens])
        if runner is not None and n_tokens == n_seqs and n_seqs <= runner.max_bucket:
            self.last_logits = runner.run_packed(records, appends, token_ids)   # every sequence feeds one token
            self._stats["graph_steps"] += 1
            path = ("decode", runner.last_key)
        elif pw is not None and pw.fits(n_tokens, n_seqs):
            self.last_logits = pw.run_packed(records, appends, token_ids)
            self._stats["piecewise_steps"] += 1
            path = ("mixed", pw.last_key)
        else:
            buf.upload(records, appends, token_ids, pad_seqs=n_seqs, pad_tokens=n_tokens)
            self.last_logits = buf.step(n_tokens, n_seqs, decode_only=False)
            path = ("eager", (n_tokens, n_seqs))
        if self.step_log is not None:                                # device-resident replay (see replay_on_device)
            self.step_log.append((path, buf.host_packed[:buf.packed_ints].clone()))
        handle = buf.queue_fetch(n_seqs)                             # greedy; one read-back for the whole batch
        self._mark("launch", gpu_end=True)
        self._resolve_pending(outputs)                               # the previous step's tokens, if still out
        run_ahead = self.lookahead and all(s.ignore_eos for s, n in zip(scheduled, chunks)
                                           if s.num_cached + n >= s.num_tokens)
        try:
            next_tokens = None if run_ahead else buf.wait_fetch(handle)
        except DeviceStatusError:
            self._abort_all()
            raise
        self._mark("wait")

        for seq, n in zip(scheduled, chunks):
            self.kv.commit(seq, n)
            seq.num_cached += n
        self._record_stats(scheduled)
        eos = self._eos
        entries = []
        for row, seq in enumerate(scheduled):
            if seq.num_cached < seq.num_tokens:
                self._stats["prefill_chunks"] += 1                   # mid-prompt chunk: nothing to sample
                seq.token_on_device = False
                continue
            tok = self._UNKNOWN if run_ahead else next_tokens[row]
            seq.output_ids.append(tok)
            seq.token_on_device = True
            finished = (tok in eos and not seq.ignore_eos) or len(seq.output_ids) >= seq.max_new_tokens
            if finished:
                self.scheduler.finish(seq)
                del self.sequences[seq.seq_id]
            if run_ahead:
                entries.append((seq, len(seq.output_ids) - 1, row, finished))
            else:
                outputs.append(StepOutput(seq.seq_id, tok, finished))
        if run_ahead:
            self._pending = (handle, entries)
        self._mark("post")
        return outputs

    def _resolve_pending(self, outputs: list[StepOutput]) -> list[StepOutput]:
        """Wait for the tokens of the step in flight (if any), put them where their stand-ins are, and append that
        step's outputs."""
        if self._pending is not None:
            handle, entries = self._pending
            self._pending = None
            try:
                tokens = self.buffers.wait_fetch(handle)
            except DeviceStatusError:
                self._abort_all()
                raise
            for seq, at, row, finished in entries:
                if not finished and seq.seq_id not in self.sequences:
                    continue                                   # aborted while its token was on the way back
                seq.output_ids[at] = tokens[row]
                outputs.append(StepOutput(seq.seq_id, tokens[row], finished))
        return outputs

    def _abort_all(self) -> None:
        """A step's results are undefined (the device reported a failed wait): drop every request and free its KV
        blocks, as the reference's engine process does when a step raises (nanoserve/engine_process.py:139-149)."""
        self._pending = None
        for seq_id in list(self.sequences):
            self.abort(seq_id)

    def _needs_unknown_token(self, scheduled, chunks) -> bool:
        """True if this step's packed record would carry the value of a token that is still on its way back: a
        sequence whose newest output is a stand-in and which does not feed it from the device's last_tokens."""
        unknown = self._UNKNOWN
        for seq, n in zip(scheduled, chunks):
            if seq.output_ids and seq.output_ids[-1] == unknown and seq.num_cached + n >= seq.num_tokens \
                    and not (n == 1 and seq.token_on_device and seq.remaining == 1):
                return True
        return False

    # ---- device-resident replay -------------------------------------------------------------------------------------
    step_log: list | None = None      # set to [] to record (path, packed step buffer) of every step

    def replay_on_device(self, log: list) -> float:
        """Re-run recorded steps with every input already in HBM and no host round trip: the packed step buffers are
        uploaded beforehand, each step copies its buffer device-to-device and replays its graph; sampled tokens stay on
        the device (last_tokens). Returns the elapsed device time in seconds (CUDA events). The KV pool is overwritten
        exactly as in the recorded run. Used to separate kernel throughput from host overhead."""
        buf = self.buffers
        sizes = [p.numel() for _, p in log]
        resident = torch.cat([p for _, p in log]).to(buf.dev_packed.device)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        off = 0
        for (kind, key), n in zip((p for p, _ in log), sizes):
            buf.dev_packed[:n].copy_(resident[off:off + n], non_blocking=True)
            off += n
            if kind == "decode":
                self.graph_runner.replay(key)
            elif kind == "mixed":
                self.piecewise_runner.replay(key)
            else:
                buf.step(key[0], key[1], decode_only=False)
        ev1.record()
        torch.cuda.synchronize()
        return ev0.elapsed_time(ev1) / 1e3

    # ---- optional per-phase timing (off unless `engine.timing = {}`) ----------------------------------------------
    timing: dict | None = None

    def _mark(self, phase: str, gpu_start: bool = False, gpu_end: bool = False) -> None:
        T = self.timing
        if T is None:
            return
        now = time.perf_counter()
        if phase == "schedule":
            if "_step_start" in T:
                T[phase] = T.get(phase, 0.0) + now - T["_step_start"]
        elif T.get("_last") is not None:
            T[phase] = T.get(phase, 0.0) + now - T["_last"]
        T["_last"] = now
        if gpu_start:
            T["_ev0"] = torch.cuda.Event(enable_timing=True)
            T["_ev0"].record()
        if gpu_end:
            T["_ev1"] = torch.cuda.Event(enable_timing=True)
            T["_ev1"].record()
        if phase == "post":
            # with a step in flight (lookahead) nothing has synchronised yet: keep the event pair and add its time once
            # the device has passed it
            T.setdefault("_evs", []).append((T["_ev0"], T["_ev1"]))
            waiting = []
            for e0, e1 in T["_evs"]:
                if e1.query():
                    T["gpu"] = T.get("gpu", 0.0) + e0.elapsed_time(e1) / 1e3
                else:
                    waiting.append((e0, e1))
            T["_evs"] = waiting
            T["steps"] = T.get("steps", 0) + 1

    def _record_stats(self, running: list[Sequence]) -> None:
        st = self._stats
        st["steps"] += 1
        st["peak_running"] = max(st["peak_running"], len(running))
        used, reserved = self.kv.usage(running)
        st["kv_used_tokens_peak"] = max(st["kv_used_tokens_peak"], used)
        st["kv_reserved_tokens_peak"] = max(st["kv_reserved_tokens_peak"], reserved)
        if reserved:
            st["kv_util_sum"] += used / reserved
            st["kv_util_samples"] += 1
