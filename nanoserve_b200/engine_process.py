"""The engine loop in its own process, one per GPU: the building block of request-level replicas.

Follows the reference's process split (nanoserve/engine_process.py:29-292): a picklable `EngineSpec`, a child started
with "spawn" that owns the GPU and runs add/abort/step in a loop, two one-way pipes, ONE message per engine step, and
the same failure rules - a step that raises fails every in-flight request of that engine, frees their KV and keeps the
engine serving; a child that dies makes every open stream raise.

What differs from the reference:
  * the child selects its GPU (`EngineSpec.device`, exported as CUDA_VISIBLE_DEVICES before CUDA is touched), so a
    parent can run one engine process per GPU; the reference always used "cuda" of its only device
    (nanoserve/engine_process.py:58,62);
  * weights are random-init of a named architecture or come from a factory ("package.module:function" returning an
    engine): checkpoints cannot be downloaded where this runs;
  * the parent side delivers events to plain callbacks, so it serves synchronous callers (the replica router, the
    benchmark loop) and asyncio callers (`generate`, the reference's interface) alike.

Nothing in this module imports torch at import time: the child must set CUDA_VISIBLE_DEVICES first.
"""
from __future__ import annotations

import importlib
import multiprocessing as mp
import os
import threading
import time
from dataclasses import dataclass, field


@dataclass
class EngineSpec:
    """Everything the child needs to build its engine (picklable: it crosses the process boundary)."""
    model: str = "qwen2.5-0.5b"          # an architecture of nanoserve_b200.synthetic.SHAPES (random-init weights)
    dtype: str = "bfloat16"
    seed: int = 0                        # weight seed
    device: int | None = None            # physical GPU index for this child; None = inherit the parent's visibility
    max_seq_len: int = 2048
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 2048
    kv_cache_tokens: int | None = None
    prefix_caching: bool = False
    lookahead: bool = False
    capture_graphs: bool = True          # capture every CUDA graph before serving
    n_layers: int | None = None          # shrink the architecture (tests)
    vocab: int | None = None
    factory: str | None = None           # "package.module:function": called with the spec, returns the engine
    factory_args: dict = field(default_factory=dict)


def build_engine(spec: EngineSpec):
    """The engine a spec describes; used by the child process and by in-process callers, so both build the same one."""
    if spec.factory:
        mod, _, fn = spec.factory.partition(":")
        return getattr(importlib.import_module(mod), fn)(spec)
    import torch
    from nanoserve_b200.engine import LLMEngine
    from nanoserve_b200.model import ModelConfig, Qwen2Model
    from nanoserve_b200.synthetic import random_state_dict
    sd, cfg = random_state_dict(spec.model, dtype=getattr(torch, spec.dtype), device="cuda", seed=spec.seed,
                                n_layers=spec.n_layers, vocab=spec.vocab)
    return LLMEngine(Qwen2Model(ModelConfig(**cfg), sd), eos_token_ids=[], max_seq_len=spec.max_seq_len,
                     max_num_seqs=spec.max_num_seqs, max_num_batched_tokens=spec.max_num_batched_tokens,
                     kv_cache_tokens=spec.kv_cache_tokens, prefix_caching=spec.prefix_caching, lookahead=spec.lookahead)


# ---------------------------------------------------------------------------------------------------- child process
def _child_stats(llm, num_aborted: int) -> dict:
    st = {"unfinished": llm.has_unfinished(), "num_aborted": num_aborted}
    kv = getattr(llm, "kv", None)
    if kv is not None and hasattr(kv, "num_free_blocks"):
        st["num_free_blocks"] = kv.num_free_blocks
    engine_stats = llm.stats
    st["engine"] = engine_stats() if callable(engine_stats) else engine_stats
    return st


def _portable(e: BaseException) -> BaseException:
    """Exceptions cross the pipe pickled; one that cannot be is replaced by a RuntimeError with its text."""
    import pickle
    try:
        pickle.loads(pickle.dumps(e))
        return e
    except Exception:
        return RuntimeError(f"{type(e).__name__}: {e}")


def _child_main(spec: EngineSpec, req_conn, out_conn) -> None:
    if spec.device is not None:
        os.environ["CUDA_VISIBLE_DEVICES"] = str(spec.device)       # before anything initialises CUDA
    try:
        llm = build_engine(spec)
        capture_s = llm.capture_graphs() if (spec.capture_graphs and hasattr(llm, "capture_graphs")) else 0.0
        out_conn.send(("ready", {"eos_token_ids": list(getattr(llm, "eos_token_ids", [])), "capture_s": capture_s,
                                 "pid": os.getpid()}))
    except BaseException as e:                                      # noqa: BLE001 - report, then leave
        out_conn.send(("fatal", f"{type(e).__name__}: {e}"))
        return
    rid_of: dict[int, int] = {}          # engine sequence id -> request id of the parent
    seq_of: dict[int, int] = {}          # request id -> engine sequence id
    num_aborted = 0
    while True:
        wait = 0.0 if llm.has_unfinished() else 0.05                # idle: block briefly instead of spinning
        try:
            while req_conn.poll(wait):
                wait = 0.0
                msg = req_conn.recv()
                kind = msg[0]
                if kind == "add":
                    _, rid, prompt, max_new, ignore_eos, t_arrival, sampling = msg
                    try:
                        kw = {"sampling": sampling} if sampling is not None else {}
                        sid = llm.add_request(prompt, max_new, ignore_eos=ignore_eos, arrival_time=t_arrival, **kw)
                    except Exception as e:                          # refused (too long, ...): tell the caller
                        out_conn.send(("error", [rid], _portable(e)))
                        continue
                    rid_of[sid], seq_of[rid] = rid, sid
                elif kind == "abort":
                    sid = seq_of.pop(msg[1], None)
                    if sid is not None:
                        llm.abort(sid)
                        del rid_of[sid]
                        num_aborted += 1
                elif kind == "stats":
                    out_conn.send(("stats", msg[1], _child_stats(llm, num_aborted)))
                elif kind == "stop":
                    return
        except (EOFError, OSError):                                 # the parent is gone
            return
        if not llm.has_unfinished():
            continue
        try:
            outputs = llm.step()
        except Exception as e:                                      # fail every in-flight request, keep serving
            out_conn.send(("error", list(seq_of), _portable(e)))
            for sid in list(rid_of):
                llm.abort(sid)
            rid_of.clear()
            seq_of.clear()
            continue
        if not outputs:
            if not getattr(llm, "lookahead", False):
                time.sleep(0.001)                                   # a policy that waits for a fuller batch
            continue
        t = time.perf_counter()
        batch = []
        for out in outputs:
            rid = rid_of.get(out.seq_id)
            if rid is None:                                         # aborted while its token was on the way back
                continue
            batch.append((rid, out.token, out.finished))
            if out.finished:
                del rid_of[out.seq_id], seq_of[rid]
        if batch:
            out_conn.send(("tokens", t, batch))


# --------------------------------------------------------------------------------------------------- parent process
class EngineProcess:
    """Parent-side handle of one engine child. Events of a request go to the callback given at `submit`:
    callback(rid, token, timestamp, finished) per token, callback(rid, exception, None, True) on failure; requests
    submitted without one are reported through `on_batch`, one list of such tuples per engine step (what the router uses:
    one hand-over per step, not per token). Both run on this object's reader thread and must not block. `generate` wraps
    the callback form for asyncio callers."""

    def __init__(self, spec: EngineSpec, start_timeout_s: float = 900.0):
        ctx = mp.get_context("spawn")
        req_r, self._req_w = ctx.Pipe(duplex=False)
        self._out_r, out_w = ctx.Pipe(duplex=False)
        self._proc = ctx.Process(target=_child_main, args=(spec, req_r, out_w), name="nanoserve-b200-engine", daemon=True)
        self._proc.start()
        req_r.close()                                               # the child holds its own copies
        out_w.close()
        if not self._out_r.poll(start_timeout_s):
            self._proc.kill()
            raise TimeoutError(f"engine process not ready after {start_timeout_s} s")
        try:
            kind, info = self._out_r.recv()
        except (EOFError, OSError):
            kind, info = "fatal", "engine process exited while starting"
        if kind != "ready":
            self._proc.join(timeout=5)
            raise RuntimeError(f"engine process failed to start: {info}")
        self.eos_token_ids: list[int] = info["eos_token_ids"]
        self.capture_s: float = info["capture_s"]
        self.pid: int = info["pid"]
        self._lock = threading.Lock()                               # guards _sinks, _next_rid and _req_w
        self._sinks: dict[int, object] = {}
        self._next_rid = 0
        self._stats_waiters: dict[int, list] = {}
        self.num_aborted = 0
        self.alive = True
        self.on_exit = None                                         # called once, from the reader thread, when the child is gone
        self.on_batch = None                                        # on_batch(self, [(rid, item, t, finished)]) for requests without a callback
        self._reader = threading.Thread(target=self._read_loop, name="nanoserve-b200-engine-reader", daemon=True)
        self._reader.start()

    def is_alive(self) -> bool:
        return self.alive and self._proc.is_alive()

    @property
    def outstanding(self) -> int:
        return len(self._sinks)

    # ---- requests
    def submit(self, prompt_ids: list[int], max_new_tokens: int, callback=None, ignore_eos: bool = False, sampling=None) -> int:
        with self._lock:
            if not self.alive:
                raise RuntimeError("engine process exited")
            rid = self._next_rid
            self._next_rid += 1
            self._sinks[rid] = callback
            try:
                self._req_w.send(("add", rid, list(prompt_ids), max_new_tokens, ignore_eos, time.perf_counter(), sampling))
            except (OSError, BrokenPipeError, ValueError) as e:
                del self._sinks[rid]
                raise RuntimeError("engine process exited") from e
        return rid

    def abort(self, rid: int) -> None:
        with self._lock:
            if self._sinks.pop(rid, None) is not None:
                self.num_aborted += 1
                try:
                    self._req_w.send(("abort", rid))
                except (OSError, BrokenPipeError, ValueError):
                    pass

    async def generate(self, prompt_ids: list[int], max_new_tokens: int, ignore_eos: bool = False, sampling=None):
        """Yield (token, timestamp) as the engine process produces them (the reference's interface,
        nanoserve/engine_process.py:199-230). Leaving the iterator early aborts the request and frees its KV."""
        import asyncio
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()

        def sink(rid, item, t, finished):
            try:
                loop.call_soon_threadsafe(q.put_nowait, (item, t, finished))
            except RuntimeError:
                pass                                                # that caller's loop has closed

        rid = self.submit(prompt_ids, max_new_tokens, sink, ignore_eos, sampling)
        done = False
        try:
            while True:
                item, t, finished = await q.get()
                if isinstance(item, BaseException):
                    done = True
                    raise item
                done = finished
                yield item, t
                if finished:
                    return
        finally:
            if not done:
                self.abort(rid)

    def stats(self, timeout_s: float = 30.0) -> dict:
        """Ask the child for its state (free KV blocks, unfinished work, abort count, engine counters)."""
        ev, box = threading.Event(), []
        with self._lock:
            key = self._next_rid
            self._next_rid += 1
            self._stats_waiters[key] = [ev, box]
            self._req_w.send(("stats", key))
        if not ev.wait(timeout_s):
            raise TimeoutError("engine process did not answer")
        if not box:
            raise RuntimeError("engine process exited")
        return box[0]

    # ---- reader thread
    def _deliver(self, events) -> None:
        """events: [(rid, item, t, finished)]; a stream ends at its first error or finished token. Requests submitted
        with a callback get one call per event; the others are handed to `on_batch` as one list per message."""
        calls, batch = [], []
        with self._lock:
            for ev in events:
                rid = ev[0]
                sink = self._sinks.get(rid, self)
                if sink is self:                                    # aborted meanwhile
                    continue
                if ev[3]:
                    del self._sinks[rid]
                if sink is None:
                    batch.append(ev)
                else:
                    calls.append((sink, ev))
        for sink, ev in calls:
            sink(*ev)
        if batch and self.on_batch is not None:
            self.on_batch(self, batch)

    def _read_loop(self) -> None:
        while True:
            try:
                msg = self._out_r.recv()
            except (EOFError, OSError):
                with self._lock:
                    self.alive = False
                    rids = list(self._sinks)
                self._deliver([(rid, RuntimeError("engine process exited"), None, True) for rid in rids])
                for ev, _ in list(self._stats_waiters.values()):
                    ev.set()
                if self.on_exit is not None:
                    self.on_exit(self)
                return
            kind = msg[0]
            if kind == "tokens":
                _, t, batch = msg
                self._deliver([(rid, tok, t, fin) for rid, tok, fin in batch])
            elif kind == "error":
                _, rids, exc = msg
                self._deliver([(rid, exc, None, True) for rid in rids])
            elif kind == "stats":
                _, key, st = msg
                with self._lock:
                    ev, box = self._stats_waiters.pop(key)
                box.append(st)
                ev.set()

    def close(self, timeout_s: float = 30.0) -> None:
        if self._proc.is_alive():
            try:
                with self._lock:
                    self._req_w.send(("stop",))
            except (OSError, BrokenPipeError, ValueError):
                pass
            self._proc.join(timeout=timeout_s)
            if self._proc.is_alive():
                self._proc.kill()
                self._proc.join(timeout=5)
        try:
            self._req_w.close()
        except OSError:
            pass
