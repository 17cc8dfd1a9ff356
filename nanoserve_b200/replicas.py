"""Request-level replicas: one independent engine per GPU, no collective on the data path.

The reference is single-GPU; its process-per-engine pattern (nanoserve/engine_process.py:160-170) is what scaling by
replicas reuses. Nothing is exchanged between replicas while they serve.

`ReplicaRouter` is the serving form: ONE request stream in, one engine process per GPU (`EngineProcess`), each request
sent to the replica with the fewest requests in flight. The helpers below it (max / sum over ranks) are the bookkeeping
of the torchrun form of the benchmark, where every rank runs its own engine and its own stream: a barrier, and the
maximum over ranks of each rank's elapsed time.
"""
from __future__ import annotations

import queue
import threading

from nanoserve_b200.engine_process import EngineProcess, EngineSpec


class ReplicaRouter:
    """Least-outstanding dispatch of one request stream over N engine processes.

    submit() returns a router-wide request id; events come back through ONE queue (one entry per engine step of a
    replica), drained with poll():
    (request id, token, timestamp, finished) per token and (request id, exception, None, True) when a request fails.
    A replica whose process dies fails its own in-flight requests ("engine process exited"), is taken out of the
    rotation, and the others keep serving; submit() raises once no replica is left. A step that raises inside a replica
    fails that replica's in-flight requests only and the replica keeps serving (nanoserve/engine_process.py:139-149).
    Ties between equally loaded replicas go round-robin, so an idle router spreads its first requests evenly."""

    def __init__(self, specs: list[EngineSpec], start_timeout_s: float = 900.0):
        if not specs:
            raise ValueError("a router needs at least one replica")
        self.events: queue.SimpleQueue = queue.SimpleQueue()
        self._lock = threading.Lock()
        self._next = 0
        self._rr = 0
        self._where: dict[int, tuple[int, int]] = {}          # router id -> (replica, replica-local id)
        self._local: list[dict[int, int]] = [dict() for _ in specs]     # replica-local id -> router id
        self.replicas: list[EngineProcess] = []
        self.dispatched = [0] * len(specs)
        started: list = [None] * len(specs)
        errors: list = []

        def start(i, spec):
            try:
                started[i] = EngineProcess(spec, start_timeout_s)
            except BaseException as e:                          # noqa: BLE001 - reported below
                errors.append((i, e))

        threads = [threading.Thread(target=start, args=(i, s)) for i, s in enumerate(specs)]   # engines build side by side
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            for ep in started:
                if ep is not None:
                    ep.close(timeout_s=5)
            i, e = errors[0]
            raise RuntimeError(f"replica {i} failed to start: {e}") from e
        self.replicas = started
        self._index = {id(r): i for i, r in enumerate(started)}
        for r in started:
            r.on_batch = self._on_batch

    @property
    def alive(self) -> list[int]:
        return [i for i, r in enumerate(self.replicas) if r.is_alive()]

    def outstanding(self, i: int) -> int:
        return len(self._local[i])

    def _pick(self) -> int:
        live = self.alive
        if not live:
            raise RuntimeError("no replica is alive")
        n = len(self.replicas)
        order = sorted(live, key=lambda i: (len(self._local[i]), (i - self._rr) % n))
        self._rr = (order[0] + 1) % n
        return order[0]

    def submit(self, prompt_ids: list[int], max_new_tokens: int, ignore_eos: bool = False, sampling=None) -> int:
        with self._lock:
            gid = self._next
            self._next += 1
            for _ in range(len(self.replicas)):
                i = self._pick()
                try:
                    # the replica's reader thread may see this request's first tokens before submit() returns its id:
                    # _on_batch resolves ids through _local under this same lock
                    lid = self.replicas[i].submit(prompt_ids, max_new_tokens, None, ignore_eos, sampling)
                except RuntimeError:
                    continue                                    # died between the check and the send: try the next one
                self._where[gid] = (i, lid)
                self._local[i][lid] = gid
                self.dispatched[i] += 1
                return gid
            raise RuntimeError("no replica is alive")

    def _on_batch(self, replica: EngineProcess, events: list) -> None:
        """One engine step's events of one replica: replica-local ids become router ids, one queue entry per step."""
        i = self._index[id(replica)]
        local = self._local[i]
        out = []
        with self._lock:
            for lid, item, t, finished in events:
                gid = local.get(lid)
                if gid is None:
                    continue
                if finished:
                    del local[lid]
                    del self._where[gid]
                out.append((gid, item, t, finished))
        if out:
            self.events.put(out)

    def abort(self, gid: int) -> None:
        with self._lock:
            where = self._where.pop(gid, None)
            if where is not None:
                del self._local[where[0]][where[1]]
        if where is not None:
            self.replicas[where[0]].abort(where[1])

    def poll(self, timeout_s: float | None = None) -> list[tuple]:
        """Every event that has arrived; blocks up to timeout_s for the first one (None = do not block)."""
        out = []
        try:
            if timeout_s:
                out.extend(self.events.get(timeout=timeout_s))
            while True:
                out.extend(self.events.get_nowait())
        except queue.Empty:
            pass
        return out

    def stats(self) -> list[dict | None]:
        return [r.stats() if r.is_alive() else None for r in self.replicas]

    def close(self) -> None:
        for r in self.replicas:
            r.close()


def serve_closed_loop(router: ReplicaRouter, requests: list, concurrency: int, timeout_s: float = 600.0):
    """Closed loop over a router in the shape of the reference's bare-loop probe (bench/runs/m11_loop_profile.py:41-59):
    keep `concurrency` requests in flight over ALL replicas, refill when one finishes. requests = [(prompt_ids,
    max_new)]. Returns ({request index: tokens}, {request index: exception})."""
    import time
    todo = list(enumerate(requests))
    todo.reverse()
    index_of: dict[int, int] = {}
    tokens: dict[int, list[int]] = {}
    failed: dict[int, BaseException] = {}

    def submit_next():
        i, (prompt, max_new) = todo.pop()
        tokens[i] = []
        index_of[router.submit(prompt, max_new, ignore_eos=True)] = i

    while todo and len(index_of) < concurrency:
        submit_next()
    deadline = time.monotonic() + timeout_s
    while index_of:
        events = router.poll(timeout_s=0.05)
        if not events and time.monotonic() > deadline:
            raise TimeoutError(f"{len(index_of)} requests still in flight after {timeout_s} s")
        for gid, item, _, finished in events:
            i = index_of.get(gid)
            if i is None:
                continue
            if isinstance(item, BaseException):
                failed[i] = item
            else:
                tokens[i].append(item)
            if finished:
                del index_of[gid]
                if todo:
                    try:
                        submit_next()
                    except RuntimeError as e:                   # no replica left: fail what was never sent
                        while todo:
                            j, _ = todo.pop()
                            failed[j] = e
    return tokens, failed


def _dist():
    import torch.distributed as dist
    return dist


def max_over_ranks(seconds: list[float], device="cpu") -> list[float]:
    """Element-wise maximum over all ranks of a short list of timings (identity without a process group)."""
    import torch
    dist = _dist()
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(seconds)
    t = torch.tensor(seconds, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def sum_over_ranks(counts: list[float], device="cpu") -> list[float]:
    """Element-wise sum over all ranks of a short list of counts (identity without a process group): replicas serve
    different request streams, so their token counts differ."""
    import torch
    dist = _dist()
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(counts)
    t = torch.tensor(counts, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t.tolist()


def aggregate_throughput(units_per_rank: int, seconds: float, device="cpu") -> tuple[float, float]:
    """Whole-job throughput of identical replicas: (world_size * units_per_rank / max-over-ranks seconds, that max)."""
    dist = _dist()
    world = dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1
    slowest = max_over_ranks([seconds], device)[0]
    return world * units_per_rank / slowest, slowest


def replica_seed(base_seed: int, rank: int) -> int:
    """Each replica serves its own request stream: a distinct, reproducible seed per rank."""
    return base_seed + 1000003 * rank
