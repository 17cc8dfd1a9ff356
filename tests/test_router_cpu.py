"""Engine process + replica router, host side only (CPU stub engines in real child processes).

Failures are made on the host, as the request stream asks for them: a step that raises (every in-flight request of that
engine fails, its KV comes back, the engine keeps serving); a child that dies without a word (every open stream of that
replica raises, the router stops sending it work, the other replica carries on); a parent that closes the pipe (the
child leaves by itself)."""
import asyncio
import random
import time

import pytest

from nanoserve_b200.engine_process import EngineProcess, EngineSpec
from nanoserve_b200.replicas import ReplicaRouter, serve_closed_loop
from tests.stub_engine import DIE_TOKEN, RAISE_TOKEN, stub_token


def spec(**args):
    return EngineSpec(factory="tests.stub_engine:make_stub", factory_args=args, max_num_seqs=8)


def requests(n, seed=0):
    rng = random.Random(seed)
    return [([rng.randrange(1000) for _ in range(rng.randint(3, 40))], rng.randint(2, 12)) for _ in range(n)]


def expected(reqs):
    return {i: [stub_token(p, k) for k in range(n)] for i, (p, n) in enumerate(reqs)}


def test_router_serves_one_stream_over_two_replicas():
    router = ReplicaRouter([spec(step_s=0.002), spec(step_s=0.002)])
    try:
        reqs = requests(40)
        tokens, failed = serve_closed_loop(router, reqs, concurrency=8, timeout_s=60)
        assert not failed and tokens == expected(reqs)
        assert sum(router.dispatched) == 40 and min(router.dispatched) >= 12      # least-outstanding keeps both busy
        for st in router.stats():
            assert st["unfinished"] is False and st["num_free_blocks"] == 1000
    finally:
        router.close()


def test_a_step_exception_fails_that_replicas_requests_and_frees_their_kv():
    router = ReplicaRouter([spec(), spec()])
    try:
        good = requests(6, seed=1)
        ids = [router.submit(p, 50, ignore_eos=True) for p, _ in good[:4]]        # long requests on both replicas
        bad = router.submit([1, 2, RAISE_TOKEN], 5, ignore_eos=True)
        where = dict(router._where)
        bad_replica = where[bad][0]
        deadline = time.monotonic() + 20
        failed, finished = {}, set()
        while time.monotonic() < deadline and (bad not in failed or len(finished) + len(failed) < 5):
            for gid, item, _, fin in router.poll(timeout_s=0.05):
                if isinstance(item, BaseException):
                    failed[gid] = item
                elif fin:
                    finished.add(gid)
        assert bad in failed and "injected step failure" in str(failed[bad])
        same_replica = {g for g in ids if where[g][0] == bad_replica}
        assert same_replica <= set(failed) and not (set(failed) - same_replica - {bad})   # neighbours on that engine fail too, nobody else
        assert finished == set(ids) - same_replica
        st = router.stats()
        assert st[bad_replica]["num_free_blocks"] == 1000 and st[bad_replica]["unfinished"] is False
        # the replica that raised keeps serving
        more = requests(10, seed=2)
        tokens, failed2 = serve_closed_loop(router, more, concurrency=4, timeout_s=30)
        assert not failed2 and tokens == expected(more) and min(router.dispatched) > 2
    finally:
        router.close()


def test_a_killed_child_fails_its_streams_and_leaves_the_rotation():
    router = ReplicaRouter([spec(), spec()])
    try:
        ids = [router.submit(p, 200, ignore_eos=True) for p, _ in requests(4, seed=3)]
        where = dict(router._where)
        killer = router.submit([DIE_TOKEN], 3, ignore_eos=True)
        dead = router._where[killer][0]
        deadline = time.monotonic() + 20
        failed, finished = {}, set()
        while time.monotonic() < deadline and len(failed) + len(finished) < 5:
            for gid, item, _, fin in router.poll(timeout_s=0.05):
                if isinstance(item, BaseException):
                    failed[gid] = item
                elif fin:
                    finished.add(gid)
        on_dead = {g for g in ids if where[g][0] == dead} | {killer}
        assert set(failed) == on_dead and all("engine process exited" in str(e) for e in failed.values())
        assert finished == set(ids) - on_dead
        assert router.alive == [1 - dead]
        more = requests(8, seed=4)
        tokens, failed2 = serve_closed_loop(router, more, concurrency=4, timeout_s=30)
        assert not failed2 and tokens == expected(more)
        assert router.stats()[dead] is None
        # the last replica dies too: submit has nowhere to go
        router.submit([DIE_TOKEN], 3, ignore_eos=True)
        deadline = time.monotonic() + 20
        while router.alive and time.monotonic() < deadline:
            router.poll(timeout_s=0.05)
        with pytest.raises(RuntimeError, match="no replica is alive"):
            router.submit([1, 2, 3], 4)
    finally:
        router.close()


def test_a_closed_pipe_ends_the_child():
    ep = EngineProcess(spec())
    ep._req_w.close()                       # the parent goes away without a stop message
    ep._proc.join(timeout=10)
    assert ep._proc.exitcode == 0
    deadline = time.monotonic() + 5
    while ep.alive and time.monotonic() < deadline:
        time.sleep(0.01)
    assert not ep.is_alive()
    with pytest.raises(RuntimeError, match="engine process exited"):
        ep.submit([1], 1, lambda *a: None)


def test_generate_streams_tokens_and_an_early_exit_aborts():
    ep = EngineProcess(spec(step_s=0.001))
    try:
        async def run():
            prompt = [5, 6, 7]
            got = [tok async for tok, _ in ep.generate(prompt, 6, ignore_eos=True)]
            assert got == [stub_token(prompt, k) for k in range(6)]
            n = 0
            async for _tok, _t in ep.generate(prompt, 1000, ignore_eos=True):
                n += 1
                if n == 3:
                    break
            with pytest.raises(ValueError):
                async for _ in ep.generate([1] * 5000, 10):
                    pass
        asyncio.run(run())
        deadline = time.monotonic() + 10
        while time.monotonic() < deadline:
            st = ep.stats()
            if not st["unfinished"]:
                break
            time.sleep(0.01)
        assert st["unfinished"] is False and st["num_aborted"] == 1 and st["num_free_blocks"] == 1000
    finally:
        ep.close()
