"""`LLMEngine(lookahead=True)` keeps one step in flight. Gates: with every request submitted up front the scheduler's
decisions (ids, chunks, block tables) and the tokens are IDENTICAL to the engine without the option, under preemption
and prefix caching too; sequences that can stop on an end-of-sequence token fall back to waiting and stop on the same
token; no stand-in token is ever returned; no KV block leaks. Tokens are also checked against the CPU oracle."""
import random

import pytest
import torch

from oracle.engine import OracleEngine, OracleModel, run_requests
from tests.golden import make_golden as G
from tests.test_engine_gpu import gpu_model, make_engine, run_traced

pytestmark = pytest.mark.gpu


def drive(eng, requests, ignore_eos, concurrency=None):
    """Closed loop over add_request/step; returns ({request: tokens}, {request: finished flags})."""
    todo = list(enumerate(requests))
    idx_of, toks, flags = {}, {}, {}
    limit = concurrency or len(requests)

    def submit():
        i, (prompt, max_new) = todo.pop(0)
        idx_of[eng.add_request(prompt, max_new, ignore_eos=ignore_eos(i))] = i
        toks[i], flags[i] = [], []

    while todo and len(idx_of) < limit:
        submit()
    calls = 0
    while eng.has_unfinished():
        calls += 1
        assert calls < 100000
        for o in eng.step():
            toks[idx_of[o.seq_id]].append(o.token)
            flags[idx_of[o.seq_id]].append(o.finished)
            if o.finished and todo:
                submit()
    return toks, flags


@pytest.mark.parametrize("kw", [
    dict(G.TINY_ENGINE_KW),
    dict(max_seq_len=128, max_num_seqs=6, max_num_batched_tokens=48, kv_cache_tokens=256),            # preempts
    dict(max_seq_len=128, max_num_seqs=3, max_num_batched_tokens=32, kv_cache_tokens=512, prefix_caching=True),
])
def test_lookahead_changes_no_decision_and_no_token(kw):
    cfg, sd = G.TINY_CFG, G.tiny_state_dict(G.TINY_CFG)
    rng = random.Random(11)
    prefix = [rng.randrange(512) for _ in range(40)]
    reqs = [(prefix + [rng.randrange(512) for _ in range(rng.randint(2, 30))], rng.randint(4, 30)) for _ in range(8)]
    model = gpu_model(cfg, sd, torch.float32)
    plain = make_engine(model, **kw)
    ahead = make_engine(model, lookahead=True, **kw)
    a, ta = run_traced(plain, reqs, None)
    b, tb = run_traced(ahead, reqs, None)
    assert len(ta) == len(tb)
    for x, y in zip(ta, tb):
        assert x["ids"] == y["ids"] and x["chunks"] == y["chunks"] and x["tables"] == y["tables"]
    assert a == b
    assert all(t >= 0 for out in b for t in out) and [len(o) for o in b] == [n for _, n in reqs]
    assert plain.stats["num_preemptions"] == ahead.stats["num_preemptions"]
    assert ahead.kv.num_free_blocks == plain.kv.num_free_blocks
    assert not ahead.has_unfinished() and ahead._pending is None
    okw = {k: v for k, v in kw.items()}
    oracle = OracleEngine(OracleModel(cfg, sd), reserve_garbage_block=True, **okw)
    want = run_requests(oracle, reqs)
    assert all(b[i] == want[i] for i in range(len(reqs))) or min(oracle.logits_gap) <= 1e-3


def test_lookahead_closed_loop_tokens_equal_the_oracle():
    cfg, sd = G.TINY_CFG, G.tiny_state_dict(G.TINY_CFG)
    reqs = G.tiny_requests()
    oracle = OracleEngine(OracleModel(cfg, sd), reserve_garbage_block=True, **G.TINY_ENGINE_KW)
    want = run_requests(oracle, reqs, concurrency=4)
    eng = make_engine(gpu_model(cfg, sd, torch.float32), lookahead=True, **G.TINY_ENGINE_KW)
    got, flags = drive(eng, reqs, lambda i: True, concurrency=4)
    # refills reach the engine one call later than without lookahead, so step composition differs; tokens do not
    assert all(got[i] == want[i] for i in range(len(reqs))) or min(oracle.logits_gap) <= 1e-3
    assert all(f[-1] and not any(f[:-1]) for f in flags.values())
    assert eng.kv.num_free_blocks == eng.kv.pool.num_blocks - 1


def test_lookahead_waits_for_sequences_that_can_hit_eos():
    from nanoserve_b200.engine import LLMEngine
    cfg, sd = G.TINY_CFG, G.tiny_state_dict(G.TINY_CFG)
    rng = random.Random(5)
    reqs = [([rng.randrange(512) for _ in range(rng.randint(5, 40))], 24) for _ in range(8)]
    model = gpu_model(cfg, sd, torch.float32)
    free_run, _ = drive(make_engine(model, **G.TINY_ENGINE_KW), reqs, lambda i: True)
    # stop tokens taken from the middle of what the odd requests generate, so they do stop early
    eos = sorted({free_run[i][len(free_run[i]) // 2] for i in range(1, len(reqs), 2)})
    mixed = lambda i: i % 2 == 0                  # even requests ignore eos (and run ahead when a step has only them)
    plain = LLMEngine(model, eos_token_ids=eos, **G.TINY_ENGINE_KW)
    ahead = LLMEngine(model, eos_token_ids=eos, lookahead=True, **G.TINY_ENGINE_KW)
    a, fa = drive(plain, reqs, mixed)
    b, fb = drive(ahead, reqs, mixed)
    assert a == b and fa == fb
    assert any(len(a[i]) < 24 for i in range(1, len(reqs), 2))          # somebody did stop on eos
    assert all(a[i][-1] in eos or len(a[i]) == 24 for i in range(1, len(reqs), 2))
    assert all(len(a[i]) == 24 for i in range(0, len(reqs), 2))
    assert ahead.kv.num_free_blocks == plain.kv.num_free_blocks
