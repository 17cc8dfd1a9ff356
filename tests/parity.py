"""Shared rule for comparing greedy token streams with a reference run.

A greedy decoder and its reference can only part ways at a step where the reference's two best logits are closer
than the numerical error of the path under test. Once they have parted the contexts differ, so only the FIRST
divergence of a request is judged, and it is judged by the reference's top-2 gap AT THAT REQUEST AND TOKEN, never
by a minimum over the whole run (the reference's own tests apply the tie rule per divergence point,
tests/test_llm_engine.py:1-17).
"""
from __future__ import annotations


def first_divergence(a, b):
    return next((k for k in range(min(len(a), len(b))) if a[k] != b[k]), None)


def check_tokens(got, want, gap_at, tie: float, first: int | None = None, what: str = "") -> tuple[int, list]:
    """got / want: token lists per request (same order); gap_at(i, j) = the reference's top-2 logit gap where request
    i sampled its j-th token; `first` limits the comparison to the first `first` tokens. Asserts that every request
    either equals the reference or first differs at a token whose reference gap is <= tie. Returns (number of
    identical requests, [(request, token index, gap)] of the accepted divergences)."""
    assert len(got) == len(want), f"{what}: {len(got)} requests, reference has {len(want)}"
    same, accepted = 0, []
    for i, (a, b) in enumerate(zip(got, want)):
        if first is not None:
            a, b = a[:first], b[:first]
        j = first_divergence(a, b)
        if j is None:
            assert len(a) == len(b), f"{what}: request {i} produced {len(a)} tokens, reference {len(b)}"
            same += 1
            continue
        gap = gap_at(i, j)
        assert gap <= tie, (f"{what}: request {i} diverges at token {j} ({a[j]} vs {b[j]}) where the reference's "
                            f"top-2 gap is {gap:.3e} > {tie:.1e}")
        accepted.append((i, j, gap))
    assert same + len(accepted) == len(want)
    return same, accepted


def run_lockstep(eng, oracle, requests, first: int | None = None):
    """Submits every request to the engine under test and to the CPU oracle engine, steps both together and compares,
    step by step, the logits row of every request that still shares the oracle's context (max-abs over the vocabulary).
    Both engines must take the same scheduling decisions (checked: same request ids per step). Returns (tokens per
    request from the engine, tokens from the oracle, worst logit error). `first` limits the logit comparison to each
    request's first `first` generated tokens."""
    oracle.keep_logits = True
    for prompt, max_new in requests:
        a = eng.add_request(prompt, max_new, ignore_eos=True)
        b = oracle.add_request(prompt, max_new, ignore_eos=True)
        assert a == b
    order: list[int] = []
    orig = eng.scheduler.schedule

    def spy(now):
        plan = orig(now)
        order[:] = [s.seq_id for s in plan.scheduled]
        return plan

    eng.scheduler.schedule = spy
    n = len(requests)
    got, want = [[] for _ in range(n)], [[] for _ in range(n)]
    parted: set[int] = set()
    worst = 0.0
    while eng.has_unfinished():
        outs = eng.step()
        ref_outs = oracle.step()
        assert order == oracle.trace[-1]["ids"], "the engine and the oracle scheduled different requests"
        logits = eng.last_logits.float().cpu()
        sampled = {o.seq_id for o in outs}
        for row, rid in enumerate(order):
            if rid in sampled and rid not in parted and (first is None or len(got[rid]) < first):
                worst = max(worst, (logits[row] - oracle.last_logits[rid].float()).abs().max().item())
        for rid, tok, _ in ref_outs:
            want[rid].append(tok)
        for o in outs:
            got[o.seq_id].append(o.token)
            k = len(got[o.seq_id]) - 1
            if k >= len(want[o.seq_id]) or want[o.seq_id][k] != o.token:
                parted.add(o.seq_id)
    assert not oracle.has_unfinished()
    return got, want, worst
