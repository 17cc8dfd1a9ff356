"""Pin the CPU oracle against outputs of the reference itself (tests/golden/, made by make_golden.py)."""
import json
from pathlib import Path

import pytest
import torch

from oracle import ops as O
from oracle.engine import OracleEngine, OracleModel, run_requests
from tests.golden import make_golden as G
from tests.parity import check_tokens

GOLD = Path(__file__).parent / "golden"


def close(a, b, dtype):
    assert a.shape == b.shape and a.dtype == b.dtype
    if dtype == torch.float32:
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    else:   # same expressions on another CPU may round a sum differently: at most one bf16 ulp, nearly all equal
        assert (a == b).float().mean().item() >= 0.995
        torch.testing.assert_close(a.float(), b.float(), rtol=2 ** -7, atol=1e-6)


@pytest.mark.parametrize("name", ["f32", "bf16"])
def test_ops_match_reference_outputs(name):
    gold = torch.load(GOLD / "ops.pt")[name]
    d = G.ops_inputs()[name]
    dt = d["x"].dtype
    close(O.rms_norm(d["x"], d["w"], 1e-6), gold["rms_norm"], dt)
    out, summed = O.add_rms_norm(d["x"], d["w"], 1e-6, d["res"])
    assert torch.equal(summed, gold["add"])
    close(out, gold["add_rms_norm"], dt)
    close(O.silu_mul(d["gate_up"]), gold["silu_mul"], dt)
    cos, sin = O.rope_cos_sin(d["positions"], 64, 1_000_000.0, dt)
    close(cos, gold["cos"], dt)
    close(sin, gold["sin"], dt)
    q, k, v = O.rope_qkv(d["qkv"], gold["cos"], gold["sin"], 14, 2, 64)
    close(q, gold["rope_q"], dt)
    close(k, gold["rope_k"], dt)
    assert torch.equal(v, d["qkv"][:, 16 * 64:].view(37, 2, 64))


@pytest.mark.parametrize("name", ["f32", "bf16"])
def test_attention_matches_reference_paths(name):
    gold = torch.load(GOLD / "ops.pt")[name]
    d = G.ops_inputs()[name]
    tables = G.attn_tables(d["perm"])
    width = max(len(t) for t in tables)
    bt = torch.tensor([t + [0] * (width - len(t)) for t in tables], dtype=torch.int32)
    lens = torch.tensor(G.ATTN_LENS, dtype=torch.int32)
    tol = 1e-5 if name == "f32" else 1e-2
    dec = O.paged_attention_decode(d["q"][:4], d["k_pool"], d["v_pool"], bt, lens, 0.125)
    assert (dec.float() - gold["decode_ref"].float()).abs().max().item() <= tol
    cu = torch.tensor([0] + list(torch.tensor(G.ATTN_QLENS).cumsum(0)), dtype=torch.int32)
    rag = O.ragged_paged_attention(d["q"], d["k_pool"], d["v_pool"], bt, lens, cu, 0.125)
    assert (rag.float() - gold["attend_mixed"].float()).abs().max().item() <= tol
    # decode rows of the ragged restatement equal the decode restatement
    one = O.ragged_paged_attention(d["q"][:4], d["k_pool"], d["v_pool"], bt, lens, None, 0.125)
    assert (one.float() - dec.float()).abs().max().item() <= tol


def drive_planner(case, make_engine, add, step):
    """Replay a planner case the way make_golden.py drove the reference: requests arrive at given step numbers."""
    reqs = G.planner_requests(case)
    pending = sorted(range(len(reqs)), key=lambda i: (reqs[i]["arrive"], i))
    eng = make_engine()
    step_no = 0
    order = []
    while pending or eng.has_unfinished():
        while pending and reqs[pending[0]]["arrive"] <= step_no:
            i = pending.pop(0)
            order.append(i)
            add(eng, i, reqs[i])
        step(eng)
        step_no += 1
    return eng, order


@pytest.mark.parametrize("name", list(G.PLANNER_CASES))
def test_oracle_engine_reproduces_reference_planner_traces(name):
    gold = json.loads((GOLD / "planner_traces.json").read_text())[name]
    case = G.PLANNER_CASES[name]
    kw = case["kw"]
    rid_to_idx = {}

    def make():
        return OracleEngine(None, max_seq_len=kw["max_seq_len"], max_num_seqs=kw["max_num_seqs"],
                            max_num_batched_tokens=kw["max_num_batched_tokens"], kv_cache_tokens=kw["kv_cache_tokens"],
                            block_size=kw["block_size"], prefix_caching=kw["prefix_caching"],
                            feed=lambda r, k: G.fed_token(rid_to_idx[r.rid], k))

    def add(eng, i, req):
        rid_to_idx[eng.add_request(req["prompt"], req["max_new"], ignore_eos=True)] = i

    eng, _ = drive_planner(case, make, add, lambda e: e.step())
    assert len(eng.trace) == len(gold["steps"])
    for got, want in zip(eng.trace, gold["steps"]):
        got = dict(got, ids=[rid_to_idx[r] for r in got["ids"]])
        assert got == want
    assert eng.preemptions == gold["preemptions"] and eng.num_free_blocks() == gold["final_free"]
    assert eng.prefix_hit_tokens == gold["prefix_hit_tokens"]


def test_oracle_engine_tiny_model_tokens():
    gold = json.loads((GOLD / "tiny_engine.json").read_text())
    model = OracleModel(G.TINY_CFG, G.tiny_state_dict(G.TINY_CFG))
    eng = OracleEngine(model, **G.TINY_ENGINE_KW)
    outs = run_requests(eng, G.tiny_requests(), concurrency=4)
    got = [outs[i] for i in range(len(outs))]
    assert len(eng.trace) == gold["steps"]
    # fp32 on the same kind of CPU is normally identical; another BLAS may flip an argmax only at a near-tie of that
    # very request and token
    check_tokens(got, gold["tokens"], lambda i, j: eng.gaps[i][j], 1e-3, what="oracle, tiny model")


def test_oracle_engine_config0_tokens():
    """benchmark configuration 0 (0.5B shape, fp32, 8 requests x 64 tokens) against the reference's own run."""
    from nanoserve_b200.synthetic import random_state_dict
    gold = json.loads((GOLD / "config0_tokens.json").read_text())
    sd, cfg = random_state_dict("qwen2.5-0.5b", dtype=torch.float32)
    eng = OracleEngine(OracleModel(cfg, sd), **G.CONFIG0_ENGINE_KW)
    outs = run_requests(eng, G.config0_requests())
    got = [outs[i] for i in range(len(outs))]
    assert len(eng.trace) == gold["steps"]
    check_tokens(got, gold["tokens"], lambda i, j: gold["step_gaps"][j][i], 1e-3, what="oracle, config 0")


def test_token_gate_fails_on_a_wrong_token():
    """The token gate must be able to fail: one changed token of the reference's stream, at the step of the first 32
    whose reference gap is furthest from a tie, is reported even under the widest (bf16) rule in use."""
    import pytest
    gold = json.loads((GOLD / "config0_tokens.json").read_text())
    toks = [list(t) for t in gold["tokens"]]
    i, j = max(((i, j) for i in range(8) for j in range(32)), key=lambda ij: gold["step_gaps"][ij[1]][ij[0]])
    toks[i][j] = (toks[i][j] + 1) % 151936
    with pytest.raises(AssertionError):
        check_tokens(toks, gold["tokens"], lambda i, j: gold["step_gaps"][j][i], 0.25, first=32)
    # and a change at a genuine near-tie is accepted by the rule it was made for, while the strict rule refuses it
    i, j = min(((i, j) for i in range(8) for j in range(32)), key=lambda ij: gold["step_gaps"][ij[1]][ij[0]])
    toks = [list(t) for t in gold["tokens"]]
    toks[i][j] = (toks[i][j] + 1) % 151936
    gap = gold["step_gaps"][j][i]
    check_tokens(toks, gold["tokens"], lambda i, j: gold["step_gaps"][j][i], gap, first=32)
    with pytest.raises(AssertionError):
        check_tokens(toks, gold["tokens"], lambda i, j: gold["step_gaps"][j][i], gap / 2, first=32)


def test_oracle_sampling_distribution_matches_the_reference_sampler():
    """The reference's sample() was run over thousands of seeds on seeded logits rows (tests/golden/sampling.json):
    every token it ever produced is a survivor of the oracle's top-k / top-p masking, every survivor the oracle gives a
    non-negligible probability was produced, and the observed frequencies sit within 5 standard deviations of the
    oracle's probabilities."""
    gold = json.loads((GOLD / "sampling.json").read_text())
    for entry in gold["support"]:
        c = entry["case"]
        logits = G.sampling_logits(c["seed"], c["vocab"])
        probs = O.sampling_probabilities(logits, c["temperature"], c["top_k"], c["top_p"])
        counts = torch.tensor(entry["counts"], dtype=torch.float64)
        n = counts.sum().item()
        assert n == c["draws"]
        assert ((counts > 0) <= (probs > 0)).all(), f"the reference produced a token the oracle drops: {c}"
        assert (counts[probs * n >= 30] > 0).all(), f"a likely survivor was never produced: {c}"
        sigma = (probs * (1 - probs) / n).sqrt()
        assert ((counts / n - probs).abs() <= 5 * sigma + 1e-9).all(), c
