"""The product's Scheduler + PagedKVManager make the reference's decisions bit for bit: scheduled ids, chunk sizes,
slots, block tables, positions, token ids, free-block counts and preemption counts of every step equal the traces
recorded from the reference (tests/golden/planner_traces.json). The packed records the engine would upload, expanded
by the CPU restatement of the metadata kernel, must reproduce the same slots / positions / tokens."""
import json
from pathlib import Path

import pytest
import torch

from nanoserve_b200.kv_manager import PagedKVManager
from nanoserve_b200.model import ModelConfig
from nanoserve_b200.scheduler import Scheduler, Sequence
from oracle import ops as O
from tests.golden import make_golden as G

GOLD = json.loads((Path(__file__).parent / "golden" / "planner_traces.json").read_text())
TINY = ModelConfig(**G.TINY_CFG)


@pytest.mark.parametrize("name", list(G.PLANNER_CASES))
def test_scheduler_and_kv_manager_reproduce_reference_traces(name):
    case, gold = G.PLANNER_CASES[name], GOLD[name]
    kw = case["kw"]
    kv = PagedKVManager(TINY, kw["kv_cache_tokens"], kw["block_size"], device="cpu", dtype=torch.float32,
                        prefix_caching=kw["prefix_caching"], max_seats=kw["max_num_seqs"])
    sch = Scheduler("continuous", max_num_seqs=kw["max_num_seqs"], max_num_batched_tokens=kw["max_num_batched_tokens"],
                    kv=kv, chunked_prefill=True)
    reqs = G.planner_requests(case)
    pending = sorted(range(len(reqs)), key=lambda i: (reqs[i]["arrive"], i))
    mirror: dict[int, list[int]] = {}          # what the device block-table mirror would hold, per seat
    last_tokens: dict[int, int] = {}
    step_no, k = 0, 0
    while pending or sch.has_unfinished():
        while pending and reqs[pending[0]]["arrive"] <= step_no:
            i = pending.pop(0)
            sch.add(Sequence(seq_id=i, prompt_ids=list(reqs[i]["prompt"]), max_new_tokens=reqs[i]["max_new"], ignore_eos=True))
        plan = sch.schedule(now=0.0)
        step_no += 1
        if not plan.scheduled:
            continue
        want = gold["steps"][k]
        k += 1
        # reference-style host lists
        kv.begin_step()
        toks, poss = [], []
        for seq, n in zip(plan.scheduled, plan.chunks):
            t, p = seq.step_tokens(n)
            toks += t
            poss += p
            kv.seq_input(seq, n)
        got = dict(ids=[s.seq_id for s in plan.scheduled], chunks=list(plan.chunks), slots=list(kv._slots),
                   tables=[list(s.block_table.blocks) for s in plan.scheduled], positions=poss, tokens=toks,
                   free=kv.num_free_blocks, preemptions=sch.num_preemptions)
        assert got == want, f"step {k - 1} differs"
        # packed records -> metadata (CPU restatement of the device kernel) must give the same arrays
        records, appends, token_ids = kv.step_records(plan.scheduled, plan.chunks)
        for a in range(0, len(appends), 3):
            seat, idx, blk = appends[a:a + 3]
            row = mirror.setdefault(seat, [])
            del row[idx:]
            row.append(blk)
        recs = [tuple(records[i:i + 4]) for i in range(0, len(records), 4)]
        meta = O.step_metadata(recs, mirror, last_tokens, token_ids, kw["block_size"], len(recs), sum(plan.chunks), 0)
        assert meta["slot_mapping"] == want["slots"] and meta["positions"] == want["positions"]
        assert meta["tokens"] == want["tokens"]
        assert [r[1] + r[2] for r in recs] == [len(s.block_table.blocks) * 0 + s.num_cached + n
                                               for s, n in zip(plan.scheduled, plan.chunks)]
        for seq, n in zip(plan.scheduled, plan.chunks):
            kv.commit(seq, n)
            seq.num_cached += n
        for seq in plan.scheduled:
            if seq.num_cached < seq.num_tokens:
                seq.token_on_device = False
                continue
            tok = G.fed_token(seq.seq_id, len(seq.output_ids))
            seq.output_ids.append(tok)
            seq.token_on_device = True
            last_tokens[seq.seat] = tok
            if len(seq.output_ids) >= seq.max_new_tokens:
                sch.finish(seq)
    assert k == len(gold["steps"])
    assert kv.num_free_blocks == gold["final_free"] and sch.num_preemptions == gold["preemptions"]
    assert kv.prefix_hit_tokens == gold["prefix_hit_tokens"] and kv.prefix_query_tokens == gold["prefix_query_tokens"]
    assert sorted(kv._free_seats) == list(range(kw["max_num_seqs"]))          # every seat returned
