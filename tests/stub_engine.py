"""A CPU stand-in with the engine's interface (add_request / step / abort / has_unfinished / stats / kv.num_free_blocks),
for host-side tests of the engine process and the replica router: no torch, no GPU. A request's n-th token is a fixed
function of its prompt; magic prompt tokens make a step raise, or make the process die, so the failure paths can be
driven from the request stream."""
from __future__ import annotations

import os
import time
from dataclasses import dataclass

RAISE_TOKEN = 900001        # a running request whose prompt holds this makes step() raise
DIE_TOKEN = 900002          # ... makes the process exit at once, without a goodbye


def stub_token(prompt: list[int], n: int) -> int:
    return (sum(prompt) * 31 + n * 7 + len(prompt)) % 1000


@dataclass
class StubOutput:
    seq_id: int
    token: int
    finished: bool


class _Kv:
    def __init__(self, blocks: int):
        self.num_free_blocks = blocks


class StubEngine:
    def __init__(self, spec=None, blocks: int = 1000, step_s: float = 0.0):
        args = getattr(spec, "factory_args", {}) or {}
        self.kv = _Kv(args.get("blocks", blocks))
        self.step_s = args.get("step_s", step_s)
        self.max_num_seqs = getattr(spec, "max_num_seqs", 64)
        self.eos_token_ids: list[int] = []
        self.seqs: dict[int, dict] = {}
        self.next_id = 0
        self.steps = 0

    def add_request(self, prompt_ids, max_new_tokens, ignore_eos=False, arrival_time=None, sampling=None) -> int:
        if len(prompt_ids) + max_new_tokens > 4096:
            raise ValueError("prompt + max_new_tokens exceeds max_seq_len")
        sid = self.next_id
        self.next_id += 1
        need = -(-(len(prompt_ids) + max_new_tokens) // 16)
        self.kv.num_free_blocks -= need
        self.seqs[sid] = dict(prompt=list(prompt_ids), max_new=max_new_tokens, out=0, blocks=need)
        return sid

    def has_unfinished(self) -> bool:
        return bool(self.seqs)

    def abort(self, seq_id: int) -> None:
        s = self.seqs.pop(seq_id, None)
        if s is not None:
            self.kv.num_free_blocks += s["blocks"]

    def step(self):
        self.steps += 1
        if self.step_s:
            time.sleep(self.step_s)
        running = list(self.seqs.items())[:self.max_num_seqs]
        for _, s in running:
            if DIE_TOKEN in s["prompt"]:
                os._exit(3)
            if RAISE_TOKEN in s["prompt"]:
                raise RuntimeError("injected step failure")
        outs = []
        for sid, s in running:
            tok = stub_token(s["prompt"], s["out"])
            s["out"] += 1
            done = s["out"] >= s["max_new"]
            if done:
                self.abort(sid)
            outs.append(StubOutput(sid, tok, done))
        return outs

    @property
    def stats(self) -> dict:
        return {"steps": self.steps}


def make_stub(spec):
    return StubEngine(spec)
