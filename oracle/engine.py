"""CPU oracle for the whole continuous-batching step — TEST INFRASTRUCTURE ONLY (see oracle/ops.py).

A compact, single-file restatement of the reference's engine loop on the CPU torch path: scheduling and
preemption (nanoserve/scheduler.py:128-200), block allocation, slots and prefix caching
(nanoserve/kv_cache.py:79-248, nanoserve/kv_manager.py:101-196), the unfused Qwen2 forward
(nanoserve/model.py:236-260,283-318,341-362) and the step loop (nanoserve/engine.py:195-260). Every step can be
recorded as a trace of integers (who ran, chunk sizes, slots, block tables, free blocks, preemptions) so the
product's decisions can be compared exactly. Parity status: PINNED against traces and tokens produced by the
reference itself (tests/golden/, tests/test_oracle_golden.py).
"""
from __future__ import annotations

from collections import OrderedDict, deque

import torch
import torch.nn.functional as F

from oracle import ops


class Req:
    def __init__(self, rid, prompt, max_new, ignore_eos):
        self.rid, self.prompt, self.max_new, self.ignore_eos = rid, list(prompt), max_new, ignore_eos
        self.out: list[int] = []
        self.cached = 0            # tokens with K/V stored
        self.blocks: list[int] | None = None
        self.stored = 0            # the block table's committed token count
        self.hashed = 0            # leading blocks already offered to the prefix cache
        self.node = 0              # trie node of the last of those

    def toks(self):
        return self.prompt + self.out

    def total(self):
        return len(self.prompt) + len(self.out)

    def remaining(self):
        return self.total() - self.cached

    def prefilling(self):
        return self.cached == 0 or self.remaining() > 1


class Pool:
    """Free list + optional prefix cache, as plain dicts (nanoserve/kv_cache.py:79-204)."""

    def __init__(self, num_blocks, block_size, prefix_caching):
        self.n, self.bs, self.prefix = num_blocks, block_size, prefix_caching
        self.free_list = list(range(num_blocks - 1, -1, -1))
        self.ref, self.block_of, self.key_of, self.node_of = {}, {}, {}, {}
        self.lru = OrderedDict()
        self.next_node = 1

    def num_free(self):
        return len(self.free_list) + len(self.lru)

    def take(self):
        if self.free_list:
            b = self.free_list.pop()
        elif self.lru:
            b, _ = self.lru.popitem(last=False)
            del self.block_of[self.key_of.pop(b)]
            del self.node_of[b]
        else:
            raise RuntimeError("pool exhausted")
        if self.prefix:
            self.ref[b] = 1
        return b

    def give_back(self, blocks):
        if not self.prefix:
            self.free_list.extend(blocks)
            return
        for b in reversed(blocks):
            self.ref[b] -= 1
            if self.ref[b] == 0:
                del self.ref[b]
                if b in self.key_of:
                    self.lru[b] = None
                else:
                    self.free_list.append(b)

    def lookup(self, toks, max_blocks):
        hits, parent = [], 0
        for i in range(min(max_blocks, len(toks) // self.bs)):
            b = self.block_of.get((parent, tuple(toks[i * self.bs:(i + 1) * self.bs])))
            if b is None:
                break
            hits.append(b)
            parent = self.node_of[b]
        return hits

    def pin(self, blocks):
        for b in blocks:
            if self.ref.get(b, 0) == 0:
                del self.lru[b]
            self.ref[b] = self.ref.get(b, 0) + 1

    def register(self, r: Req):
        toks = r.toks()
        for i in range(r.hashed, r.stored // self.bs):
            key = (r.node, tuple(toks[i * self.bs:(i + 1) * self.bs]))
            have = self.block_of.get(key)
            if have is None:
                b, node = r.blocks[i], self.next_node
                self.next_node += 1
                self.block_of[key], self.key_of[b], self.node_of[b] = b, key, node
            else:
                node = self.node_of[have]
            r.node, r.hashed = node, i + 1


class OracleModel:
    """Unfused Qwen2 forward on CPU tensors, attention over the paged pool (nanoserve/model.py:236-260,283-318)."""

    def __init__(self, cfg: dict, sd: dict):
        self.cfg, self.sd = cfg, sd
        self.dtype = sd["model.embed_tokens.weight"].dtype
        self.lm_head = sd["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else sd["lm_head.weight"]

    def new_pool(self, num_blocks, block_size):
        c = self.cfg
        shape = (c["n_layers"], num_blocks, block_size, c["n_kv_heads"], c["head_dim"])
        return torch.zeros(shape, dtype=self.dtype), torch.zeros(shape, dtype=self.dtype)

    @torch.inference_mode()
    def forward(self, tokens, positions, tables, seq_lens, cu, slots, k_pool, v_pool):
        """tokens/positions/slots: flat lists; tables: list of block-id lists per sequence; returns logits of each
        sequence's last token [S, vocab]."""
        c, sd = self.cfg, self.sd
        nh, nkv, hd, eps = c["n_heads"], c["n_kv_heads"], c["head_dim"], c["rms_norm_eps"]
        N = len(tokens)
        x = F.embedding(torch.tensor(tokens), sd["model.embed_tokens.weight"])
        cos, sin = ops.rope_cos_sin(torch.tensor(positions), hd, c["rope_theta"], self.dtype)
        cs, sn = cos[:, None, :], sin[:, None, :]
        width = max(len(t) for t in tables)
        tab = torch.tensor([t + [0] * (width - len(t)) for t in tables], dtype=torch.int32)
        lens_t, cu_t, slot_t = torch.tensor(seq_lens, dtype=torch.int32), torch.tensor(cu, dtype=torch.int32), torch.tensor(slots)
        for i in range(c["n_layers"]):
            p = f"model.layers.{i}."
            h = ops.rms_norm(x, sd[p + "input_layernorm.weight"], eps)
            q = F.linear(h, sd[p + "self_attn.q_proj.weight"], sd[p + "self_attn.q_proj.bias"]).view(N, nh, hd)
            k = F.linear(h, sd[p + "self_attn.k_proj.weight"], sd[p + "self_attn.k_proj.bias"]).view(N, nkv, hd)
            v = F.linear(h, sd[p + "self_attn.v_proj.weight"], sd[p + "self_attn.v_proj.bias"]).view(N, nkv, hd)
            q = q * cs + ops.rotate_half(q) * sn
            k = k * cs + ops.rotate_half(k) * sn
            ops.kv_write(k_pool[i], v_pool[i], k, v, slot_t)
            o = ops.ragged_paged_attention(q, k_pool[i], v_pool[i], tab, lens_t, cu_t, hd ** -0.5)
            x = x + F.linear(o.reshape(N, nh * hd), sd[p + "self_attn.o_proj.weight"])
            h = ops.rms_norm(x, sd[p + "post_attention_layernorm.weight"], eps)
            x = x + F.linear(F.silu(F.linear(h, sd[p + "mlp.gate_proj.weight"])) * F.linear(h, sd[p + "mlp.up_proj.weight"]),
                             sd[p + "mlp.down_proj.weight"])
        x = ops.rms_norm(x, sd["model.norm.weight"], eps)
        last = torch.tensor(cu[1:]) - 1
        return F.linear(x[last], self.lm_head)


class OracleEngine:
    """Step loop of the reference on the CPU (nanoserve/engine.py:195-260) with the paged KV manager, chunked
    prefill and optional prefix caching. model=None runs the integer logic only: `feed` supplies the tokens."""

    def __init__(self, model: OracleModel | None, eos_ids=(), max_seq_len=2048, max_num_seqs=8,
                 max_num_batched_tokens=2048, kv_cache_tokens=None, block_size=16, chunked_prefill=True,
                 prefix_caching=False, reserve_garbage_block=False, watermark=0.01, feed=None):
        self.model, self.eos, self.max_seq_len = model, set(eos_ids), max_seq_len
        self.max_seqs, self.bs, self.chunked = max_num_seqs, block_size, chunked_prefill
        self.budget = max_num_batched_tokens if chunked_prefill else max(max_num_batched_tokens, max_seq_len)
        tokens = kv_cache_tokens if kv_cache_tokens is not None else 32 * max_seq_len
        self.num_blocks = -(-tokens // block_size)
        self.pool = Pool(self.num_blocks, block_size, prefix_caching)
        self.watermark = int(watermark * self.num_blocks)
        self.garbage = self.pool.free_list.pop() if reserve_garbage_block else None   # the graphs' padding block
        self.kv = model.new_pool(self.num_blocks, block_size) if model is not None else None
        self.waiting, self.running = deque(), []
        self.preemptions = self.prefix_hit_tokens = self.prefix_query_tokens = 0
        self.next_id, self.trace, self.feed = 0, [], feed
        self.logits_gap: list[float] = []      # top-2 logit gap of every sampled token (tie analysis)
        self.gaps: dict[int, list[float]] = {}  # the same gaps per request id, indexed by output token
        self.keep_logits = False               # True: last_logits = {request id: logits row} of the newest step
        self.last_logits: dict[int, torch.Tensor] = {}

    # -- requests
    def add_request(self, prompt, max_new, ignore_eos=False):
        if len(prompt) + max_new > self.max_seq_len:
            raise ValueError("prompt + max_new_tokens exceeds max_seq_len")
        if -(-(len(prompt) + max_new) // self.bs) > self.num_blocks:
            raise ValueError("request could never fit the KV budget")
        r = Req(self.next_id, prompt, max_new, ignore_eos)
        self.next_id += 1
        self.waiting.append(r)
        return r.rid

    def has_unfinished(self):
        return bool(self.waiting or self.running)

    # -- KV manager
    def _need(self, r: Req, n_new):
        return max(0, -(-(r.stored + n_new) // self.bs) - len(r.blocks))

    def _hits(self, r: Req):
        if not self.pool.prefix:
            return []
        t = r.toks()
        return self.pool.lookup(t, (len(t) - 1) // self.bs)

    def _release(self, r: Req):
        self.pool.give_back(r.blocks)
        r.blocks, r.stored = None, 0

    def _can_admit(self, r: Req):
        hits = self._hits(r)
        parked = sum(1 for b in hits if self.pool.ref.get(b, 0) == 0)
        need = -(-r.remaining() // self.bs) - len(hits) + parked
        return need <= self.pool.num_free() - self.watermark

    def _admit(self, r: Req):
        r.blocks, r.stored, r.hashed, r.node = [], 0, 0, 0
        if self.pool.prefix:
            hits = self._hits(r)
            self.prefix_query_tokens += r.total()
            if hits:
                self.pool.pin(hits)
                r.blocks, r.hashed, r.stored = list(hits), len(hits), len(hits) * self.bs
                r.node = self.pool.node_of[hits[-1]]
                r.cached = r.stored
                self.prefix_hit_tokens += r.stored
        for _ in range(self._need(r, r.remaining())):
            r.blocks.append(self.pool.take())

    # -- scheduler
    def _schedule(self):
        i = 0
        while i < len(self.running):
            r = self.running[i]
            if self._need(r, 1) <= self.pool.num_free():
                for _ in range(self._need(r, 1)):
                    r.blocks.append(self.pool.take())
                i += 1
                continue
            victim = self.running.pop()
            self._release(victim)
            victim.cached = 0
            self.waiting.appendleft(victim)
            self.preemptions += 1
        budget, sched, chunks, partial = self.budget, [], [], []
        for r in self.running:
            if r.prefilling():
                partial.append(r)
            else:
                sched.append(r)
                chunks.append(1)
                budget -= 1
        for r in partial:
            n = min(r.remaining(), budget) if self.chunked else r.remaining()
            if n > 0:
                sched.append(r)
                chunks.append(n)
                budget -= n
        admitted = []
        while (self.waiting and len(self.running) + len(admitted) < self.max_seqs
               and (budget > 0 if self.chunked else self.waiting[0].remaining() <= budget)
               and self._can_admit(self.waiting[0])):
            r = self.waiting.popleft()
            self._admit(r)
            n = min(r.remaining(), budget) if self.chunked else r.remaining()
            budget -= n
            admitted.append(r)
            sched.append(r)
            chunks.append(n)
        self.running.extend(admitted)
        return sched, chunks

    # -- one step
    def step(self):
        sched, chunks = self._schedule()
        if not sched:
            return []
        tokens, positions, slots, tables, lens, cu = [], [], [], [], [], [0]
        for r, n in zip(sched, chunks):
            all_toks = r.toks()
            tokens += all_toks[r.cached:r.cached + n]
            positions += list(range(r.cached, r.cached + n))
            slots += [r.blocks[p // self.bs] * self.bs + p % self.bs for p in range(r.stored, r.stored + n)]
            tables.append(list(r.blocks))
            lens.append(r.cached + n)
            cu.append(cu[-1] + n)
        self.trace.append(dict(ids=[r.rid for r in sched], chunks=list(chunks), slots=list(slots),
                               tables=[list(t) for t in tables], positions=list(positions), tokens=list(tokens),
                               free=self.pool.num_free(), preemptions=self.preemptions))
        if self.model is not None:
            logits = self.model.forward(tokens, positions, [t[:-(-L // self.bs)] for t, L in zip(tables, lens)], lens, cu,
                                        slots, *self.kv)
            top2 = logits.float().topk(2, dim=-1).values
            gaps = (top2[:, 0] - top2[:, 1]).tolist()
            nxt = logits.argmax(-1).tolist()
            if self.keep_logits:
                self.last_logits = {r.rid: logits[i] for i, r in enumerate(sched)}
        else:
            nxt, gaps = [self.feed(r, len(r.out)) for r in sched], [1.0] * len(sched)
        for r, n in zip(sched, chunks):
            r.stored += n
            if self.pool.prefix and r.stored // self.bs > r.hashed:
                self.pool.register(r)
            r.cached += n
        outs = []
        for r, tok, gap in zip(sched, nxt, gaps):
            if r.cached < r.total():
                continue
            r.out.append(tok)
            self.logits_gap.append(gap)
            self.gaps.setdefault(r.rid, []).append(gap)
            done = (tok in self.eos and not r.ignore_eos) or len(r.out) >= r.max_new
            if done:
                self.running.remove(r)
                self._release(r)
            outs.append((r.rid, tok, done))
        return outs

    def num_free_blocks(self):
        return self.pool.num_free()


def run_requests(engine, requests, concurrency=None):
    """Closed loop in the shape of the reference's bare-loop probe (bench/runs/m11_loop_profile.py:41-59): keep
    `concurrency` requests in flight (default: all at once), refill when one finishes. requests =
    [(prompt_ids, max_new)]. Returns {request index: generated tokens}. Works for OracleEngine and for engines with
    the reference's add_request/step interface."""
    queue = deque(enumerate(requests))
    idx_of, outs = {}, {}
    limit = concurrency or len(requests)

    def submit():
        i, (prompt, max_new) = queue.popleft()
        idx_of[engine.add_request(prompt, max_new, ignore_eos=True)] = i
        outs[i] = []

    while queue and len(idx_of) < limit:
        submit()
    while engine.has_unfinished():
        for o in engine.step():
            rid, tok, done = (o.seq_id, o.token, o.finished) if hasattr(o, "seq_id") else o
            outs[idx_of[rid]].append(tok)
            if done and queue:
                submit()
    return outs
