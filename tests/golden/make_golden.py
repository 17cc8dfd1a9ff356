"""Generate the golden fixtures in this folder by running the REFERENCE itself (imported from its read-only
checkout) on seeded inputs. Run where the reference is available:

    python tests/golden/make_golden.py [/path/to/reference]

Outputs (committed):
  planner_traces.json   step-by-step integer decisions of the reference Scheduler + PagedKVManager
  ops.pt                outputs of the reference's torch ops / attention paths on seeded inputs
  tiny_engine.json      tokens of the reference LLMEngine (CPU, fp32) on a tiny random Qwen2-shaped model
  config0_tokens.json   tokens + top-2 logit gaps of the reference LLMEngine on the 0.5B shape (benchmark configuration 0)
The tests regenerate the same inputs from the same seeds (helpers below are imported by the tests).
"""
from __future__ import annotations

import json
import random
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# ------------------------------------------------------------------------------------------------ seeded inputs
TINY_CFG = dict(vocab_size=512, hidden_size=128, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=32,
                intermediate_size=256, rope_theta=1_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)

PLANNER_CASES = {
    # name: engine kwargs + request stream (prompt_len, max_new, arrival step)
    "roomy": dict(kw=dict(max_num_seqs=6, max_num_batched_tokens=64, kv_cache_tokens=2048, block_size=16,
                          max_seq_len=512, prefix_caching=False), n=14, prompt=(5, 90), out=(3, 30), seed=1),
    "tight_preempt": dict(kw=dict(max_num_seqs=8, max_num_batched_tokens=48, kv_cache_tokens=320, block_size=16,
                                  max_seq_len=256, prefix_caching=False), n=12, prompt=(20, 70), out=(20, 40), seed=2),
    "block4_chunked": dict(kw=dict(max_num_seqs=4, max_num_batched_tokens=10, kv_cache_tokens=256, block_size=4,
                                   max_seq_len=128, prefix_caching=False), n=9, prompt=(1, 40), out=(1, 12), seed=3),
    "prefix_evict": dict(kw=dict(max_num_seqs=6, max_num_batched_tokens=64, kv_cache_tokens=480, block_size=16,
                                 max_seq_len=256, prefix_caching=True), n=16, prompt=(4, 40), out=(4, 20), seed=4,
                         shared_prefix=70),
}


def planner_requests(case: dict):
    rng = random.Random(case["seed"])
    prefix = [rng.randrange(1000) for _ in range(case.get("shared_prefix", 0))]
    reqs = []
    for i in range(case["n"]):
        plen = rng.randint(*case["prompt"])
        own = [rng.randrange(1000) for _ in range(plen)]
        use_prefix = bool(prefix) and i % 4 != 3
        reqs.append(dict(prompt=(prefix + own) if use_prefix else own, max_new=rng.randint(*case["out"]),
                         arrive=rng.randint(0, 12)))
    return reqs


def fed_token(rid: int, k: int) -> int:
    """Deterministic stand-in for the sampled token (request id, index of the output token)."""
    return (rid * 7919 + k * 104729 + 13) % 1000


def tiny_state_dict(cfg: dict, seed: int = 0, dtype=torch.float32) -> dict:
    g = torch.Generator().manual_seed(seed)
    H, NH, NKV, HD, I, V = (cfg[k] for k in ("hidden_size", "n_heads", "n_kv_heads", "head_dim", "intermediate_size",
                                              "vocab_size"))

    def mat(*shape, std=0.05):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    sd = {"model.embed_tokens.weight": mat(V, H, std=0.5), "model.norm.weight": torch.ones(H, dtype=dtype)}
    for i in range(cfg["n_layers"]):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"] = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
        sd[p + "post_attention_layernorm.weight"] = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
        for nm, rows in (("q", NH * HD), ("k", NKV * HD), ("v", NKV * HD)):
            sd[p + f"self_attn.{nm}_proj.weight"] = mat(rows, H, std=0.15)
            sd[p + f"self_attn.{nm}_proj.bias"] = mat(rows, std=0.1)
        sd[p + "self_attn.o_proj.weight"] = mat(H, NH * HD, std=0.1)
        sd[p + "mlp.gate_proj.weight"] = mat(I, H, std=0.1)
        sd[p + "mlp.up_proj.weight"] = mat(I, H, std=0.1)
        sd[p + "mlp.down_proj.weight"] = mat(H, I, std=0.1)
    return sd


def tiny_requests(seed: int = 5, n: int = 7):
    rng = random.Random(seed)
    return [([rng.randrange(TINY_CFG["vocab_size"]) for _ in range(rng.randint(3, 60))], rng.randint(4, 24))
            for _ in range(n)]


TINY_ENGINE_KW = dict(max_seq_len=128, max_num_seqs=4, max_num_batched_tokens=32, kv_cache_tokens=512, block_size=16)


def config0_requests():
    """benchmark configuration 0: 8 requests, prompt lengths uniform in 32-256, uniform token ids, 64 greedy tokens."""
    rng = random.Random(0)
    reqs = []
    for _ in range(8):
        n = rng.randint(32, 256)
        reqs.append(([rng.randrange(151936) for _ in range(n)], 64))
    return reqs


CONFIG0_ENGINE_KW = dict(max_seq_len=2048, max_num_seqs=8, max_num_batched_tokens=2048, block_size=16)


def ops_inputs():
    """Seeded inputs of the op-level fixtures (sizes follow the reference's own op tests)."""
    g = torch.Generator().manual_seed(1234)
    out = {}
    for name, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        d = {}
        d["x"] = (torch.randn(37, 896, generator=g) * 3).to(dt)
        d["res"] = torch.randn(37, 896, generator=g).to(dt)
        d["w"] = (1 + 0.1 * torch.randn(896, generator=g)).to(dt)
        d["gate_up"] = (torch.randn(11, 2 * 4864, generator=g) * 2).to(dt)
        d["qkv"] = torch.randn(37, (14 + 4) * 64, generator=g).to(dt)
        d["positions"] = torch.randint(0, 8192, (37,), generator=g)
        # attention: pool + mixed batch (2 decodes, fresh prefill of 40, chunk of 22 on 30 cached)
        nb = 24
        d["k_pool"] = torch.randn(nb, 16, 2, 64, generator=g).to(dt)
        d["v_pool"] = torch.randn(nb, 16, 2, 64, generator=g).to(dt)
        d["perm"] = torch.randperm(nb, generator=g)
        d["q"] = torch.randn(1 + 1 + 40 + 22, 14, 64, generator=g).to(dt)
        out[name] = d
    return out


ATTN_LENS, ATTN_QLENS = [100, 17, 40, 52], [1, 1, 40, 22]


def attn_tables(perm):
    tables, used = [], 0
    for L in ATTN_LENS:
        nb = -(-L // 16)
        tables.append(perm[used:used + nb].tolist())
        used += nb
    return tables


# ------------------------------------------------------------------------------------------------ generation
def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from nanoserve.engine import LLMEngine
    from nanoserve.kernels.paged_attention import paged_attention_reference
    from nanoserve.kv_manager import PagedKVManager
    from nanoserve.model import ModelConfig, Qwen2Model, SeqInput, rms_norm, rotate_half
    from nanoserve.scheduler import Scheduler, Sequence
    import torch.nn.functional as F

    # ---- 1. planner traces: the reference Scheduler + PagedKVManager driven like LLMEngine.step drives them
    traces = {}
    tiny = ModelConfig(**TINY_CFG)
    for name, case in PLANNER_CASES.items():
        kw = case["kw"]
        kv = PagedKVManager(tiny, kw["kv_cache_tokens"], kw["block_size"], device="cpu", dtype=torch.float32,
                            prefix_caching=kw["prefix_caching"])
        sch = Scheduler("continuous", max_num_seqs=kw["max_num_seqs"], max_num_batched_tokens=kw["max_num_batched_tokens"],
                        kv=kv, chunked_prefill=True)
        reqs = planner_requests(case)
        pending = sorted(range(len(reqs)), key=lambda i: (reqs[i]["arrive"], i))
        steps, step_no = [], 0
        while pending or sch.has_unfinished():
            while pending and reqs[pending[0]]["arrive"] <= step_no:
                i = pending.pop(0)
                sch.add(Sequence(seq_id=i, prompt_ids=list(reqs[i]["prompt"]), max_new_tokens=reqs[i]["max_new"],
                                 ignore_eos=True))
            plan = sch.schedule(now=0.0)
            step_no += 1
            if not plan.scheduled:
                continue
            kv.begin_step()
            toks, poss = [], []
            for seq, n in zip(plan.scheduled, plan.chunks):
                t, p = seq.step_tokens(n)
                toks += t
                poss += p
                kv.seq_input(seq, n)
            steps.append(dict(ids=[s.seq_id for s in plan.scheduled], chunks=list(plan.chunks), slots=list(kv._slots),
                              tables=[list(s.block_table.blocks) for s in plan.scheduled], positions=poss, tokens=toks,
                              free=kv.num_free_blocks, preemptions=sch.num_preemptions))
            for seq, n in zip(plan.scheduled, plan.chunks):
                kv.commit(seq, n)
                seq.num_cached += n
            for seq in plan.scheduled:
                if seq.num_cached < seq.num_tokens:
                    continue
                seq.output_ids.append(fed_token(seq.seq_id, len(seq.output_ids)))
                if len(seq.output_ids) >= seq.max_new_tokens:
                    sch.finish(seq)
        traces[name] = dict(steps=steps, final_free=kv.num_free_blocks, preemptions=sch.num_preemptions,
                            prefix_hit_tokens=kv.prefix_hit_tokens, prefix_query_tokens=kv.prefix_query_tokens)
        print(f"planner {name}: {len(steps)} steps, {sch.num_preemptions} preemptions, hits {kv.prefix_hit_tokens}")
    (HERE / "planner_traces.json").write_text(json.dumps(traces, separators=(",", ":")))

    # ---- 2. op-level outputs of the reference's torch paths
    res = {}
    for name, d in ops_inputs().items():
        dt = d["x"].dtype
        r = {}
        r["rms_norm"] = rms_norm(d["x"], d["w"], 1e-6)
        summed = d["res"] + d["x"]
        r["add"] = summed
        r["add_rms_norm"] = rms_norm(summed, d["w"], 1e-6)
        r["silu_mul"] = F.silu(d["gate_up"][..., :4864]) * d["gate_up"][..., 4864:]
        stub = Qwen2Model.__new__(Qwen2Model)
        stub.cfg = ModelConfig(vocab_size=8, hidden_size=896, n_layers=1, n_heads=14, n_kv_heads=2, head_dim=64,
                               intermediate_size=8, rope_theta=1_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)
        stub.dtype, stub.fused = dt, False
        stub.inv_freq = 1.0 / (1_000_000.0 ** (torch.arange(0, 64, 2, dtype=torch.float) / 64))
        cos, sin = stub.rope(d["positions"])
        r["cos"], r["sin"] = cos[0], sin[0]
        q0 = d["qkv"][:, :14 * 64].view(37, 14, 64)
        k0 = d["qkv"][:, 14 * 64:16 * 64].view(37, 2, 64)
        c, s = cos[0][:, None, :], sin[0][:, None, :]
        r["rope_q"] = q0 * c + rotate_half(q0) * s
        r["rope_k"] = k0 * c + rotate_half(k0) * s
        # decode oracle of the reference (gather + SDPA) on 4 rows
        tables = attn_tables(d["perm"])
        width = max(len(t) for t in tables)
        bt = torch.tensor([t + [0] * (width - len(t)) for t in tables], dtype=torch.int32)
        lens = torch.tensor(ATTN_LENS, dtype=torch.int32)
        r["decode_ref"] = paged_attention_reference(d["q"][:4], d["k_pool"], d["v_pool"], bt, lens, 0.125)
        # the reference's _attend on the mixed batch (SDPA loop: decode rows, fresh prefill, chunk on context)
        from nanoserve.kv_cache import PagedKVCache
        pool = PagedKVCache.__new__(PagedKVCache)
        pool.cfg, pool.k, pool.v, pool.block_size = stub.cfg, d["k_pool"][None], d["v_pool"][None], 16
        seqs, q = [], d["q"]
        for L, T, t in zip(ATTN_LENS, ATTN_QLENS, tables):
            seqs.append(SeqInput(T, block_table=torch.tensor(t), ctx_len=L - T))
        # fresh prefill rows read this step's K/V densely in the reference: hand it the same values the pool holds
        N = q.shape[0]
        k_dense = torch.zeros(N, 2, 64, dtype=dt)
        v_dense = torch.zeros(N, 2, 64, dtype=dt)
        start = 0
        for L, T, t in zip(ATTN_LENS, ATTN_QLENS, tables):
            pos = torch.arange(L - T, L)
            rows = torch.tensor(t)[pos // 16] * 16 + pos % 16
            k_dense[start:start + T] = d["k_pool"].view(-1, 2, 64)[rows]
            v_dense[start:start + T] = d["v_pool"].view(-1, 2, 64)[rows]
            start += T
        r["attend_mixed"] = stub._attend(0, q[None], k_dense[None], v_dense[None], seqs, paged=pool)[0].view(N, 14, 64)
        res[name] = r
    torch.save(res, HERE / "ops.pt")
    print("ops fixtures:", {k: list(v) for k, v in res.items()}["f32"])

    # ---- 3. tiny end-to-end engine, CPU fp32, chunked prefill with a small budget
    model = Qwen2Model(ModelConfig(**TINY_CFG), tiny_state_dict(TINY_CFG))
    eng = LLMEngine(model, eos_token_ids=[], **TINY_ENGINE_KW)
    from oracle.engine import run_requests
    outs = run_requests(eng, tiny_requests(), concurrency=4)
    (HERE / "tiny_engine.json").write_text(json.dumps(dict(tokens=[outs[i] for i in range(len(outs))],
                                                           steps=eng.stats["steps"],
                                                           prefill_chunks=eng.stats["prefill_chunks"])))
    print("tiny engine:", eng.stats["steps"], "steps")

    # ---- 4. benchmark configuration 0 on the full 0.5B shape (random init), CPU fp32
    from nanoserve_b200.synthetic import random_state_dict
    sd, cfg = random_state_dict("qwen2.5-0.5b", dtype=torch.float32)
    model = Qwen2Model(ModelConfig(**cfg), sd)
    eng = LLMEngine(model, eos_token_ids=[], **CONFIG0_ENGINE_KW)
    gaps = []
    orig = model.forward_batch

    def spy(*a, **k):
        logits = orig(*a, **k)
        top2 = logits.float().topk(2, dim=-1).values
        gaps.append((top2[:, 0] - top2[:, 1]).tolist())
        return logits

    model.forward_batch = spy
    import time
    t0 = time.perf_counter()
    outs = run_requests(eng, config0_requests())
    dt_s = time.perf_counter() - t0
    (HERE / "config0_tokens.json").write_text(json.dumps(dict(tokens=[outs[i] for i in range(len(outs))], step_gaps=gaps,
                                                              steps=eng.stats["steps"])))
    print(f"config 0: {eng.stats['steps']} steps, {sum(len(v) for v in outs.values())} tokens in {dt_s:.1f} s")


# ---- sampling host pieces: per-request seeds and parameter validation (integers and flags only) -------------------
SAMPLING_SEEDS = [(0, 0), (1, 0), (0, 1), (12345, 7), (2 ** 62 - 1, 255), (2 ** 63 + 5, 3), (987654321987, 1_000_000),
                  (2 ** 64 - 1, 2 ** 32), (42, 41), (42, 42), (42, 43)]
SAMPLING_PARAMS = [dict(), dict(temperature=0.0, top_k=5), dict(temperature=0.7), dict(temperature=1.0, top_k=1),
                   dict(temperature=0.5, top_p=0.9, top_k=40, seed=7), dict(temperature=-0.1), dict(temperature=float("nan")),
                   dict(top_p=0.0), dict(top_p=1.0001), dict(top_p=1.0), dict(top_k=-1), dict(top_k=0, temperature=2.0)]


SAMPLING_SUPPORT_CASES = [
    dict(seed=0, vocab=64, temperature=1.0, top_k=0, top_p=1.0, draws=4000),
    dict(seed=1, vocab=64, temperature=0.7, top_k=8, top_p=1.0, draws=4000),
    dict(seed=2, vocab=64, temperature=1.3, top_k=0, top_p=0.6, draws=4000),
    dict(seed=3, vocab=64, temperature=0.9, top_k=12, top_p=0.8, draws=4000),
    dict(seed=4, vocab=64, temperature=2.0, top_k=3, top_p=0.3, draws=2000),
    dict(seed=5, vocab=200, temperature=0.5, top_k=0, top_p=0.95, draws=4000),
]


def sampling_logits(seed: int, vocab: int) -> torch.Tensor:
    """A seeded fp32 logits row (standard deviation 2: a few tokens dominate, as in a language model's output)."""
    return torch.randn(vocab, generator=torch.Generator().manual_seed(1000 + seed)) * 2.0


def sampling_main(ref_root: str) -> None:
    """Records the reference's mix_seed values, which SamplingParams it accepts (and whether they are greedy), and how
    often its sample() picked each token of seeded logits rows over thousands of seeds (its support and frequencies)."""
    sys.path.insert(0, ref_root)
    from nanoserve.sampling import SamplingParams, mix_seed, sample
    seeds = [[s, n, mix_seed(s, n)] for s, n in SAMPLING_SEEDS]
    params = []
    for kw in SAMPLING_PARAMS:
        try:
            params.append(dict(ok=True, greedy=bool(SamplingParams(**kw).greedy)))
        except ValueError:
            params.append(dict(ok=False, greedy=None))
    # which tokens the reference's sample() can produce: its support over many seeds, per (logits row, parameters)
    support = []
    for case in SAMPLING_SUPPORT_CASES:
        logits = sampling_logits(case["seed"], case["vocab"])
        p = SamplingParams(temperature=case["temperature"], top_k=case["top_k"], top_p=case["top_p"])
        counts = [0] * case["vocab"]
        B = 8
        for s in range(0, case["draws"], B):
            toks = sample(logits[None].repeat(B, 1), [p] * B, list(range(s, s + B)), [3] * B)
            for t in toks:
                counts[t] += 1
        support.append(dict(case=case, counts=counts))
    (HERE / "sampling.json").write_text(json.dumps(dict(mix_seed=seeds, params=params, support=support)))
    print(f"sampling: {len(seeds)} seeds, {len(params)} parameter sets, {len(support)} support cases")


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[2] == "sampling":
        sampling_main(sys.argv[1])
    elif len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of the reference project> [sampling]")
    else:
        main(sys.argv[1])
        sampling_main(sys.argv[1])
