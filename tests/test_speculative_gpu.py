"""Speculative decoding on the ragged kernel: the text must equal plain greedy decoding with the target, whatever the
draft proposes (nanoserve/speculative.py:1-22). Checked against the CPU oracle's greedy run of the target (tie rule of
tests/parity.py) and against this library's plain engine; a draft equal to the target is accepted every time; KV
blocks of both pools come back; the draft's tokens reach the host once per step."""
import random

import pytest
import torch

from oracle.engine import OracleEngine, OracleModel, run_requests
from tests.golden import make_golden as G
from tests.parity import check_tokens

pytestmark = pytest.mark.gpu


def _model(cfg, sd, dtype):
    from nanoserve_b200.model import ModelConfig, Qwen2Model
    return Qwen2Model(ModelConfig(**cfg), {k: v.to(dtype).cuda() for k, v in sd.items()})


def _requests(vocab, n=7, seed=5, prompt=(3, 60), out=(4, 24)):
    rng = random.Random(seed)
    return [([rng.randrange(vocab) for _ in range(rng.randint(*prompt))], rng.randint(*out)) for _ in range(n)]


@pytest.mark.parametrize("k", [1, 3, 4])
@pytest.mark.parametrize("same_draft", [True, False])
@pytest.mark.parametrize("graphs", [False, True])
def test_tiny_fp32_speculative_text_equals_greedy_target(k, same_draft, graphs):
    from nanoserve_b200.speculative import SpeculativeEngine
    cfg, sd = G.TINY_CFG, G.tiny_state_dict(G.TINY_CFG)
    dcfg = dict(cfg) if same_draft else dict(cfg, n_layers=2)
    dsd = sd if same_draft else G.tiny_state_dict(dcfg, seed=1)
    if not same_draft:
        dsd["model.embed_tokens.weight"] = sd["model.embed_tokens.weight"]      # a related draft: some guesses land
    reqs = _requests(cfg["vocab_size"])
    eng = SpeculativeEngine(_model(cfg, sd, torch.float32), _model(dcfg, dsd, torch.float32), eos_token_ids=[],
                            num_speculative_tokens=k, max_seq_len=128, max_num_seqs=4, cuda_graphs=graphs)
    free_t, free_d = eng.tpool.allocator.num_free, eng.dpool.allocator.num_free
    got = run_requests(eng, reqs, concurrency=4)
    oracle = OracleEngine(OracleModel(cfg, sd), max_seq_len=128, max_num_seqs=4, max_num_batched_tokens=4096)
    want = run_requests(oracle, reqs, concurrency=4)
    n = len(reqs)
    same, accepted = check_tokens([got[i] for i in range(n)], [want[i] for i in range(n)], lambda i, j: oracle.gaps[i][j],
                                  1e-3, what=f"speculative k={k}")
    st = eng.stats
    print(f"k={k} same_draft={same_draft} graphs={graphs}: {same}/{n} identical, acceptance {st['acceptance_rate']:.2f}, "
          f"{st['tokens_per_target_forward']:.2f} tokens per target forward, host syncs {st['host_syncs']} in {st['steps']} steps")
    assert all(len(got[i]) == reqs[i][1] for i in range(n))
    assert eng.tpool.allocator.num_free == free_t and eng.dpool.allocator.num_free == free_d
    assert st["host_syncs"] <= 2 * st["steps"]
    assert st["num_speculative_tokens"] == k and st["cuda_graphs"] == graphs
    if same_draft and same == n:
        assert st["acceptance_rate"] > 0.95                     # the draft IS the target: (nearly) every guess is taken
    if graphs and k > 1:
        assert st["graph_draft_steps"] > 0


def test_bf16_speculative_on_the_tensor_core_kernels_equals_the_plain_engine():
    """0.5B layer shape (head_dim 64: the tcgen05 prefill kernel serves the k+1-token verification rows, the decode kernel
    the draft steps), bf16, 2-layer target and 1-layer draft: the speculative text equals the plain engine's greedy text
    except where the CPU oracle's top-2 gap is within the bf16 tie rule."""
    from nanoserve_b200.engine import LLMEngine
    from nanoserve_b200.speculative import SpeculativeEngine
    from nanoserve_b200.synthetic import random_state_dict
    sd32, cfg = random_state_dict("qwen2.5-0.5b", dtype=torch.float32, n_layers=2, vocab=8192)
    dsd32, dcfg = random_state_dict("qwen2.5-0.5b", dtype=torch.float32, n_layers=1, vocab=8192)
    sd16 = {k: v.to(torch.bfloat16) for k, v in sd32.items()}
    target = _model(cfg, sd16, torch.bfloat16)
    reqs = _requests(8192, n=10, seed=8, prompt=(8, 90), out=(6, 20))
    eng = SpeculativeEngine(target, _model(dcfg, dsd32, torch.bfloat16), eos_token_ids=[], num_speculative_tokens=3,
                            max_seq_len=256, max_num_seqs=6)
    got = run_requests(eng, reqs, concurrency=6)
    plain = run_requests(LLMEngine(target, eos_token_ids=[], max_seq_len=256, max_num_seqs=6), reqs, concurrency=6)
    oracle = OracleEngine(OracleModel(cfg, {k: v.float() for k, v in sd16.items()}), max_seq_len=256, max_num_seqs=6,
                          max_num_batched_tokens=4096)
    want = run_requests(oracle, reqs, concurrency=6)
    n = len(reqs)
    tie = 2 * 0.06                                   # bf16 logit tolerance of this shape (see tests/test_engine_gpu.py)
    same, _ = check_tokens([got[i] for i in range(n)], [want[i] for i in range(n)], lambda i, j: oracle.gaps[i][j], tie,
                           what="speculative bf16 vs oracle")
    same_plain = sum(got[i] == plain[i] for i in range(n))
    print(f"bf16 speculative: {same}/{n} identical to the oracle, {same_plain}/{n} to the plain engine; "
          f"acceptance {eng.stats['acceptance_rate']:.2f}")
    check_tokens([plain[i] for i in range(n)], [want[i] for i in range(n)], lambda i, j: oracle.gaps[i][j], tie,
                 what="plain bf16 vs oracle")


def test_refusals():
    from nanoserve_b200.sampling import SamplingParams
    from nanoserve_b200.speculative import SpeculativeEngine
    cfg, sd = G.TINY_CFG, G.tiny_state_dict(G.TINY_CFG)
    m = _model(cfg, sd, torch.float32)
    eng = SpeculativeEngine(m, m, eos_token_ids=[], max_seq_len=64, max_num_seqs=2, cuda_graphs=False)
    with pytest.raises(ValueError):
        eng.add_request([1, 2, 3], 4, sampling=SamplingParams(temperature=0.8))
    with pytest.raises(ValueError):
        eng.add_request([1] * 60, 10)
    other = dict(cfg, vocab_size=256)
    with pytest.raises(ValueError):
        SpeculativeEngine(m, _model(other, G.tiny_state_dict(other), torch.float32), eos_token_ids=[])
    sid = eng.add_request([1, 2, 3], 5)
    eng.step()
    eng.abort(sid)
    assert not eng.has_unfinished() and eng.tpool.allocator.num_free == eng.tpool.num_blocks - 1
