"""Device sampling (ns_sample_rows behind nanoserve_b200.sampling.sample and inside the engine's graphs) against the CPU
oracle's restatement of the reference's sampler (oracle.ops.sampling_survivors / sampling_probabilities, pinned to the
reference's observed frequencies in tests/test_oracle_golden.py).

The reference draws from a host generator, so equal samples are not reachable on the device; parity is defined as:
  * the set of tokens that survive top-k / top-p equals the oracle's on seeded logits (count and threshold; exact for
    top-k, and for top-p up to a rounding of 2e-6 in the cumulative probability of a 152K-term sum);
  * temperature -> 0 and top_k = 1 give the argmax;
  * a row's token depends only on its logits, parameters and seed: not on its neighbours, its row index or the batch size;
  * over >= 1e5 draws the frequencies are within 5 standard deviations of softmax(logits / T) on the survivors;
  * in the engine, a request's text is reproducible from its seed and survives preemption + recompute unchanged.
"""
import random

import pytest
import torch

from oracle import ops as O
from tests.golden import make_golden as G

pytestmark = pytest.mark.gpu

CASES = [dict(temperature=1.0, top_k=0, top_p=1.0), dict(temperature=0.7, top_k=8, top_p=1.0),
         dict(temperature=1.3, top_k=0, top_p=0.6), dict(temperature=0.9, top_k=12, top_p=0.8),
         dict(temperature=2.0, top_k=3, top_p=0.3), dict(temperature=0.5, top_k=0, top_p=0.95),
         dict(temperature=1.0, top_k=50, top_p=0.9), dict(temperature=0.8, top_k=0, top_p=0.999)]


def _params(**kw):
    from nanoserve_b200.sampling import SamplingParams
    return SamplingParams(**kw)


@pytest.mark.parametrize("vocab", [64, 1000, 151936])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_survivors_equal_the_oracle(vocab, dtype):
    from nanoserve_b200.sampling import sample
    g = torch.Generator().manual_seed(vocab)
    logits = (torch.randn(len(CASES), vocab, generator=g) * 2.0).to(dtype)
    # bf16 rows are full of equal values: a group of equal values is kept or dropped as a whole on both sides. The
    # kernel sums probability mass exactly (fixed point), so the oracle sums in float64 here.
    toks, info = sample(logits.cuda(), [_params(**c) for c in CASES], list(range(len(CASES))), [0] * len(CASES),
                        return_survivors=True)
    for i, c in enumerate(CASES):
        x, keep = O.sampling_survivors(logits[i], c["temperature"], c["top_k"], c["top_p"], mass_dtype=torch.float64)
        thr, kept = info[i]
        assert keep[toks[i]], "the sampled token is not a survivor"
        assert kept == int((x >= thr).sum()), "survivors are exactly the values >= the reported threshold"
        if c["top_p"] >= 1:
            assert kept == int(keep.sum()), (c, vocab)                    # top-k alone: exact
        else:
            # the nucleus boundary is a comparison of a sum of up to 152K fp32 exponentials with p: the kernel's and
            # the oracle's sums differ in the last bits, so the count must lie between the oracle's for p -/+ 2e-6
            lo = int(O.sampling_survivors(logits[i], c["temperature"], c["top_k"], c["top_p"] - 2e-6, torch.float64)[1].sum())
            hi = int(O.sampling_survivors(logits[i], c["temperature"], c["top_k"], min(1.0, c["top_p"] + 2e-6), torch.float64)[1].sum())
            assert lo <= kept <= hi, (c, vocab, lo, kept, hi)
        if kept == int(keep.sum()) and kept < vocab:
            assert thr == x[keep].min().item(), (c, vocab)


def test_greedy_limits_equal_argmax():
    from nanoserve_b200.sampling import sample
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(6, 5000, generator=g)
    want = logits.argmax(-1).tolist()
    dev = logits.cuda()
    assert sample(dev, [None] * 6, [0] * 6, [0] * 6) == want
    assert sample(dev, [_params(temperature=0.0, top_p=0.5)] * 6, [1] * 6, [2] * 6) == want
    assert sample(dev, [_params(temperature=1.5, top_k=1)] * 6, [1] * 6, [2] * 6) == want
    assert sample(dev, [_params(temperature=1e-4)] * 6, [3] * 6, [4] * 6) == want       # gaps >> 1e-4 * Gumbel noise
    assert sample(dev, [_params(temperature=1.0, top_p=1e-6)] * 6, [3] * 6, [4] * 6) == want   # only the best token survives


def test_a_row_does_not_depend_on_its_neighbours():
    from nanoserve_b200.sampling import sample
    g = torch.Generator().manual_seed(2)
    row = torch.randn(151936, generator=g) * 1.5
    p = _params(temperature=0.9, top_k=200, top_p=0.95)
    alone = sample(row[None].cuda(), [p], [77], [5])[0]
    others = torch.randn(9, 151936, generator=g)
    for pos in (0, 4, 9):
        batch = torch.cat([others[:pos], row[None], others[pos:]]).cuda()
        params = [_params(temperature=1.0 + 0.1 * j) if j % 2 else None for j in range(10)]
        params[pos] = p
        seeds = list(range(100, 110))
        seeds[pos] = 77
        assert sample(batch, params, seeds, [5] * 10)[pos] == alone
    assert sample(row[None].cuda(), [p], [77], [6])[0] != alone or sample(row[None].cuda(), [p], [78], [5])[0] != alone


@pytest.mark.parametrize("case", [0, 1, 3, 6])
def test_frequencies_follow_the_oracle_distribution(case):
    """256 rows of the same logits x 400 draw numbers = 102,400 draws per case."""
    from nanoserve_b200.sampling import sample
    c = CASES[case]
    vocab = 300
    logits = G.sampling_logits(10 + case, vocab)
    probs = O.sampling_probabilities(logits, c["temperature"], c["top_k"], c["top_p"])
    dev = logits[None].repeat(256, 1).cuda()
    params = [_params(**c)] * 256
    counts = torch.zeros(vocab, dtype=torch.float64)
    for step in range(400):
        toks = sample(dev, params, list(range(256)), [step] * 256)
        counts += torch.bincount(torch.tensor(toks), minlength=vocab).double()
    n = counts.sum().item()
    assert n == 102400
    assert ((counts > 0) <= (probs > 0)).all()
    sigma = (probs * (1 - probs) / n).sqrt()
    worst = ((counts / n - probs).abs() / (sigma + 1e-12))[probs > 0].max().item()
    print(f"case {c}: {int((probs > 0).sum())} survivors, worst deviation {worst:.2f} sigma")
    assert ((counts / n - probs).abs() <= 5 * sigma + 1e-9).all()


def _engine(kv_tokens, dtype=torch.float32, **kw):
    from tests.test_engine_gpu import gpu_model, make_engine
    cfg, sd = G.TINY_CFG, G.tiny_state_dict(G.TINY_CFG)
    return make_engine(gpu_model(cfg, sd, dtype), max_seq_len=128, max_num_seqs=6, max_num_batched_tokens=48,
                       kv_cache_tokens=kv_tokens, **kw)


def _run(eng, reqs, params):
    ids = {}
    for i, ((prompt, n), p) in enumerate(zip(reqs, params)):
        ids[eng.add_request(prompt, n, ignore_eos=True, sampling=p)] = i
    outs = {i: [] for i in range(len(reqs))}
    while eng.has_unfinished():
        for o in eng.step():
            outs[ids[o.seq_id]].append(o.token)
    return [outs[i] for i in range(len(reqs))]


@pytest.mark.parametrize("lookahead", [False, True])
def test_engine_sampling_is_reproducible_and_survives_preemption(lookahead):
    rng = random.Random(4)
    reqs = [([rng.randrange(512) for _ in range(rng.randint(20, 50))], 30) for _ in range(6)]
    params = [_params(temperature=0.8, top_p=0.9, seed=11), None, _params(temperature=1.2, top_k=20, seed=12),
              _params(temperature=0.0), _params(temperature=0.6, seed=13), _params(temperature=1.0, top_k=5, top_p=0.7, seed=14)]
    roomy = _run(_engine(2048, lookahead=lookahead), reqs, params)
    again = _run(_engine(2048, lookahead=lookahead), reqs, params)
    assert roomy == again                                             # same seeds, same text
    tight_eng = _engine(256, lookahead=lookahead)
    tight = _run(tight_eng, reqs, params)
    assert tight_eng.stats["num_preemptions"] > 0
    assert tight == roomy                                             # draw n is keyed by (seed, n): recompute redraws the same
    greedy = _run(_engine(2048), reqs, [None] * 6)
    assert roomy[1] == greedy[1] and roomy[3] == greedy[3]            # greedy rows beside sampling rows are untouched
    assert roomy[0] != greedy[0] or roomy[2] != greedy[2]             # and the sampling rows really sample
    other = _run(_engine(2048), reqs, [_params(temperature=0.8, top_p=0.9, seed=99)] + params[1:])
    assert other[0] != roomy[0] and other[2] == roomy[2]              # another seed, another text; neighbours unchanged
