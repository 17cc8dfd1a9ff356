"""Host side of per-request sampling against values recorded from the reference (tests/golden/sampling.json, written by
tests/golden/make_golden.py): per-token seeds are bit-exact, parameter validation accepts and refuses the same sets,
and the engine runs greedy parameters and refuses the others."""
import json
from pathlib import Path

import pytest

from nanoserve_b200.sampling import SamplingParams, mix_seed
from tests.golden import make_golden as G

GOLD = json.loads((Path(__file__).parent / "golden" / "sampling.json").read_text())


def test_mix_seed_is_bit_exact():
    assert [(s, n) for s, n, _ in GOLD["mix_seed"]] == [tuple(x) for x in G.SAMPLING_SEEDS]
    for seed, step, want in GOLD["mix_seed"]:
        got = mix_seed(seed, step)
        assert got == want and 0 <= got < 2 ** 63


def test_consecutive_steps_give_unrelated_seeds():
    seen = {mix_seed(42, n) for n in range(1000)} | {mix_seed(s, 0) for s in range(1000)}
    assert len(seen) == 2000 - 1          # (42, 0) appears in both sets


def test_parameter_validation_matches_the_reference():
    assert len(GOLD["params"]) == len(G.SAMPLING_PARAMS)
    for kw, want in zip(G.SAMPLING_PARAMS, GOLD["params"]):
        if want["ok"]:
            assert SamplingParams(**kw).greedy == want["greedy"], kw
        else:
            with pytest.raises(ValueError):
                SamplingParams(**kw)


def test_params_are_immutable_and_hashable():
    p = SamplingParams(temperature=0.7, top_k=40, seed=3)
    with pytest.raises(Exception):
        p.temperature = 1.0
    assert p == SamplingParams(temperature=0.7, top_k=40, seed=3) and hash(p) == hash(SamplingParams(temperature=0.7, top_k=40, seed=3))
