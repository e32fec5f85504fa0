"""Sampling options and the plain sampler (no GPU)."""

import math

import pytest
import torch

from llm_runtime_study_b200.errors import SamplingError
from llm_runtime_study_b200.sampling.config import SamplingConfig
from tests.plain import sampling_plain as plain


@pytest.mark.parametrize("kwargs", [
    dict(temperature=-0.1), dict(temperature=float("nan")), dict(temperature=float("inf")),
    dict(top_k=0), dict(top_k=-3), dict(top_p=0.0), dict(top_p=1.5), dict(top_p=float("nan")), dict(seed=-1),
])
def test_bad_options(kwargs):
    with pytest.raises(SamplingError):
        SamplingConfig(**kwargs)


def test_defaults_are_greedy():
    c = SamplingConfig()
    assert (c.temperature, c.top_k, c.top_p, c.seed) == (0.0, None, 1.0, None)


def test_plain_filters_follow_the_reference_rules():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 3.0])
    assert plain.kept_mask(logits, 1.0, 2, 1.0).tolist() == [True, False, False, False, True]
    probs = torch.softmax(logits, 0)                 # sorted: 3.0, 2.0, 1.0, 0.5, -1.0
    p = float(probs[4]) + 1e-6                       # just above the top token's mass: second stays too
    assert plain.kept_mask(logits, 1.0, None, p).tolist() == [True, False, False, False, True]
    assert plain.kept_mask(logits, 1.0, None, 1e-9).tolist() == [False, False, False, False, True]
    assert plain.kept_mask(logits, 1.0, None, 1.0).all()


def test_plain_sampler_is_seeded_and_follows_softmax():
    logits = torch.tensor([0.0, 1.0, 2.0, -1.0])
    a = [plain.sample(logits, 0.8, None, 1.0, 5, c)[0] for c in range(20)]
    b = [plain.sample(logits, 0.8, None, 1.0, 5, c)[0] for c in range(20)]
    assert a == b and len(set(a)) > 1
    counts = torch.zeros(4)
    for c in range(3000):
        counts[plain.sample(logits, 1.0, None, 1.0, 9, c)[0]] += 1
    assert float((counts / 3000 - torch.softmax(logits, 0)).abs().max()) < 0.03
    u = plain.uniforms(1, 2, 1000)
    assert 0 < float(u.min()) and float(u.max()) < 1 and abs(float(u.mean()) - 0.5) < 0.05
    assert plain.sample(logits, 0.0, None, 1.0, 0, 0)[0] == 2 and math.isfinite(float(u.sum()))
