"""Sampling on the host: the generator, the uniform draw, and parameter validation."""

import pytest

from zephyr_b200.config import InvalidArgumentError
from zephyr_b200.sampling import GREEDY_TEMPERATURE, MT19937_64, SamplingParams


def test_generator_matches_the_standard():
    g = MT19937_64()
    for _ in range(9999):
        g.next_u64()
    assert g.next_u64() == 9981545732273789042           # the C++ standard's check value for mt19937_64
    assert [MT19937_64(42).next_u64() for _ in range(1)] == [13930160852258120406]   # std::mt19937_64(42)()


def test_uniform_draw():
    g, h = MT19937_64(7), MT19937_64(7)
    for _ in range(100):
        u = g.next_uniform()
        assert 0.0 <= u < 1.0 and u == float(h.next_u64() >> 40) * 2.0 ** -24
        assert u * 2 ** 24 == int(u * 2 ** 24)             # exactly representable in float32


def test_parameters():
    assert SamplingParams(temperature=0.0).greedy and SamplingParams(temperature=GREEDY_TEMPERATURE / 2).greedy
    assert not SamplingParams(temperature=0.7).greedy
    SamplingParams(temperature=0.7).validate(100)
    SamplingParams(temperature=0.0, top_p=1.0, top_k=0, min_p=0.0).validate(100)
    SamplingParams(temperature=0.9, top_p=0.9, top_k=40, min_p=0.05, frequency_penalty=0.1, presence_penalty=-0.1,
                   repetition_penalty=1.2, logits_bias={3: -float("inf")}, top_logprobs=5).validate(100)
    assert SamplingParams(repetition_penalty=1.1).uses_history and not SamplingParams(top_k=3).uses_history
    for bad in (dict(temperature=-1.0), dict(temperature=float("nan")), dict(repetition_penalty=0.0),
                dict(logits_bias={100: 1.0}), dict(logits_bias={1: float("inf")}), dict(top_logprobs=-1),
                dict(top_p=float("inf"))):
        with pytest.raises(InvalidArgumentError):
            SamplingParams(**bad).validate(100)
