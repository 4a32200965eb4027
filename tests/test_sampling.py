"""Sampling parameters and the sampler on the CPU."""

import pytest

import sampling_cases as sc
from emulated_ops import TorchOps
from qwen3_runtime_b200 import SamplingParams


def test_params_defaults_and_validation():
    p = SamplingParams()
    assert p.is_greedy() and p.temperature == 0.0 and p.top_p == 1.0 and p.top_k == 0 and p.min_p == 0.0
    assert not p.has_penalties() and not p.needs_filter()
    for bad in (dict(temperature=float("nan")), dict(top_p=0.0), dict(top_p=1.5), dict(min_p=-0.1), dict(min_p=2.0),
                dict(min_tokens=-1), dict(repetition_penalty=0.0)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    assert SamplingParams(temperature=0.7, top_k=3).needs_filter() and SamplingParams(presence_penalty=0.1).has_penalties()


@pytest.mark.parametrize("case", [sc.case_greedy_and_equivalents, sc.case_seeded_draws,
                                  sc.case_filters_restrict_the_support, sc.case_bias_and_penalties],
                         ids=lambda f: f.__name__[5:])
def test_sampler(case):
    case(TorchOps(), "cpu")
