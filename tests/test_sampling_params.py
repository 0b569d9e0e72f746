"""SamplingParams: the reference's names, defaults and checks (src/dli/sampling.py:22-56).  No GPU."""

import dataclasses

import pytest

from dli_b200 import SamplingParams


def test_defaults_and_greedy():
    p = SamplingParams()
    assert (p.max_tokens, p.temperature, p.top_k, p.top_p, p.seed, p.stop_token_ids, p.ignore_eos) == (16, 0.0, -1, 1.0, None, (), False)
    assert p.greedy and SamplingParams(temperature=0.7, top_k=1).greedy and not SamplingParams(temperature=0.7).greedy
    with pytest.raises(dataclasses.FrozenInstanceError):
        p.max_tokens = 3


@pytest.mark.parametrize("bad", [dict(max_tokens=0), dict(temperature=-0.1), dict(temperature=2.5), dict(temperature=float("nan")),
                                 dict(top_k=0), dict(top_k=-2), dict(top_p=0.0), dict(top_p=1.5)])
def test_values_out_of_range_are_refused(bad):
    with pytest.raises(ValueError, match=next(iter(bad))):
        SamplingParams(**bad)


def test_the_edges_are_allowed():
    SamplingParams(max_tokens=1, temperature=2.0, top_k=1, top_p=1.0)
    SamplingParams(temperature=0.0, top_p=1e-9, stop_token_ids=(1, 2), seed=2**62, ignore_eos=True)
