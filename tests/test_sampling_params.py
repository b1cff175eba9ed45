"""``SamplingParams``: the reference's fields and defaults (src/qwen25vl_lite/sampling.py) and what
``validate`` refuses, each with a message that names the field, the value and the rule."""

import pytest

from qwen25vl_lite.sampling.params import SamplingParams


def test_defaults_are_greedy_and_valid():
    p = SamplingParams()
    p.validate()
    assert p.temperature == 0.0 and p.top_p == 1.0 and p.min_p == 0.0 and p.repetition_penalty == 1.0
    assert not p.has_penalties and not p.has_filters


@pytest.mark.parametrize("field,value", [("temperature", -0.1), ("top_p", 0.0), ("top_p", 1.5), ("max_tokens", 0),
                                         ("repetition_penalty", 0.0), ("min_p", -0.1), ("min_p", 1.1)])
def test_values_outside_their_range_are_refused_by_name(field, value):
    p = SamplingParams(**{field: value})
    with pytest.raises(ValueError, match=rf"SamplingParams\.{field} = {value!r}: must be"):
        p.validate()


def test_penalties_and_filters_are_seen():
    assert SamplingParams(repetition_penalty=1.2).has_penalties
    assert SamplingParams(presence_penalty=0.5).has_penalties and SamplingParams(frequency_penalty=0.5).has_penalties
    assert SamplingParams(temperature=0.8, top_k=40).has_filters
    assert SamplingParams(temperature=0.8, top_p=0.9).has_filters and SamplingParams(temperature=0.8, min_p=0.1).has_filters
    assert not SamplingParams(temperature=0.0, top_k=40, top_p=0.9).has_filters      # greedy takes the maximum whatever the filters
    assert not SamplingParams(temperature=0.8, top_k=-1).has_filters
