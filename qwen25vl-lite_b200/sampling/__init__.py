"""Sampling parameters and the device sampler."""

from .params import SamplingParams  # noqa: F401
from .sampler import Sampler, filter_scores, new_seed  # noqa: F401
