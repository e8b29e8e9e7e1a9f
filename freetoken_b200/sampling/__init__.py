"""Sampling options and the device sampler."""

from .params import SamplingParams

__all__ = ["SamplingParams"]
