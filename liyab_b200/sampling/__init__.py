"""Greedy, temperature, top-k and top-p sampling."""
from .params import SamplingParams, uniform_draw

__all__ = ["SamplingParams", "uniform_draw"]
