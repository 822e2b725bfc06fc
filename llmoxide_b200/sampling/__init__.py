"""Greedy, temperature, top-k, top-p and repetition-penalty sampling."""

from .params import Rng, Sampling

__all__ = ["Rng", "Sampling"]
