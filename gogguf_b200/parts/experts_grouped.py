"""Routed experts on the tensor cores: (token, choice) pairs sorted by expert, one product per expert."""
from __future__ import annotations


def try_make(part):
    return None
