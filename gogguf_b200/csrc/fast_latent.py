"""Host side of the tensor-core latent attention kernels (csrc/latent_attention.cu)."""
from __future__ import annotations


def try_make(heads: int, latent_dim: int, rope_dim: int, scale: float, window: int):
    return None
