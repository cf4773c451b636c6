"""Position encodings.  A mixer builds the one its spec names and asks it for per-step tables."""
from __future__ import annotations

from typing import Any, Dict, Tuple

import torch

from ..csrc import kernels as K
from .base import Runtime, StepContext
from .registry import register_position


@register_position("rope_neox")
class RotaryNeoX:
    """Rotary positions with NeoX pairing (i, i + rotary_dim/2): angle = pos * theta^(-2i/rotary_dim)
    (pkg/ops/rope_tables.go:6-20, pkg/ops/rope_heads.go:30-38).  Angles, cos and sin are computed in
    float64 once per step for all layers that share (theta, rotary_dim) and stored as float32."""

    pairing = "halves"

    def __init__(self, params: Dict[str, Any], rt: Runtime):
        self.theta = float(params["theta"])
        self.rotary_dim = int(params["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {self.rotary_dim}")
        half = self.rotary_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        self.inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                  -2.0 * i / self.rotary_dim).to(rt.device)
        self.key = ("rope", self.theta, self.rotary_dim)     # the tables do not depend on the pairing

    def tables(self, ctx: StepContext) -> Tuple[torch.Tensor, torch.Tensor]:
        got = ctx.shared.get(self.key)
        if got is None:
            half = self.rotary_dim // 2
            cos = ctx.ws.get(f"rope_cos_{self.theta}_{self.rotary_dim}", (ctx.n_tokens, half), torch.float32)
            sin = ctx.ws.get(f"rope_sin_{self.theta}_{self.rotary_dim}", (ctx.n_tokens, half), torch.float32)
            K.rope_tables(ctx.positions, self.inv_freq, cos, sin)
            got = ctx.shared[self.key] = (cos, sin)
        return got


@register_position("rope_adjacent")
class RotaryAdjacent(RotaryNeoX):
    """The same angles with the other pairing: element 2i turns with element 2i + 1 (the interleaved layout),
    angle = pos * theta^(-2i/rotary_dim).  The tables are those of `RotaryNeoX` (column i is pair i), so layers
    of both kinds with equal base and size share them; which elements form a pair is the business of the
    kernel that applies them, and a mixer states the pairing it implements in `pairing`."""

    pairing = "adjacent"
