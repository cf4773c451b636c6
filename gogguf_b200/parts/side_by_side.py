"""A mixer made of several mixers that read the same input side by side; its output is their weighted sum.

Spec parameters: `members`, a list of dicts with `kind` (a registered mixer kind), `params` (that mixer's own
parameters), `prefix` (added to the part's prefix for the member's tensors) and `weight` (the factor on the
member's output, default 1).  Each member keeps a cache or state of its own: the part's cache request is the tuple
of its members' requests and it is handed the tuple of their views.  A member that takes its factor into its own
last step (`scale_output(w) -> bool`) adds straight into the output; any other member writes into a zeroed buffer
that is added with its factor.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Runtime, StepContext
from .registry import MIXERS, lookup, register_mixer


def _members(spec: PartSpec) -> List[Tuple[PartSpec, type, float]]:
    out = []
    for m in spec["members"]:
        ps = PartSpec(kind=m["kind"], params=dict(m.get("params") or {}), prefix=m.get("prefix", ""))
        out.append((ps, lookup(MIXERS, ps.kind, "mixer"), float(m.get("weight", 1.0))))
    if not out:
        raise ValueError("side_by_side: no members")
    return out


@register_mixer("side_by_side")
class SideBySideMixer:
    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        t: Dict[str, TensorDecl] = {}
        for ps, mcls, _ in _members(spec):
            for local, decl in mcls.tensors(ps).items():
                if ps.prefix + local in t:
                    raise ValueError(f"side_by_side: two members declare the tensor {ps.prefix + local!r}")
                t[ps.prefix + local] = decl
        return t

    @classmethod
    def cache_request(cls, spec: PartSpec):
        return tuple(mcls.cache_request(ps) for ps, mcls, _ in _members(spec))

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.members = []
        for ps, mcls, w in _members(spec):
            own = {local: weights[ps.prefix + local] for local in mcls.tensors(ps) if ps.prefix + local in weights}
            part = mcls(ps, own, rt)
            take = getattr(part, "scale_output", None)
            direct = w == 1.0 or (take is not None and bool(take(w)))
            self.members.append((part, w, direct))

    def absorb_norm(self, norm) -> bool:
        """The norm before this mixer goes into every member's first projection, or into none: all members read
        the same input."""
        parts = [p for p, _, _ in self.members]
        if not all(getattr(p, "can_absorb_norm", None) is not None and p.can_absorb_norm(norm) for p in parts):
            return False
        return all([bool(p.absorb_norm(norm)) for p in parts])

    @property
    def capturable(self) -> bool:
        return all(getattr(p, "capturable", True) for p, _, _ in self.members)

    def prepare(self, ctx: StepContext) -> None:
        for part, _, _ in self.members:
            prep = getattr(part, "prepare", None)
            if prep is not None:
                prep(ctx)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache, writes_cache: bool = True) -> None:
        if not isinstance(cache, tuple) or len(cache) != len(self.members):
            raise ValueError("side_by_side: one cache view per member is expected")
        for (part, w, direct), view in zip(self.members, cache):
            if direct:
                part.forward(h, residual, ctx, view, writes_cache)
                continue
            buf = ctx.ws.get("side_by_side_out", tuple(residual.shape), torch.float32)
            buf.zero_()
            part.forward(h, buf, ctx, view, writes_cache)
            K.residual_axpy(residual, buf, w)
