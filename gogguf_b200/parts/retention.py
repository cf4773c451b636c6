"""Retention mixer: linear attention with a fixed decay per head, no softmax and no denominator.

Per head h with sizes d (queries, keys) and dv (values), for the tokens of one sequence in order:

    q_t, k_t = rotate(W_q x_t), rotate(W_k x_t) * d^(-1/2)        (rotation first, then the factor on k)
    S_t = decay_h S_(t-1) + k_t v_t^T,   S_(-1) = 0               (S: [d, dv], float32, one per sequence)
    o_t = S_t^T q_t
    y_t = W_o ( concat_h( o_t / rms(o_t) ) * silu(W_g x_t) )      (rms over dv, eps inside the root, no weight)

What a layer keeps per sequence is S alone (`StateRequest`), whatever the sequence's length; the state is read at
the start of a step and written back at its end, so prompts may come in portions and decoding goes on from them.
Rotation, decays, the state, the outputs' norm and the gate's product are float32 in both compute paths; the four
projections of x run as one product in the compute dtype.

Spec parameters: hidden_size, num_heads, head_dim, value_dim, decay (one number per head), eps, position (a
rotation of the `rope_neox` family), key_scale (default head_dim^(-1/2)), names (keys q, k, v, g, o).
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from ..cache.sequence_cache import StateRequest, StateView
from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Linear, Runtime, StepContext
from .registry import POSITIONS, lookup, register_mixer

CHUNKED_FROM = 64       # new tokens of one sequence from which a step takes the chunked form


@register_mixer("retention")
class RetentionMixer:
    @classmethod
    def _names(cls, spec: PartSpec) -> Dict[str, str]:
        n = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", g="g_proj.weight", o="o_proj.weight")
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        h, H, d, dv = spec["hidden_size"], spec["num_heads"], spec["head_dim"], spec["value_dim"]
        n = cls._names(spec)
        return {n["q"]: TensorDecl(shape=(H * d, h)), n["k"]: TensorDecl(shape=(H * d, h)),
                n["v"]: TensorDecl(shape=(H * dv, h)), n["g"]: TensorDecl(shape=(H * dv, h)),
                n["o"]: TensorDecl(shape=(h, H * dv))}

    @classmethod
    def cache_request(cls, spec: PartSpec) -> StateRequest:
        return StateRequest(shape=(int(spec["num_heads"]), int(spec["head_dim"]), int(spec["value_dim"])),
                            dtype=torch.float32)

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.hidden = int(spec["hidden_size"])
        self.H, self.d, self.dv = int(spec["num_heads"]), int(spec["head_dim"]), int(spec["value_dim"])
        decay = [float(x) for x in spec["decay"]]
        if len(decay) != self.H:
            raise ValueError(f"retention: {len(decay)} decays for {self.H} heads")
        if not all(0.0 <= a <= 1.0 for a in decay):
            raise ValueError("retention: every decay must lie in [0, 1]")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=rt.device)
        self.eps = float(spec["eps"])
        self.key_scale = float(spec.get("key_scale") or self.d ** -0.5)
        pos = dict(spec["position"])
        self.position = lookup(POSITIONS, pos["kind"], "position encoding")(pos, rt)
        if getattr(self.position, "pairing", "halves") != "halves":
            raise ValueError("retention: the rotation must pair element i with element i + rotary_dim / 2")
        self.rot = int(pos.get("rotary_dim", self.d))
        if self.rot > self.d:
            raise ValueError("retention: rotary_dim exceeds head_dim")
        n = self._names(spec)
        mats = [rt.matrix(weights[n[k]]) for k in ("q", "k", "v", "g")]
        if len({m.dtype for m in mats}) != 1:
            mats = [m.float() for m in mats]
        # rows: all q heads, all k heads, all v heads, the gate
        self.qkvg = Linear(torch.cat(mats, dim=0), rt)
        self.o = Linear(weights[n["o"]], rt)
        self.out_scale = 1.0
        # prompts: chunks over many CTAs where the head sizes allow (GOGGUF_B200_RETENTION_CHUNKED=1: chunks in
        # one CTA per head, the twin; =0: token by token, the form of decode steps)
        mode = os.environ.get("GOGGUF_B200_RETENTION_CHUNKED", "2")
        self._many = mode == "2" and max(self.d, self.dv) <= K.RETENTION_CHUNKS_MAX_HEAD
        self._chunked = mode != "0" and K.retention_chunk_takes(self.d, self.dv)

    def can_absorb_norm(self, norm) -> bool:
        return self.qkvg.can_fold and norm.size == self.hidden

    def absorb_norm(self, norm) -> bool:
        """Take the block's pre-norm into the q/k/v/gate projection; `forward` then gets RowStats as `h`."""
        if not self.can_absorb_norm(norm):
            return False
        self.qkvg.fold_input_norm(norm.weight, norm.eps)
        return True

    def scale_output(self, mult: float) -> bool:
        """A factor on this mixer's output: it multiplies the gated heads in float32, before the output product."""
        self.out_scale = float(mult)
        return True

    def prepare(self, ctx: StepContext) -> None:
        self.position.tables(ctx)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache: StateView,
                writes_cache: bool = True) -> None:
        if not writes_cache:
            raise ValueError("retention: a layer's state cannot be read by another layer")
        T, H, d, dv = ctx.n_tokens, self.H, self.d, self.dv
        dt = self.rt.dtype
        width = 2 * H * d + 2 * H * dv
        x = ctx.ws.get("retention_qkvg", (T, width), dt)
        self.qkvg(h, x, ws=ctx.ws)
        cos, sin = self.position.tables(ctx)
        y = ctx.ws.get("retention_out", (T, H * dv), dt)
        raw = ctx.ws.get("retention_raw", (T, H * dv), torch.float32)
        if self._many and ctx.max_new >= CHUNKED_FROM:
            n = K.retention_chunks_scratch(T, ctx.n_seqs, H, d, dv)
            K.retention_chunks(x, y, ctx.ws.get("retention_chunk_states", (n,), torch.float32), cache.state, cos, sin,
                               ctx.cu_seqlens, ctx.slots, ctx.seq_of_token, self.decay, T, ctx.n_seqs, H, d, dv,
                               self.rot, self.key_scale, self.eps, self.out_scale)
            self.o(y, residual, accumulate=True, ws=ctx.ws)
            return
        form = 1 if (self._chunked and ctx.max_new >= CHUNKED_FROM) else 0
        K.retention(x, y, raw, cache.state, cos, sin, ctx.cu_seqlens, ctx.slots, ctx.seq_of_token, self.decay,
                    T, ctx.n_seqs, H, d, dv, self.rot, self.key_scale, self.eps, self.out_scale, form)
        self.o(y, residual, accumulate=True, ws=ctx.ws)
