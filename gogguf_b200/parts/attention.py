"""Grouped-query attention mixer with optional per-head q/k RMSNorm and a position encoding.

Order of operations as in the reference (pkg/model/qwen3/model.go:215-260): q, k, v projections
without bias; each q and k head normed over its `head_dim` slice with one shared weight (before the
rotation); rotation of q and k; k (normed, rotated) and v (raw) appended to the cache; attention of
every new token over the cached positions it may see; output projection added to the residual.
Score scale is 1/sqrt(head_dim) unless the spec gives `scale` (pkg/ops/attention.go:24).

Further parameters of the spec, each with the default that leaves the above unchanged: `value_dim` (head size of
v and of the attention output where it differs from `head_dim`), `qk_norm` = "whole" (q normed over its whole
projection with a weight of that size, k alike, instead of head by head), `sink` (a stored number per query head
that joins the softmax's denominator as exp(sink_h), without key, value or scale), `names` (the stored tensors'
local names; keys q, k, v, o, q_norm, k_norm, sink).  `scale_output(m)` puts a factor on the attention output
in float32, before it is rounded for the output projection.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional

import torch

from ..cache.sequence_cache import KVRequest, KVView
from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..csrc import tcgen05_gemm
from ..weights.loader import TensorDecl
from .base import Linear, Runtime, StepContext
from .registry import POSITIONS, lookup, register_mixer

MAX_HEAD_DIM = 256


@register_mixer("attention")
class AttentionMixer:
    @classmethod
    def _names(cls, spec: PartSpec) -> Dict[str, str]:
        n = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight",
                 q_norm="q_norm.weight", k_norm="k_norm.weight", sink="sink")
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def _norm_mode(cls, spec: PartSpec) -> int:
        """0: no q/k norm; 1: head by head; 2: over the whole projection."""
        v = spec.get("qk_norm")
        if not v:
            return 0
        if v is True or v == "head":
            return 1
        if v == "whole":
            return 2
        raise ValueError(f"attention: qk_norm={v!r} is not known (False, True / 'head', 'whole')")

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        h, nq, nkv, d = spec["hidden_size"], spec["num_heads"], spec["num_kv_heads"], spec["head_dim"]
        dv = spec.get("value_dim") or d
        n = cls._names(spec)
        t = {
            n["q"]: TensorDecl(shape=(nq * d, h)),
            n["k"]: TensorDecl(shape=(nkv * d, h)),
            n["v"]: TensorDecl(shape=(nkv * dv, h)),
            n["o"]: TensorDecl(shape=(h, nq * dv)),
        }
        mode = cls._norm_mode(spec)
        if mode:
            t[n["q_norm"]] = TensorDecl(shape=(d if mode == 1 else nq * d,), init="ones_normal")
            t[n["k_norm"]] = TensorDecl(shape=(d if mode == 1 else nkv * d,), init="ones_normal")
        if spec.get("sink"):
            t[n["sink"]] = TensorDecl(shape=(nq,), init="small_normal")
        return t

    @classmethod
    def cache_request(cls, spec: PartSpec) -> KVRequest:
        d, dv = int(spec["head_dim"]), int(spec.get("value_dim") or spec["head_dim"])
        return KVRequest(num_kv_heads=int(spec["num_kv_heads"]), head_dim=d, window=spec.get("window"),
                         value_dim=None if dv == d else dv)

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.hidden = int(spec["hidden_size"])
        self.nq = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec.get("value_dim") or self.d)
        if self.nq % self.nkv:
            raise ValueError(f"attention: {self.nq} query heads are not a multiple of {self.nkv} kv heads")
        if self.d > MAX_HEAD_DIM or self.d % 2:
            raise ValueError(f"attention: head_dim={self.d} is not supported (even, at most {MAX_HEAD_DIM})")
        if self.dv > MAX_HEAD_DIM:
            raise ValueError(f"attention: value_dim={self.dv} is not supported (at most {MAX_HEAD_DIM})")
        self.window = int(spec.get("window") or 0)
        self.scale = float(spec.get("scale") or 1.0 / math.sqrt(self.d))
        self.eps = float(spec.get("qk_norm_eps", 0.0))
        pos = dict(spec["position"])
        self.position = lookup(POSITIONS, pos["kind"], "position encoding")(pos, rt)
        self.rot = int(pos.get("rotary_dim", self.d))
        if self.rot > self.d:
            raise ValueError("attention: rotary_dim exceeds head_dim")
        names = self._names(spec)
        q, k, v = (rt.matrix(weights[names[n]]) for n in ("q", "k", "v"))
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = q.float(), k.float(), v.float()
        # rows: all q heads, then all k heads, then all v heads
        self.qkv = Linear(torch.cat([q, k, v], dim=0), rt)
        self.o = Linear(weights[names["o"]], rt)
        self.norm_mode = self._norm_mode(spec)
        if self.norm_mode:
            self.q_norm = rt.vector(weights[names["q_norm"]])
            self.k_norm = rt.vector(weights[names["k_norm"]])
        else:
            self.q_norm = self.k_norm = None
        self.sink = rt.vector(weights[names["sink"]]) if spec.get("sink") else None
        self.out_scale = 1.0
        # what the kernels written for one head size, a norm head by head and a plain softmax do not take
        self._general = self.dv != self.d or self.norm_mode == 2
        self._fast = None
        if rt.fast and rt.dtype == torch.bfloat16 and self.dv == self.d:
            from ..csrc import fast_attention
            self._fast = fast_attention.try_make(self.nq, self.nkv, self.d, self.scale, self.window)
        # head size 128 with a full rotation by cos/sin tables: the decode form of the q/k/v product can do
        # the per-head work itself (one head per 128-row weight tile)
        self._fused_rope = (self.qkv.tensor_core and self.d == 128 and self.rot == self.d and not self._general
                            and os.environ.get("GOGGUF_B200_FUSE_QKV_ROPE", "1") != "0")

    def can_absorb_norm(self, norm) -> bool:
        return self.qkv.can_fold and norm.size == self.hidden

    def absorb_norm(self, norm) -> bool:
        """Take the block's pre-norm into the q/k/v projection; `forward` then gets RowStats as `h`."""
        if not self.can_absorb_norm(norm):
            return False
        self.qkv.fold_input_norm(norm.weight, norm.eps)
        return True

    def scale_output(self, mult: float) -> bool:
        """A factor on this mixer's output: the attention kernels apply it to their float32 result."""
        self.out_scale = float(mult)
        return True

    def prepare(self, ctx: StepContext) -> None:
        self.position.tables(ctx)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache: KVView,
                writes_cache: bool = True) -> None:
        T, nq, nkv, d, dv = ctx.n_tokens, self.nq, self.nkv, self.d, self.dv
        dt = self.rt.dtype
        q = ctx.ws.get("attn_q", (T, nq * d), dt)
        o = ctx.ws.get("attn_out", (T, nq * dv), dt)
        cos, sin = self.position.tables(ctx)
        table = ctx.page_tables[cache.group]
        if self._fused_rope and tcgen05_gemm.qkv_rope_takes(T):
            # norm, rotation and cache write happen in the projection's epilogue
            self.qkv.qkv_rope(h, T, ws=ctx.ws, q_out=q, qw=self.q_norm, kw=self.k_norm, eps=self.eps, cos=cos, sin=sin,
                              positions=ctx.positions, seq_of_token=ctx.seq_of_token, page_table=table,
                              page_size=cache.page_size, k_pool=cache.k if writes_cache else None,
                              v_pool=cache.v if writes_cache else None, nq=nq, nkv=nkv)
        elif self._general:
            qkv = ctx.ws.get("attn_qkv", (T, (nq + nkv) * d + nkv * dv), dt)
            self.qkv(h, qkv, ws=ctx.ws)
            K.qkv_prep(qkv, q, self.q_norm, self.k_norm, self.eps, self.norm_mode, cos, sin, ctx.positions,
                       ctx.seq_of_token, table, cache.page_size, cache.k if writes_cache else None,
                       cache.v if writes_cache else None, T, nq, nkv, d, dv, self.rot)
        else:
            qkv = ctx.ws.get("attn_qkv", (T, (nq + 2 * nkv) * d), dt)
            self.qkv(h, qkv, ws=ctx.ws)
            K.qk_norm_rope_cache(qkv, q, self.q_norm, self.k_norm, self.eps, cos, sin, ctx.positions,
                                 ctx.seq_of_token, table, cache.page_size,
                                 cache.k if writes_cache else None, cache.v if writes_cache else None,
                                 T, nq, nkv, d, self.rot)
        if self._fast is not None:
            self._fast(q, cache.k, cache.v, o, ctx, table, cache.page_size, sink=self.sink, out_scale=self.out_scale)
        else:
            K.attention_plain(q, cache.k, cache.v, o, ctx.positions, ctx.seq_of_token, table,
                              cache.page_size, T, nq, nkv, d, self.scale, self.window, dv=dv, sink=self.sink,
                              out_scale=self.out_scale)
        self.o(o, residual, accumulate=True, ws=ctx.ws, emit=ctx.shared.get("row_stats"))
