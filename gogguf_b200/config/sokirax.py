"""Typed configuration of the Sokirax decoder, read from its config.json keys.

A Sokirax model is a list of layers that may differ from one another.  A layer has a norm before and after each
of its two parts: x += norm1b(mixer(norm1(x))), x += norm2b(ff(norm2(x))); the feed-forward may be absent.  The
mixer is softmax attention inside a sliding window (type "attention": q/k normed head by head, rotation with
stretched frequencies where `rot.scaling` is given) or two mixers side by side (type "parallel"): windowed
attention whose q and k are normed over the whole projection and whose softmax has a sink per head, and retention
(linear attention with a fixed decay per head and a state per sequence), summed with `left_scale` and
`right_scale`.  The feed-forward is a gated unit or routed experts (softmax over the chosen logits) with one shared
gated unit.  A layer with `weights_of: j` runs layer j's tensors with a cache and state of its own.  The head is a
matrix of its own.

config.json keys (every size and constant comes from here):

    architecture   "Sokirax"
    vocab, width   vocabulary and width of the residual stream
    norm.eps       epsilon of every RMS norm
    layers[i]      type "attention": mixer {heads, kv_heads, dim, vdim, scale, mask {size},
                                            rot {base, dims, scaling {factor, original, fast, slow}}}
                   type "parallel":  mixer {left {heads, kv_heads, dim, vdim, scale, mask {size}, rot {base, dims}},
                                            right {heads, dim, vdim, decay [..], rot {base, dims}},
                                            left_scale, right_scale}
                   mlp null | {kind "dense", ff} |
                       {kind "moe", expert {ff}, router {experts, top}, shared {ff}}
                   weights_of j (optional): the layer has no tensors of its own

Tensor names: ``embed``, ``final.norm``, ``head`` and per layer i ``l<i>.norm{1,1b,2,2b}``;
``l<i>.mix.{q,k,v,o,q.norm,k.norm}`` or ``l<i>.mix.left.{q,k,v,o,q.norm,k.norm,sink}`` with
``l<i>.mix.right.{q,k,v,g,o}``; ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.router``,
``l<i>.mlp.e<k>.{gate,up,down}`` and ``l<i>.mlp.shared.{gate,up,down}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .registry import ConfigError, register_architecture
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry

# the design has no position table and no trained context length: positions are bounded by what a
# float32 angle still resolves, which is far beyond any cache
MAX_POSITIONS = 1 << 22

# constant the design fixes: cos and sin of a stretched rotation are multiplied by SLOPE ln(factor) + 1
YARN_MAGNITUDE_SLOPE = 0.1


def _need(d: Any, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"sokirax config: {where} needs {key!r}")
    return d[key]


def _pos_int(d: Any, key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"sokirax config: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _number(d: Any, key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"sokirax config: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None      # factor, original, fast, slow

    @classmethod
    def from_dict(cls, d: Any, dim: int, where: str) -> "RotaryConfig":
        dims = _pos_int(d, "dims", where)
        if dims % 2 or dims > dim:
            raise ConfigError(f"sokirax config: {where}.dims={dims} must be even and at most the head size {dim}")
        base = _number(d, "base", where)
        if not base > 1:
            raise ConfigError(f"sokirax config: {where}.base must be above one")
        sc = d.get("scaling")
        scaling = None
        if sc is not None:
            scaling = tuple(_number(sc, k, where + ".scaling") for k in ("factor", "original", "fast", "slow"))
            if not all(v > 0 for v in scaling):
                raise ConfigError(f"sokirax config: {where}.scaling values must be positive")
        return cls(base=base, dims=dims, scaling=scaling)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = dict(base=self.base, dims=self.dims)
        if self.scaling is not None:
            f, o, fa, sl = self.scaling
            d["scaling"] = dict(factor=f, original=int(o) if float(o).is_integer() else o, fast=fa, slow=sl)
        return d

    def position(self) -> Dict[str, Any]:
        if self.scaling is None:
            return dict(kind="rope_neox", theta=self.base, rotary_dim=self.dims)
        f, o, fa, sl = self.scaling
        return dict(kind="rope_yarn", theta=self.base, rotary_dim=self.dims, factor=f, original=o, fast=fa, slow=sl,
                    magnitude_slope=YARN_MAGNITUDE_SLOPE)


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    rot: RotaryConfig

    @classmethod
    def from_dict(cls, d: Any, where: str) -> "WindowAttentionConfig":
        heads, kv = _pos_int(d, "heads", where), _pos_int(d, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"sokirax config: {where}.heads={heads} is not a multiple of kv_heads={kv}")
        dim = _pos_int(d, "dim", where)
        window = (d.get("mask") or {}).get("size")
        if window is not None and (isinstance(window, bool) or not isinstance(window, int) or window <= 0):
            raise ConfigError(f"sokirax config: {where}.mask.size must be a positive integer, got {window!r}")
        return cls(heads=heads, kv_heads=kv, dim=dim, vdim=_pos_int(d, "vdim", where),
                   scale=_number(d, "scale", where), window=window,
                   rot=RotaryConfig.from_dict(_need(d, "rot", where), dim, where + ".rot"))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                                 scale=self.scale, rot=self.rot.to_dict())
        if self.window is not None:
            d["mask"] = dict(size=self.window)
        return d

    def part(self, width: int, eps: float, prefix: str, qk_norm: str, sink: bool) -> Dict[str, Any]:
        names = dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm", sink="sink")
        return dict(kind="attention", prefix=prefix, params=dict(
            hidden_size=width, num_heads=self.heads, num_kv_heads=self.kv_heads, head_dim=self.dim,
            value_dim=self.vdim, scale=self.scale, window=self.window, qk_norm=qk_norm, qk_norm_eps=eps,
            sink=sink, position=self.rot.position(), names=names))


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: RotaryConfig

    @classmethod
    def from_dict(cls, d: Any, where: str) -> "RetentionConfig":
        heads, dim = _pos_int(d, "heads", where), _pos_int(d, "dim", where)
        decay = _need(d, "decay", where)
        if not isinstance(decay, (list, tuple)) or len(decay) != heads:
            raise ConfigError(f"sokirax config: {where}.decay must list one number per head ({heads})")
        decay = tuple(float(a) for a in decay)
        if not all(0.0 <= a <= 1.0 for a in decay):
            raise ConfigError(f"sokirax config: {where}.decay values must lie in [0, 1]")
        return cls(heads=heads, dim=dim, vdim=_pos_int(d, "vdim", where), decay=decay,
                   rot=RotaryConfig.from_dict(_need(d, "rot", where), dim, where + ".rot"))

    def to_dict(self) -> Dict[str, Any]:
        return dict(heads=self.heads, dim=self.dim, vdim=self.vdim, decay=list(self.decay), rot=self.rot.to_dict())

    def part(self, width: int, eps: float, prefix: str) -> Dict[str, Any]:
        return dict(kind="retention", prefix=prefix, params=dict(
            hidden_size=width, num_heads=self.heads, head_dim=self.dim, value_dim=self.vdim, decay=list(self.decay),
            eps=eps, position=self.rot.position(), names=dict(q="q", k="k", v="v", g="g", o="o")))


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: WindowAttentionConfig
    right: RetentionConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, d: Any, where: str) -> "ParallelMixerConfig":
        return cls(left=WindowAttentionConfig.from_dict(_need(d, "left", where), where + ".left"),
                   right=RetentionConfig.from_dict(_need(d, "right", where), where + ".right"),
                   left_scale=_number(d, "left_scale", where), right_scale=_number(d, "right_scale", where))

    def to_dict(self) -> Dict[str, Any]:
        return dict(left=self.left.to_dict(), right=self.right.to_dict(), left_scale=self.left_scale,
                    right_scale=self.right_scale)


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                   # "dense" or "moe"
    ff: int                     # inner width (of one expert for "moe")
    experts: int = 0
    top: int = 0
    shared_ff: int = 0          # inner width of the shared unit (0: none)

    @classmethod
    def from_dict(cls, d: Any, where: str) -> "FeedForwardConfig":
        kind = _need(d, "kind", where)
        if kind == "dense":
            return cls(kind="dense", ff=_pos_int(d, "ff", where))
        if kind == "moe":
            ex, ro = _need(d, "expert", where), _need(d, "router", where)
            experts, top = _pos_int(ro, "experts", where + ".router"), _pos_int(ro, "top", where + ".router")
            if top > experts:
                raise ConfigError(f"sokirax config: {where}.router.top={top} exceeds experts={experts}")
            sh = d.get("shared")
            return cls(kind="moe", ff=_pos_int(ex, "ff", where + ".expert"), experts=experts, top=top,
                       shared_ff=_pos_int(sh, "ff", where + ".shared") if sh is not None else 0)
        raise ConfigError(f"sokirax config: {where}.kind={kind!r} is not known (dense, moe)")

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return dict(kind="dense", ff=self.ff)
        d: Dict[str, Any] = dict(kind="moe", expert=dict(ff=self.ff), router=dict(experts=self.experts, top=self.top))
        if self.shared_ff:
            d["shared"] = dict(ff=self.shared_ff)
        return d


@dataclass(frozen=True)
class SokiraxLayer:
    type: str                                   # "attention" or "parallel"
    mixer: object                               # WindowAttentionConfig or ParallelMixerConfig
    mlp: Optional[FeedForwardConfig]
    weights_of: Optional[int] = None


@register_architecture("Sokirax", "sokirax")
@dataclass(frozen=True)
class SokiraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[SokiraxLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.05

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "SokiraxConfig":
        raw = _need(d, "layers", "config")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("sokirax config: 'layers' must be a non-empty list")
        layers: List[SokiraxLayer] = []
        for i, ld in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(ld, "type", where)
            if kind == "attention":
                mixer = WindowAttentionConfig.from_dict(_need(ld, "mixer", where), where + ".mixer")
            elif kind == "parallel":
                mixer = ParallelMixerConfig.from_dict(_need(ld, "mixer", where), where + ".mixer")
            else:
                raise ConfigError(f"sokirax config: {where}.type={kind!r} is not known (attention, parallel)")
            mlp = ld.get("mlp")
            src = ld.get("weights_of")
            if src is not None and (isinstance(src, bool) or not isinstance(src, int) or not (0 <= src < len(raw))
                                    or src == i):
                raise ConfigError(f"sokirax config: {where}.weights_of={src!r} must name another layer")
            layers.append(SokiraxLayer(type=kind, mixer=mixer, weights_of=src,
                                       mlp=None if mlp is None else FeedForwardConfig.from_dict(mlp, where + ".mlp")))
        for i, layer in enumerate(layers):
            # the layer whose tensors are used (before or after this one) must have tensors, and the same parts:
            # both run one set of built parts, each with a cache and state of its own
            if layer.weights_of is None:
                continue
            src = layers[layer.weights_of]
            if src.weights_of is not None:
                raise ConfigError(f"sokirax config: layers[{i}].weights_of={layer.weights_of} names a layer without tensors")
            if (layer.type, layer.mixer, layer.mlp) != (src.type, src.mixer, src.mlp):
                raise ConfigError(f"sokirax config: layers[{i}] uses the tensors of layer {layer.weights_of} "
                                  "but describes other sizes")
        eps = _number(_need(d, "norm", "config"), "eps", "norm")
        if not eps > 0:
            raise ConfigError(f"sokirax config: norm.eps must be > 0, got {eps}")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(x) for x in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"), norm_eps=eps,
                   layers=tuple(layers), eos_token_ids=eos_ids,
                   initializer_range=float(d.get("initializer_range", 0.05)))

    # ------------------------------------------------------------------ write
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for l in self.layers:
            ld: Dict[str, Any] = {"type": l.type, "mixer": l.mixer.to_dict(),
                                  "mlp": None if l.mlp is None else l.mlp.to_dict()}
            if l.weights_of is not None:
                ld["weights_of"] = l.weights_of
            layers.append(ld)
        d: Dict[str, Any] = {"architecture": "Sokirax", "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d

    # ------------------------------------------------------------- derived
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def parameter_count(self) -> int:
        W = self.width
        n = 2 * self.vocab * W + W

        def attn(a: WindowAttentionConfig, whole: bool, sink: bool) -> int:
            m = (a.heads + a.kv_heads) * a.dim * W + a.kv_heads * a.vdim * W + W * a.heads * a.vdim
            m += (a.heads + a.kv_heads) * a.dim if whole else 2 * a.dim
            return m + (a.heads if sink else 0)

        for l in self.layers:
            if l.weights_of is not None:
                continue
            n += 2 * W
            if l.type == "attention":
                n += attn(l.mixer, False, False)
            else:
                r = l.mixer.right
                n += attn(l.mixer.left, True, True) + 2 * r.heads * r.dim * W + 3 * r.heads * r.vdim * W
            f = l.mlp
            if f is not None:
                n += 2 * W
                n += 3 * f.ff * W if f.kind == "dense" else f.experts * (3 * f.ff * W + W) + 3 * f.shared_ff * W
        return n

    def kv_bytes_per_token(self, itemsize: int = 2) -> int:
        """Bytes a token adds to the paged caches (the retention states do not grow with the sequence)."""
        n = 0
        for l in self.layers:
            a = l.mixer if l.type == "attention" else l.mixer.left
            n += a.kv_heads * (a.dim + a.vdim) * itemsize
        return n

    # ---------------------------------------------------------------- spec
    def to_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        blocks: List[BlockSpec] = []
        block_of: Dict[int, int] = {}
        schedule: List[ScheduleEntry] = []

        def norm(p: str, name: str) -> PartSpec:
            return PartSpec(kind="rmsnorm", prefix=p, params=dict(size=W, eps=eps, tensor=name))

        for i, l in enumerate(self.layers):
            if l.weights_of is not None:
                continue
            p = f"l{i}."
            if l.type == "attention":
                m = l.mixer.part(W, eps, p + "mix.", qk_norm="head", sink=False)
                mixer = PartSpec(kind=m["kind"], prefix=m["prefix"], params=m["params"])
            else:
                left = l.mixer.left.part(W, eps, "left.", qk_norm="whole", sink=True)
                right = l.mixer.right.part(W, eps, "right.")
                left["weight"], right["weight"] = l.mixer.left_scale, l.mixer.right_scale
                mixer = PartSpec(kind="side_by_side", prefix=p + "mix.", params=dict(members=[left, right]))
            parts: Dict[str, PartSpec] = {"mixer": mixer, "mixer_norm": norm(p, "norm1"),
                                          "mixer_post_norm": norm(p, "norm1b")}
            f = l.mlp
            if f is not None:
                names = dict(gate="gate", up="up", down="down")
                if f.kind == "dense":
                    ff = PartSpec(kind="swiglu", prefix=p + "mlp.", params=dict(
                        hidden_size=W, intermediate_size=f.ff, names=names))
                else:
                    params = dict(hidden_size=W, intermediate_size=f.ff, num_experts=f.experts, top_k=f.top,
                                  score="softmax", renormalize=True, weight_on="output",
                                  activation=dict(kind="silu_glu"),
                                  names=dict(router="router", expert="e{}.", **names))
                    if f.shared_ff:
                        params["shared"] = dict(intermediate_size=f.shared_ff, prefix="shared.", names=names)
                    ff = PartSpec(kind="routed_experts", prefix=p + "mlp.", params=params)
                parts.update(feed_forward=ff, feed_forward_norm=norm(p, "norm2"),
                             feed_forward_post_norm=norm(p, "norm2b"))
            block_of[i] = len(blocks)
            blocks.append(BlockSpec("sandwich_norm", parts))
        # a layer that names another layer's tensors is that layer's block once more, with a cache and state of its own
        for i, l in enumerate(self.layers):
            schedule.append(ScheduleEntry(block=block_of[i if l.weights_of is None else l.weights_of]))
        spec = ModelSpec(
            architecture="Sokirax", vocab_size=self.vocab, hidden_size=W, max_positions=MAX_POSITIONS,
            blocks=tuple(blocks), schedule=tuple(schedule),
            embedding=PartSpec(kind="embedding", prefix="", params=dict(vocab_size=self.vocab, hidden_size=W,
                                                                        tensor="embed")),
            final_norm=PartSpec(kind="rmsnorm", prefix="final.", params=dict(size=W, eps=eps, tensor="norm")),
            head=PartSpec(kind="linear_head", prefix="", params=dict(vocab_size=self.vocab, hidden_size=W,
                                                                     tensor="head")),
            stop_token_ids=self.eos_token_ids,
        )
        spec.validate()
        return spec
