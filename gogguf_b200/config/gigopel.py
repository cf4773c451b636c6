"""Typed configuration of the Gigopel decoder, read from its config.json keys.

A Gigopel model is a list of layers that may differ from one another.  Every layer is a *parallel* block:
one norm whose output both the mixer and the feed-forward read, their sum multiplied by ``residual_mult``
and added to the residual stream.  The norms store their weight as an offset from one.  The mixer is latent
attention inside a sliding window; the feed-forward is absent, dense (one up and one down matrix around the
xIELU activation) or a set of routed experts.  The head is the embedding table.

config.json keys (all sizes come from here, none from the code):

    architecture   "Gigopel"
    vocab, width   vocabulary and width of the residual stream
    residual_mult  factor on what a layer adds to the stream
    norm.eps       epsilon of every RMS norm
    layers[i]      type ("latent_attention"), mixer {heads, dim, rot_dim, vdim, kv_rank, scale,
                   rot {base, dims}, mask {size}}, mlp null | {kind "dense", ff} |
                   {kind "moe", expert {ff, limit}, router {experts, top}}

Tensor names: ``embed``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,o}``,
``l<i>.mlp.{up,down,act}`` or ``l<i>.mlp.router`` with ``l<i>.mlp.e<k>.{gate,up,down}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .registry import ConfigError, register_architecture
from .spec import BlockSpec, ModelSpec, PartSpec, default_schedule

# the design has no position table and no trained context length: positions are bounded by what a
# float32 angle still resolves, which is far beyond any cache
MAX_POSITIONS = 1 << 22

# constants the design fixes
GLU_SIGMOID_SLOPE = 1.702      # the experts' gate is g * sigmoid(1.702 g)


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"gigopel config: {where} needs {key!r}")
    return d[key]


def _pos_int(d: Dict[str, Any], key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"gigopel config: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _number(d: Dict[str, Any], key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"gigopel config: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int            # per head: query/key elements that are not rotated
    rot_dim: int        # per head: rotated query elements; the one rotated key part all heads share
    vdim: int           # per head: value elements
    kv_rank: int        # size of the cached latent
    scale: float        # factor on the scores
    rot_base: float
    rot_dims: int       # how many of the rot_dim elements are rotated (the rest pass unchanged)
    window: Optional[int]   # a position sees itself and the window - 1 before it; None: everything before it

    @classmethod
    def from_dict(cls, d: Dict[str, Any], where: str) -> "LatentAttentionConfig":
        rot_dim = _pos_int(d, "rot_dim", where)
        rot = d.get("rot") or {}
        dims = int(rot.get("dims", rot_dim))
        if dims <= 0 or dims % 2 or dims > rot_dim:
            raise ConfigError(f"gigopel config: {where}.rot.dims={dims} must be even and at most rot_dim={rot_dim}")
        mask = d.get("mask") or {}
        window = mask.get("size")
        if window is not None and (isinstance(window, bool) or not isinstance(window, int) or window <= 0):
            raise ConfigError(f"gigopel config: {where}.mask.size must be a positive integer, got {window!r}")
        base = float(rot.get("base", 10000.0))
        if not base > 0:
            raise ConfigError(f"gigopel config: {where}.rot.base must be > 0")
        return cls(heads=_pos_int(d, "heads", where), dim=_pos_int(d, "dim", where), rot_dim=rot_dim,
                   vdim=_pos_int(d, "vdim", where), kv_rank=_pos_int(d, "kv_rank", where),
                   scale=_number(d, "scale", where) if d.get("scale") is not None
                   else (_pos_int(d, "dim", where) + rot_dim) ** -0.5,
                   rot_base=base, rot_dims=dims, window=window)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = dict(heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim,
                                 kv_rank=self.kv_rank, scale=self.scale,
                                 rot=dict(base=self.rot_base, dims=self.rot_dims))
        if self.window is not None:
            d["mask"] = dict(size=self.window)
        return d


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                   # "dense" or "moe"
    ff: int                     # inner width (of one expert for "moe")
    experts: int = 0
    top: int = 0
    limit: float = 0.0

    @classmethod
    def from_dict(cls, d: Dict[str, Any], where: str) -> "FeedForwardConfig":
        kind = _need(d, "kind", where)
        if kind == "dense":
            return cls(kind="dense", ff=_pos_int(d, "ff", where))
        if kind == "moe":
            ex, ro = _need(d, "expert", where), _need(d, "router", where)
            experts, top = _pos_int(ro, "experts", where + ".router"), _pos_int(ro, "top", where + ".router")
            if top > experts:
                raise ConfigError(f"gigopel config: {where}.router.top={top} exceeds experts={experts}")
            limit = _number(ex, "limit", where + ".expert")
            if not limit > 0:
                raise ConfigError(f"gigopel config: {where}.expert.limit must be > 0")
            return cls(kind="moe", ff=_pos_int(ex, "ff", where + ".expert"), experts=experts, top=top, limit=limit)
        raise ConfigError(f"gigopel config: {where}.kind={kind!r} is not known (dense, moe)")

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return dict(kind="dense", ff=self.ff)
        return dict(kind="moe", expert=dict(ff=self.ff, limit=self.limit),
                    router=dict(experts=self.experts, top=self.top))


@dataclass(frozen=True)
class GigopelLayer:
    mixer: LatentAttentionConfig
    mlp: Optional[FeedForwardConfig]


@register_architecture("Gigopel", "gigopel")
@dataclass(frozen=True)
class GigopelConfig:
    vocab: int
    width: int
    residual_mult: float
    norm_eps: float
    layers: Tuple[GigopelLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.05

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GigopelConfig":
        raw = _need(d, "layers", "config")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("gigopel config: 'layers' must be a non-empty list")
        layers: List[GigopelLayer] = []
        for i, ld in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(ld, "type", where)
            if kind != "latent_attention":
                raise ConfigError(f"gigopel config: {where}.type={kind!r} is not known (latent_attention)")
            mixer = LatentAttentionConfig.from_dict(_need(ld, "mixer", where), where + ".mixer")
            mlp = ld.get("mlp")
            layers.append(GigopelLayer(mixer=mixer,
                                       mlp=None if mlp is None else FeedForwardConfig.from_dict(mlp, where + ".mlp")))
        eps = _number(_need(d, "norm", "config"), "eps", "norm")
        if not eps > 0:
            raise ConfigError(f"gigopel config: norm.eps must be > 0, got {eps}")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(x) for x in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"),
                   residual_mult=_number(d, "residual_mult", "config") if d.get("residual_mult") is not None else 1.0,
                   norm_eps=eps, layers=tuple(layers),
                   eos_token_ids=eos_ids, initializer_range=float(d.get("initializer_range", 0.05)))

    # ------------------------------------------------------------------ write
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": "Gigopel",
            "vocab": self.vocab, "width": self.width, "residual_mult": self.residual_mult,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": "latent_attention", "mixer": l.mixer.to_dict(),
                        "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers],
        }
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
        n = self.vocab * self.width + self.width
        for l in self.layers:
            a = l.mixer
            n += self.width + a.heads * (a.dim + a.rot_dim) * self.width + (a.kv_rank + a.rot_dim) * self.width \
                + a.kv_rank + a.heads * (a.dim + a.vdim) * a.kv_rank + self.width * a.heads * a.vdim
            f = l.mlp
            if f is not None and f.kind == "dense":
                n += 2 * f.ff * self.width + 2
            elif f is not None:
                n += f.experts * (3 * f.ff * self.width + self.width)
        return n

    def kv_bytes_per_token(self, itemsize: int = 2) -> int:
        return sum((l.mixer.kv_rank + l.mixer.rot_dim) * itemsize for l in self.layers)

    # ---------------------------------------------------------------- spec
    def to_spec(self) -> ModelSpec:
        blocks: List[BlockSpec] = []
        W = self.width
        for i, l in enumerate(self.layers):
            p = f"l{i}."
            a = l.mixer
            parts: Dict[str, PartSpec] = {
                "norm": PartSpec(kind="rmsnorm", prefix=p,
                                 params=dict(size=W, eps=self.norm_eps, tensor="norm1", weight_offset=1.0)),
                "mixer": PartSpec(kind="latent_attention", prefix=p + "mix.", params=dict(
                    hidden_size=W, num_heads=a.heads, nope_dim=a.dim, rope_dim=a.rot_dim, value_dim=a.vdim,
                    latent_dim=a.kv_rank, scale=a.scale, window=a.window, latent_norm_eps=self.norm_eps,
                    position=dict(kind="rope_adjacent", theta=a.rot_base, rotary_dim=a.rot_dims),
                    names=dict(q="q", down="dkv", latent_norm="dkv.norm", up_k="uk", up_v="uv", out="o"))),
            }
            f = l.mlp
            if f is not None and f.kind == "dense":
                parts["feed_forward"] = PartSpec(kind="xielu_mlp", prefix=p + "mlp.", params=dict(
                    hidden_size=W, intermediate_size=f.ff, names=dict(up="up", down="down", act="act")))
            elif f is not None:
                parts["feed_forward"] = PartSpec(kind="routed_experts", prefix=p + "mlp.", params=dict(
                    hidden_size=W, intermediate_size=f.ff, num_experts=f.experts, top_k=f.top,
                    score="sigmoid", renormalize=False, weight_on="input",
                    activation=dict(kind="clamped_glu", limit=f.limit, slope=GLU_SIGMOID_SLOPE),
                    names=dict(router="router", expert="e{}.", gate="gate", up="up", down="down")))
            blocks.append(BlockSpec("parallel", parts, params=dict(residual_mult=self.residual_mult)))
        spec = ModelSpec(
            architecture="Gigopel", vocab_size=self.vocab, hidden_size=W, max_positions=MAX_POSITIONS,
            blocks=tuple(blocks), schedule=default_schedule(len(blocks)),
            embedding=PartSpec(kind="embedding", prefix="", params=dict(vocab_size=self.vocab, hidden_size=W,
                                                                        tensor="embed")),
            final_norm=PartSpec(kind="rmsnorm", prefix="final.",
                                params=dict(size=W, eps=self.norm_eps, tensor="norm", weight_offset=1.0)),
            head=PartSpec(kind="linear_head", prefix="head.",
                          params=dict(vocab_size=self.vocab, hidden_size=W, tied_to="embed")),
            stop_token_ids=self.eos_token_ids,
        )
        spec.validate()
        return spec
