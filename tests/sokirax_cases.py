"""Tiny Sokirax configurations for the tests, model folders made from them, and the plain implementation's view
of a folder.  The configurations differ from one another in every size, in the order of their layers, in their
windows and constants; some take values that another model may happen to make equal or one."""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch


def rot(base, dims, scaling=None):
    r = dict(base=base, dims=dims)
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def attn(heads, kv_heads, dim, vdim, scale, window, r):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=r)
    if window is not None:
        m["mask"] = dict(size=window)
    return m


def ret(heads, dim, vdim, decay, r):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay), rot=r)


def par(left, right, left_scale, right_scale):
    return dict(left=left, right=right, left_scale=left_scale, right_scale=right_scale)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, experts, top, shared=None):
    d = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared:
        d["shared"] = dict(ff=shared)
    return d


def layer(kind, mixer, mlp, weights_of=None):
    d = dict(type=kind, mixer=mixer, mlp=mlp)
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


_A = attn(4, 2, 24, 40, 0.21, 70, rot(70000.0, 16, (4.0, 512, 16.0, 2.0)))
_P = par(attn(6, 3, 16, 24, 0.3, 9, rot(900.0, 8)), ret(3, 12, 20, (0.9, 0.97, 0.995), rot(5000.0, 12)), 0.7, 1.6)
# sizes no tensor-core kernel takes; a stretched rotation; a window shorter than a page and one that crosses a page
# border; key and value head sizes that differ; a layer run twice on one set of tensors; a layer without feed-forward
CASE_S = dict(
    architecture="Sokirax", vocab=211, width=96, norm=dict(eps=2e-6),
    layers=[
        layer("parallel", _P, moe(40, 5, 2, shared=56)),
        layer("attention", _A, dense(136)),
        layer("parallel", _P, moe(40, 5, 2, shared=56), weights_of=0),
        layer("attention", attn(3, 3, 10, 6, 0.4, None, rot(123.0, 10)), None),
        layer("attention", _A, dense(136), weights_of=1),
    ])
# values that happen to be one or equal: one head, one key/value head per query head, a window of one position (a
# token sees only itself), one expert of which one is taken, no shared unit, both factors one, decays of one (nothing
# fades) and zero (only the token itself), the whole head rotated, a stretch factor of one
CASE_ONE = dict(
    architecture="Sokirax", vocab=97, width=64, norm=dict(eps=1e-5),
    layers=[
        layer("parallel", par(attn(1, 1, 16, 16, 0.25, 1, rot(10000.0, 16)),
                              ret(2, 16, 16, (1.0, 0.0), rot(10000.0, 16)), 1.0, 1.0), moe(48, 1, 1)),
        layer("attention", attn(2, 2, 16, 16, 0.25, 33, rot(10000.0, 16, (1.0, 64, 8.0, 1.0))), dense(64)),
    ])
# sizes the tensor-core kernels take: head sizes 64 and 128 with equal key and value sizes, wide products, experts
# whose products are large enough for the grouped form, retention heads that the chunked form holds
CASE_W = dict(
    architecture="Sokirax", vocab=523, width=256, norm=dict(eps=3e-6),
    layers=[
        layer("attention", attn(4, 1, 128, 128, 0.09, 150, rot(100000.0, 64, (6.0, 256, 24.0, 1.5))), moe(128, 6, 2, shared=192)),
        layer("parallel", par(attn(8, 2, 64, 64, 0.12, 90, rot(10000.0, 32)),
                              ret(4, 64, 128, (0.96, 0.99, 0.999, 0.9995), rot(10000.0, 32)), 1.3, 0.8), dense(384)),
        layer("parallel", par(attn(4, 4, 64, 64, 0.12, 200, rot(50000.0, 64)),
                              ret(2, 128, 64, (0.98, 0.9999), rot(777.0, 2)), 0.5, 1.0), moe(64, 9, 3)),
    ])


def every_expert(cfg: dict) -> dict:
    """The same configuration with every expert chosen for every token (top = experts).  The bfloat16 comparisons
    of whole models run on these: where the choice is among close logits, rounding alone may take another expert
    and change that token's row by far more than rounding; the choice itself is held exactly by the float32 runs
    and by the feed-forward's own test."""
    import copy
    c = copy.deepcopy(cfg)
    for l in c["layers"]:
        if l["mlp"] is not None and l["mlp"]["kind"] == "moe":
            l["mlp"]["router"]["top"] = l["mlp"]["router"]["experts"]
    return c


# whole heads rotated: head size 128 with a norm head by head takes the q/k/v product's own epilogue (norm, rotation
# by the stretched and lengthened tables, cache write); head size 64 with sinks takes the tensor-core attention;
# a query group of 32 heads per key/value head, which those kernels do not take; retention heads wider than long
CASE_F = dict(
    architecture="Sokirax", vocab=307, width=256, norm=dict(eps=1e-5),
    layers=[
        layer("attention", attn(6, 3, 128, 128, 0.1, 100, rot(30000.0, 128, (5.0, 128, 20.0, 2.0))), dense(320)),
        layer("parallel", par(attn(4, 1, 64, 64, 0.15, 70, rot(2000.0, 64, (3.0, 64, 8.0, 1.0))),
                              ret(2, 32, 96, (0.97, 0.999), rot(2000.0, 32, (3.0, 64, 8.0, 1.0))), 0.9, 1.4), dense(192)),
        layer("attention", attn(32, 1, 64, 64, 0.12, None, rot(10000.0, 64)), None),
        layer("attention", attn(6, 3, 128, 128, 0.1, 100, rot(30000.0, 128, (5.0, 128, 20.0, 2.0))), dense(320), weights_of=0),
    ])
CASES = {"S": (CASE_S, 3), "ONE": (CASE_ONE, 4), "W": (CASE_W, 6), "F": (CASE_F, 8)}
CASES.update({"SB": (every_expert(CASE_S), 3), "WB": (every_expert(CASE_W), 6)})


def make_folder(tmp, name: str, store_dtype: str = "float32", std: float = 0.12, norm_std: float = 0.1) -> str:
    """Write case `name` with the product's random-weights mode; returns the folder."""
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine.model import write_random_model
    cfg, seed = CASES[name]
    folder = os.path.join(str(tmp), f"sokirax_{name}_{store_dtype}_{std}")
    if not os.path.isdir(folder):
        write_random_model(config_from_dict(cfg), seed, folder, dtype=store_dtype, std=std, norm_std=norm_std)
    return folder


def plain_logits(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None):
    import plain_sokirax as plain
    if layers_out is None:
        return plain.forward(cfg, w, tokens, torch.float64)
    logits, states = plain.forward(cfg, w, tokens, torch.float64, keep_layers=True)
    layers_out.extend(states)
    return logits


def draw_case(seed: int) -> dict:
    """A configuration nobody chose: every size, the order of the layers, windows and constants from a seeded
    generator."""
    import random
    r = random.Random(seed)
    width = r.choice([8, 16, 24]) * r.choice([3, 5, 7, 9])

    def draw_rot(dim):
        dims = r.choice([d for d in (2, 4, 8, 16, 32, 64) if d <= dim])
        sc = r.choice([None, None, (r.choice([2.0, 6.0, 40.0]), r.choice([64, 1024]), r.choice([4.0, 24.0]), r.choice([0.5, 1.5]))])
        return rot(r.choice([100.0, 1e4, 300000.0]), dims, sc)

    def draw_attn():
        kv = r.choice([1, 2, 3])
        dim = r.choice([4, 8, 16, 24, 40, 64])
        return attn(kv * r.choice([1, 2, 4]), kv, dim, r.choice([4, 8, 16, 24, 56, 64]), r.choice([0.05, 0.11, 0.3]),
                    r.choice([None, 1, 2, 17, 63, 64, 65, 128, 200]), draw_rot(dim))

    def draw_par():
        H = r.choice([1, 2, 3, 5])
        dim = r.choice([4, 8, 20, 32, 64])
        right = ret(H, dim, r.choice([4, 8, 24, 32, 72]), [r.choice([0.5, 0.9, 0.99, 0.999, 1.0]) for _ in range(H)],
                    draw_rot(dim))
        return par(draw_attn(), right, r.choice([0.4, 1.0, 1.7]), r.choice([0.6, 1.0, 2.0]))

    shapes = [("attention", draw_attn()) if r.random() < 0.5 else ("parallel", draw_par()) for _ in range(r.choice([1, 2, 3]))]
    layers = []
    for i in range(r.choice([1, 2, 3, 4, 5])):
        own = [j for j, l in enumerate(layers) if "weights_of" not in l]
        if own and r.random() < 0.25:
            j = r.choice(own)
            layers.append(dict(layers[j], weights_of=j))
            continue
        kind = r.choice(["none", "dense", "moe", "moe"])
        experts = r.choice([1, 2, 4, 7, 13])
        mlp = None if kind == "none" else dense(r.choice([8, 24, 40, 72, 200])) if kind == "dense" else \
            moe(r.choice([8, 16, 40, 96]), experts, r.randint(1, min(experts, 4)), shared=r.choice([None, 16, 88]))
        t, m = r.choice(shapes)
        layers.append(layer(t, m, mlp))
    return dict(architecture="Sokirax", vocab=r.choice([53, 211, 641, 1031]), width=width,
                norm=dict(eps=r.choice([1e-6, 1e-5, 3e-4])), layers=layers)


_STEADY = {}


def steady_first_token(cfg: dict, w: Dict[str, torch.Tensor]) -> int:
    """A token id for the first position of a bfloat16 comparison.  A sequence's first token leaves retention with
    +-v over its length, the sign being that of q . k: where q and k happen to be nearly orthogonal, rounding
    decides the sign and with it the whole row (and what later positions read of it).  This returns the first id
    whose q and k are at an angle of cos >= 0.1 in every retention head of every layer run (or, where no id is,
    the one whose least cosine is largest), by the plain implementation in float64; float32 comparisons take any
    token."""
    import plain_sokirax as plain
    key = id(w)
    if key in _STEADY:
        return _STEADY[key]
    eps = float(cfg["norm"]["eps"])
    best = (-1.0, 0)
    for tok in range(min(int(cfg["vocab"]), 64)):
        x = w["embed"].double()[[tok]]
        worst = 1.0
        for i, ld in enumerate(cfg["layers"]):
            p = f"l{ld.get('weights_of', i)}."
            if ld["type"] == "parallel":
                mx = ld["mixer"]["right"]
                H, d = mx["heads"], mx["dim"]
                h = plain.wnorm(x, w[p + "norm1"], eps)
                q = plain.rotate_halves((h @ w[p + "mix.right.q"].double().T).view(1, H, d), mx["rot"])
                k = plain.rotate_halves((h @ w[p + "mix.right.k"].double().T).view(1, H, d), mx["rot"])
                cos = (q * k).sum(-1) / (q.norm(dim=-1) * k.norm(dim=-1)).clamp_min(1e-30)
                worst = min(worst, float(cos.abs().min()))
            x = plain.layer(x, w, p, ld, eps)
        best = max(best, (worst, -tok))
        if worst >= 0.1:
            break
    _STEADY[key] = -best[1]
    return -best[1]


def steady(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype: str) -> List[int]:
    """`tokens` as a bfloat16 comparison takes them: with a steady first token (see above); unchanged for float32."""
    if dtype != "bfloat16" or not tokens:
        return list(tokens)
    return [steady_first_token(cfg, w)] + list(tokens[1:])
