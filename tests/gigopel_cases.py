"""Tiny Gigopel configurations for the tests, model folders made from them, and the plain implementation's
view of a folder.  The configurations differ from one another in every size, in the order of their layers, in
their windows and constants; some take values that another model may happen to make equal or one."""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch


def mixer(heads, dim, rot_dim, vdim, kv_rank, scale, base, dims=None, window=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
             rot=dict(base=base, dims=rot_dim if dims is None else dims))
    if window is not None:
        m["mask"] = dict(size=window)
    return m


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, limit, experts, top):
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top))


def layer(mx, mlp):
    return dict(type="latent_attention", mixer=mx, mlp=mlp)


# sizes the tensor-core kernels take (latent and rotated sizes multiples of 16); a window that crosses a page
# border, one shorter than a tile, one layer without a window; two of five experts; a layer without feed-forward
CASE_T = dict(
    architecture="Gigopel", vocab=211, width=96, residual_mult=0.45, norm=dict(eps=2e-6),
    layers=[
        layer(mixer(3, 24, 16, 40, 48, 0.21, 70000.0, window=70), dense(136)),
        layer(mixer(3, 24, 16, 40, 48, 0.21, 70000.0, window=7), moe(72, 1.5, 5, 2)),
        layer(mixer(2, 8, 32, 16, 80, 0.3, 900.0, dims=16), None),
        layer(mixer(3, 24, 16, 40, 48, 0.21, 70000.0, window=70), moe(40, 0.7, 3, 3)),
    ])
# one head, one expert of which one is taken, a window of one position (a token sees only itself), a factor of
# one on the residual, equal plain and value sizes
CASE_ONE = dict(
    architecture="Gigopel", vocab=97, width=64, residual_mult=1.0, norm=dict(eps=1e-5),
    layers=[
        layer(mixer(1, 16, 16, 16, 32, 0.25, 10000.0, window=1), moe(48, 2.0, 1, 1)),
        layer(mixer(1, 16, 16, 16, 32, 0.25, 10000.0, window=33), dense(64)),
    ])
# sizes that no tensor-core kernel takes: every product and the attention run on the plain kernels in bfloat16 too
CASE_ODD = dict(
    architecture="Gigopel", vocab=131, width=50, residual_mult=0.8, norm=dict(eps=1e-6),
    layers=[
        layer(mixer(5, 10, 6, 12, 40, 0.4, 5000.0, dims=4, window=21), moe(30, 1.0, 7, 3)),
        layer(mixer(2, 14, 10, 6, 24, 0.15, 123456.0, window=64), dense(70)),
    ])
# wide enough for the tensor-core products of more than 128 tokens and for the experts' grouped products
CASE_W = dict(
    architecture="Gigopel", vocab=523, width=256, residual_mult=0.35, norm=dict(eps=3e-6),
    layers=[
        layer(mixer(8, 32, 32, 32, 128, 0.13, 100000.0, window=150), moe(128, 1.0, 6, 2)),
        layer(mixer(4, 64, 16, 64, 272, 0.11, 10000.0, window=90), dense(384)),
        layer(mixer(8, 32, 32, 32, 128, 0.13, 100000.0, window=150), moe(64, 3.0, 9, 1)),
    ])
CASES = {"T": (CASE_T, 3), "ONE": (CASE_ONE, 4), "ODD": (CASE_ODD, 5), "W": (CASE_W, 6)}


def make_folder(tmp, name: str, store_dtype: str = "float32", std: float = 0.12, norm_std: float = 0.1) -> str:
    """Write case `name` with the product's random-weights mode; returns the folder."""
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine.model import write_random_model
    cfg, seed = CASES[name]
    folder = os.path.join(str(tmp), f"gigopel_{name}_{store_dtype}_{std}")
    if not os.path.isdir(folder):
        write_random_model(config_from_dict(cfg), seed, folder, dtype=store_dtype, std=std, norm_std=norm_std)
    return folder


def plain_logits(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None):
    import plain_gigopel as plain
    return plain.forward(tokens, w, cfg, torch.float64, layers_out)
