"""A plain, slow restatement of the Gigopel decoder, one function per mechanism, on the CPU.

It shares no code with the package: tensors come in as a dict of torch tensors by name, the
configuration as the parsed config.json.  Everything is computed in the dtype of `x` (float64 in
the tests), whole sequences at a time, with explicit loops where a loop is the clearest statement.

Notation: x [n, W] is the residual stream of one sequence, positions are 0..n-1.

    layer:   h = znorm(x; w1),  x <- x + m * (mixer(h) + ff(h))          (one norm, two readers)
    znorm:   x / sqrt(mean(x^2) + eps) * (1 + w)
    mixer:   latent attention (below), causal inside a window of `mask.size` positions
    ff:      none, dense (xIELU) or routed experts
    output:  logits = E znorm(x; w_final),  E the embedding table
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

SQRT_2_OVER_PI = math.sqrt(2.0 / math.pi)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def znorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The block norm and the final norm: the stored weight is the offset from one."""
    return rms_unit(x, eps) * (1.0 + w.to(x.dtype))


def wnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The norm of the latent: the stored weight is the factor itself."""
    return rms_unit(x, eps) * w.to(x.dtype)


def rotate_adjacent(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotary positions on the first `dims` elements of the last axis of v [n, ..., d]; element 2i
    is paired with 2i+1, angle a = p * base^(-2i/dims); (u, v) -> (u cos a - v sin a, v cos a + u sin a)."""
    out = v.clone()
    n = v.shape[0]
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        a = positions.to(torch.float64) * f
        shape = [n] + [1] * (v.dim() - 2)
        c, s = torch.cos(a).to(v.dtype).view(shape), torch.sin(a).to(v.dtype).view(shape)
        u, w = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u * c - w * s
        out[..., 2 * i + 1] = w * c + u * s
    return out


def visible(n: int, window: Optional[int]) -> torch.Tensor:
    """mask[i, j]: may position i read position j?  0 <= i - j (< window)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    m = (i - j) >= 0
    if window is not None:
        m &= (i - j) < window
    return m


def latent_attention(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, mx: dict, eps: float) -> torch.Tensor:
    """q = Wq h, per head [dim plain | rot_dim rotated];  Wdkv h = [latent (kv_rank) | shared rotated key (rot_dim)];
    c = wnorm(latent);  k_plain = Wuk c, v = Wuv c per head;  score = (q_plain . k_plain + q_rot . k_rot) * scale;
    softmax over the visible positions; out = Wo concat(heads)."""
    n = h.shape[0]
    H, d, r, dv, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    dt = h.dtype
    W = lambda name: t[p + name].to(dt)
    pos = torch.arange(n)
    q = (h @ W("q").T).view(n, H, d + r)
    dkv = h @ W("dkv").T
    c = wnorm(dkv[:, :R], t[p + "dkv.norm"], eps)
    kr = dkv[:, R:R + r]
    rot = mx.get("rot") or {}
    dims, base = int(rot.get("dims", r)), float(rot.get("base", 10000.0))
    q_plain, q_rot = q[..., :d], rotate_adjacent(q[..., d:], pos, base, dims)
    k_rot = rotate_adjacent(kr, pos, base, dims)
    k_plain = (c @ W("uk").T).view(n, H, d)
    v = (c @ W("uv").T).view(n, H, dv)
    mask = mx.get("mask") or {}
    see = visible(n, mask.get("size"))
    out = torch.zeros(n, H, dv, dtype=dt)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * mx["scale"]
        s = s.masked_fill(~see, float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ v[:, hd]
    return out.reshape(n, H * dv) @ W("o").T


def softplus(z):
    return torch.log1p(torch.exp(z))


def xielu(z: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    ap, aq = softplus(p.to(z.dtype)), 0.5 + softplus(q.to(z.dtype))
    return torch.where(z > 0, ap * z * z + 0.5 * z, aq * (torch.expm1(z) - z) + 0.5 * z)


def dense_ff(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    dt = h.dtype
    a = t[p + "act"]
    return xielu(h @ t[p + "up"].to(dt).T, a[0], a[1]) @ t[p + "down"].to(dt).T


def expert(hin: torch.Tensor, t: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    """g = min(Wg h, L), u = clamp(Wu h, -L, L), y = g sigmoid(1.702 g) (u + 1), out = Wd y."""
    dt = hin.dtype
    g = torch.clamp(hin @ t[p + "gate"].to(dt).T, max=limit)
    u = torch.clamp(hin @ t[p + "up"].to(dt).T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ t[p + "down"].to(dt).T


def routed_ff(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    """scores = sigmoid(Wr h); the `top` largest are chosen; each chosen expert reads score * h."""
    dt = h.dtype
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    limit = mlp["expert"]["limit"]
    s = torch.sigmoid(h @ t[p + "router"].to(dt).T)
    out = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=dt)
    for i in range(h.shape[0]):
        chosen = torch.topk(s[i], top).indices.tolist()
        for e in chosen:
            out[i] += expert((s[i, e] * h[i])[None], t, f"{p}e{e}.", limit)[0]
    return out


def feed_forward(h, t, p, mlp: Optional[dict]):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return dense_ff(h, t, p)
    if mlp["kind"] == "moe":
        return routed_ff(h, t, p, mlp)
    raise ValueError(mlp["kind"])


def layer(x, t, i: int, lc: dict, cfg: dict):
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    h = znorm(x, t[f"l{i}.norm1"], eps)
    if lc["type"] != "latent_attention":
        raise ValueError(lc["type"])
    y = latent_attention(h, t, f"l{i}.mix.", lc["mixer"], eps)
    f = feed_forward(h, t, f"l{i}.mlp.", lc.get("mlp"))
    if f is not None:
        y = y + f
    return x + m * y


def forward(tokens: List[int], t: Dict[str, torch.Tensor], cfg: dict, dtype=torch.float64, layers_out=None):
    """Logits [n, vocab] of one whole sequence; `layers_out` (a list) receives the stream after every layer."""
    E = t["embed"].to(dtype)
    x = E[torch.tensor(tokens, dtype=torch.long)]
    for i, lc in enumerate(cfg["layers"]):
        x = layer(x, t, i, lc, cfg)
        if layers_out is not None:
            layers_out.append(x.clone())
    return znorm(x, t["final.norm"], cfg["norm"]["eps"]) @ E.T
