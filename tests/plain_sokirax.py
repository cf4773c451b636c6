"""A plain, slow restatement of the Sokirax decoder, one function per mechanism, on the CPU.

It shares no code with the package: tensors come in as a dict of torch tensors by name, the configuration as
the parsed config.json.  Everything is computed in the dtype of `x` (float64 in the tests), one whole sequence
at a time, with explicit loops where a loop is the clearest statement.

Notation: x [n, W] is the residual stream of one sequence, positions are 0..n-1.

    layer:      x <- x + N1b(mixer(N1(x)));  x <- x + N2b(ff(N2(x)))      (a norm on either side of each part)
    N(x; w):    x / sqrt(mean(x^2) + eps) * w
    mixer:      windowed softmax attention, or attention beside retention ("parallel")
    ff:         none, a gated unit, or routed experts with one shared gated unit
    output:     logits = W_head N(x; w_final)
    layer i with weights_of j reads every tensor of layer j.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ----------------------------------------------------------------------------------------------- norms
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def wnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w.to(x.dtype)


# ----------------------------------------------------------------------------------------------- rotation
def rotary_frequencies(rot: dict) -> (List[float], float):
    """f_i = base^(-2i/dims), i < dims/2, and the factor on cos and sin.  With `scaling` (factor s, original L,
    fast b, slow a): the pair index at which a wave makes t turns within L positions is
    d(t) = dims ln(L / (2 pi t)) / (2 ln base); lo = max(floor d(b), 0), hi = min(ceil d(a), dims - 1);
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); f_i <- f_i / s * r_i + f_i (1 - r_i); the factor is
    0.1 ln s + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    s, L = float(sc["factor"]), float(sc["original"])

    def d(t: float) -> float:
        return dims * math.log(L / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(d(float(sc["fast"]))), 0)
    hi = min(math.ceil(d(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / s * r + fi * (1.0 - r))
    return out, 0.1 * math.log(s) + 1.0


def rotate_halves(v: torch.Tensor, rot: dict) -> torch.Tensor:
    """Rotary positions on the first `dims` elements of the last axis of v [n, heads, d]: element i turns with
    element i + dims/2 by the angle p f_i; (u, w) -> (u c - w s, w c + u s) with c, s the (scaled) cos and sin."""
    dims = int(rot["dims"])
    half = dims // 2
    freq, mag = rotary_frequencies(rot)
    n = v.shape[0]
    out = v.clone()
    p = torch.arange(n, dtype=torch.float64)
    for i in range(half):
        a = p * freq[i]
        c = (torch.cos(a) * mag).to(v.dtype)[:, None]
        s = (torch.sin(a) * mag).to(v.dtype)[:, None]
        u, w = v[..., i], v[..., i + half]
        out[..., i] = u * c - w * s
        out[..., i + half] = w * c + u * s
    return out


# ----------------------------------------------------------------------------------------------- attention
def windowed_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                               window: Optional[int], sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [n, H, d], k [n, G, d], v [n, G, dv] -> [n, H, dv].  Position i reads j with 0 <= i - j (< window); query
    head h reads key/value head h // (H / G).  With a sink, exp(sink_h) joins the softmax's denominator: it has no
    key, no value and no scale."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(n):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = s.max()
            if sink is not None:
                m = torch.maximum(m, sink[h].to(q.dtype))
            e = torch.exp(s - m)
            den = e.sum()
            if sink is not None:
                den = den + torch.exp(sink[h].to(q.dtype) - m)
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


def attention_mixer(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, mx: dict, eps: float,
                    whole_norm: bool, sink: bool) -> torch.Tensor:
    """q, k, v projections; q and k normed (per head with one weight of the head's size, or over the whole
    projection with a weight of its size) and then rotated; windowed softmax; output projection."""
    n = h.shape[0]
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    dt = h.dtype
    W = lambda name: t[p + name].to(dt)
    q, k, v = h @ W("q").T, h @ W("k").T, h @ W("v").T
    if whole_norm:
        q, k = wnorm(q, t[p + "q.norm"], eps), wnorm(k, t[p + "k.norm"], eps)
        q, k = q.view(n, H, d), k.view(n, G, d)
    else:
        q, k = wnorm(q.view(n, H, d), t[p + "q.norm"], eps), wnorm(k.view(n, G, d), t[p + "k.norm"], eps)
    q, k = rotate_halves(q, mx["rot"]), rotate_halves(k, mx["rot"])
    window = (mx.get("mask") or {}).get("size")
    o = windowed_softmax_attention(q, k, v.view(n, G, dv), float(mx["scale"]), window,
                                   t[p + "sink"] if sink else None)
    return o.reshape(n, H * dv) @ W("o").T


# ----------------------------------------------------------------------------------------------- retention
def retention_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: List[float]) -> torch.Tensor:
    """Per head: S_t = decay_h S_(t-1) + k_t v_t^T (S_-1 = 0), o_t = S_t^T q_t.  q, k [n, H, d], v [n, H, dv]."""
    n, H, d = q.shape
    dv = v.shape[-1]
    out = torch.zeros(n, H, dv, dtype=q.dtype)
    for h in range(H):
        S = torch.zeros(d, dv, dtype=q.dtype)
        for i in range(n):
            S = decay[h] * S + torch.outer(k[i, h], v[i, h])
            out[i, h] = S.T @ q[i, h]
    return out


def retention_mixer(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, mx: dict, eps: float) -> torch.Tensor:
    """q, k rotated, k times dim^(-1/2) after the rotation; the recurrence; every head's output divided by its
    root mean square (no weight); heads joined, times silu(W_g h), output projection."""
    n = h.shape[0]
    H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
    dt = h.dtype
    W = lambda name: t[p + name].to(dt)
    q = rotate_halves((h @ W("q").T).view(n, H, d), mx["rot"])
    k = rotate_halves((h @ W("k").T).view(n, H, d), mx["rot"]) * d ** -0.5
    v = (h @ W("v").T).view(n, H, dv)
    o = rms_unit(retention_recurrence(q, k, v, [float(x) for x in mx["decay"]]), eps).reshape(n, H * dv)
    g = h @ W("g").T
    return (o * (g * torch.sigmoid(g))) @ W("o").T


def parallel_mixer(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, mx: dict, eps: float) -> torch.Tensor:
    left = attention_mixer(h, t, p + "left.", mx["left"], eps, whole_norm=True, sink=True)
    right = retention_mixer(h, t, p + "right.", mx["right"], eps)
    return float(mx["left_scale"]) * left + float(mx["right_scale"]) * right


# ----------------------------------------------------------------------------------------------- feed-forward
def gated_unit(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    """W_down (silu(W_gate h) * (W_up h))."""
    dt = h.dtype
    g, u = h @ t[p + "gate"].to(dt).T, h @ t[p + "up"].to(dt).T
    return (g * torch.sigmoid(g) * u) @ t[p + "down"].to(dt).T


def routed_experts(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    """z = W_router h; the `top` largest logits are chosen, their weights are the softmax over the chosen logits;
    the weighted sum of the chosen experts' outputs, plus the shared unit's output for every token."""
    dt = h.dtype
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ t[p + "router"].to(dt).T
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(z[i, e]), e))[:top]
        w = torch.softmax(z[i, order], dim=0)
        for e, we in zip(order, w):
            out[i] += we * gated_unit(h[i:i + 1], t, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_unit(h, t, p + "shared.")
    return out


def feed_forward(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return gated_unit(h, t, p)
    if mlp["kind"] == "moe":
        return routed_experts(h, t, p, mlp)
    raise ValueError(mlp["kind"])


# ----------------------------------------------------------------------------------------------- the model
def layer(x: torch.Tensor, t: Dict[str, torch.Tensor], p: str, ld: dict, eps: float) -> torch.Tensor:
    h = wnorm(x, t[p + "norm1"], eps)
    if ld["type"] == "attention":
        m = attention_mixer(h, t, p + "mix.", ld["mixer"], eps, whole_norm=False, sink=False)
    elif ld["type"] == "parallel":
        m = parallel_mixer(h, t, p + "mix.", ld["mixer"], eps)
    else:
        raise ValueError(ld["type"])
    x = x + wnorm(m, t[p + "norm1b"], eps)
    if ld.get("mlp") is not None:
        f = feed_forward(wnorm(x, t[p + "norm2"], eps), t, p + "mlp.", ld["mlp"])
        x = x + wnorm(f, t[p + "norm2b"], eps)
    return x


def forward(cfg: dict, t: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            keep_layers: bool = False):
    """Logits [n, vocab] of one sequence (and, on request, the residual stream after every layer run)."""
    eps = float(cfg["norm"]["eps"])
    x = t["embed"].to(dtype)[torch.tensor(tokens, dtype=torch.long)]
    states = []
    for i, ld in enumerate(cfg["layers"]):
        src = ld.get("weights_of", i)
        x = layer(x, t, f"l{src}.", ld, eps)
        if keep_layers:
            states.append(x.clone())
    logits = wnorm(x, t["final.norm"], eps) @ t["head"].to(dtype).T
    return (logits, states) if keep_layers else logits
