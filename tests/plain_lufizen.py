"""A plain, slow Lufizen: whole sequences on the CPU, one function per mechanism.

Written from the design's equations and nothing else; it shares no code with the package.  Everything is torch on
the CPU in ``dtype`` (float64 by default).  ``weights`` maps checkpoint tensor names to tensors, ``config`` is the
dict of a config.json.

    x = embed[token] * embedding.scale
    per layer i:   x <- x + N(mixer(x); norm1);   x <- x + N(ff(x); norm2)  (if the layer has a feed-forward)
    logits = logit_scale * head . N(x; final.norm)
    N(y; w) = y / sqrt(mean(y^2) + eps) * w           (the norm sits on a sublayer's OUTPUT; sublayers read x itself)

Mixers: ``attention`` (grouped queries, values that ARE the projected keys, half-split rotation with stretched
frequencies, a weightless per-head norm after the rotation, a learned sink) and ``latent_attention`` (queries through
a normed latent, keys and values out of a normed latent plus one rotated key part for all heads, a gate per head).
Feed-forward: routed experts (sigmoid scores, a correction that only the choice sees, groups ranked by their two
best members) plus a gated shared expert.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------------------------ small pieces
def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) (* w) over the last axis."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2i / dims), i < dims / 2, then (if ``scaling`` is given) stretched by wavelength l = 2 pi / f:
    kept where l < original / high, divided by ``factor`` where l > original / low, and in between blended with
    s = (original / l - low) / (high - low): (1 - s) f / factor + s f."""
    dims = rot["dims"]
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(rot["base"]), dtype=torch.float64), -2.0 * i / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for fi in f.tolist():
            l = 2.0 * math.pi / fi
            if l < orig / high:
                out.append(fi)
            elif l > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / l - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=torch.float64)
    return f


def rotate(x: torch.Tensor, f: torch.Tensor, pairing: str, first_position: int = 0,
           angle_dtype: torch.dtype = torch.float64) -> torch.Tensor:
    """x [T, heads, d]: the first 2 * len(f) coordinates of every head are rotated, the others pass.  Frequency i
    turns coordinates (i, i + len(f)) (``half``) or (2i, 2i + 1) (``interleaved``): the pair (u, v) of the token at
    position p becomes (u cos a - v sin a, v cos a + u sin a), a = p f_i.  ``angle_dtype`` float32 rounds the
    frequency and the product to 32 bits, as a 32-bit implementation does."""
    T, half = x.shape[0], f.shape[0]
    a = ((first_position + torch.arange(T, dtype=torch.float64)).to(angle_dtype)[:, None]
         * f.to(angle_dtype)[None, :]).double()
    cos, sin = torch.cos(a).to(x.dtype)[:, None, :], torch.sin(a).to(x.dtype)[:, None, :]
    out = x.clone()
    if pairing == "half":
        u, v = x[..., :half], x[..., half:2 * half]
        out[..., :half] = u * cos - v * sin
        out[..., half:2 * half] = v * cos + u * sin
    else:
        u, v = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
        out[..., 0:2 * half:2] = u * cos - v * sin
        out[..., 1:2 * half:2] = v * cos + u * sin
    return out


def causal_mask(T: int) -> torch.Tensor:
    return torch.arange(T)[None, :] <= torch.arange(T)[:, None]


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask: torch.Tensor,
                      sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, d], k [T, H, d], v [T, H, dv] (keys and values already spread over the query heads).
    p_ij = exp(s_ij) / (sum over visible j of exp(s_ij) + exp(sink_h)), s = scale q.k; the sink term (one learned
    number a head, not scaled, no value) is absent when ``sink`` is None."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.to(s.dtype)[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.to(s.dtype)[:, None, None] - m)
    return torch.einsum("hij,jhd->ihd", e / den, v)


# ------------------------------------------------------------------------------------------------ the mixers
def attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Grouped-query attention whose values are the keys as projected (before rotation and norm)."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, G, d)
    v = k
    rot = m.get("rot")
    if rot:
        f = frequencies(rot)
        q, k = rotate(q, f, "half"), rotate(k, f, "half")
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    rep = H // G
    o = softmax_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1), m["scale"], causal_mask(T),
                          w[p + "sink"])
    return o.reshape(T, H * d) @ w[p + "o"].T


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Keys and values expanded from a normed latent; here they are really formed, head by head."""
    T = h.shape[0]
    H, d, r, dv, c = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, d + r)
    down = h @ w[p + "dkv"].T
    lat = rms_norm(down[:, :c], w[p + "dkv.norm"], eps)
    f = frequencies(m["rot"])
    k_rot = rotate(down[:, None, c:], f, "interleaved")                       # [T, 1, r]
    q_rot = rotate(q[..., d:], f, "interleaved")
    k_plain = (lat @ w[p + "uk"].T).reshape(T, H, d)
    v = (lat @ w[p + "uv"].T).reshape(T, H, dv)
    qq = torch.cat([q[..., :d], q_rot], -1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, r)], -1)
    o = softmax_attention(qq, kk, v, m["scale"], causal_mask(T))
    o = o * sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------------------------------------------ feed-forward
def expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(z: torch.Tensor, correction: torch.Tensor, top: int, groups: int, keep: int, scale: float):
    """z [T, E] router logits -> (chosen experts [T, top], their weights).  s = sigmoid(z); the choice looks at
    s + correction: a group's score is the sum of its two largest members (its only member's score if it has one),
    only the ``keep`` best groups stay open, the ``top`` largest open members are chosen; the weights are s (without
    the correction) times ``scale``."""
    T, E = z.shape
    s = sigmoid(z)
    c = s + correction
    per = E // groups
    grouped = c.reshape(T, groups, per)
    score = grouped.topk(min(2, per), -1).values.sum(-1)
    best = score.topk(keep, -1).indices
    allowed = torch.zeros(T, groups, dtype=torch.bool).scatter_(1, best, True).repeat_interleave(per, 1)
    chosen = c.masked_fill(~allowed, float("-inf")).topk(top, -1).indices
    return chosen, s.gather(1, chosen) * scale


def route_margin(z: torch.Tensor, correction: torch.Tensor, top: int, groups: int, keep: int) -> torch.Tensor:
    """How far every token's choice is from another one, in choice scores [T]: the gap between the last group kept and
    the first one left out, and between the last member chosen and the first one left out among the open groups."""
    T, E = z.shape
    c = sigmoid(z) + correction
    per = E // groups
    score = c.reshape(T, groups, per).topk(min(2, per), -1).values.sum(-1)
    ranked = score.sort(-1, descending=True).values
    gap = torch.full((T,), float("inf"), dtype=z.dtype)
    if keep < groups:
        gap = torch.minimum(gap, ranked[:, keep - 1] - ranked[:, keep])
    best = score.topk(keep, -1).indices
    allowed = torch.zeros(T, groups, dtype=torch.bool).scatter_(1, best, True).repeat_interleave(per, 1)
    members = c.masked_fill(~allowed, float("-inf")).sort(-1, descending=True).values
    if top < keep * per:
        gap = torch.minimum(gap, members[:, top - 1] - members[:, top])
    return gap


def experts_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict,
               margins: Optional[list] = None) -> torch.Tensor:
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    z = h @ w[p + "router"].T
    if margins is not None:
        margins.append(route_margin(z, w[p + "correction"], r["top"], groups["count"], groups["keep"]))
    chosen, weight = route(z, w[p + "correction"], r["top"], groups["count"], groups["keep"], r["scale"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            out[t] += g * expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + expert(h, w, p + "shared.") * sigmoid(h @ w[p + "shared.sg"].T)
    return out


# ------------------------------------------------------------------------------------------------ the model
def forward(config: dict, weights: Dict[str, torch.Tensor], ids: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None, margins_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: a list that receives x after every layer;
    ``margins_out``: one that receives every router's ``route_margin`` [T]."""
    w = {n: (t if not t.is_floating_point() else t.to(dtype)) for n, t in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(ids)] * config["embedding"]["scale"]
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        mixer = attention if layer["type"] == "attention" else latent_attention
        x = x + rms_norm(mixer(x, w, p + "mix.", m, eps), w[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp:
            x = x + rms_norm(experts_ff(x, w, p + "mlp.", mlp, margins_out), w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T * config["logit_scale"]
