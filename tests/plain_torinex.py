"""A plain, slow Torinex: whole sequences on the CPU, one function per mechanism.

Written from the design's equations and nothing else; it shares no code with the package.  Everything is torch on
the CPU in ``dtype`` (float64 by default).  ``weights`` maps checkpoint tensor names to tensors, ``config`` is the
dict of a config.json.

    x = embed[token]
    per layer i:   x <- x + N(mixer(x); norm1);   x <- x + N(ff(x); norm2)  (if the layer has a feed-forward)
                   x <- x + N(side.proj (gelu_tanh(side.gate x) * side.embed[token][i]); side.norm)   (if token_side)
    logits = embed . N(x; final.norm)
    N(y; w) = y / sqrt(mean(y^2) + eps) * w           (the norm sits on a sublayer's OUTPUT; sublayers read x itself)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------------------------ small pieces
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) ** 2


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def rotate_pairs(x: torch.Tensor, base: float, dims: int, first_position: int = 0,
                 angle_dtype: torch.dtype = torch.float64) -> torch.Tensor:
    """x [T, heads, d]: of every head's first ``dims`` coordinates, coordinate 2i is paired with 2i + 1 and the pair
    (u, v) of the token at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i / dims); the
    other coordinates pass.  ``angle_dtype`` float32 rounds the frequency and the product p * f to 32 bits as a
    32-bit implementation does (at position 3000 that moves an angle by 1e-4); cos and sin are exact after that."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims).to(angle_dtype)
    a = ((first_position + torch.arange(T, dtype=torch.float64)).to(angle_dtype)[:, None] * f[None, :]).double()
    cos, sin = torch.cos(a).to(x.dtype)[:, None, :], torch.sin(a).to(x.dtype)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def causal_mask(T: int) -> torch.Tensor:
    return torch.arange(T)[None, :] <= torch.arange(T)[:, None]


def chunk_mask(T: int, size: int) -> torch.Tensor:
    """[T, T] True where query i reads key j: j <= i and both lie in the same block of ``size`` positions counted
    from position 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def sink_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                           mask: torch.Tensor) -> torch.Tensor:
    """q [T, H, d], k [T, H, d], v [T, H, dv] (keys and values already spread over the query heads).
    p_ij = exp(s_ij) / (1 + sum over visible j of exp(s_ij)), s = scale q.k: a sink of score 0 without a value."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True) + torch.exp(-m)
    return torch.einsum("hij,jhd->ihd", e / den, v)


# ------------------------------------------------------------------------------------------------ the mixer
def attention_keys_values(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """Keys (normed over the whole projection, rotated) and values of a layer that has projections of its own:
    k [T, G, d], v [T, G, dv]."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = rms_norm(h @ w[p + "k"].T + w[p + "k.b"], w[p + "k.norm"], eps).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        k = rotate_pairs(k, rot["base"], rot["dims"])
    return k, v


def attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, k: torch.Tensor,
              v: torch.Tensor) -> torch.Tensor:
    """Grouped-query attention with biased projections, one RMS norm over ALL of q's rows at once (before the split
    into heads), a rotation of each head's first coordinates, blocks of positions, the sink in the denominator."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ w[p + "q"].T + w[p + "q.b"], w[p + "q.norm"], eps).reshape(T, H, d)
    rot = m.get("rot")
    if rot:
        q = rotate_pairs(q, rot["base"], rot["dims"])
    rep = H // G
    mask = chunk_mask(T, m["mask"]["size"]) if m.get("mask") else causal_mask(T)
    o = sink_softmax_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1), m["scale"], mask)
    return o.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


# ------------------------------------------------------------------------------------------------ feed-forward
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return relu_squared(h @ w[p + "up"].T) @ w[p + "down"].T


def clamped_expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    """g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(z: torch.Tensor, top: int, groups: int, keep: int):
    """z [T, E] router logits -> (chosen experts [T, top], their weights).  Scores are the softmax over all experts;
    experts form ``groups`` equal groups of neighbours, a group's score is its largest score, only experts of the
    ``keep`` best groups can be chosen; the ``top`` largest of those are taken with their scores as weights."""
    T, E = z.shape
    s = torch.softmax(z, -1)
    per = E // groups
    best = s.reshape(T, groups, per).max(-1).values.topk(keep, -1).indices
    allowed = torch.zeros(T, groups, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    masked = s.masked_fill(~allowed.repeat_interleave(per, 1), -1.0)
    chosen = masked.topk(top, -1).indices
    return chosen, s.gather(1, chosen)


def route_margin(z: torch.Tensor, top: int, groups: int, keep: int) -> torch.Tensor:
    """How far every token's choice is from another one, in logits [T]: the gap between the last group kept and the
    first one left out (by their largest logits), and between the last expert chosen and the first one left out among
    the experts of the kept groups.  A choice within rounding of another is a close call."""
    T, E = z.shape
    per = E // groups
    best = z.reshape(T, groups, per).max(-1).values.sort(-1, descending=True).values
    gap = torch.full((T,), float("inf"), dtype=z.dtype)
    if keep < groups:
        gap = torch.minimum(gap, best[:, keep - 1] - best[:, keep])
    chosen_groups = z.reshape(T, groups, per).max(-1).values.topk(keep, -1).indices
    allowed = torch.zeros(T, groups, dtype=torch.bool).scatter_(1, chosen_groups, True).repeat_interleave(per, 1)
    ranked = z.masked_fill(~allowed, float("-inf")).sort(-1, descending=True).values
    if top < keep * per:
        gap = torch.minimum(gap, ranked[:, top - 1] - ranked[:, top])
    return gap


def experts_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict,
               margins: Optional[list] = None) -> torch.Tensor:
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    if margins is not None:
        margins.append(route_margin(h @ w[p + "router"].T, r["top"], groups["count"], groups["keep"]))
    chosen, weight = route(h @ w[p + "router"].T, r["top"], groups["count"], groups["keep"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            out[t] += g * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def token_side(x: torch.Tensor, ids: List[int], w: Dict[str, torch.Tensor], p: str, layer: int, dim: int,
               eps: float) -> torch.Tensor:
    """What a layer adds from the per-layer token table: N(side.proj (gelu_tanh(side.gate x) * e); side.norm)."""
    e = w["side.embed"][torch.tensor(ids)][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + "side.gate"].T) * e) @ w[p + "side.proj"].T
    return rms_norm(y, w[p + "side.norm"], eps)


# ------------------------------------------------------------------------------------------------ the model
def forward(config: dict, weights: Dict[str, torch.Tensor], ids: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None, margins_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: a list that receives x after every layer;
    ``margins_out``: one that receives every router's ``route_margin`` [T]."""
    w = {n: (t if not t.is_floating_point() else t.to(dtype)) for n, t in weights.items()}
    eps = config["norm"]["eps"]
    side = config.get("token_side")
    x = w["embed"][torch.tensor(ids)]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if m.get("kv_from") is None:
            kept[i] = attention_keys_values(x, w, p + "mix.", m, eps)
        k, v = kept[i if m.get("kv_from") is None else m["kv_from"]]
        x = x + rms_norm(attention(x, w, p + "mix.", m, eps, k, v), w[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp:
            y = dense_ff(x, w, p + "mlp.") if mlp["kind"] == "dense" else experts_ff(x, w, p + "mlp.", mlp, margins_out)
            x = x + rms_norm(y, w[p + "norm2"], eps)
        if side:
            x = x + token_side(x, ids, w, p, i, side["dim"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T
