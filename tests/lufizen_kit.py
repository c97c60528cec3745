"""Small Lufizen configurations, random weights for them and helpers that run them through the engine.

The configurations differ from one another in every size and option: head counts and groups of query heads, head
sizes of every kernel family, rotations over a part of a head, over all of it or none, with and without stretched
frequencies, latent layers with narrow and wide latents and values wider and narrower than keys, the two kinds of
layer in several orders, routed experts with and without groups (also groups of one member), one to all experts a
token, with and without a shared expert, layers without a feed-forward, embedding and logit factors other than 1.
Weights are drawn with torch's generator and are representable in bfloat16, so that the float32 engine, the bfloat16
engine and the plain implementation read the same numbers.
"""
from __future__ import annotations

from typing import Dict, Sequence

import numpy as np
import torch

import plain_lufizen as P
from kefetar_kit import bf16_values, check, make_engine, run_alone, tokens  # noqa: F401  (shared helpers)
from mukenex_kit import write_model  # noqa: F401


def attention(heads, kv_heads, dim, scale, rot=None, mlp=None):
    """rot: (base, dims) or (base, dims, (factor, low, high, original)) or None."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if len(rot) > 2 and rot[2] is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), rot[2]))
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": scale, "rot": {"base": base, "dims": rot_dim}}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def moe(ff, experts, top, scale, groups=None, shared=None):
    """groups: (count, keep) or None; shared: ff or None."""
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def config(vocab, width, eps, layers, embedding_scale=1.5, logit_scale=1.0):
    return {"architecture": "Lufizen", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embedding_scale}, "logit_scale": logit_scale, "layers": layers}


STRETCH = (8.0, 1.0, 4.0, 64)      # wavelengths of 16 to 64 positions are blended, longer ones stretched eightfold

CONFIGS = {
    # two KV heads, a rotation over a part of a head with stretched frequencies, a latent layer between two attention
    # layers, groups of experts ranked by two members, a shared expert, a layer without feed-forward
    "L1": config(97, 40, 1e-5, [
        attention(4, 2, 12, 0.3, (300.0, 8, STRETCH), mlp=moe(20, 8, 3, 2.0, (4, 2), 28)),
        latent(3, 10, 4, 14, 24, 18, 0.25, 1000.0, mlp=moe(16, 5, 2, 0.7)),
        attention(2, 2, 10, 0.4),
        attention(6, 2, 12, 0.25, (10000.0, 12), mlp=moe(12, 6, 2, 1.0, (3, 2))),
    ], embedding_scale=2.0, logit_scale=0.5),
    # head sizes of the tensor-core kernels, four query heads a KV head, every expert for every token, latent layers
    # first and last, values narrower than keys, groups of one member
    "L2": config(211, 64, 1e-6, [
        latent(4, 16, 16, 8, 48, 32, 0.18, 500.0, mlp=moe(24, 3, 3, 1.5, None, 40)),
        attention(8, 2, 32, 0.18, (500.0, 32), mlp=moe(32, 4, 2, 2.25, (4, 3), 16)),
        attention(4, 4, 16, 0.3, (77.0, 2, (2.0, 1.0, 3.0, 32))),
        latent(2, 32, 8, 48, 56, 80, 0.2, 40000.0, mlp=moe(24, 6, 4, 1.0, (2, 2))),
    ], embedding_scale=1.0, logit_scale=2.0),
    # heads of 64 and wider than 128, one KV head, a latent wider than 128
    "L3": config(73, 72, 3e-6, [
        attention(2, 1, 64, 0.12, (1e6, 64), mlp=moe(40, 4, 2, 2.0, (2, 1), 16)),
        latent(3, 24, 16, 40, 160, 24, 0.15, 100.0),
        attention(3, 1, 160, 0.08, (100.0, 30, STRETCH), mlp=moe(16, 9, 3, 3.0, (3, 2))),
    ], embedding_scale=0.7, logit_scale=0.25),
}

# One layer alone, with scores so sharp that a single key (or the sink) decides a position's result.
ONLY_ATTENTION = config(89, 48, 1e-5, [attention(6, 3, 16, 0.9, (200000.0, 10, (4.0, 1.0, 4.0, 256)))])
ONLY_LATENT = config(89, 36, 1e-5, [latent(4, 12, 8, 10, 40, 28, 1.6, 5000.0)])
# One expert a token: a near tie between the two best experts would show in full, so this one is compared in float32.
ONE_EXPERT = config(61, 32, 1e-5, [attention(2, 1, 8, 0.3, (100.0, 4), mlp=moe(12, 6, 1, 2.0, (3, 1), 10))])


def random_weights(raw: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors by name, float32 with bfloat16-representable values."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, std=1.0, mean=0.0):
        return bf16_values(mean + std * torch.randn(tuple(shape), generator=g))

    w, width = {}, raw["width"]
    w["embed"] = normal(raw["vocab"], width)
    w["head"] = normal(raw["vocab"], width, std=width ** -0.5)
    w["final.norm"] = normal(width, std=0.2, mean=1.0)
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        w[p + "norm1"] = normal(width, std=0.3, mean=1.0)
        if layer["type"] == "attention":
            w[p + "mix.q"] = normal(H * d, width, std=width ** -0.5)
            w[p + "mix.k"] = normal(m["kv_heads"] * d, width, std=width ** -0.5)
            # sinks of the size of a position's best scores (d * scale at most): they take a share nearly everywhere
            w[p + "mix.sink"] = normal(H, std=1.5, mean=0.6 * d * m["scale"])
        else:
            r, c, qr = m["rot_dim"], m["kv_rank"], m["q_rank"]
            w[p + "mix.dq"] = normal(qr, width, std=width ** -0.5)
            w[p + "mix.dq.norm"] = normal(qr, std=0.3, mean=1.0)
            w[p + "mix.uq"] = normal(H * (d + r), qr, std=qr ** -0.5)
            w[p + "mix.dkv"] = normal(c + r, width, std=0.5 * width ** -0.5)
            w[p + "mix.dkv.norm"] = normal(c, std=0.3, mean=1.0)
            w[p + "mix.uk"] = normal(H * d, c, std=c ** -0.5)
            w[p + "mix.uv"] = normal(H * dv, c, std=c ** -0.5)
            w[p + "mix.g"] = normal(H, width, std=width ** -0.5)
        w[p + "mix.o"] = normal(width, H * dv, std=(H * dv) ** -0.5)
        mlp = layer.get("mlp")
        if mlp:
            w[p + "norm2"] = normal(width, std=0.3, mean=1.0)
            ff, experts = mlp["expert"]["ff"], mlp["router"]["experts"]
            # scores that lie apart (the stream has a root mean square of a few units) and corrections that reorder them
            w[p + "mlp.router"] = normal(experts, width, std=0.5 * width ** -0.5)
            w[p + "mlp.correction"] = normal(experts, std=0.3)
            names = [f"e{e}" for e in range(experts)] + (["shared"] if mlp.get("shared") else [])
            for e in names:
                f = mlp["shared"]["ff"] if e == "shared" else ff
                w[f"{p}mlp.{e}.gate"] = normal(f, width, std=width ** -0.5)
                w[f"{p}mlp.{e}.up"] = normal(f, width, std=width ** -0.5)
                w[f"{p}mlp.{e}.down"] = normal(width, f, std=f ** -0.5)
            if mlp.get("shared"):
                w[p + "mlp.shared.sg"] = normal(1, width, std=width ** -0.5)
    return w


def oracle(raw: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int]) -> np.ndarray:
    """The plain implementation's logits in float64, [T, vocab]."""
    return P.forward(raw, weights, list(ids), dtype=torch.float64).numpy()


CLOSE_CALL = 0.02        # in scores (sigmoids); a bfloat16 engine's router logits differ from the plain ones by hundredths


def oracle_and_close_calls(raw: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int]):
    """The plain logits [T, vocab] and, per position, whether one of its routers chose within ``CLOSE_CALL`` of
    another choice: there a bfloat16 engine may take the other expert, and the difference is no rounding matter."""
    margins = []
    logits = P.forward(raw, weights, list(ids), dtype=torch.float64, margins_out=margins).numpy()
    close = np.zeros(len(ids), dtype=bool)
    for m in margins:
        close |= (m < CLOSE_CALL).numpy()
    return logits, close


TOL = {"float32": 3e-5, "bfloat16": 4e-2}
# The one-layer models have scores of tens: q and k rounded to bfloat16 (2^-9 each) move such a score by a tenth, and
# so a key's weight by a tenth.  Their bfloat16 bound is that share of the logits' scale; their float32 bound is the
# common one, and that is the run which shows a wrong key.
SHARP_BF16_TOL = 0.15


def tolerance(name: str, dtype: str) -> float:
    return SHARP_BF16_TOL if (name in ("attention", "latent") and dtype == "bfloat16") else TOL[dtype]


def check_clear(got: np.ndarray, want: np.ndarray, close: np.ndarray, dtype: str, what: str, tol: float = None) -> None:
    """``check`` on every position in float32.  In bfloat16, on the positions whose routers made no close call (which
    are most: the rest must not be many), and one position in twenty (or one) may lie beyond the bound, though not
    beyond five times it: a norm on a sublayer's output magnifies the rounding of an output whose terms cancel (these
    models are a few dozen columns wide, so one rounded term weighs much), and the float32 run, which allows no
    exception, is the one that shows a wrong mechanism."""
    tol = TOL[dtype] if tol is None else tol
    if dtype == "bfloat16":
        assert close.mean() < 0.4, f"{what}: too many close calls for the test to mean much"
        got, want = got[~close], want[~close]
        bound = tol * max(1.0, float(np.abs(want).max()))
        err = np.abs(got.astype(np.float64) - want).max(axis=1)
        beyond = np.nonzero(err > bound)[0]
        if 0 < beyond.size <= max(1, len(err) // 20) and err.max() <= 5.0 * bound:
            keep = np.ones(len(err), dtype=bool)
            keep[beyond] = False
            got, want = got[keep], want[keep]
    check(got, want, dtype, what, tol)


def clear_weights(raw: dict, seed: int, ids: Sequence[int], tries: int = 16) -> Dict[str, torch.Tensor]:
    """Of ``tries`` random weight sets, the one whose routers are farthest from a close call on ``ids``: a bfloat16
    engine may then round as it likes without choosing another group or expert than the plain implementation."""
    best, best_gap = None, -1.0
    for k in range(tries):
        w = random_weights(raw, seed + 1000 * k)
        margins = []
        P.forward(raw, w, list(ids), dtype=torch.float64, margins_out=margins)
        gap = min(float(m.min()) for m in margins) if margins else float("inf")
        if gap > best_gap:
            best, best_gap = w, gap
        if gap > 0.05:
            break
    return best


def standout_case(kind: str, raw: dict, weights: Dict[str, torch.Tensor], far: int, T: int, seed: int):
    """Token ids and weights of a one-layer model in which the key at position ``far`` fits the queries of a marked
    token that comes again right behind it, a page later and hundreds of positions later, so that one far key among
    hundreds carries those positions' results.  Returns (ids, weights, the marked positions).

    attention: q and k are normed, so nothing stands out by its size; instead W_q is made W_k with the width's
    coordinates permuted, and the marked token's embedding is the far token's with the inverse permutation: the marked
    token's query IS the far token's key (up to the rotation by their distance), while its own key and value are
    unrelated to the far token's.  latent: the rotated key part is the one part of a latent key that is not normed;
    all but its slowest pair are made small, the far token's embedding row is scaled up, and the rotated query rows of
    every head are made rank one, so that the marked token's rotated query is a multiple of the far token's rotated
    key part."""
    g = torch.Generator().manual_seed(seed)
    vocab, width = raw["vocab"], raw["width"]
    far_token, marked = vocab - 1, vocab - 2
    ids = torch.randint(0, vocab - 2, (T,), generator=g).tolist()
    places = [p for p in (far + 1, far + 2, far + 16, far + 17, T // 2, T - 34, T - 2, T - 1) if far < p < T]
    ids[far] = far_token
    for p in places:
        ids[p] = marked
    w = dict(weights)
    w["embed"] = weights["embed"].clone()
    if kind == "attention":
        m = raw["layers"][0]["mixer"]
        perm = torch.randperm(width, generator=g)
        rep = m["heads"] // m["kv_heads"]
        k = weights["l0.mix.k"].reshape(m["kv_heads"], m["dim"], width)
        w["l0.mix.q"] = k.repeat_interleave(rep, 0)[:, :, perm].reshape(m["heads"] * m["dim"], width).contiguous()
        # q(marked) = W_q e_marked = W_k[:, perm] e_marked = W_k e_far  when  e_far[perm] = e_marked
        w["embed"][marked] = w["embed"][far_token][perm]
    else:
        m = raw["layers"][0]["mixer"]
        H, d, r, c = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
        eps, scale = raw["norm"]["eps"], raw["embedding"]["scale"]
        w["embed"][far_token] = bf16_values(weights["embed"][far_token] * 12.0)
        dkv = weights["l0.mix.dkv"].clone()
        dkv[c:c + r - 2] *= 0.05
        w["l0.mix.dkv"] = bf16_values(dkv)
        k_far = (w["l0.mix.dkv"][c:].double() @ (w["embed"][far_token].double() * scale))
        cq = P.rms_norm((weights["l0.mix.dq"].double() @ (w["embed"][marked].double() * scale))[None],
                        weights["l0.mix.dq.norm"].double(), eps)[0]
        gain = 12.0 / (m["scale"] * float(k_far @ k_far))              # the marked token's score for the far key: 12
        uq = weights["l0.mix.uq"].clone().reshape(H, d + r, -1)
        uq[:, d:] = (gain * k_far[:, None] * cq[None, :] / float(cq @ cq)).float()
        w["l0.mix.uq"] = bf16_values(uq.reshape(H * (d + r), -1))
        w["l0.mix.uk"] = bf16_values(weights["l0.mix.uk"] * 0.25)       # the unrotated scores: a few units, not tens
    return ids, w, places
