"""Small Torinex configurations, random weights for them and helpers that run them through the engine.

The configurations differ from one another in every size and option: head counts and groups, key and value widths,
rotations over a part of a head, over all of it or none, blocks of positions of many sizes (also the page's size, one
position, or none), layers that read an earlier layer's keys and values in several orders, dense, routed (with and
without groups, with and without a shared expert, one to all experts a token) and absent feed-forwards, with and
without the per-layer token input.  Weights are drawn with torch's generator and are representable in bfloat16, so
that the float32 engine, the bfloat16 engine and the plain implementation read the same numbers.
"""
from __future__ import annotations

from typing import Dict, Sequence

import numpy as np
import torch

import plain_torinex as P
from kefetar_kit import bf16_values, check, make_engine, run_alone, tokens  # noqa: F401  (shared helpers)
from mukenex_kit import write_model  # noqa: F401


def attention(heads, kv_heads, dim, vdim, scale, block=None, rot=None, kv_from=None, mlp=None):
    """rot: (base, dims) or None."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if block is not None:
        m["mask"] = {"size": block}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, top, groups=None, shared=None):
    """groups: (count, keep) or None; shared: (ff, limit) or None."""
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def config(vocab, width, eps, layers, side=None):
    raw = {"architecture": "Torinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if side is not None:
        raw["token_side"] = {"dim": side}
    return raw


CONFIGS = {
    # two KV heads, values narrower than keys, a rotation over a part of a head, blocks that are no multiple of a
    # page, groups of experts, a shared expert, layers that read the first and the third layer's keys, a layer
    # without mask, rotation or feed-forward, a layer with one expert a token out of ungrouped experts
    "T1": config(97, 40, 1e-5, [
        attention(4, 2, 12, 8, 0.3, 24, (10000.0, 8), mlp=moe(20, 1.5, 8, 3, (4, 2), (28, 2.5))),
        attention(4, 2, 12, 8, 0.25, 24, (10000.0, 8), kv_from=0, mlp=dense(56)),
        attention(2, 2, 10, 14, 0.4),
        attention(2, 2, 10, 14, 0.35, 30, kv_from=2, mlp=moe(16, 3.0, 5, 2)),
    ], side=6),
    # head sizes of the tensor-core kernels, four query heads a KV head, every expert for every token, no token
    # input, blocks one position longer than two pages, three layers on one layer's keys
    "T2": config(211, 64, 1e-6, [
        attention(8, 2, 32, 32, 0.18, 33, (500.0, 32), mlp=dense(96)),
        attention(8, 2, 32, 32, 0.2, 33, (500.0, 32), kv_from=0, mlp=moe(24, 2.0, 3, 3, None, (40, 1.0))),
        attention(4, 4, 16, 16, 0.3, 16, (77.0, 2), mlp=moe(32, 4.0, 6, 2, (2, 1))),
        attention(4, 4, 16, 16, 0.3, 16, (77.0, 2), kv_from=2),
        attention(4, 4, 16, 16, 0.22, 16, (77.0, 2), kv_from=2, mlp=dense(24)),
    ]),
    # heads of 64 and wider than 128, a token input one column wide, blocks of one page, as many groups as experts
    "T3": config(73, 72, 3e-6, [
        attention(2, 1, 64, 64, 0.12, 8, (1e6, 64), mlp=moe(40, 2.0, 4, 2, (4, 3), (16, 2.0))),
        attention(3, 1, 160, 136, 0.08, 50, (100.0, 30), mlp=dense(48)),
        attention(3, 1, 160, 136, 0.07, 50, (100.0, 30), kv_from=1, mlp=dense(40)),
    ], side=1),
}

# One layer alone, with scores so sharp that a single key (or the sink) decides a position's result.
ONLY_BLOCKS = config(89, 36, 1e-5, [attention(4, 2, 12, 14, 3.0, 48, (10000.0, 12))])
ONLY_FAR = config(89, 48, 1e-5, [attention(6, 3, 16, 16, 2.5, 470, (200000.0, 10)),
                                 attention(6, 3, 16, 16, 2.5, 470, (200000.0, 10), kv_from=0)])
# One expert a token: a near tie between the two best experts would show in full, so this one is compared in float32.
ONE_EXPERT = config(61, 32, 1e-5, [attention(2, 1, 8, 8, 0.3, 20, (100.0, 4), mlp=moe(12, 1.0, 6, 1, (3, 1)))], side=3)


def random_weights(raw: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Checkpoint tensors by name, float32 with bfloat16-representable values."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, std=1.0, mean=0.0):
        return bf16_values(mean + std * torch.randn(tuple(shape), generator=g))

    w, width = {}, raw["width"]
    w["embed"] = normal(raw["vocab"], width)
    w["final.norm"] = normal(width, std=0.2, mean=1.0)
    side = (raw.get("token_side") or {}).get("dim", 0)
    if side:
        w["side.embed"] = normal(raw["vocab"], side * len(raw["layers"]))
    wide = 2.0 * width ** -0.5
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        w[p + "norm1"] = normal(width, std=0.3, mean=1.0)
        rows = [("q", H * d)] + ([("k", G * d), ("v", G * dv)] if m.get("kv_from") is None else [])
        for name, n in rows:
            w[p + "mix." + name] = normal(n, width, std=wide if name != "v" else width ** -0.5)
            w[p + "mix." + name + ".b"] = normal(n, std=0.5)
            if name != "v":
                w[p + "mix." + name + ".norm"] = normal(n, std=0.3, mean=1.0)
        w[p + "mix.o"] = normal(width, H * dv, std=(H * dv) ** -0.5)
        w[p + "mix.o.b"] = normal(width, std=0.3)
        mlp = layer.get("mlp")
        if mlp:
            w[p + "norm2"] = normal(width, std=0.3, mean=1.0)
            if mlp["kind"] == "dense":
                w[p + "mlp.up"] = normal(mlp["ff"], width, std=width ** -0.5)
                w[p + "mlp.down"] = normal(width, mlp["ff"], std=mlp["ff"] ** -0.5)
            else:
                ff = mlp["expert"]["ff"]
                # a router whose logits lie far apart: ties between experts are rare and the lesser experts count little
                w[p + "mlp.router"] = normal(mlp["router"]["experts"], width, std=3.0 * width ** -0.5)
                names = [f"e{e}" for e in range(mlp["router"]["experts"])] + (["shared"] if mlp.get("shared") else [])
                for e in names:
                    f = mlp["shared"]["ff"] if e == "shared" else ff
                    w[f"{p}mlp.{e}.gate"] = normal(f, width, std=1.5 * width ** -0.5)      # some gates beyond the limit
                    w[f"{p}mlp.{e}.up"] = normal(f, width, std=1.5 * width ** -0.5)
                    w[f"{p}mlp.{e}.down"] = normal(width, f, std=f ** -0.5)
        if side:
            w[p + "side.gate"] = normal(side, width, std=width ** -0.5)
            w[p + "side.proj"] = normal(width, side, std=1.0)
            w[p + "side.norm"] = normal(width, std=0.3, mean=0.7)
    return w


def oracle(raw: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int]) -> np.ndarray:
    """The plain implementation's logits in float64, [T, vocab]."""
    return P.forward(raw, weights, list(ids), dtype=torch.float64).numpy()


CLOSE_CALL = 0.08        # logits; a bfloat16 engine's logits differ from the plain ones by a few hundredths


def oracle_and_close_calls(raw: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int]):
    """The plain logits [T, vocab] and, per position, whether one of its routers chose within ``CLOSE_CALL`` of
    another choice: there a bfloat16 engine may take the other expert, and the difference is no rounding matter."""
    margins = []
    logits = P.forward(raw, weights, list(ids), dtype=torch.float64, margins_out=margins).numpy()
    close = np.zeros(len(ids), dtype=bool)
    for m in margins:
        close |= (m < CLOSE_CALL).numpy()
    return logits, close


def check_clear(got: np.ndarray, want: np.ndarray, close: np.ndarray, dtype: str, what: str, tol: float = None) -> None:
    """``check`` on every position in float32.  In bfloat16, on the positions whose routers made no close call (which
    are most: the rest must not be many), and one position in fifty (or one) may lie beyond the bound, though not
    beyond four times it: a norm on a sublayer's output magnifies the rounding of an output whose terms cancel, and
    the float32 run, which allows no exception, is the one that shows a wrong mechanism."""
    tol = TOL[dtype] if tol is None else tol
    if dtype == "bfloat16":
        assert close.mean() < 0.25, f"{what}: too many close calls for the test to mean much"
        got, want = got[~close], want[~close]
        bound = tol * max(1.0, float(np.abs(want).max()))
        err = np.abs(got.astype(np.float64) - want).max(axis=1)
        beyond = np.nonzero(err > bound)[0]
        if 0 < beyond.size <= max(1, len(err) // 50) and err.max() <= 4.0 * bound:
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
        if gap > 0.5:
            break
    return best


TOL = {"float32": 3e-5, "bfloat16": 4e-2}
# The one-layer models have scores of tens: q and k rounded to bfloat16 (2^-9 each) move such a score by a tenth, and
# so a key's weight by a tenth.  Their bfloat16 bound is that share of the logits' scale; their float32 bound is the
# common one, and that is the run which shows a wrong key.
SHARP_BF16_TOL = 0.15


def tolerance(name: str, dtype: str) -> float:
    return SHARP_BF16_TOL if (name in ("blocks", "far") and dtype == "bfloat16") else TOL[dtype]
