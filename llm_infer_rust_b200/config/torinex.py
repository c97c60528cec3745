"""Typed configuration of Torinex, read from its own config.json keys.

    architecture    "Torinex"
    vocab, width    sizes of the embedding table (which is also the output head) and of the residual
    norm.eps        eps of every RMS norm of the model (inside the root)
    token_side      {dim}: every layer adds a gated read of its own ``dim`` columns of a second token table
                    (absent: no such input)
    layers[i]       type ("attention"), mixer (sizes and constants, below), mlp: null,
                    {"kind": "dense", "ff": F} or {"kind": "moe", "expert": {"ff", "limit"},
                    "router": {"experts", "top", "groups": {"count", "keep"}}, "shared": {"ff", "limit"}}
                    (``groups`` absent: one group; ``shared`` absent: no shared expert)

    attention       heads, kv_heads, dim, vdim, scale, rot {base, dims} (absent: no rotation), mask {size} (blocks of
                    that many positions; absent: every earlier key), kv_from: j (absent: keys and values of its own)

Nothing here is a default for a size: a key that the design needs and the file lacks is an error.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .kefetar import MAX_POSITIONS, _int, _number
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry


@dataclass(frozen=True)
class TorinexExpert:
    ff: int
    limit: float


@dataclass(frozen=True)
class TorinexFF:
    kind: str                  # "dense" | "moe"
    ff: int = 0                # dense
    expert: Optional[TorinexExpert] = None
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    shared: Optional[TorinexExpert] = None


@dataclass(frozen=True)
class TorinexLayer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    ff: Optional[TorinexFF]
    chunk: Optional[int] = None        # blocks of positions; None: every earlier key
    rot_base: float = 0.0
    rot_dims: int = 0                  # 0: no rotation
    kv_from: Optional[int] = None      # the layer whose keys and values this one reads


@dataclass(frozen=True)
class TorinexConfig:
    vocab: int
    width: int
    eps: float
    side_dim: int                      # 0: no per-layer token input
    layers: Tuple[TorinexLayer, ...]

    architecture = "Torinex"
    model_type = None

    @staticmethod
    def _expert(raw: Any, where: str) -> TorinexExpert:
        if not isinstance(raw, dict):
            raise ConfigError(f"{where[:-1]} must be an object with ff and limit")
        return TorinexExpert(_int(raw, "ff", where), _number(raw, "limit", where))

    @staticmethod
    def _feed_forward(mlp: Any, where: str) -> Optional[TorinexFF]:
        if mlp is None:
            return None
        if not isinstance(mlp, dict):
            raise ConfigError(f"invalid {where}mlp: an object or null is required")
        kind = mlp.get("kind")
        if kind == "dense":
            return TorinexFF("dense", ff=_int(mlp, "ff", where + "mlp."))
        if kind == "moe":
            router = mlp.get("router")
            if not isinstance(router, dict):
                raise ConfigError(f"{where}mlp needs a router object")
            r = where + "mlp.router."
            experts, top = _int(router, "experts", r), _int(router, "top", r)
            groups, keep = 1, 1
            if router.get("groups") is not None:
                if not isinstance(router["groups"], dict):
                    raise ConfigError(f"invalid {r}groups: an object with count and keep")
                groups, keep = _int(router["groups"], "count", r + "groups."), _int(router["groups"], "keep", r + "groups.")
            if experts % groups or keep > groups:
                raise ConfigError(f"{r}groups: count must divide experts and keep be at most count")
            if top > keep * (experts // groups):
                raise ConfigError(f"{r}top: {top} experts cannot be chosen from {keep} groups of {experts // groups}")
            shared = TorinexConfig._expert(mlp["shared"], where + "mlp.shared.") if mlp.get("shared") is not None else None
            return TorinexFF("moe", expert=TorinexConfig._expert(mlp.get("expert"), where + "mlp.expert."),
                             experts=experts, top=top, groups=groups, keep=keep, shared=shared)
        raise ConfigError(f"unsupported {where}mlp.kind: {kind!r} (dense and moe are known)")

    @staticmethod
    def parse(raw: Any) -> "TorinexConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config must be an object")
        vocab, width = _int(raw, "vocab", ""), _int(raw, "width", "")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("missing norm (an object with eps)")
        eps = _number(norm, "eps", "norm.")
        side_dim = 0
        if raw.get("token_side") is not None:
            if not isinstance(raw["token_side"], dict):
                raise ConfigError("invalid token_side: an object with dim")
            side_dim = _int(raw["token_side"], "dim", "token_side.")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"{where}mixer must be an object")
            if entry.get("type") != "attention":
                raise ConfigError(f"unsupported {where}type: {entry.get('type')!r} (attention is known)")
            m, w = entry["mixer"], where + "mixer."
            heads, kv_heads = _int(m, "heads", w), _int(m, "kv_heads", w)
            dim, vdim = _int(m, "dim", w), _int(m, "vdim", w)
            if heads % kv_heads:
                raise ConfigError(f"{w}heads must be a multiple of kv_heads")
            if dim % 2 or vdim % 2 or dim > 512 or vdim > 512:
                raise ConfigError(f"{w}dim and vdim must be even and at most 512")
            chunk = None
            if m.get("mask") is not None:
                if not isinstance(m["mask"], dict):
                    raise ConfigError(f"invalid {w}mask: an object with size")
                chunk = _int(m["mask"], "size", w + "mask.")
            rot_base, rot_dims = 0.0, 0
            if m.get("rot") is not None:
                if not isinstance(m["rot"], dict):
                    raise ConfigError(f"invalid {w}rot: an object with base and dims")
                rot_base, rot_dims = _number(m["rot"], "base", w + "rot."), _int(m["rot"], "dims", w + "rot.", 2)
                if rot_dims % 2 or rot_dims > dim:
                    raise ConfigError(f"invalid {w}rot.dims: {rot_dims} (even and at most dim = {dim})")
            kv_from = None
            if m.get("kv_from") is not None:
                kv_from = _int(m, "kv_from", w, 0)
                if kv_from >= i or layers[kv_from].kv_from is not None:
                    raise ConfigError(f"{w}kv_from: {kv_from} must name an earlier layer that has keys of its own")
                src = layers[kv_from]
                if (src.kv_heads, src.dim, src.vdim) != (kv_heads, dim, vdim):
                    raise ConfigError(f"{w}kv_from: layer {kv_from} has other kv_heads, dim or vdim")
            layers.append(TorinexLayer(heads, kv_heads, dim, vdim, _number(m, "scale", w),
                                       TorinexConfig._feed_forward(entry.get("mlp"), where), chunk, rot_base,
                                       rot_dims, kv_from))
        return TorinexConfig(vocab, width, eps, side_dim, tuple(layers))

    # ------------------------------------------------------------------ parts
    def model_spec(self) -> ModelSpec:
        norm = PartSpec("output_rms_norm", {"width": self.width, "eps": self.eps})
        encodings: Dict[str, PartSpec] = {}
        names: Dict[tuple, str] = {}

        def encoding(base: float, dims: int) -> str:
            key = (base, dims)
            if key not in names:
                names[key] = f"rot{len(names)}"
                encodings[names[key]] = PartSpec("rotary_frequencies", {"rotary_dim": dims, "theta": base,
                                                                        "pairing": "interleaved"})
            return names[key]

        layers, run = [], []
        for i, l in enumerate(self.layers):
            mixer = {"hidden_size": self.width, "num_heads": l.heads, "num_kv_heads": l.kv_heads, "head_dim": l.dim,
                     "v_head_dim": l.vdim, "bias": True, "out_bias": True, "qk_norm_eps": self.eps,
                     "qk_norm_scope": "projection", "softmax_scale": l.scale, "chunk": l.chunk, "sink": "zero",
                     "own_kv": l.kv_from is None}
            if l.rot_dims:
                mixer.update(rot_dims=l.rot_dims, position_encoding=encoding(l.rot_base, l.rot_dims))
            parts = {"mixer": PartSpec("grouped_attention", mixer), "mixer_norm": norm}
            if l.ff is not None:
                parts["ff_norm"] = norm
                if l.ff.kind == "dense":
                    parts["feed_forward"] = PartSpec("dense_act", {"hidden_size": self.width,
                                                                   "intermediate_size": l.ff.ff,
                                                                   "activation": "relu_squared"})
                else:
                    f = l.ff
                    parts["feed_forward"] = PartSpec("routed_experts", {
                        "hidden_size": self.width, "intermediate_size": f.expert.ff, "experts": f.experts,
                        "top": f.top, "groups": f.groups, "keep_groups": f.keep, "scores": "softmax",
                        "renormalize": False, "activation": "clamped_swish_glu", "limit": f.expert.limit,
                        "shared_intermediate_size": f.shared.ff if f.shared else 0,
                        "shared_limit": f.shared.limit if f.shared else 0.0})
            if self.side_dim:
                parts["token_side"] = PartSpec("token_side_input", {
                    "hidden_size": self.width, "dim": self.side_dim, "column": i * self.side_dim,
                    "table_width": len(self.layers) * self.side_dim, "vocab_size": self.vocab, "eps": self.eps,
                    "activation": "gelu_tanh"})
            layers.append(LayerSpec(PartSpec("post_norm_stream"), parts))
            run.append(RunEntry(i, reads=l.kv_from))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "out_dtype": "float32"}),
            layers=tuple(layers), run_list=tuple(run), final_norm=norm,
            lm_head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": True}),
            position_encodings=encodings)
        spec.validate()
        return spec
