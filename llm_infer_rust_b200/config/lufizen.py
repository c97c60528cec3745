"""Typed configuration of Lufizen, read from its own config.json keys.

    architecture      "Lufizen"
    vocab, width      sizes of the embedding table, of the output head and of the residual
    embedding.scale   every embedding row is multiplied by it
    logit_scale       the logits are multiplied by it
    norm.eps          eps of every RMS norm of the model (inside the root)
    layers[i]         type ("attention" | "latent_attention"), mixer (sizes and constants, below), mlp: null or
                      {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale",
                      "groups": {"count", "keep"}}, "shared": {"ff"}}
                      (``groups`` absent: one group; ``shared`` absent: no shared expert)

    attention         heads, kv_heads, dim, vdim (= dim: the values are the keys as projected; may be absent), scale,
                      rot {base, dims, scaling {factor, low, high, original}} (``rot`` absent: no rotation;
                      ``scaling`` absent: the plain frequencies)
    latent_attention  heads, dim (unrotated query/key size), rot_dim (rotated size), vdim, kv_rank, q_rank, scale,
                      rot {base, dims} (dims = rot_dim)

Nothing here is a default for a size: a key that the design needs and the file lacks is an error.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .kefetar import MAX_POSITIONS, _int, _number
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

# A group of experts is ranked by the sum of this many of its best members (fixed by the design).
GROUP_MEMBERS = 2


@dataclass(frozen=True)
class LufizenRotation:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None      # factor, low, high, original


@dataclass(frozen=True)
class LufizenFF:
    ff: int
    experts: int
    top: int
    scale: float
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0           # 0: no shared expert


@dataclass(frozen=True)
class LufizenLayer:
    kind: str                    # "attention" | "latent_attention"
    heads: int
    dim: int
    vdim: int
    scale: float
    ff: Optional[LufizenFF]
    rot: Optional[LufizenRotation] = None
    kv_heads: int = 0            # attention
    rot_dim: int = 0             # latent_attention
    kv_rank: int = 0
    q_rank: int = 0


@dataclass(frozen=True)
class LufizenConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_scale: float
    layers: Tuple[LufizenLayer, ...]

    architecture = "Lufizen"
    model_type = None

    @staticmethod
    def _rotation(m: dict, w: str, widest: int) -> Optional[LufizenRotation]:
        rot = m.get("rot")
        if rot is None:
            return None
        if not isinstance(rot, dict):
            raise ConfigError(f"invalid {w}rot: an object with base and dims")
        base, dims = _number(rot, "base", w + "rot."), _int(rot, "dims", w + "rot.", 2)
        if dims % 2 or dims > widest:
            raise ConfigError(f"invalid {w}rot.dims: {dims} (even and at most {widest})")
        scaling = None
        if rot.get("scaling") is not None:
            sc, sw = rot["scaling"], w + "rot.scaling."
            if not isinstance(sc, dict):
                raise ConfigError(f"invalid {w}rot.scaling: an object with factor, low, high and original")
            scaling = (_number(sc, "factor", sw), _number(sc, "low", sw), _number(sc, "high", sw),
                       _number(sc, "original", sw))
            if scaling[2] <= scaling[1]:
                raise ConfigError(f"{sw}high must be larger than low")
        return LufizenRotation(base, dims, scaling)

    @staticmethod
    def _feed_forward(mlp: Any, where: str) -> Optional[LufizenFF]:
        if mlp is None:
            return None
        if not isinstance(mlp, dict):
            raise ConfigError(f"invalid {where}mlp: an object or null is required")
        if mlp.get("kind") != "moe":
            raise ConfigError(f"unsupported {where}mlp.kind: {mlp.get('kind')!r} (moe is known)")
        router, expert = mlp.get("router"), mlp.get("expert")
        if not isinstance(router, dict) or not isinstance(expert, dict):
            raise ConfigError(f"{where}mlp needs a router object and an expert object")
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
        shared_ff = 0
        if mlp.get("shared") is not None:
            if not isinstance(mlp["shared"], dict):
                raise ConfigError(f"invalid {where}mlp.shared: an object with ff")
            shared_ff = _int(mlp["shared"], "ff", where + "mlp.shared.")
        return LufizenFF(_int(expert, "ff", where + "mlp.expert."), experts, top, _number(router, "scale", r),
                         groups, keep, shared_ff)

    @staticmethod
    def parse(raw: Any) -> "LufizenConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config must be an object")
        vocab, width = _int(raw, "vocab", ""), _int(raw, "width", "")
        norm, embedding = raw.get("norm"), raw.get("embedding")
        if not isinstance(norm, dict):
            raise ConfigError("missing norm (an object with eps)")
        if not isinstance(embedding, dict):
            raise ConfigError("missing embedding (an object with scale)")
        eps = _number(norm, "eps", "norm.")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"{where}mixer must be an object")
            kind, m, w = entry.get("type"), entry["mixer"], where + "mixer."
            ff = LufizenConfig._feed_forward(entry.get("mlp"), where)
            heads, dim = _int(m, "heads", w), _int(m, "dim", w)
            # an attention layer's values are its keys: a file may leave their size out, but not contradict it
            vdim = _int(m, "vdim", w) if (kind != "attention" or "vdim" in m) else dim
            scale = _number(m, "scale", w)
            if kind == "attention":
                kv_heads = _int(m, "kv_heads", w)
                if heads % kv_heads:
                    raise ConfigError(f"{w}heads must be a multiple of kv_heads")
                if vdim != dim:
                    raise ConfigError(f"{w}vdim must equal dim: the values are the keys as projected")
                if dim % 2 or dim > 512:
                    raise ConfigError(f"{w}dim must be even and at most 512")
                layers.append(LufizenLayer(kind, heads, dim, vdim, scale, ff, LufizenConfig._rotation(m, w, dim),
                                           kv_heads=kv_heads))
            elif kind == "latent_attention":
                rot_dim, kv_rank, q_rank = _int(m, "rot_dim", w), _int(m, "kv_rank", w), _int(m, "q_rank", w)
                if kv_rank % 2 or rot_dim % 2 or kv_rank + rot_dim > 512:
                    raise ConfigError(f"{w}kv_rank and rot_dim must be even and kv_rank + rot_dim at most 512")
                rot = LufizenConfig._rotation(m, w, rot_dim)
                if rot is None or rot.dims != rot_dim:
                    raise ConfigError(f"{w}rot.dims must equal rot_dim: the rotated part is rotated as a whole")
                layers.append(LufizenLayer(kind, heads, dim, vdim, scale, ff, rot, rot_dim=rot_dim, kv_rank=kv_rank,
                                           q_rank=q_rank))
            else:
                raise ConfigError(f"unsupported {where}type: {kind!r} (attention and latent_attention are known)")
        return LufizenConfig(vocab, width, eps, _number(embedding, "scale", "embedding."),
                             _number(raw, "logit_scale", ""), tuple(layers))

    # ------------------------------------------------------------------ parts
    def model_spec(self) -> ModelSpec:
        norm = PartSpec("output_rms_norm", {"width": self.width, "eps": self.eps})
        encodings: Dict[str, PartSpec] = {}
        names: Dict[tuple, str] = {}

        def encoding(rot: LufizenRotation, pairing: str) -> str:
            key = (rot, pairing)
            if key not in names:
                names[key] = f"rot{len(names)}"
                params = {"rotary_dim": rot.dims, "theta": rot.base, "pairing": pairing}
                if rot.scaling is not None:
                    params["wavelength_scaling"] = dict(zip(("factor", "low", "high", "original"), rot.scaling))
                encodings[names[key]] = PartSpec("rotary_frequencies", params)
            return names[key]

        layers = []
        for l in self.layers:
            if l.kind == "attention":
                mixer = {"hidden_size": self.width, "num_heads": l.heads, "num_kv_heads": l.kv_heads,
                         "head_dim": l.dim, "v_head_dim": l.vdim, "values_from_keys": True, "qk_norm_eps": self.eps,
                         "qk_norm_weight": False, "qk_norm_order": "after_rotation", "softmax_scale": l.scale,
                         "sink": True}
                if l.rot is not None:
                    mixer.update(rot_dims=l.rot.dims, position_encoding=encoding(l.rot, "half_split"))
                parts = {"mixer": PartSpec("grouped_attention", mixer), "mixer_norm": norm}
            else:
                parts = {"mixer": PartSpec("latent_attention", {
                    "hidden_size": self.width, "num_heads": l.heads, "head_dim": l.dim, "rot_dim": l.rot_dim,
                    "v_head_dim": l.vdim, "kv_rank": l.kv_rank, "q_rank": l.q_rank, "eps": self.eps,
                    "softmax_scale": l.scale, "gate": "head", "rot_dims": l.rot.dims,
                    "position_encoding": encoding(l.rot, "interleaved")}), "mixer_norm": norm}
            if l.ff is not None:
                f = l.ff
                parts["ff_norm"] = norm
                parts["feed_forward"] = PartSpec("routed_experts", {
                    "hidden_size": self.width, "intermediate_size": f.ff, "experts": f.experts, "top": f.top,
                    "groups": f.groups, "keep_groups": f.keep, "scores": "sigmoid", "renormalize": False,
                    "correction": True, "group_members": GROUP_MEMBERS, "weight_scale": f.scale,
                    "activation": "swiglu", "shared_intermediate_size": f.shared_ff, "shared_gated": f.shared_ff > 0})
            layers.append(LayerSpec(PartSpec("post_norm_stream"), parts))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "out_dtype": "float32", "scale": self.embedding_scale}),
            layers=tuple(layers), run_list=tuple(RunEntry(i) for i in range(len(layers))), final_norm=norm,
            lm_head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False,
                                             "logit_scale": self.logit_scale}),
            position_encodings=encodings)
        spec.validate()
        return spec
