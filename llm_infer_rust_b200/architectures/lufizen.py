"""Lufizen as a registry entry: configuration, parts and checkpoint names.

Checkpoint names: ``embed``, ``head``, ``final.norm``; per layer i ``l<i>.norm1`` and, with a feed-forward,
``l<i>.norm2``; the mixer's tensors ``l<i>.mix.*`` and the feed-forward's ``l<i>.mlp.*``:

    attention         q, k, sink, o                                   (q and k rows are packed; there is no v)
    latent_attention  dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o    (dq, dkv and g rows are packed into one matrix)
    moe               router, correction; e<j>.gate, e<j>.up, e<j>.down for every expert j;
                      shared.gate, shared.up, shared.down, shared.sg

Linear weights are [out, in].
"""
from __future__ import annotations

from typing import List

from ..config.lufizen import LufizenConfig
from ..config.registry import Architecture, register_architecture
from ..weights.plan import SourceTensor, WeightBinding


def lufizen_weight_plan(c: LufizenConfig) -> List[WeightBinding]:
    w = c.width
    plan = [WeightBinding("embedding.weight", (SourceTensor("embed", (c.vocab, w)),))]
    for i, l in enumerate(c.layers):
        src, dst = f"l{i}.", f"layers.{i}."
        m = src + "mix."
        if l.kind == "attention":
            plan += [WeightBinding(dst + "mixer.qkv_proj", (
                         SourceTensor(m + "q", (l.heads * l.dim, w)), SourceTensor(m + "k", (l.kv_heads * l.dim, w)))),
                     WeightBinding(dst + "mixer.sink", (SourceTensor(m + "sink", (l.heads,)),)),
                     WeightBinding(dst + "mixer.o_proj", (SourceTensor(m + "o", (w, l.heads * l.vdim)),))]
        else:
            q_rows, out_rows = l.heads * (l.dim + l.rot_dim), l.heads * l.vdim
            plan += [WeightBinding(dst + "mixer.qdkv_proj", (
                         SourceTensor(m + "dq", (l.q_rank, w)), SourceTensor(m + "dkv", (l.kv_rank + l.rot_dim, w)),
                         SourceTensor(m + "g", (l.heads, w)))),
                     WeightBinding(dst + "mixer.q_latent_norm", (SourceTensor(m + "dq.norm", (l.q_rank,), "norm"),)),
                     WeightBinding(dst + "mixer.uq_proj", (SourceTensor(m + "uq", (q_rows, l.q_rank)),)),
                     WeightBinding(dst + "mixer.latent_norm", (SourceTensor(m + "dkv.norm", (l.kv_rank,), "norm"),)),
                     WeightBinding(dst + "mixer.uk_proj", (SourceTensor(m + "uk", (l.heads * l.dim, l.kv_rank)),)),
                     WeightBinding(dst + "mixer.uv_proj", (SourceTensor(m + "uv", (out_rows, l.kv_rank)),)),
                     WeightBinding(dst + "mixer.o_proj", (SourceTensor(m + "o", (w, out_rows)),))]
        plan.append(WeightBinding(dst + "mixer_norm.weight", (SourceTensor(src + "norm1", (w,), "norm"),)))
        if l.ff is not None:
            plan.append(WeightBinding(dst + "ff_norm.weight", (SourceTensor(src + "norm2", (w,), "norm"),)))
            f, ff = src + "mlp.", l.ff.ff
            gate_up, down = [], []
            for e in range(l.ff.experts):
                gate_up += [SourceTensor(f"{f}e{e}.gate", (ff, w)), SourceTensor(f"{f}e{e}.up", (ff, w))]
                down.append(SourceTensor(f"{f}e{e}.down", (w, ff)))
            plan += [WeightBinding(dst + "feed_forward.router", (SourceTensor(f + "router", (l.ff.experts, w)),)),
                     WeightBinding(dst + "feed_forward.correction", (SourceTensor(f + "correction", (l.ff.experts,)),)),
                     WeightBinding(dst + "feed_forward.gate_up_proj", tuple(gate_up)),
                     WeightBinding(dst + "feed_forward.down_proj", tuple(down))]
            if l.ff.shared_ff:
                sf = l.ff.shared_ff
                plan += [WeightBinding(dst + "feed_forward.shared_gate_up_proj", (
                             SourceTensor(f + "shared.gate", (sf, w)), SourceTensor(f + "shared.up", (sf, w)))),
                         WeightBinding(dst + "feed_forward.shared_down_proj",
                                       (SourceTensor(f + "shared.down", (w, sf)),)),
                         WeightBinding(dst + "feed_forward.shared_gate_row", (SourceTensor(f + "shared.sg", (1, w)),))]
    plan.append(WeightBinding("final_norm.weight", (SourceTensor("final.norm", (w,), "norm"),)))
    plan.append(WeightBinding("lm_head.weight", (SourceTensor("head", (c.vocab, w)),)))
    return plan


LUFIZEN = Architecture(name=LufizenConfig.architecture, model_type=LufizenConfig.model_type,
                       parse_config=LufizenConfig.parse, model_spec=LufizenConfig.model_spec,
                       weight_plan=lufizen_weight_plan, checkpoint_dtype=lambda c: "bfloat16")

register_architecture(LUFIZEN, replace=True)
