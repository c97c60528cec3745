"""Torinex as a registry entry: configuration, parts and checkpoint names.

Checkpoint names: ``embed`` (also the output head), ``final.norm``, ``side.embed`` [vocab, layers * dim] with a
per-layer token input; per layer i ``l<i>.norm1`` and, with a feed-forward, ``l<i>.norm2``; ``l<i>.side.{gate,proj,norm}``;
the mixer's tensors ``l<i>.mix.*`` and the feed-forward's ``l<i>.mlp.*``:

    attention         q, k, v, o with q.b, k.b, v.b, o.b; q.norm, k.norm over the whole projection (q, k, v rows and
                      biases are packed; a layer that reads another layer's keys and values has q, q.b, q.norm, o, o.b)
    dense             up, down
    moe               router; e<j>.gate, e<j>.up, e<j>.down for every expert j; shared.gate, shared.up, shared.down

Linear weights are [out, in].
"""
from __future__ import annotations

from typing import List

from ..config.registry import Architecture, register_architecture
from ..config.torinex import TorinexConfig
from ..weights.plan import SourceTensor, WeightBinding


def torinex_weight_plan(c: TorinexConfig) -> List[WeightBinding]:
    w = c.width
    plan = [WeightBinding("embedding.weight", (SourceTensor("embed", (c.vocab, w)),))]
    side_table = None
    for i, l in enumerate(c.layers):
        src, dst = f"l{i}.", f"layers.{i}."
        m = src + "mix."
        q_rows, k_rows, v_rows = l.heads * l.dim, l.kv_heads * l.dim, l.kv_heads * l.vdim
        if l.kv_from is None:
            plan += [WeightBinding(dst + "mixer.qkv_proj", (
                         SourceTensor(m + "q", (q_rows, w)), SourceTensor(m + "k", (k_rows, w)),
                         SourceTensor(m + "v", (v_rows, w)))),
                     WeightBinding(dst + "mixer.qkv_bias", (
                         SourceTensor(m + "q.b", (q_rows,)), SourceTensor(m + "k.b", (k_rows,)),
                         SourceTensor(m + "v.b", (v_rows,)))),
                     WeightBinding(dst + "mixer.k_norm", (SourceTensor(m + "k.norm", (k_rows,), "norm"),))]
        else:
            plan += [WeightBinding(dst + "mixer.qkv_proj", (SourceTensor(m + "q", (q_rows, w)),)),
                     WeightBinding(dst + "mixer.qkv_bias", (SourceTensor(m + "q.b", (q_rows,)),))]
        plan += [WeightBinding(dst + "mixer.q_norm", (SourceTensor(m + "q.norm", (q_rows,), "norm"),)),
                 WeightBinding(dst + "mixer.o_proj", (SourceTensor(m + "o", (w, l.heads * l.vdim)),)),
                 WeightBinding(dst + "mixer.o_bias", (SourceTensor(m + "o.b", (w,)),)),
                 WeightBinding(dst + "mixer_norm.weight", (SourceTensor(src + "norm1", (w,), "norm"),))]
        if l.ff is not None:
            plan.append(WeightBinding(dst + "ff_norm.weight", (SourceTensor(src + "norm2", (w,), "norm"),)))
            f = src + "mlp."
            if l.ff.kind == "dense":
                plan += [WeightBinding(dst + "feed_forward.up_proj", (SourceTensor(f + "up", (l.ff.ff, w)),)),
                         WeightBinding(dst + "feed_forward.down_proj", (SourceTensor(f + "down", (w, l.ff.ff)),))]
            else:
                ff = l.ff.expert.ff
                gate_up, down = [], []
                for e in range(l.ff.experts):
                    gate_up += [SourceTensor(f"{f}e{e}.gate", (ff, w)), SourceTensor(f"{f}e{e}.up", (ff, w))]
                    down.append(SourceTensor(f"{f}e{e}.down", (w, ff)))
                plan += [WeightBinding(dst + "feed_forward.router", (SourceTensor(f + "router", (l.ff.experts, w)),)),
                         WeightBinding(dst + "feed_forward.gate_up_proj", tuple(gate_up)),
                         WeightBinding(dst + "feed_forward.down_proj", tuple(down))]
                if l.ff.shared is not None:
                    sf = l.ff.shared.ff
                    plan += [WeightBinding(dst + "feed_forward.shared_gate_up_proj", (
                                 SourceTensor(f + "shared.gate", (sf, w)), SourceTensor(f + "shared.up", (sf, w)))),
                             WeightBinding(dst + "feed_forward.shared_down_proj",
                                           (SourceTensor(f + "shared.down", (w, sf)),))]
        if c.side_dim:
            s = src + "side."
            if side_table is None:
                side_table = dst + "token_side.table"
                plan.append(WeightBinding(side_table, (SourceTensor("side.embed", (c.vocab, len(c.layers) * c.side_dim)),)))
            else:      # one table for all layers; each reads its own columns
                plan.append(WeightBinding(dst + "token_side.table", (), optional=True, alias_of=side_table))
            plan += [WeightBinding(dst + "token_side.gate_proj", (SourceTensor(s + "gate", (c.side_dim, w)),)),
                     WeightBinding(dst + "token_side.out_proj", (SourceTensor(s + "proj", (w, c.side_dim)),)),
                     WeightBinding(dst + "token_side.norm", (SourceTensor(s + "norm", (w,), "norm"),))]
    plan.append(WeightBinding("final_norm.weight", (SourceTensor("final.norm", (w,), "norm"),)))
    plan.append(WeightBinding("lm_head.weight", (), optional=True, alias_of="embedding.weight"))
    return plan


TORINEX = Architecture(name=TorinexConfig.architecture, model_type=TorinexConfig.model_type,
                       parse_config=TorinexConfig.parse, model_spec=TorinexConfig.model_spec,
                       weight_plan=torinex_weight_plan, checkpoint_dtype=lambda c: "bfloat16")

register_architecture(TORINEX, replace=True)
