"""Token embedding and output head."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import ParamDecl, Part
from .registry import register_part


class TokenEmbedding(Part):
    """h[t] = table[ids[t]], unscaled (reference: src/layers/linear.rs:9-11).  ``out_dtype`` "float32": the
    rows come out in float32 whatever the table's dtype (for a model whose residual stream is float32).
    ``scale``: every row is multiplied by it (in float, before the one rounding)."""
    category = "embedding"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.out_dtype = torch.float32 if spec.get("out_dtype") == "float32" else env.dtype
        self.scale = float(spec.get("scale", 1.0))

    def param_decls(self):
        return {"weight": ParamDecl((self.vocab, self.hidden))}

    def forward(self, token_ids):
        return ops.embedding(token_ids, self.params["weight"], self.out_dtype, self.scale)


class LinearHead(Part):
    """logits = x W^T in float32, no scale (reference: src/layers/linear.rs:15-20); with ``softcap`` c the logits
    become c * tanh(logits / c), in float; with ``logit_scale`` s they are multiplied by s, in float.

    With ``tied`` and no stored head the weight is the embedding table itself.
    """
    category = "head"
    chainable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.tied = bool(spec.get("tied", False))
        self.softcap = float(spec.get("softcap") or 0.0)
        self.logit_scale = float(spec.get("logit_scale", 1.0))

    def param_decls(self):
        return {"weight": ParamDecl((self.vocab, self.hidden))}

    def takes_pending(self, rows: int) -> bool:
        return ops.few_row_takes(rows, self.params["weight"], self.env.dtype, ops.EPI_PLAIN_F32)

    def forward(self, x):
        if isinstance(x, ops.PendingNorm):
            if self.takes_pending(x.shape[0]) and not self.softcap > 0.0 and self.logit_scale == 1.0:
                return ops.few_row_linear(x, self.params["weight"], ops.EPI_PLAIN_F32, lazy=True)
            x = x.materialize()
        logits = ops.linear(x, self.params["weight"], out_dtype=torch.float32)
        if self.logit_scale != 1.0:
            logits = ops.scale_floats(logits, self.logit_scale)
        return ops.tanh_cap(logits, self.softcap) if self.softcap > 0.0 else logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", LinearHead)
