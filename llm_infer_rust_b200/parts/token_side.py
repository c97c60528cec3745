"""A per-layer input from a second token table."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import ParamDecl, Part
from .registry import register_part


class TokenSideInput(Part):
    """What a layer adds to a float32 stream x from a second embedding table, gated by x:

        e = table[token][column : column + dim];   g = act(gate_proj x) * e;   y = out_proj g
        x <- x + y / sqrt(mean(y^2) + eps) * norm

    ``table`` [vocab, table_width] is one table for all layers (every layer's part is bound to the same tensor and
    reads its own ``dim`` columns from ``column`` on); ``gate_proj`` [dim, hidden], ``out_proj`` [hidden, dim],
    ``norm`` [hidden] a plain RMS-norm weight; ``activation`` by name (``ops.ACTIVATIONS``).  The products read the
    stream rounded to the engine's dtype; the activation, the norm and the add are taken in float.  A step of few
    tokens (``ops.TOKEN_SIDE_FEW``) takes one kernel for all of it; its y stays in float instead of being rounded."""
    category = "token_side"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.dim = int(spec["dim"])
        self.column = int(spec.get("column", 0))
        self.table_width = int(spec.get("table_width", self.dim))
        self.vocab = int(spec["vocab_size"])
        self.eps = float(spec["eps"])
        self.activation = str(spec.get("activation", "gelu_tanh"))
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is refused: {sorted(ops.ACTIVATIONS)}")
        if self.column < 0 or self.column + self.dim > self.table_width:
            raise ValueError("the layer's columns lie outside the table")

    def param_decls(self):
        return {"table": ParamDecl((self.vocab, self.table_width)), "gate_proj": ParamDecl((self.dim, self.hidden)),
                "out_proj": ParamDecl((self.hidden, self.dim)), "norm": ParamDecl((self.hidden,), "vector")}

    def bind(self, name, tensor):
        super().bind(name, tensor)
        if name == "norm":
            self.params[name] = tensor.to(torch.float32).contiguous()

    def add_into(self, stream, x, ctx):
        """``stream``: the float32 x (changed in place); ``x``: the same rounded to the engine's dtype.  Returns the
        new stream rounded to the engine's dtype."""
        p = self.params
        if x.shape[0] <= ops.TOKEN_SIDE_FEW:       # a decode step: one kernel instead of four
            return ops.token_side_few(stream, x, p["gate_proj"], p["table"], ctx.token_ids, self.column, p["out_proj"],
                                      p["norm"], self.eps, self.activation, cast_to=self.env.dtype)
        z = ops.linear(x, p["gate_proj"])
        g = ops.act_table_mul(z, self.activation, p["table"], ctx.token_ids, self.column)
        y = ops.linear(g, p["out_proj"])
        return ops.norm_add(stream, y, p["norm"], self.eps, cast_to=self.env.dtype)


register_part("token_side", "token_side_input", TokenSideInput)
