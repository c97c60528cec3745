"""Feed-forward parts."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import ParamDecl, Part
from .registry import register_part


class SwiGLU(Part):
    """down(silu(gate(x)) * up(x)) with gate and up packed into one matrix, no bias.

    ``gate_up_proj`` is [2 I, H] with the gate rows first (reference:
    src/layers/mlp.rs:7-25, packing src/models/qwen3/model.rs:577-586).
    """
    category = "feed_forward"
    chainable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])

    def param_decls(self):
        return {"gate_up_proj": ParamDecl((2 * self.inter, self.hidden)),
                "down_proj": ParamDecl((self.hidden, self.inter))}

    def takes_pending(self, tokens: int) -> bool:
        """Whether a step of ``tokens`` tokens runs the norm before it as the prologue of the gate/up product."""
        return ops.few_row_takes(tokens, self.params["gate_up_proj"], self.env.dtype, ops.EPI_SWIGLU)

    def forward(self, x):
        if ops.few_row_takes(x.shape[0], self.params["gate_up_proj"], self.env.dtype, ops.EPI_SWIGLU):
            # few tokens: norm (if pending), gate and up projections and silu(gate) * up in one kernel
            return ops.linear(ops.few_row_linear(x, self.params["gate_up_proj"], ops.EPI_SWIGLU, lazy=True),
                              self.params["down_proj"], lazy=True)
        if isinstance(x, ops.PendingNorm):
            x = x.materialize()
        if ops.gemm_tc_pays(x, self.params["gate_up_proj"], ops.GEMM_SWIGLU):
            # many tokens, large matrices: gate and up projections with silu(gate) * up as the epilogue, on tcgen05
            return ops.linear(ops.gemm_tc(x, self.params["gate_up_proj"], ops.GEMM_SWIGLU), self.params["down_proj"])
        gate_up = ops.linear(x, self.params["gate_up_proj"])
        return ops.linear(ops.silu_mul(gate_up), self.params["down_proj"])


class PolyNormFF(Part):
    """down(act(up(x))) with act = PolyNorm: a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N the
    division of a token's vector by its root mean square (in float).  ``act`` holds (a, b, c, e).  No bias."""
    category = "feed_forward"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.eps = float(spec["eps"])

    def param_decls(self):
        return {"up_proj": ParamDecl((self.inter, self.hidden)), "down_proj": ParamDecl((self.hidden, self.inter)),
                "act": ParamDecl((4,), "vector")}

    def bind(self, name, tensor):
        super().bind(name, tensor)
        if name == "act":
            self.params[name] = tensor.to(torch.float32).contiguous()

    def forward(self, x):
        z = ops.linear(x, self.params["up_proj"])
        return ops.linear(ops.poly_norm(z, self.params["act"], self.eps), self.params["down_proj"])


class DenseActFF(Part):
    """down(act(up(x))), no gate and no bias; ``activation``: gelu_erf (the exact gelu), gelu_tanh, silu or
    relu_squared (max(z, 0)^2), computed in float on the rounded projection and rounded once."""
    category = "feed_forward"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.activation = str(spec.get("activation", "gelu_erf"))
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is refused: {sorted(ops.ACTIVATIONS)}")

    def param_decls(self):
        return {"up_proj": ParamDecl((self.inter, self.hidden)), "down_proj": ParamDecl((self.hidden, self.inter))}

    def forward(self, x):
        z = ops.linear(x, self.params["up_proj"])
        return ops.linear(ops.activate(z, self.activation, in_place=True), self.params["down_proj"])


class TableExperts(Part):
    """A mixture of gated experts without a router: row ``token id`` of an integer ``table`` [vocab, top] names the
    token's experts (the entries of a row differ), and each counts 1 / top:

        y = (1 / top) sum_k down[e_k] (silu(gate[e_k] x) * (up[e_k] x))

    ``gate_up_proj`` [experts * 2 ff, hidden] holds expert after expert, each its gate rows and then its up rows;
    ``down_proj`` [experts * hidden, ff].  No biases.  The output is float32 (it is summed in float)."""
    category = "feed_forward"
    needs_context = True          # the choice depends on the step's token ids

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.experts = int(spec["experts"])
        self.top = int(spec["top"])
        self.vocab = int(spec["vocab_size"])
        if not 1 <= self.top <= self.experts:
            raise ValueError("a token takes between one and all experts")

    def param_decls(self):
        return {"gate_up_proj": ParamDecl((self.experts * 2 * self.inter, self.hidden)),
                "down_proj": ParamDecl((self.experts * self.hidden, self.inter)),
                "table": ParamDecl((self.vocab, self.top), "table")}

    def forward(self, x, ctx):
        p = self.params
        return ops.table_experts(x, ctx.token_ids, p["table"],
                                 p["gate_up_proj"].view(self.experts, 2 * self.inter, self.hidden),
                                 p["down_proj"].view(self.experts, self.hidden, self.inter))


class RoutedExperts(Part):
    """A mixture of gated experts chosen by a router, with an optional shared expert that every token takes:

        z = router x (in float);  s = softmax(z) over all experts (``scores`` "sigmoid": a sigmoid of each)
        the choice compares c = s + correction (``correction``: a stored float an expert; else c = s)
        experts form ``groups`` equal groups of neighbours; a group's score is the sum of its ``group_members``
        largest c (1, the default: its largest); only experts of the ``keep_groups`` best groups can be chosen; the
        ``top`` largest c of those are, with weights s (divided by their sum if ``renormalize``) times ``weight_scale``
        y = sum_k s_k down[e_k] glu(gate[e_k] x, up[e_k] x)  +  a shared_down glu(shared_gate x, shared_up x)
        a = 1, or with ``shared_gated`` sigmoid(shared_gate_row x): one number a token (``shared_gate_row`` [1, hidden])

    ``activation``: "swiglu" (silu(g) u) or "clamped_swish_glu" (g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit),
    u' = clamp(u, -limit, limit); ``alpha`` 1.702 unless given; the shared expert has its own ``shared_limit``).
    ``gate_up_proj`` [experts * 2 ff, hidden] holds expert after expert, each its gate rows and then its up rows;
    ``down_proj`` [experts * hidden, ff]; the shared expert's ``shared_gate_up_proj`` [2 sff, hidden] and
    ``shared_down_proj`` [hidden, sff] exist if ``shared_intermediate_size`` > 0.  No biases.  The output is float32
    (the weighted sum and the shared expert's share are added in float)."""
    category = "feed_forward"
    _GLU = {"swiglu": "silu", "clamped_swish_glu": "clamped_swish"}

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.experts = int(spec["experts"])
        self.top = int(spec["top"])
        self.groups = int(spec.get("groups") or 1)
        self.keep = int(spec.get("keep_groups") or self.groups)
        self.scores = str(spec.get("scores", "softmax"))
        self.renormalize = bool(spec.get("renormalize", False))
        self.activation = str(spec.get("activation", "swiglu"))
        self.limit = float(spec.get("limit") or 0.0)
        self.alpha = float(spec.get("alpha") or 1.702)
        self.shared_inter = int(spec.get("shared_intermediate_size") or 0)
        self.shared_limit = float(spec.get("shared_limit") or 0.0)
        self.correction = bool(spec.get("correction", False))
        self.group_members = int(spec.get("group_members") or 1)
        self.weight_scale = float(spec.get("weight_scale", 1.0))
        self.shared_gated = bool(spec.get("shared_gated", False)) and self.shared_inter > 0
        if self.activation not in self._GLU:
            raise ValueError(f"activation {self.activation!r} is refused: {sorted(self._GLU)}")
        if self.experts % self.groups or not 1 <= self.keep <= self.groups or \
                not 1 <= self.top <= self.keep * (self.experts // self.groups):
            raise ValueError("groups must divide the experts, and top experts must fit the groups that are kept")

    def param_decls(self):
        decls = {"router": ParamDecl((self.experts, self.hidden)),
                 "gate_up_proj": ParamDecl((self.experts * 2 * self.inter, self.hidden)),
                 "down_proj": ParamDecl((self.experts * self.hidden, self.inter))}
        if self.shared_inter:
            decls["shared_gate_up_proj"] = ParamDecl((2 * self.shared_inter, self.hidden))
            decls["shared_down_proj"] = ParamDecl((self.hidden, self.shared_inter))
        if self.shared_gated:
            decls["shared_gate_row"] = ParamDecl((1, self.hidden))
        if self.correction:
            decls["correction"] = ParamDecl((self.experts,), "vector")
        return decls

    def bind(self, name, tensor):
        super().bind(name, tensor)
        if name == "correction":
            self.params[name] = tensor.to(torch.float32).contiguous()

    def _shared_expert(self, x, glu):
        """The shared expert's output.  Its SwiGLU form is the dense feed-forward's, and takes that part's fused
        products: gate, up and silu(gate) * up in one few-row kernel for a step of few tokens, or as the epilogue of
        the tcgen05 product for a large portion."""
        p = self.params
        w = p["shared_gate_up_proj"]
        if glu == "silu" and x.dtype == torch.bfloat16:
            if ops.few_row_takes(x.shape[0], w, self.env.dtype, ops.EPI_SWIGLU, norm=False):
                return ops.linear(ops.few_row_linear(x, w, ops.EPI_SWIGLU), p["shared_down_proj"])
            if ops.gemm_tc_pays(x, w, ops.GEMM_SWIGLU):
                return ops.linear(ops.gemm_tc(x, w, ops.GEMM_SWIGLU), p["shared_down_proj"])
        a = ops.glu_columns(ops.linear(x, w), glu, self.shared_limit, self.alpha)
        return ops.linear(a, p["shared_down_proj"])

    def forward(self, x):
        p = self.params
        glu = self._GLU[self.activation]
        routed = ops.expert_router(x, p["router"], self.top, self.groups, self.keep, self.scores, self.renormalize,
                                   correction=p.get("correction"), group_members=self.group_members,
                                   gain_scale=self.weight_scale, gate=p.get("shared_gate_row"))
        choice, gains = routed[0], routed[1]
        shared_scale = routed[2] if self.shared_gated else None
        shared = self._shared_expert(x, glu) if self.shared_inter else None
        return ops.routed_experts(x, choice, gains, p["gate_up_proj"].view(self.experts, 2 * self.inter, self.hidden),
                                  p["down_proj"].view(self.experts, self.hidden, self.inter), glu, self.limit,
                                  self.alpha, add=shared, add_scale=shared_scale)


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "routed_experts", RoutedExperts)
register_part("feed_forward", "dense_act", DenseActFF)
register_part("feed_forward", "table_experts", TableExperts)
register_part("feed_forward", "poly_norm", PolyNormFF)
