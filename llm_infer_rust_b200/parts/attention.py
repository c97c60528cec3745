"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import PagedKVSpec, ParamDecl, Part, StateSpec
from .registry import register_part

_KEYS_PER_CTA_AT_LEAST = 512      # fewer keys per CTA leave its warps' copy pipelines half empty
# Latent rows are two to four times as wide as a head of 128 and one CTA serves up to 16 query heads on them: a CTA
# is busy with far fewer keys (measured at 8 rows x 16 heads on rows of 320 columns, 2,048 keys: 43.0 us in 4 splits,
# 27.5 us in 16; 32 heads on rows of 448: 128.0 against 91.1 us; one row of 8,192 keys: 246.8 against 82.9 us).
_LATENT_KEYS_PER_CTA_AT_LEAST = 128


def decode_splits(ctas_per_split: int, kv_len_bound: int, sm_count: int,
                  keys_per_cta: int = _KEYS_PER_CTA_AT_LEAST) -> int:
    """How many CTAs share one row's keys.

    With ``ctas_per_split`` CTAs for each split, the number of splits is chosen so that the
    grid fills whole waves of SMs as well as it can while every CTA keeps at least ``keys_per_cta`` keys.
    """
    ctas_per_split = max(1, ctas_per_split)
    if 8 * ctas_per_split >= 7 * sm_count:
        # A grid that fills the SMs without splits stays whole: with several waves the splits are combined by a kernel
        # of its own, which costs more than the last wave's idle SMs (measured at 4,096 keys a row: 32 rows x 8 KV
        # heads 90.8 us whole against 103.8 us in the four splits that fill the waves best, 64 rows 177.5 against
        # 182.3 us in two).
        return 1
    most = max(1, min(64, kv_len_bound // max(1, keys_per_cta)))
    best, best_fill = 1, 0.0
    for splits in range(1, most + 1):
        if splits == 8 and 2 * ctas_per_split * splits > sm_count:
            # Eight splits of a grid that fits one wave are the CTAs of one cluster, and more than a handful of clusters
            # of eight do not find room side by side: measured at 2 rows x 8 KV heads, 18.1 us against 12.4 us with six
            # splits (one row: 8 clusters of eight, 9.6 us, the best there).
            continue
        ctas = ctas_per_split * splits
        fill = ctas / (sm_count * -(-ctas // sm_count))
        if fill > best_fill * 1.05:
            best, best_fill = splits, fill
    return best


class GQAttention(Part):
    """q, k, v = x W_qkv^T; per-head RMSNorm of q and k; rotary encoding; keys and
    values go to the cache; causal (optionally windowed) attention over the cache;
    output projection.  No bias.

    Order and formulas: src/models/qwen3/model.rs:462-534 of the reference; one
    packed QKV matrix with q rows, then k rows, then v rows (src/layers/linear.rs:25-78).
    Parameters of the part: head counts, head size, the norm's eps (None: no QK
    norm), the window (None: all keys), the softmax scale and the name of the
    model's position encoding.
    """
    category = "mixer"
    chainable = True          # reads its input through ops.* only, and may return a product that still waits (ops.few_row_linear)

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        self.qk_eps = spec.get("qk_norm_eps")
        self.window = spec.get("window")
        self.scale = float(spec.get("softmax_scale", 1.0 / math.sqrt(self.d)))
        if self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.d % 2 or not 2 <= self.d <= 512:
            raise ValueError(f"head_dim {self.d} is refused: the attention kernels take even head sizes up to 512")
        name = spec.get("position_encoding")
        self.rope = env.position_encodings[name] if name else None

    def param_decls(self):
        decls = {"qkv_proj": ParamDecl(((self.nh + 2 * self.nkv) * self.d, self.hidden)),
                 "o_proj": ParamDecl((self.hidden, self.nh * self.d))}
        if self.qk_eps is not None:
            decls["q_norm"] = ParamDecl((self.d,), "vector")
            decls["k_norm"] = ParamDecl((self.d,), "vector")
        return decls

    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.d, self.window)

    def state_spec(self):
        return None

    def takes_pending(self, tokens: int) -> bool:
        """Whether a step of ``tokens`` tokens runs the input norm as the prologue of the QKV product."""
        return ops.few_row_takes(tokens, self.params["qkv_proj"], self.env.dtype, ops.EPI_QKV, self.d)

    def forward(self, x, ctx, cache):
        p = self.params
        tokens = x.shape[0]
        rope = self.rope
        q = torch.empty((tokens, self.nh * self.d), dtype=x.dtype, device=x.device)
        slots = ctx.slots[cache.group] if cache.writes else None
        if ops.few_row_takes(tokens, p["qkv_proj"], self.env.dtype, ops.EPI_QKV, self.d):
            # few tokens: norm (if pending), projection, per-head norm, rotation and cache store in one kernel
            ops.few_row_linear(x, p["qkv_proj"], ops.EPI_QKV, qkv=dict(
                head_dim=self.d, num_heads=self.nh, num_kv_heads=self.nkv, q_out=q, k_cache=cache.k, v_cache=cache.v,
                q_weight=p.get("q_norm"), k_weight=p.get("k_norm"), eps=float(self.qk_eps or 0.0),
                cos=rope.cos if rope else None, sin=rope.sin if rope else None,
                rot_dim=rope.rot_dim if rope else 0, positions=ctx.positions, slots=slots), lazy=True)
        else:
            if isinstance(x, ops.PendingNorm):
                x = x.materialize()
            qkv = ops.linear(x, p["qkv_proj"])
            ops.qkv_post(qkv, q, cache.k, cache.v, p.get("q_norm"), p.get("k_norm"),
                         float(self.qk_eps or 0.0), rope.cos if rope else None, rope.sin if rope else None,
                         rope.rot_dim if rope else 0, ctx.positions, slots, self.nh, self.nkv, self.d)
        out = torch.empty_like(q)
        g = cache.group
        page = ctx.page_sizes[g]
        if ctx.num_prefill:
            ops.prefill_attention(q, cache.k, cache.v, out, ctx.block_tables[g], ctx.cu_q, ctx.kv_len,
                                  ctx.prefix_len, ctx.prefill_rows, ctx.num_prefill, ctx.max_q_len,
                                  self.nh, self.nkv, self.d, page, self.window, self.scale)
        if ctx.num_decode:
            bound = min(ctx.kv_len_bound, self.window) if self.window else ctx.kv_len_bound
            per_split = ops.decode_ctas_per_split(q.dtype, ctx.num_decode, self.nh, self.nkv, self.d, page)
            splits = decode_splits(per_split, bound, ctx.sm_count)
            need = ops.decode_scratch_floats(ctx.num_decode, self.nh, self.d, splits)
            scratch = ctx.scratch(need) if need else None
            ops.decode_attention(q, cache.k, cache.v, out, scratch, ctx.block_tables[g], ctx.cu_q,
                                 ctx.kv_len, ctx.decode_rows, ctx.num_decode, self.nh, self.nkv, self.d,
                                 page, self.window, self.scale, splits)
        return ops.linear(out, p["o_proj"], lazy=True)


class GatedConvAttention(Part):
    """Grouped-query softmax attention over the paged cache whose q, k and v pass through a short causal
    convolution over time, with soft-capped scores, values mixed with an earlier layer's and a sigmoid gate.

    q, k, v, g = x W^T (one packed matrix: q rows, k rows, v rows, gate rows; keys are ``head_dim`` wide, values
    ``v_head_dim``); then, each optional and a parameter of the part:
      * ``conv_taps`` >= 1: a causal convolution on every channel of q, k and v (``conv`` [channels, taps]; its
        last taps - 1 inputs are the request's state);
      * ``position_encoding``: half-split rotation of q and k;
      * ``v_mix`` "source": this layer's v is kept for the step under the name ``v_mix_group``; "mix": v becomes
        (1 - vmix) v + vmix v_source, and that is what the cache holds;
      * ``softcap``: score <- cap * tanh(score / cap) after ``softmax_scale``; the softmax weights stay floats
        (all-sizes kernel) or enter the product with the values as two bfloat16 terms (tensor-core kernel);
      * ``window``: only the last W keys are read;
      * ``gate``: the heads' outputs are multiplied by sigmoid(g) before the output projection.
    No bias."""
    category = "mixer"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec.get("v_head_dim") or self.d)
        self.taps = int(spec.get("conv_taps") or 0)           # 0: no convolution; 1: a gain per channel
        self.window = spec.get("window")
        self.scale = float(spec.get("softmax_scale", 1.0 / math.sqrt(self.d)))
        self.softcap = float(spec.get("softcap") or 0.0)
        self.gate = bool(spec.get("gate", True))
        self.v_mix = spec.get("v_mix")                          # None | "source" | "mix"
        self.v_mix_group = str(spec.get("v_mix_group", "v"))
        if self.v_mix not in (None, "source", "mix"):
            raise ValueError(f"v_mix {self.v_mix!r} is refused: source, mix or nothing")
        if self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        for width in (self.d, self.dv):
            if width % 2 or not 2 <= width <= 512:
                raise ValueError(f"head size {width} is refused: the attention kernels take even head sizes up to 512")
        if not 0 <= self.taps <= 8:
            raise ValueError(f"{self.taps} taps are refused: the convolution kernels take up to 8")
        name = spec.get("position_encoding")
        self.rope = env.position_encodings[name] if name else None
        if self.rope is not None and self.rope.rot_dim > self.d:
            raise ValueError("the rotation is wider than a head")
        self.qkv_channels = (self.nh + self.nkv) * self.d + self.nkv * self.dv

    def param_decls(self):
        rows = self.qkv_channels + (self.nh * self.dv if self.gate else 0)
        decls = {"qkvg_proj": ParamDecl((rows, self.hidden)), "o_proj": ParamDecl((self.hidden, self.nh * self.dv))}
        if self.taps >= 1:
            decls["conv"] = ParamDecl((self.qkv_channels, self.taps))
        if self.v_mix is not None:
            decls["vmix"] = ParamDecl((), "vector")
        return decls

    def bind(self, name, tensor):
        super().bind(name, tensor)
        if name == "conv":
            self.params[name] = tensor.to(torch.float32).contiguous()
        elif name == "vmix":
            self.params[name] = tensor.to(torch.float32).reshape(1).contiguous()

    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.d, self.window, self.dv if self.dv != self.d else None)

    def state_spec(self):
        return StateSpec((self.taps - 1, self.qkv_channels), torch.float32) if self.taps > 1 else None

    def forward(self, x, ctx, cache):
        p = self.params
        tokens = x.shape[0]
        rope = self.rope
        packed = ops.linear(x, p["qkvg_proj"])
        q = torch.empty((tokens, self.nh * self.d), dtype=packed.dtype, device=packed.device)
        slots = ctx.slots[cache.group] if cache.writes else None
        v_first, v_mode = None, 0
        if self.v_mix == "source":
            v_first = torch.empty((tokens, self.nkv * self.dv), dtype=torch.float32, device=packed.device)
            ctx.extras["v_mix:" + self.v_mix_group] = v_first
            v_mode = 1
        elif self.v_mix == "mix":
            v_first = ctx.extras.get("v_mix:" + self.v_mix_group)
            if v_first is None or v_first.shape != (tokens, self.nkv * self.dv):
                raise RuntimeError("a layer mixes its values with those of a layer that did not run in this step "
                                   "(or whose values have another width)")
            v_mode = 2
        ops.conv_qkv_post(packed, p.get("conv"), cache.state, ctx, q, cache.k, cache.v,
                          rope.inv_freq if rope else None, rope.rot_dim if rope else 0, slots, self.nh, self.nkv,
                          self.d, self.dv, vmix=p.get("vmix") if v_mode == 2 else None, v_first=v_first, v_mode=v_mode)
        out = torch.empty((tokens, self.nh * self.dv), dtype=packed.dtype, device=packed.device)
        g = cache.group
        page = ctx.page_sizes[g]
        if ctx.num_prefill:
            ops.prefill_attention(q, cache.k, cache.v, out, ctx.block_tables[g], ctx.cu_q, ctx.kv_len,
                                  ctx.prefix_len, ctx.prefill_rows, ctx.num_prefill, ctx.max_q_len,
                                  self.nh, self.nkv, self.d, page, self.window, self.scale,
                                  v_head_dim=self.dv, softcap=self.softcap, precise_weights=True)
        if ctx.num_decode:
            bound = min(ctx.kv_len_bound, self.window) if self.window else ctx.kv_len_bound
            plain = self.dv == self.d
            per_split = ops.decode_ctas_per_split(q.dtype, ctx.num_decode, self.nh, self.nkv, self.d, page, plain)
            splits = decode_splits(per_split, bound, ctx.sm_count)
            need = ops.decode_scratch_floats(ctx.num_decode, self.nh, max(self.d, self.dv), splits)
            scratch = ctx.scratch(need) if need else None
            ops.decode_attention(q, cache.k, cache.v, out, scratch, ctx.block_tables[g], ctx.cu_q,
                                 ctx.kv_len, ctx.decode_rows, ctx.num_decode, self.nh, self.nkv, self.d,
                                 page, self.window, self.scale, splits, v_head_dim=self.dv, softcap=self.softcap,
                                 precise_weights=True)
        if self.gate:
            ops.sigmoid_gate_mul(out, packed, self.qkv_channels)
        return ops.linear(out, p["o_proj"])


def _masked_attention(part, q, out, ctx, cache, num_heads, num_kv_heads, head_dim, v_head_dim, sinks,
                      shared_values=False):
    """Attention of a step's rows over the paged cache for a mixer with ``window``, ``chunk`` and ``scale``: prompt
    portions and single decoded tokens, softmax weights in float.  ``shared_values``: a value is the first
    ``v_head_dim`` columns of its key's row (one KV head)."""
    g = cache.group
    page = ctx.page_sizes[g]
    if ctx.num_prefill:
        ops.prefill_attention(q, cache.k, cache.v, out, ctx.block_tables[g], ctx.cu_q, ctx.kv_len,
                              ctx.prefix_len, ctx.prefill_rows, ctx.num_prefill, ctx.max_q_len,
                              num_heads, num_kv_heads, head_dim, page, part.window, part.scale,
                              v_head_dim=v_head_dim, precise_weights=True, chunk=part.chunk, sinks=sinks,
                              shared_values=shared_values)
    if ctx.num_decode:
        bound = ctx.kv_len_bound
        for limit in (part.window, part.chunk):
            if limit:
                bound = min(bound, limit)
        plain = v_head_dim == head_dim
        keys_per_cta = _KEYS_PER_CTA_AT_LEAST
        if shared_values and ops.latent_uses_tensor_cores(q.dtype, num_heads, head_dim, v_head_dim, page):
            per_split = ctx.num_decode * (num_heads // ops.latent_head_group(num_heads))
            keys_per_cta = _LATENT_KEYS_PER_CTA_AT_LEAST
        else:
            per_split = ops.decode_ctas_per_split(q.dtype, ctx.num_decode, num_heads, num_kv_heads, head_dim, page, plain)
        splits = decode_splits(per_split, bound, ctx.sm_count, keys_per_cta)
        need = ops.decode_scratch_floats(ctx.num_decode, num_heads, max(head_dim, v_head_dim), splits)
        scratch = ctx.scratch(need) if need else None
        ops.decode_attention(q, cache.k, cache.v, out, scratch, ctx.block_tables[g], ctx.cu_q,
                             ctx.kv_len, ctx.decode_rows, ctx.num_decode, num_heads, num_kv_heads, head_dim,
                             page, part.window, part.scale, splits, v_head_dim=v_head_dim, precise_weights=True,
                             chunk=part.chunk, sinks=sinks, shared_values=shared_values)


class GroupedAttention(Part):
    """Grouped-query softmax attention over the paged cache with keys ``head_dim`` wide and values ``v_head_dim``
    wide, from one packed projection (q rows, k rows, v rows, then gate rows if gated).  Each of these is a
    parameter of the part and may be absent:
      * ``bias``: q, k and v have biases (one packed vector, added in float before anything else);  ``out_bias``: so
        has the output projection (``o_bias``; a block that adds the mixer's output through a kernel of its own may
        take the bias into that kernel, ``defer_output_bias``);
      * ``qk_norm_eps``: q and k are RMS-normed, ``qk_norm_scope`` "head": per head with one weight vector each
        (``q_norm``, ``k_norm`` of a head's size), "projection": over all of a token's q columns at once, before they
        are split into heads, and over all of its k columns (weights of the projections' sizes);
        ``qk_norm_weight`` False: the per-head norm has no weights (x / sqrt(mean(x^2) + eps));
        ``qk_norm_order`` "after_rotation": the per-head norm follows the rotation instead of preceding it;
      * ``values_from_keys``: there is no value projection (the packed matrix holds q rows and k rows): a token's
        value is its key as projected, before norm and rotation;
      * ``position_encoding`` / ``rot_dims``: the first rot_dims coordinates of every q and k head are rotated
        (the encoding says whether pairs are interleaved or half-split);
      * ``window`` W: a query at position p reads keys p - W < j <= p;  ``chunk`` C: only keys from p - p % C on
        (its own block of C positions, blocks counted from the sequence's start); both masks may be set;
      * ``sink``: a learned number per head whose exponential joins the softmax's denominator (no key, no value,
        not scaled); "zero": the number is 0 for every head and no parameter (one is added to the denominator);
      * ``own_kv`` False: the layer has no key and value projections (the packed matrix and bias hold q alone) and
        reads the cache of the run-list entry that its own entry names, with its own queries, masks and scale;
      * ``gate``: the heads' outputs are multiplied by sigmoid(g) before the output projection.
    Softmax weights stay floats."""
    category = "mixer"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec.get("v_head_dim") or self.d)
        self.bias = bool(spec.get("bias", False))
        self.qk_eps = spec.get("qk_norm_eps")
        self.window = spec.get("window")
        self.chunk = spec.get("chunk")
        self.scale = float(spec.get("softmax_scale", 1.0 / math.sqrt(self.d)))
        self.zero_sink = spec.get("sink") == "zero"
        self.sink = bool(spec.get("sink", False)) and not self.zero_sink
        self.gate = bool(spec.get("gate", False))
        self.out_bias = bool(spec.get("out_bias", False))
        self.norm_scope = str(spec.get("qk_norm_scope", "head"))
        self.own_kv = bool(spec.get("own_kv", True))
        self.norm_weight = bool(spec.get("qk_norm_weight", True))
        self.norm_order = str(spec.get("qk_norm_order", "before_rotation"))
        self.values_from_keys = bool(spec.get("values_from_keys", False))
        if self.norm_scope not in ("head", "projection"):
            raise ValueError(f"qk_norm_scope {self.norm_scope!r} is refused: head or projection")
        if self.norm_order not in ("before_rotation", "after_rotation"):
            raise ValueError(f"qk_norm_order {self.norm_order!r} is refused: before_rotation or after_rotation")
        if self.norm_scope != "head" and (not self.norm_weight or self.norm_order != "before_rotation" or
                                          self.values_from_keys):
            raise ValueError("a norm without weights, a norm after the rotation and values that are the keys are "
                             "served with per-head norms")
        if self.values_from_keys and (self.dv != self.d or not self.own_kv):
            raise ValueError("values that are the keys are as wide as the keys, and the layer has keys of its own")
        if self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        for width in (self.d, self.dv):
            if width % 2 or not 2 <= width <= 512:
                raise ValueError(f"head size {width} is refused: the attention kernels take even head sizes up to 512")
        if not self.own_kv and (self.gate or self.norm_scope != "projection"):
            raise ValueError("a layer without keys of its own is served with projection-wide norms and no gate")
        name = spec.get("position_encoding")
        self.rope = env.position_encodings[name] if name else None
        self.rot_dims = int(spec.get("rot_dims") or (self.rope.rot_dim if self.rope else 0))
        if self.rope is not None and (self.rot_dims != self.rope.rot_dim or self.rot_dims > self.d):
            raise ValueError("the rotation does not fit the head or the encoding")
        self.q_channels = self.nh * self.d
        self.qkv_channels = self.q_channels + (self.nkv * (self.d + (0 if self.values_from_keys else self.dv))
                                               if self.own_kv else 0)
        self.bias_deferred = False
        self.zero_sinks = torch.zeros(self.nh, dtype=torch.float32, device=env.device) if self.zero_sink else None

    def param_decls(self):
        rows = self.qkv_channels + (self.nh * self.dv if self.gate else 0)
        decls = {"qkv_proj": ParamDecl((rows, self.hidden)), "o_proj": ParamDecl((self.hidden, self.nh * self.dv))}
        if self.bias:
            decls["qkv_bias"] = ParamDecl((self.qkv_channels,), "vector")
        if self.out_bias:
            decls["o_bias"] = ParamDecl((self.hidden,), "vector")
        if self.qk_eps is not None and self.norm_weight:
            joint = self.norm_scope == "projection"
            decls["q_norm"] = ParamDecl((self.q_channels if joint else self.d,), "vector")
            if self.own_kv:
                decls["k_norm"] = ParamDecl((self.nkv * self.d if joint else self.d,), "vector")
        if self.sink:
            decls["sink"] = ParamDecl((self.nh,), "vector")
        return decls

    def bind(self, name, tensor):
        super().bind(name, tensor)
        if name in ("qkv_bias", "q_norm", "k_norm", "sink", "o_bias"):
            self.params[name] = tensor.to(torch.float32).contiguous()

    def defer_output_bias(self) -> bool:
        """Asked by a block whose next kernel can add the output projection's bias (``params["o_bias"]``) in float:
        True if there is one, and from then on ``forward`` returns the projection without it."""
        self.bias_deferred = self.out_bias
        return self.bias_deferred

    def cache_spec(self):
        # a chunk's earlier blocks are never read again, but their pages are kept: only a window gives pages back
        return PagedKVSpec(self.nkv, self.d, self.window, self.dv if self.dv != self.d else None)

    def state_spec(self):
        return None

    def _fused_projection(self, tokens: int, x) -> bool:
        """Whether a step of ``tokens`` tokens runs the projection, the rotation, the per-head norm and the cache
        store in ONE few-row kernel (the dense models' fused QKV step, with this part's forms as its options): per-head
        norms, no bias and no gate (the packed matrix holds nothing but heads), keys of its own as wide as the values,
        half-split pairs, a head size that the kernel takes."""
        if not (self.norm_scope == "head" and not self.bias and not self.gate and self.own_kv and self.dv == self.d
                and x.dtype == torch.bfloat16 and ops.few_row_route != "chain"):
            return False
        if self.rope is not None and getattr(self.rope, "pairing", "half_split") != "half_split":
            return False
        return ops.few_row_takes(tokens, self.params["qkv_proj"], self.env.dtype, ops.EPI_QKV, self.d, norm=False)

    def forward(self, x, ctx, cache):
        p = self.params
        tokens = x.shape[0]
        rope = self.rope
        if cache.writes and not self.own_kv:
            raise RuntimeError("a layer without keys of its own must read the cache of another run-list entry")
        if cache.writes and self._fused_projection(tokens, x):
            q = torch.empty((tokens, self.nh * self.d), dtype=x.dtype, device=x.device)
            ops.few_row_linear(x, p["qkv_proj"], ops.EPI_QKV, qkv=dict(
                head_dim=self.d, num_heads=self.nh, num_kv_heads=self.nkv, q_out=q, k_cache=cache.k, v_cache=cache.v,
                q_weight=p.get("q_norm"), k_weight=p.get("k_norm"), eps=float(self.qk_eps or 0.0),
                inv_freq=rope.inv_freq if rope else None, rot_dim=self.rot_dims if rope else 0,
                positions=ctx.positions, slots=ctx.slots[cache.group],
                plain_norm=self.qk_eps is not None and not self.norm_weight,
                norm_after_rotation=self.norm_order == "after_rotation", values_are_keys=self.values_from_keys))
            out = torch.empty((tokens, self.nh * self.dv), dtype=x.dtype, device=x.device)
            _masked_attention(self, q, out, ctx, cache, self.nh, self.nkv, self.d, self.dv,
                              self.zero_sinks if self.zero_sink else p.get("sink"))
            y = ops.linear(out, p["o_proj"])
            if self.out_bias and not self.bias_deferred:
                ops.add_row_bias(y, p["o_bias"])
            return y
        packed = ops.linear(x, p["qkv_proj"])
        q = torch.empty((tokens, self.nh * self.d), dtype=packed.dtype, device=packed.device)
        slots = ctx.slots[cache.group] if cache.writes else None
        prepare = ops.joint_heads_prepare if self.norm_scope == "projection" else ops.heads_prepare
        extra = {"has_kv": self.own_kv} if self.norm_scope == "projection" else \
            {"plain_norm": self.qk_eps is not None and not self.norm_weight,
             "norm_after_rotation": self.norm_order == "after_rotation", "values_are_keys": self.values_from_keys}
        prepare(packed, q, cache.k, cache.v, ctx.positions, slots, self.nh, self.nkv, self.d, self.dv,
                bias=p.get("qkv_bias"), q_weight=p.get("q_norm"), k_weight=p.get("k_norm"),
                eps=float(self.qk_eps or 0.0), inv_freq=rope.inv_freq if rope else None,
                rot_dims=self.rot_dims if rope else 0,
                interleaved=getattr(rope, "pairing", "half_split") == "interleaved", **extra)
        out = torch.empty((tokens, self.nh * self.dv), dtype=packed.dtype, device=packed.device)
        _masked_attention(self, q, out, ctx, cache, self.nh, self.nkv, self.d, self.dv,
                          self.zero_sinks if self.zero_sink else p.get("sink"))
        if self.gate:
            ops.sigmoid_gate_mul(out, packed, self.qkv_channels)
        y = ops.linear(out, p["o_proj"])
        if self.out_bias and not self.bias_deferred:
            ops.add_row_bias(y, p["o_bias"])
        return y


class LatentAttention(Part):
    """Attention whose keys and values are expanded from a narrow latent, so that only the latent is cached.

    One packed projection gives, per head, [``head_dim`` plain | ``rot_dim`` rotated] query coordinates, then the
    down projection [``kv_rank`` latent | ``rot_dim`` rotated key part that all heads share], then the gate rows if
    gated.  The latent c is RMS-normed (``latent_norm``, eps ``eps``); head h's plain key is W_uk[h] c and its value
    W_uv[h] c; score = (q_plain . k_plain + q_rot . k_rot) * scale.  Computed without ever forming a head's keys:

        q_plain . (W_uk[h] c) = (W_uk[h]^T q_plain) . c,        sum_j p_j W_uv[h] c_j = W_uv[h] (sum_j p_j c_j)

    so the cache holds ONE row per token, [c | k_rot] (kv_rank + rot_dim wide, one KV head for all query heads): it
    is the token's key, and its first kv_rank columns are the token's value (no value tensor is kept); a head's query is [W_uk[h]^T q_plain | q_rot] and its output W_uv[h] times the attention's
    result.  ``window``, ``chunk``, ``sink``, ``gate``, ``position_encoding`` / ``rot_dims``: as in
    ``grouped_attention``; ``gate`` "head": one gate a head (heads gate rows instead of heads * v_head_dim).

    ``q_rank`` R: the queries go through a latent of their own.  The packed projection then holds [R query latent |
    kv_rank + rot_dim down projection | gate rows]; the query latent is RMS-normed (``q_latent_norm``, eps ``eps``)
    and ``uq_proj`` [heads * (head_dim + rot_dim), R] gives the heads' query coordinates."""
    category = "mixer"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["num_heads"])
        self.d = int(spec["head_dim"])
        self.r = int(spec["rot_dim"])
        self.dv = int(spec["v_head_dim"])
        self.c = int(spec["kv_rank"])
        self.eps = float(spec["eps"])
        self.window = spec.get("window")
        self.chunk = spec.get("chunk")
        self.scale = float(spec.get("softmax_scale", 1.0 / math.sqrt(self.d + self.r)))
        self.sink = bool(spec.get("sink", False))
        self.gate = bool(spec.get("gate", False))
        self.gate_per_head = spec.get("gate") == "head"
        self.q_rank = int(spec.get("q_rank") or 0)
        if (self.c + self.r) % 2 or self.c % 2 or self.c + self.r > 512:
            raise ValueError("kv_rank and kv_rank + rot_dim must be even and at most 512 (the attention kernels' head sizes)")
        name = spec.get("position_encoding")
        self.rope = env.position_encodings[name] if name else None
        self.rot_dims = int(spec.get("rot_dims") or (self.rope.rot_dim if self.rope else 0))
        if self.rope is not None and (self.rot_dims != self.rope.rot_dim or self.rot_dims > self.r):
            raise ValueError("the rotation does not fit the rotated part or the encoding")
        self.q_channels = self.nh * (self.d + self.r)
        self.down_column = self.q_rank if self.q_rank else self.q_channels
        self.gate_column = self.down_column + self.c + self.r
        self.gate_rows = (self.nh if self.gate_per_head else self.nh * self.dv) if self.gate else 0
        self.uk_t = None

    def param_decls(self):
        rows = self.gate_column + self.gate_rows
        decls = {"qdkv_proj": ParamDecl((rows, self.hidden)), "latent_norm": ParamDecl((self.c,), "vector"),
                 "uk_proj": ParamDecl((self.nh * self.d, self.c)), "uv_proj": ParamDecl((self.nh * self.dv, self.c)),
                 "o_proj": ParamDecl((self.hidden, self.nh * self.dv))}
        if self.sink:
            decls["sink"] = ParamDecl((self.nh,), "vector")
        if self.q_rank:
            decls["q_latent_norm"] = ParamDecl((self.q_rank,), "vector")
            decls["uq_proj"] = ParamDecl((self.q_channels, self.q_rank))
        return decls

    def bind(self, name, tensor):
        super().bind(name, tensor)
        if name in ("latent_norm", "sink", "q_latent_norm"):
            self.params[name] = tensor.to(torch.float32).contiguous()
        elif name == "uk_proj":
            # per head transposed, [heads, kv_rank, head_dim]: the product q_plain W_uk[h] as rows times rows
            self.uk_t = tensor.view(self.nh, self.d, self.c).transpose(1, 2).contiguous()

    def cache_spec(self):
        return PagedKVSpec(1, self.c + self.r, self.window, self.c, shared_values=True)

    def state_spec(self):
        return None

    def forward(self, x, ctx, cache):
        p = self.params
        tokens = x.shape[0]
        rope = self.rope
        packed = ops.linear(x, p["qdkv_proj"])
        if self.q_rank:
            queries = ops.linear(ops.columns_rms_norm(packed, self.q_rank, p["q_latent_norm"], self.eps), p["uq_proj"])
        else:
            queries = packed
        q_plain = queries[:, :self.q_channels].view(tokens, self.nh, self.d + self.r)[:, :, :self.d].transpose(0, 1)
        q_lat = ops.head_products(q_plain, self.uk_t)                                   # [heads, tokens, kv_rank]
        width = self.c + self.r
        q = torch.empty((tokens, self.nh * width), dtype=packed.dtype, device=packed.device)
        slots = ctx.slots[cache.group] if cache.writes else None
        ops.latent_prepare(queries, q_lat, q, cache.k, cache.v, p["latent_norm"], self.eps, ctx.positions, slots,
                           self.nh, self.d, self.r, self.c, inv_freq=rope.inv_freq if rope else None,
                           rot_dims=self.rot_dims if rope else 0,
                           interleaved=getattr(rope, "pairing", "half_split") == "interleaved",
                           down=packed[:, self.down_column:])
        o_lat = torch.empty((tokens, self.nh * self.c), dtype=packed.dtype, device=packed.device)
        _masked_attention(self, q, o_lat, ctx, cache, self.nh, 1, width, self.c, p.get("sink"), shared_values=True)
        out = torch.empty((tokens, self.nh * self.dv), dtype=packed.dtype, device=packed.device)
        ops.head_products(o_lat.view(tokens, self.nh, self.c).transpose(0, 1),
                          p["uv_proj"].view(self.nh, self.dv, self.c),
                          out=out.view(tokens, self.nh, self.dv).transpose(0, 1))
        if self.gate:
            ops.sigmoid_gate_mul(out, packed, self.gate_column, per=self.dv if self.gate_per_head else 1)
        return ops.linear(out, p["o_proj"])


register_part("mixer", "gqa_attention", GQAttention)
register_part("mixer", "grouped_attention", GroupedAttention)
register_part("mixer", "latent_attention", LatentAttention)
register_part("mixer", "gated_conv_attention", GatedConvAttention)
