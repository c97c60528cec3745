"""Arrangements of a layer's parts."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import ParamDecl, Part
from .registry import build_part, register_part


class PreNormDeferredAdd:
    """Pre-norm residual block whose adds are folded into the following norm.

    x = norm_in(h + residual); a = mixer(x); x = norm_post(a + residual);
    h = feed_forward(x).  The feed-forward's output is NOT added here: the next
    block's input norm (or the model's final norm) adds it.  The first block gets
    ``residual is None``: then residual = h and x = norm_in(h).
    Reference: src/models/qwen3/model.rs:424-460, :516-534 and :181-208.
    """
    category = "block"

    def __init__(self, layer_spec, env):
        self.spec = layer_spec
        self.input_norm = build_part("norm", layer_spec["input_norm"], env)
        self.post_mixer_norm = build_part("norm", layer_spec["post_mixer_norm"], env)
        self.mixer = build_part("mixer", layer_spec["mixer"], env)
        self.feed_forward = build_part("feed_forward", layer_spec["feed_forward"], env)

    def children(self):
        return {"input_norm": self.input_norm, "mixer": self.mixer,
                "post_mixer_norm": self.post_mixer_norm, "feed_forward": self.feed_forward}

    @staticmethod
    def _fuses(norm, consumer, tokens):
        """A norm is handed on unrun when it can be (``pending_add``) and its consumer ``takes_pending``."""
        takes = getattr(consumer, "takes_pending", None)
        return hasattr(norm, "pending_add") and takes is not None and takes(tokens)

    @staticmethod
    def _settle(part):
        """Products of few rows may wait to be launched together (``ops.few_row_linear``).  A part that says
        ``chainable = True`` touches activations through ``ops`` alone and may be handed such tensors; before any
        other part runs, everything that waits is launched."""
        if not getattr(part, "chainable", False):
            ops.flush_chain()

    def forward(self, h, residual, ctx, cache):
        tokens = h.shape[0]
        self._settle(self.input_norm)
        self._settle(self.mixer)
        if residual is None:
            residual = h
            if hasattr(self.input_norm, "pending") and self._fuses(self.input_norm, self.mixer, tokens):
                x = self.input_norm.pending(h)
            else:
                x = self.input_norm.forward(h)
        elif self._fuses(self.input_norm, self.mixer, tokens):
            x = self.input_norm.pending_add(h, residual)
            residual = x.residual_out
        else:
            x = self.input_norm.forward_add(h, residual, out=h)
        a = self.mixer.forward(x, ctx, cache)
        self._settle(self.post_mixer_norm)
        self._settle(self.feed_forward)
        if self._fuses(self.post_mixer_norm, self.feed_forward, tokens):
            x = self.post_mixer_norm.pending_add(a, residual)
            residual = x.residual_out
        else:
            x = self.post_mixer_norm.forward_add(a, residual, out=a)
        return self.feed_forward.forward(x), residual


class PreNormInputConv:
    """Pre-norm residual block over a float32 stream whose sublayers read their normed input through a short
    causal convolution over time:

        x <- x + mixer(conv_m(norm_in(x)));    x <- x + feed_forward(conv_f(norm_post(x)))

    The stream x is float32 whatever the engine's dtype, and every sum into it is taken in float.  Parts by name:
    ``input_norm``, ``mixer``, and optionally ``mixer_conv``, and (all or none) ``post_mixer_norm``,
    ``feed_forward``, optionally ``ff_conv``; a layer without a feed-forward has only the first sublayer.  The
    norms hand their scale on (``scale(x, add)``), the convolutions multiply by it as they read.  As in the
    deferred-add block the last sublayer's output is not added here: the block returns (output, stream), and the
    next block's first norm (or the model's final norm) adds it.  Each convolution keeps its last inputs in a
    state of the block's own (``state_specs``), beside the mixer's."""
    category = "block"

    def __init__(self, layer_spec, env):
        self.spec = layer_spec
        self.env = env
        parts = layer_spec.parts
        self.input_norm = build_part("norm", layer_spec["input_norm"], env)
        self.mixer = build_part("mixer", layer_spec["mixer"], env)
        self.mixer_conv = build_part("token_conv", parts["mixer_conv"], env) if "mixer_conv" in parts else None
        self.feed_forward = build_part("feed_forward", parts["feed_forward"], env) if "feed_forward" in parts else None
        self.post_mixer_norm = self.ff_conv = None
        if self.feed_forward is not None:
            self.post_mixer_norm = build_part("norm", layer_spec["post_mixer_norm"], env)
            self.ff_conv = build_part("token_conv", parts["ff_conv"], env) if "ff_conv" in parts else None

    def children(self):
        named = {"input_norm": self.input_norm, "mixer_conv": self.mixer_conv, "mixer": self.mixer,
                 "post_mixer_norm": self.post_mixer_norm, "ff_conv": self.ff_conv, "feed_forward": self.feed_forward}
        return {name: part for name, part in named.items() if part is not None}

    def state_specs(self):
        """Per-request states of the block itself, by name (the mixer's own is asked of the mixer)."""
        specs = {}
        for name, conv in (("mixer_conv", self.mixer_conv), ("ff_conv", self.ff_conv)):
            if conv is not None and conv.state_spec() is not None:
                specs[name] = conv.state_spec()
        return specs

    def _read(self, norm, conv, name, x, add, ctx, cache):
        if conv is not None and hasattr(conv, "forward_after_norm") and hasattr(norm, "eps"):
            # a decode step: add, norm, convolution and state in one kernel
            fused = conv.forward_after_norm(x, add, norm.params["weight"], norm.eps, ctx, cache.states.get(name),
                                            self.env.dtype)
            if fused is not None:
                return fused
        scale = norm.scale(x, add)                     # x += add, in float
        if conv is None:
            return ops.scaled_rows(x, scale, None, self.env.dtype)
        return conv.forward(x, scale, ctx, cache.states.get(name), self.env.dtype)

    def forward(self, h, residual, ctx, cache):
        ops.flush_chain()
        x, add = (h, None) if residual is None else (residual, h)
        y = self.mixer.forward(self._read(self.input_norm, self.mixer_conv, "mixer_conv", x, add, ctx, cache), ctx, cache)
        if self.feed_forward is None:
            return y, x
        y = self.feed_forward.forward(self._read(self.post_mixer_norm, self.ff_conv, "ff_conv", x, y, ctx, cache))
        return y, x


class StreamMix(Part):
    """The coefficients with which one sublayer meets a residual of S streams: ``in`` [S] (what it reads),
    ``out`` [S] (where its output goes) and ``mix`` [S, S] (how the old streams pass on, indexed [from, to]).
    They are kept as one packed float32 vector (in, out, mix).  Without parameters (``fixed``: S = 1) it is
    the ordinary residual sum: in = out = mix = 1."""
    category = "stream_mix"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.streams = int(spec.get("streams", 1))
        self.fixed = bool(spec.get("fixed", False))
        if self.fixed and self.streams != 1:
            raise ValueError("fixed coefficients stand for one stream")
        self.packed = torch.ones(3, dtype=torch.float32, device=env.device) if self.fixed else None

    def param_decls(self):
        if self.fixed:
            return {}
        s = self.streams
        return {"in": ParamDecl((s,), "vector"), "out": ParamDecl((s,), "vector"), "mix": ParamDecl((s, s), "vector")}

    def bind(self, name, tensor):
        super().bind(name, tensor)
        if all(n in self.params for n in ("in", "out", "mix")):
            self.packed = torch.cat([self.params[n].to(torch.float32).reshape(-1) for n in ("in", "out", "mix")]).contiguous()


class MultiStreamPreNorm:
    """Pre-norm block over a residual of S float32 streams ("hyper-connections"; S = 1 with fixed coefficients is
    the ordinary x <- x + sublayer(norm(x))).  For each sublayer q (the mixer, then the feed-forward if the layer
    has one), with its coefficients in_q, out_q, mix_q:

        u = sum_s in_q[s] X_s;    y = sublayer(norm_q(u));    X_t <- sum_s mix_q[s, t] X_s + out_q[t] y   (all t at once)

    The write-back of a sublayer is owed to the next read: the norm part (``stream_rms_norm``) does the write-back
    of the sublayer before, the read and the norm in one kernel, and the block returns (y of its last sublayer,
    the carry with that sublayer's coefficients pending); the next block's first read, or the model's last norm,
    settles it.  Parts by name: ``input_norm``, ``mixer``, ``mixer_mix`` and, all or none, ``post_mixer_norm``,
    ``feed_forward``, ``ff_mix``.  A feed-forward that says ``needs_context`` is also given the step's context."""
    category = "block"

    def __init__(self, layer_spec, env):
        self.spec = layer_spec
        self.env = env
        parts = layer_spec.parts
        self.input_norm = build_part("norm", layer_spec["input_norm"], env)
        self.mixer = build_part("mixer", layer_spec["mixer"], env)
        self.mixer_mix = build_part("stream_mix", layer_spec["mixer_mix"], env)
        self.feed_forward = build_part("feed_forward", parts["feed_forward"], env) if "feed_forward" in parts else None
        self.post_mixer_norm = self.ff_mix = None
        if self.feed_forward is not None:
            self.post_mixer_norm = build_part("norm", layer_spec["post_mixer_norm"], env)
            self.ff_mix = build_part("stream_mix", layer_spec["ff_mix"], env)

    def children(self):
        named = {"input_norm": self.input_norm, "mixer_mix": self.mixer_mix, "mixer": self.mixer,
                 "post_mixer_norm": self.post_mixer_norm, "ff_mix": self.ff_mix, "feed_forward": self.feed_forward}
        return {name: part for name, part in named.items() if part is not None}

    def forward(self, h, residual, ctx, cache):
        ops.flush_chain()
        carry = self.input_norm.open(h) if residual is None else residual
        y = self.mixer.forward(self.input_norm.read(h, carry, self.mixer_mix.packed), ctx, cache)
        carry.pending = self.mixer_mix.packed
        if self.feed_forward is not None:
            x = self.post_mixer_norm.read(y, carry, self.ff_mix.packed)
            y = self.feed_forward.forward(x, ctx) if getattr(self.feed_forward, "needs_context", False) \
                else self.feed_forward.forward(x)
            carry.pending = self.ff_mix.packed
        return y, carry


class PostNormStream:
    """A layer whose norms sit on the sublayers' outputs, over a float32 stream x; the sublayers read x itself:

        x <- x + norm_m(mixer(x));    x <- x + norm_f(feed_forward(x));    x <- x + token_side(x, token ids)

    Parts by name: ``mixer`` and ``mixer_norm``; all or none of ``feed_forward`` and ``ff_norm``; optionally
    ``token_side`` (a per-layer read of a second token table that brings its own norm).  The norms are
    ``output_rms_norm``: each add is one kernel that also hands on the new x rounded to the engine's dtype, which the
    next sublayer's products read (the block passes it on as ``residual``; the stream itself is ``h``).  A mixer that
    has an output bias and offers ``defer_output_bias()`` leaves the bias to that kernel.  A feed-forward that says
    ``needs_context`` is also given the step's context."""
    category = "block"

    def __init__(self, layer_spec, env):
        self.spec = layer_spec
        self.env = env
        parts = layer_spec.parts
        self.mixer = build_part("mixer", layer_spec["mixer"], env)
        self.mixer_norm = build_part("norm", layer_spec["mixer_norm"], env)
        self.feed_forward = build_part("feed_forward", parts["feed_forward"], env) if "feed_forward" in parts else None
        self.ff_norm = build_part("norm", layer_spec["ff_norm"], env) if self.feed_forward is not None else None
        self.token_side = build_part("token_side", parts["token_side"], env) if "token_side" in parts else None
        for norm in (self.mixer_norm, self.ff_norm):
            if norm is not None and not hasattr(norm, "add_into"):
                raise ValueError("this block needs norms that add into the stream (output_rms_norm)")
        defer = getattr(self.mixer, "defer_output_bias", None)
        self.mixer_bias_here = bool(defer()) if defer is not None else False

    def children(self):
        named = {"mixer": self.mixer, "mixer_norm": self.mixer_norm, "feed_forward": self.feed_forward,
                 "ff_norm": self.ff_norm, "token_side": self.token_side}
        return {name: part for name, part in named.items() if part is not None}

    def forward(self, h, residual, ctx, cache):
        ops.flush_chain()
        x = ops.cast(h, self.env.dtype) if residual is None else residual
        y = self.mixer.forward(x, ctx, cache)
        x = self.mixer_norm.add_into(h, y, bias=self.mixer.params.get("o_bias") if self.mixer_bias_here else None)
        if self.feed_forward is not None:
            y = self.feed_forward.forward(x, ctx) if getattr(self.feed_forward, "needs_context", False) \
                else self.feed_forward.forward(x)
            x = self.ff_norm.add_into(h, y)
        if self.token_side is not None:
            x = self.token_side.add_into(h, x, ctx)
        return h, x


register_part("stream_mix", "stream_mix", StreamMix)
register_part("block", "post_norm_stream", PostNormStream)
register_part("block", "pre_norm_deferred_add", PreNormDeferredAdd)
register_part("block", "multi_stream_pre_norm", MultiStreamPreNorm)
register_part("block", "pre_norm_input_conv", PreNormInputConv)
