"""RMSNorm with an optional fused residual add."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import ParamDecl, Part
from .registry import register_part


class RMSNorm(Part):
    """y = x * rsqrt(mean(x^2) + eps) * weight, in float, rounded once.

    ``forward_add`` adds a residual first: the float sum is normalised unrounded
    and stored rounded as the new residual (reference: src/layers/ops.rs:8-35,
    src/layers/fused_ops.cu:49-106).
    """
    category = "norm"
    chainable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.width = int(spec["width"])
        self.eps = float(spec["eps"])

    def param_decls(self):
        return {"weight": ParamDecl((self.width,), "vector")}

    def forward(self, x, out=None, rows=None):
        return ops.rms_norm(x, self.params["weight"], self.eps, out=out, rows=rows)

    def forward_add(self, x, residual, out=None, rows=None, write_residual=True):
        return ops.add_rms_norm(x, residual, self.params["weight"], self.eps, out=out, rows=rows,
                                write_residual=write_residual)

    def pending_add(self, x, residual, rows=None, write_residual=True):
        """The same add + norm, not run yet: a consumer that ``takes_pending`` fuses it into its product.
        The new residual will be in ``.residual_out`` of the result (``residual`` itself is left alone)."""
        return ops.PendingNorm(x, residual, self.params["weight"], self.eps, rows=rows,
                               write_residual=write_residual)


    def pending(self, x, rows=None):
        """The plain norm of ``x``, not run yet (for a consumer that ``takes_pending``)."""
        return ops.PendingNorm(x, None, self.params["weight"], self.eps, rows=rows, write_residual=False)


class ScalarRMSNorm(Part):
    """y = x / sqrt(mean(x^2) + eps) * g with ONE gain g for all coordinates, over a float32 stream.

    The norm is handed on as a per-token scale (``scale``: g / sqrt(mean(x^2) + eps), float32 [tokens]), so that
    whatever reads the normed vector next (a convolution over time, a row gather for the head) multiplies as
    it reads; ``scale`` can add a sublayer's output to the stream first, the sum in float.  ``forward`` is the
    norm itself for chosen rows, rounded once to the engine's dtype."""
    category = "norm"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.eps = float(spec["eps"])

    def param_decls(self):
        return {"weight": ParamDecl((), "vector")}

    def bind(self, name, tensor):
        super().bind(name, tensor)
        self.params[name] = tensor.to(torch.float32).reshape(1).contiguous()

    def scale(self, x, add=None):
        return ops.residual_scale(x, add, self.params["weight"], self.eps)

    def forward(self, x, out=None, rows=None):
        return ops.scaled_rows(x, self.scale(x), rows, self.env.dtype)

    def forward_add(self, x, residual, out=None, rows=None, write_residual=True):
        """The norm of residual + x for chosen rows; the sum stays in ``residual`` (the float32 stream)."""
        return ops.scaled_rows(residual, self.scale(residual, x), rows, self.env.dtype)


class StreamCarry:
    """A residual held as S float32 streams [tokens, S, width], with the write-back that is still owed to it:
    ``pending`` holds the packed coefficients (in, out, mix) of the sublayer whose output comes with the next read.
    ``start``: the streams do not exist yet and begin as copies of this [tokens, width] float32 tensor."""

    def __init__(self, streams, start=None):
        self.streams = streams
        self.start = start
        self.pending = None


class StreamRMSNorm(Part):
    """RMS norm that reads a residual of S float32 streams (``streams``; 1: the ordinary residual sum).

    ``read(y, carry, coefficients)``: the write-back that ``carry`` still owes (X_t <- sum_s mix[s, t] X_s + out[t] y,
    with the coefficients of the sublayer that produced ``y``), then u = sum_s in[s] X_s with the reading sublayer's
    ``in``, then u / sqrt(mean(u^2) + eps) * (weight + offset), rounded once to the engine's dtype: one kernel.
    ``offset`` 1 is a weight stored around zero.  ``forward_add`` is the model's last read: in = 1 (the sum of the
    streams), chosen rows, nothing stored."""
    category = "norm"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.width = int(spec["width"])
        self.eps = float(spec["eps"])
        self.offset = float(spec.get("offset", 0.0))
        self.streams = int(spec.get("streams", 1))
        if not 1 <= self.streams <= ops.MAX_STREAMS:
            raise ValueError(f"{self.streams} streams are refused: the kernel takes 1 to {ops.MAX_STREAMS}")

    def param_decls(self):
        return {"weight": ParamDecl((self.width,), "vector")}

    def bind(self, name, tensor):
        super().bind(name, tensor)
        self.params[name] = tensor.to(torch.float32).contiguous()

    def open(self, h):
        """A carry whose streams begin as copies of ``h`` (float32 [tokens, width])."""
        streams = torch.empty((h.shape[0], self.streams, self.width), dtype=torch.float32, device=h.device)
        return StreamCarry(streams, start=h)

    def read(self, y, carry, coefficients, rows=None, store=True):
        read_in = None if coefficients is None else coefficients[:self.streams]
        out = ops.stream_step(carry.streams, self.params["weight"], self.offset, self.eps, self.env.dtype,
                              start=carry.start, y=y if carry.start is None else None,
                              before=carry.pending if carry.start is None else None, read_in=read_in, rows=rows,
                              store=store)
        if store:
            carry.start, carry.pending = None, None
        return out

    def forward(self, x, out=None, rows=None):
        """The norm of a plain float32 [tokens, width] tensor (a model of one layer-less stream)."""
        carry = self.open(x)
        return self.read(None, carry, None, rows=rows, store=False)

    def forward_add(self, x, residual, out=None, rows=None, write_residual=True):
        return self.read(x, residual, None, rows=rows, store=write_residual)


class OutputRMSNorm(Part):
    """RMS norm on a sublayer's OUTPUT, for a residual stream that is float32 whatever the engine's dtype:

        ``add_into(stream, y)``:  stream <- stream + (y + bias) / sqrt(mean((y + bias)^2) + eps) * weight

    in float and in place, one kernel; it returns the new stream rounded once to the engine's dtype (the stream itself
    in a float32 engine), which is what the next sublayer's first product reads.  ``bias`` (float32, per column) is an
    output projection's bias that its owner left to this kernel.  ``forward`` / ``forward_add`` are the plain norm of
    the stream itself at chosen rows (a model's last norm); ``forward_add`` is handed the rounded copy that the blocks
    pass on as ``residual`` and does not need it."""
    category = "norm"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.width = int(spec["width"])
        self.eps = float(spec["eps"])

    def param_decls(self):
        return {"weight": ParamDecl((self.width,), "vector")}

    def bind(self, name, tensor):
        super().bind(name, tensor)
        self.params[name] = tensor.to(torch.float32).contiguous()

    def add_into(self, stream, y, bias=None):
        return ops.norm_add(stream, y, self.params["weight"], self.eps, bias=bias, cast_to=self.env.dtype)

    def forward(self, x, out=None, rows=None):
        return ops.norm_rows(x, self.params["weight"], self.eps, self.env.dtype, rows=rows)

    def forward_add(self, x, residual, out=None, rows=None, write_residual=True):
        return ops.norm_rows(x, self.params["weight"], self.eps, self.env.dtype, rows=rows)


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "output_rms_norm", OutputRMSNorm)
register_part("norm", "stream_rms_norm", StreamRMSNorm)
register_part("norm", "scalar_rms_norm", ScalarRMSNorm)
