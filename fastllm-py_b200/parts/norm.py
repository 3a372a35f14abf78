"""RMSNorm: x * (mean(x^2) + eps)^-1/2 * w, eps inside the root, the weight
multiplies (no "+1").  fastllm_py/kernels/ops.py:19-27; the fused
residual-add form is fastllm_py/graph_decode.py:300-324."""
from __future__ import annotations

import torch

from ..native import ops
from .base import Part
from .registry import register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """params: size, eps.  tensors: weight [size]."""
    category = "norm"
    takes_partial = True                 # split-K partial sums are added while the row is read
    takes_post_norm = True               # a pending sum that passes another RMSNorm first: one kernel does both
    takes_extra = True                   # two tensors pending: both are added while the row is read

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    def weight_shapes(self):
        return {"weight": (self.size,)}

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def apply(self, stream, out, rows=None):
        """Norm the residual stream into `out`, adding the pending sum first.
        With `rows` (int32 indices) only those rows are normed, into out[0..m), and the
        pending sum (a tensor then: `ResidualStream.norm_into` sees to it) stays pending."""
        post = getattr(stream, "pending_norm", None)
        if getattr(stream, "extra", None) is not None:
            # two sums pending (tensors; `ResidualStream.norm_into` sees to it): x += pending + extra; out = self(x)
            ops.norm_pair(stream.x, stream.pending, stream.extra, self.weight, None, out, None, self.eps, rows)
            if rows is None:
                stream.pending = stream.extra = None
            return
        if stream.pending is not None and post is not None:
            # x += post(pending); out = self(x): the layer norms the sublayer's output before adding it
            if not isinstance(stream.pending, torch.Tensor):         # split-K partial sums (never with rows)
                ops.sandwich_norm_partial(stream.x, stream.pending, post.weight, post.eps, self.weight, self.eps, out)
            else:
                ops.sandwich_norm(stream.x, stream.pending, post.weight, post.eps, self.weight, self.eps, out, rows)
            if rows is None:
                stream.pending = stream.pending_norm = None
            return
        if stream.pending is not None:
            if not isinstance(stream.pending, torch.Tensor):         # split-K partial sums
                if rows is not None:
                    raise RuntimeError("a gathered norm cannot take partial sums")
                ops.add_rmsnorm_partial(stream.x, stream.pending, self.weight, out, self.eps)
                stream.pending = None
                return
            ops.add_rmsnorm(stream.x, stream.pending, self.weight, out, self.eps, rows)
            if rows is None:
                stream.pending = None
        else:
            ops.rmsnorm(stream.x, self.weight, out, self.eps, rows)

    def add_normed(self, stream):
        """stream.x += rmsnorm(stream.pending) * weight: this part as the norm of a sublayer's output."""
        ops.sandwich_norm(stream.x, stream.pending, self.weight, self.eps, None, 0.0, None)
        stream.pending = stream.pending_norm = None

    def pairs_with(self, other) -> bool:
        """Whether `apply_pair` can norm a row for this part and `other` at once."""
        return isinstance(other, RMSNorm) and other.size == self.size and other.eps == self.eps and \
            other.weight.dtype == self.weight.dtype

    def apply_pair(self, stream, other, out, out_other):
        """x += pending (+ extra); out = self(x), out_other = other(x): the two norms share the row's root
        mean square, so one pass serves both.  The pending sum must be a tensor (or none) without a norm of its own."""
        ops.norm_pair(stream.x, stream.pending, stream.extra, self.weight, other.weight, out, out_other, self.eps)
        stream.pending = stream.extra = None


@register_part("norm", "layernorm")
class LayerNorm(Part):
    """(x - mean) / sqrt(var + eps) * weight + bias, the variance being the mean of the squared deviations.
    params: size, eps, bias (True).  tensors: weight [size] and, with bias, bias [size].  Adds the stream's pending
    sum, multiplied by the stream's `pending_scale`, while it reads."""
    category = "norm"
    native_libraries = ("norm_mix",)
    takes_scale = True                   # the pending sum times a number: added while the row is read
    takes_partial = True                 # split-K partial sums are added while the row is read
    PARTIAL_FROM = 64                    # ... in steps of this many rows and more: one block reads a row's slabs, which
                                         # for a handful of rows is slower than the reduce kernel's many blocks

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.has_bias = bool(spec.params.get("bias", True))
        self.weight = self.bias = None

    def weight_shapes(self):
        shapes = {"weight": (self.size,)}
        if self.has_bias:
            shapes["bias"] = (self.size,)
        return shapes

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()
        if self.has_bias:
            self.bias = tensors["bias"].to(self.weight.dtype).contiguous()

    def apply(self, stream, out, rows=None):
        """Norm the residual stream into `out`, adding the pending sum (a tensor, or split-K partial sums) first.
        With `rows` only those rows are normed, into out[0..m), and the pending sum (a tensor then:
        `ResidualStream.norm_into` sees to it) stays pending."""
        if stream.pending is not None and not isinstance(stream.pending, torch.Tensor) and \
                stream.x.shape[0] < self.PARTIAL_FROM:
            stream.pending = stream.pending.reduce_into(stream.spill())
        ops.add_layernorm(stream.x, stream.pending, stream.pending_scale, self.weight, self.bias, out, self.eps, rows)
        if rows is None:
            stream.pending, stream.pending_scale = None, 1.0


@register_part("norm", "rmsnorm_scalar")
class ScalarRMSNorm(RMSNorm):
    """RMSNorm whose weight is ONE stored number g for all coordinates: x * (mean(x^2) + eps)^-1/2 * g.
    With a `scale` tensor (one factor per coordinate applied to the normed row, a layer scale) the two are one
    vector, g * scale, formed in float32 at load; every kernel of RMSNorm then serves.
    params: size, eps.  tensors: weight [] and, optionally, scale [size]."""

    def weight_shapes(self):
        shapes = {"weight": ()}
        if "scale" in self.spec.tensors:
            shapes["scale"] = (self.size,)
        return shapes

    def load(self, tensors):
        g = tensors["weight"].float().reshape(1)
        if "scale" in tensors:
            self.weight = (g * tensors["scale"].float()).contiguous()
        else:
            self.weight = g.expand(self.size).contiguous()
