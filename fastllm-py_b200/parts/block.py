"""Block arrangements: how a layer's mixer, feed-forward and norms are wired.

"prenorm" is the Llama layer (fastllm_py/model.py:464-470):
    x = x + mixer(norm_mixer(x));  x = x + feed_forward(norm_ff(x))
The sums are left pending on the residual stream and folded into the next norm.  With `residual_scale`
m both sums are multiplied by m as they are added, and the layer may have no feed-forward.

"sandwich" norms each sublayer on both sides:
    x = x + norm_mixer_out(mixer(norm_mixer_in(x)));  x = x + norm_ff_out(ff(norm_ff_in(x)))
and may have no feed-forward at all.  The sublayer's output is left pending with
its norm; the next norm of the stream does norm, add and norm in one kernel.

"parallel" runs mixer and feed-forward side by side on the same x, each behind a norm of its own:
    x = x + mixer(norm_mixer(x)) + feed_forward(norm_ff(x))
and may have no feed-forward.  Both outputs are left pending; the next layer's two norms share
the row's root mean square, so one kernel adds both sums and writes both normed rows.
"""
from __future__ import annotations

import torch

from .base import Part
from .registry import build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Part):
    """norm roles: "mixer" and, with a feed-forward, "feed_forward".  params: residual_scale (1)."""
    category = "block"

    def __init__(self, layer_spec, ctx):
        super().__init__(layer_spec, ctx)
        self.mixer = build_part("mixer", layer_spec.mixer, ctx)
        self.norm_mixer = build_part("norm", layer_spec.norms["mixer"], ctx)
        self.feed_forward = self.norm_ff = None
        if layer_spec.feed_forward is not None:
            self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, ctx)
            self.norm_ff = build_part("norm", layer_spec.norms["feed_forward"], ctx)
        self.hidden = self.norm_mixer.size
        self.scale = float(layer_spec.params.get("residual_scale", 1.0))

    def children(self):
        parts = [self.mixer, self.norm_mixer]
        if self.feed_forward is not None:
            parts += [self.feed_forward, self.norm_ff]
        return parts

    def forward(self, stream, step, cache):
        n = stream.x.shape[0]
        dt = self.ctx.dtype
        h = step.workspace.rows("normed", n, self.hidden, dt)
        delta = step.workspace.rows("delta", n, self.hidden, dt)
        # a mixer or feed-forward returns None when it wrote `delta`, or the
        # split-K partial sums of its last product, which the next norm adds up
        stream.norm_into(self.norm_mixer, h)
        left = self.mixer.forward(h, delta, step, cache)
        stream.pending, stream.pending_scale = (delta if left is None else left), self.scale
        if self.feed_forward is None:
            return
        stream.norm_into(self.norm_ff, h)
        left = self.feed_forward.forward(h, delta, step)
        stream.pending, stream.pending_scale = (delta if left is None else left), self.scale


@register_part("block", "sandwich")
class SandwichBlock(Part):
    """norm roles: "mixer_in", "mixer_out" and, with a feed-forward, "ff_in", "ff_out"."""
    category = "block"

    def __init__(self, layer_spec, ctx):
        super().__init__(layer_spec, ctx)
        self.mixer = build_part("mixer", layer_spec.mixer, ctx)
        self.norm_mixer_in = build_part("norm", layer_spec.norms["mixer_in"], ctx)
        self.norm_mixer_out = build_part("norm", layer_spec.norms["mixer_out"], ctx)
        self.feed_forward = self.norm_ff_in = self.norm_ff_out = None
        if layer_spec.feed_forward is not None:
            self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, ctx)
            self.norm_ff_in = build_part("norm", layer_spec.norms["ff_in"], ctx)
            self.norm_ff_out = build_part("norm", layer_spec.norms["ff_out"], ctx)
        self.hidden = self.norm_mixer_in.size

    def children(self):
        parts = [self.mixer, self.norm_mixer_in, self.norm_mixer_out]
        if self.feed_forward is not None:
            parts += [self.feed_forward, self.norm_ff_in, self.norm_ff_out]
        return parts

    def forward(self, stream, step, cache):
        n = stream.x.shape[0]
        dt = self.ctx.dtype
        h = step.workspace.rows("normed", n, self.hidden, dt)
        delta = step.workspace.rows("delta", n, self.hidden, dt)
        stream.norm_into(self.norm_mixer_in, h)
        left = self.mixer.forward(h, delta, step, cache)
        stream.pending, stream.pending_norm = (delta if left is None else left), self.norm_mixer_out
        if self.feed_forward is not None:
            stream.norm_into(self.norm_ff_in, h)
            left = self.feed_forward.forward(h, delta, step)
            stream.pending, stream.pending_norm = (delta if left is None else left), self.norm_ff_out


@register_part("block", "parallel")
class ParallelBlock(Part):
    """norm roles: "mixer" and, with a feed-forward, "feed_forward"."""
    category = "block"

    def __init__(self, layer_spec, ctx):
        super().__init__(layer_spec, ctx)
        self.mixer = build_part("mixer", layer_spec.mixer, ctx)
        self.norm_mixer = build_part("norm", layer_spec.norms["mixer"], ctx)
        self.feed_forward = self.norm_ff = None
        if layer_spec.feed_forward is not None:
            self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, ctx)
            self.norm_ff = build_part("norm", layer_spec.norms["feed_forward"], ctx)
        self.hidden = self.norm_mixer.size

    def children(self):
        parts = [self.mixer, self.norm_mixer]
        if self.feed_forward is not None:
            parts += [self.feed_forward, self.norm_ff]
        return parts

    def forward(self, stream, step, cache):
        n = stream.x.shape[0]
        dt = self.ctx.dtype
        ws = step.workspace
        h = ws.rows("normed", n, self.hidden, dt)
        delta = ws.rows("delta", n, self.hidden, dt)
        if self.feed_forward is None:
            stream.norm_into(self.norm_mixer, h)
        else:
            h_ff = ws.rows("normed_ff", n, self.hidden, dt)
            pairs = getattr(self.norm_mixer, "pairs_with", None)
            if pairs is not None and pairs(self.norm_ff) and stream.pending_norm is None:
                if stream.pending is not None and not isinstance(stream.pending, torch.Tensor):
                    stream.pending = stream.pending.reduce_into(stream.spill())
                self.norm_mixer.apply_pair(stream, self.norm_ff, h, h_ff)
            else:
                stream.norm_into(self.norm_mixer, h)          # adds what was pending
                stream.norm_into(self.norm_ff, h_ff)
        # the split-K scratch is shared: partial sums are added up before the other sublayer's products run
        left = self.mixer.forward(h, delta, step, cache)
        if left is not None:
            left.reduce_into(delta)
        stream.pending = delta
        if self.feed_forward is not None:
            delta_ff = ws.rows("delta_ff", n, self.hidden, dt)
            left = self.feed_forward.forward(h_ff, delta_ff, step)
            if left is not None:
                left.reduce_into(delta_ff)
            stream.extra = delta_ff


@register_part("block", "gated_postnorm")
class GatedPostNormBlock(Part):
    """A layer whose sublayers read the residual stream itself and are normed on their OUTPUT only:
        h = x;  hc = h + conv(h);  x <- x + norm_out(sublayer(hc) * sigmoid(W_gate h + b_gate))
    for the mixer and then (if the layer has one) the feed-forward.  conv is a causal convolution over time on each
    channel with `taps` taps (no bias; zeros before the sequence's start), whose last taps - 1 input rows per
    sublayer are per-request state, filed by position; the gate reads h as it was before the convolution.
    params: hidden_size, taps (0: no convolution), gate (bool).  norm roles: "mixer_out" and, with a feed-forward,
    "ff_out".  tensors: conv_mixer, conv_ff [hidden, taps]; gate_mixer, gate_ff [hidden, hidden] with
    gate_mixer_bias, gate_ff_bias [hidden]."""
    category = "block"
    native_libraries = ("gated_block",)

    def __init__(self, layer_spec, ctx):
        super().__init__(layer_spec, ctx)
        p = layer_spec.params
        self.hidden = int(p["hidden_size"])
        self.taps = int(p.get("taps") or 0)
        self.gated = bool(p.get("gate", True))
        self.mixer = build_part("mixer", layer_spec.mixer, ctx)
        self.norm_mixer_out = build_part("norm", layer_spec.norms["mixer_out"], ctx)
        self.feed_forward = self.norm_ff_out = None
        if layer_spec.feed_forward is not None:
            self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, ctx)
            self.norm_ff_out = build_part("norm", layer_spec.norms["ff_out"], ctx)
        self.subs = ["mixer"] + (["ff"] if self.feed_forward is not None else [])
        self.conv, self.gate, self.gate_bias, self._w_out = {}, {}, {}, {}

    def children(self):
        parts = [self.mixer, self.norm_mixer_out]
        if self.feed_forward is not None:
            parts += [self.feed_forward, self.norm_ff_out]
        return parts

    def weight_shapes(self):
        shapes = {}
        for s in self.subs:
            if self.taps:
                shapes[f"conv_{s}"] = (self.hidden, self.taps)
            if self.gated:
                shapes[f"gate_{s}"] = (self.hidden, self.hidden)
                shapes[f"gate_{s}_bias"] = (self.hidden,)
        return shapes

    def load(self, tensors):
        from .linear import Linear
        for s in self.subs:
            if self.taps:
                self.conv[s] = tensors[f"conv_{s}"].float().contiguous()
            else:                                             # one tap of weight zero: hc = h
                self.conv[s] = torch.zeros((self.hidden, 1), dtype=torch.float32, device=self.ctx.device)
            if self.gated:
                self.gate[s] = Linear([tensors[f"gate_{s}"]])
                self.gate_bias[s] = tensors[f"gate_{s}_bias"].float().contiguous()

    def state_need(self):
        from ..cache.needs import FixedState
        back = self.taps - 1
        return FixedState((len(self.subs) * back * self.hidden,), "float32") if back > 0 else None

    def reserve(self, limits):
        for lin in self.gate.values():
            lin.reserve(self.ctx.dtype, limits.max_tokens, side=True)

    def _out_weight(self, s, norm):
        w = self._w_out.get(s)
        if w is None:
            w = self._w_out[s] = norm.weight.float().contiguous()
        return w

    def _sublayer(self, s, index, norm, run, stream, step, state):
        from ..native import ops
        n = stream.x.shape[0]
        dt = self.ctx.dtype
        ws = step.workspace
        taps = max(self.taps, 1)
        ring = None
        if taps > 1:
            span = (taps - 1) * self.hidden
            ring = state.tensor[:, index * span:(index + 1) * span]
        h = ws.rows("normed", n, self.hidden, dt) if self.gated else None
        hc = ws.rows("conv_in", n, self.hidden, dt)
        ops.input_conv(stream.x, self.conv[s], taps, ring, step, h, hc)
        gate = None
        if self.gated:
            # before the sublayer, into the second scratch buffer: both this product and the sublayer's last one may
            # then stay split-K partial sums until the kernel below adds them up
            gate = ws.rows("branch_gate", n, self.hidden, dt)
            gate = self.gate[s].forward(h, gate, defer=True, side=True) or gate
        delta = ws.rows("delta", n, self.hidden, dt)
        left = run(hc, delta)
        ops.gated_norm_add(stream.x, delta if left is None else left, gate, self.gate_bias.get(s),
                           self._out_weight(s, norm), norm.eps, step, ring, taps, dtype=dt)

    def forward(self, stream, step, cache, state=None):
        stream.settle()                                       # the sublayers read x itself
        self._sublayer("mixer", 0, self.norm_mixer_out, lambda hc, out: self.mixer.forward(hc, out, step, cache),
                       stream, step, state)
        if self.feed_forward is not None:
            self._sublayer("ff", 1, self.norm_ff_out, lambda hc, out: self.feed_forward.forward(hc, out, step),
                           stream, step, state)
