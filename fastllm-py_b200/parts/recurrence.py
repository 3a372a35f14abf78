"""Gated recurrence mixer: a linear recurrence per channel with gates made from the input (the
real-gated linear recurrent unit), between a gate branch and an input branch.

    y = gelu_tanh(W_y h + b_y)                                 gate branch, `width` channels
    u = conv(W_x h + b_x)                                      causal convolution per channel, `taps` taps, with bias
    r = sigmoid(A_b u_b + a_b),  i = sigmoid(I_b u_b + i_b)    per block b of width / blocks channels
    a = exp(-rate * r * softplus(lam))                         `rate` 8 unless given
    S <- a S + sqrt(1 - a^2) * i * u;     out = W_o (S * y)

One stacked matrix serves y | x.  The request's state row holds S and the convolution's last taps - 1
inputs; it is float and carried from step to step by the cache manager's state slots.  Everything
after the projection is float: the convolution, the block products of the gates, decays, the state.
"""
from __future__ import annotations

import torch

from ..cache.needs import FixedState
from ..native import ops
from .base import Part
from .linear import Linear
from .registry import register_part


@register_part("mixer", "gated_recurrence")
class GatedRecurrence(Part):
    """params: hidden_size, width, blocks, taps, rate (8.0).  tensors: y, x [width, hidden] with y_bias, x_bias [width];
    conv [width, taps], conv_bias [width]; gate_a, gate_i [blocks, width / blocks, width / blocks] with gate_a_bias,
    gate_i_bias [blocks, width / blocks]; lam [width]; o [hidden, width]."""
    category = "mixer"
    native_libraries = ("rglru",)

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden, self.width = int(p["hidden_size"]), int(p["width"])
        self.blocks, self.taps = int(p["blocks"]), int(p["taps"])
        self.rate = float(p.get("rate", 8.0))
        if self.width % self.blocks:
            raise ValueError(f"gated_recurrence: {self.blocks} blocks do not divide the width {self.width}")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"gated_recurrence: {self.taps} taps are beyond the kernels' 16")
        if (self.width // self.blocks) * 16 * 4 > 48 * 1024:
            raise ValueError(f"gated_recurrence: blocks of {self.width // self.blocks} channels exceed the kernel's 768")
        self.proj = self.o = None

    def cache_need(self):
        return FixedState((self.width * self.taps,), "float32")

    def weight_shapes(self):
        w, bw = self.width, self.width // self.blocks
        return {"y": (w, self.hidden), "x": (w, self.hidden), "y_bias": (w,), "x_bias": (w,), "conv": (w, self.taps),
                "conv_bias": (w,), "gate_a": (self.blocks, bw, bw), "gate_i": (self.blocks, bw, bw),
                "gate_a_bias": (self.blocks, bw), "gate_i_bias": (self.blocks, bw), "lam": (w,), "o": (self.hidden, w)}

    def load(self, tensors):
        if tensors["y"].dtype != tensors["x"].dtype:
            raise ValueError("gated_recurrence: the two branches' matrices must be stored in one dtype")
        self.proj = Linear([tensors["y"], tensors["x"]])
        self.o = Linear([tensors["o"]])
        self.bias = torch.cat([tensors["y_bias"].float(), tensors["x_bias"].float()]).contiguous()
        self.conv_w = tensors["conv"].float().contiguous()
        self.conv_b = tensors["conv_bias"].float().contiguous()
        self.gate_a = tensors["gate_a"].contiguous()
        self.gate_i = tensors["gate_i"].to(self.gate_a.dtype).contiguous()
        self.gate_a_bias = tensors["gate_a_bias"].float().reshape(-1).contiguous()
        self.gate_i_bias = tensors["gate_i_bias"].float().reshape(-1).contiguous()
        # the exponent's factor per channel, formed in double and rounded once
        self.rate_c = (-self.rate * torch.nn.functional.softplus(tensors["lam"].double())).float().contiguous()

    def reserve(self, limits):
        for lin in (self.proj, self.o):
            if lin is not None:
                lin.reserve(self.ctx.dtype, limits.max_tokens)

    def forward(self, h, out, step, cache):
        n = h.shape[0]
        dt = self.ctx.dtype
        ws = step.workspace
        proj = ws.rows("recurrence_proj", n, 2 * self.width, dt)
        self.proj.forward(h, proj)
        u = ws.rows("recurrence_u", n, self.width, torch.float32)
        a = ws.rows("recurrence_a", n, self.width, torch.float32)
        bx = ws.rows("recurrence_bx", n, self.width, torch.float32)
        gated = ws.rows("recurrence_out", n, self.width, dt)
        ops.rglru(proj, self.bias, self.conv_w, self.conv_b, self.gate_a, self.gate_i, self.gate_a_bias, self.gate_i_bias,
                  self.rate_c, cache.tensor, step, u, a, bx, gated, self.width, self.blocks, self.taps,
                  fixed_order=dt == torch.float32)        # the 32-bit path: cuts and batches agree bit for bit
        return self.o.forward(gated, out, defer=True)
