"""Gated linear attention mixer: linear attention whose state decays per key channel by a number
made from the token; no softmax and no denominator.

For a head with state S [dim x vdim] (float, one per request, zero at the start):

    alpha = sigmoid(W_a2 (W_a1 h) + b_a2)^(1 / tau)            one number per head and key channel
    S <- diag(alpha) S + k v^T;   o = S^T (q * q_scale)        q_scale dim^-1/2 unless given

q, k (`heads` x `dim`) and v (`heads` x `vdim`) are projections of the input.  Each head's o is divided by
its root mean square over vdim and multiplied by a weight [vdim] that the heads share; the heads are
concatenated, multiplied by silu(W_g h) and projected by W_o.

One stacked matrix serves q | k | v | gate | the decay's low-rank input; the small second matrix of the
decay is applied in float by the preparing kernel.  The request's state row holds S for every head; it
is float and carried from step to step by the cache manager's state slots.  Everything after the
projection is float.
"""
from __future__ import annotations

import torch

from ..cache.needs import FixedState
from ..native import ops
from .base import Part
from .linear import Linear
from .registry import register_part


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Part):
    """params: hidden_size, heads, dim, vdim, tau, norm_eps, q_scale (None: dim^-1/2).  tensors: q, k [heads * dim, hidden],
    v, g [heads * vdim, hidden], a1 [rank, hidden], a2 [heads * dim, rank], a2_bias [heads * dim], norm [vdim],
    o [hidden, heads * vdim]; `rank` is a1's row count, a parameter too."""
    category = "mixer"
    native_libraries = ("gla",)

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim, self.vdim = int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.rank = int(p["rank"])
        self.tau = float(p["tau"])
        self.norm_eps = float(p["norm_eps"])
        self.q_scale = float(p["q_scale"]) if p.get("q_scale") is not None else self.dim ** -0.5
        if self.dim > 256:
            raise ValueError(f"gated_linear_attention: dim {self.dim} is beyond the scan kernel's limit of 256")
        self.hd, self.hv = self.heads * self.dim, self.heads * self.vdim
        self.proj_cols = 2 * self.hd + 2 * self.hv + self.rank          # q | k | v | gate | low
        self.proj = self.o = None

    def cache_need(self):
        return FixedState((self.heads * self.vdim * self.dim,), "float32")

    def weight_shapes(self):
        w = self.hidden
        return {"q": (self.hd, w), "k": (self.hd, w), "v": (self.hv, w), "g": (self.hv, w), "a1": (self.rank, w),
                "a2": (self.hd, self.rank), "a2_bias": (self.hd,), "norm": (self.vdim,), "o": (w, self.hv)}

    def load(self, tensors):
        mats = [tensors[s] for s in ("q", "k", "v", "g", "a1")]
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("gated_linear_attention: the projections must be stored in one dtype")
        self.proj = Linear(mats)
        self.o = Linear([tensors["o"]])
        self.a2 = tensors["a2"].float().t().contiguous()               # [rank, heads * dim]: the kernel reads along heads * dim
        self.a2_bias = tensors["a2_bias"].float().contiguous()
        self.norm_w = tensors["norm"].contiguous()

    def reserve(self, limits):
        for lin in (self.proj, self.o):
            if lin is not None:
                lin.reserve(self.ctx.dtype, limits.max_tokens)

    def forward(self, h, out, step, cache):
        n = h.shape[0]
        dt = self.ctx.dtype
        ws = step.workspace
        proj = ws.rows("gla_proj", n, self.proj_cols, dt)
        self.proj.forward(h, proj)
        work = ws.rows("gla_work", n, 3 * self.hd + self.hv, torch.float32)
        ops.gla_prep(proj, self.a2, self.a2_bias, work, self.heads, self.dim, self.vdim, self.rank, self.q_scale, self.tau)
        o = ws.rows("gla_o", n, self.hv, torch.float32)
        ops.gla_scan(work, o, cache.tensor, step, self.heads, self.dim, self.vdim,
                     fixed_order=dt == torch.float32)     # the 32-bit path: cuts and batches agree bit for bit
        y = ws.rows("gla_y", n, self.hv, dt)
        ops.gla_gated_norm(o, proj[:, 2 * self.hd + self.hv:2 * self.hd + 2 * self.hv], self.norm_w, y, self.heads,
                           self.vdim, self.norm_eps)
        return self.o.forward(y, out, defer=True)
