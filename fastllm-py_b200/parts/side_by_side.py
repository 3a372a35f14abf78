"""Two mixers side by side: both read the same input, and the layer's result is the weighted sum of
their results, each first normed over the model width.

    out = weight * (rms(left(h)) * w_left + rms(right(h)) * w_right)       (weight 1/2: their average)

Each of the two is a mixer part of its own with whatever cache or state it needs; this part asks the
cache manager for both (`cache_needs`) and hands each its view.  Either may leave its last product as
split-K partial sums, which the one kernel that norms both rows and mixes them adds up as it reads.
The scratch for partial sums is one buffer and a second one beside it: a left mixer that says
`honours_partial_side` is told (`partial_side = True`) to leave its sums in the second, where the right
mixer's products do not overwrite them; one that does not gets its sums added up before the right runs.
"""
from __future__ import annotations

from ..native import ops
from .base import Part
from .registry import build_part, register_part


@register_part("mixer", "side_by_side")
class SideBySide(Part):
    """params: hidden_size, left (PartSpec), right (PartSpec), norm_eps, weight (0.5).
    tensors: left_out, right_out [hidden]."""
    category = "mixer"
    native_libraries = ("norm_mix",)
    SIDES = ("left", "right")
    PARTIAL_FROM = 64                    # rows from which the mix kernel adds partial sums up itself

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.norm_eps = float(p["norm_eps"])
        self.weight = float(p.get("weight", 0.5))
        self.left = build_part("mixer", p["left"], ctx)
        self.right = build_part("mixer", p["right"], ctx)
        if getattr(self.left, "honours_partial_side", False):
            self.left.partial_side = True
        self.w_left = self.w_right = None

    def children(self):
        return [self.left, self.right]

    def cache_need(self):
        return None

    def cache_needs(self) -> dict:
        """name -> need of the mixers that want a cache or a state; the step's views come back under the same names."""
        needs = {side: getattr(self, side).cache_need() for side in self.SIDES}
        return {side: need for side, need in needs.items() if need is not None}

    def weight_shapes(self):
        return {"left_out": (self.hidden,), "right_out": (self.hidden,)}

    def load(self, tensors):
        self.w_left = tensors["left_out"].contiguous()
        self.w_right = tensors["right_out"].to(self.w_left.dtype).contiguous()

    # what the two decide on the host per step is theirs: the decoder asks this part, which asks them
    def plan_step(self, step):
        for side in (self.left, self.right):
            if hasattr(side, "plan_step"):
                side.plan_step(step)

    def graph_key(self, step):
        return tuple(side.graph_key(step) for side in (self.left, self.right) if hasattr(side, "graph_key"))

    @property
    def plan_key(self):
        return ("side_by_side", getattr(self.left, "plan_key", id(self.left)), getattr(self.right, "plan_key", id(self.right)))

    def forward(self, h, out, step, cache):
        n = h.shape[0]
        dt = self.ctx.dtype
        ws = step.workspace
        results = []
        for side in self.SIDES:
            buf = ws.rows(f"side_{side}", n, self.hidden, dt)
            part = getattr(self, side)
            left = part.forward(h, buf, step, None if cache is None else cache.get(side))
            if left is not None and (n < self.PARTIAL_FROM or
                                     (side == "left" and not getattr(part, "partial_side", False))):
                # a handful of rows: the reduce kernel's many blocks are faster than one block a row; a left mixer
                # that used the first scratch buffer: the right mixer's products would overwrite the sums
                left = left.reduce_into(buf)
            results.append(buf if left is None else left)
        ops.rms_mix(results[0], results[1], self.w_left, self.w_right, out, self.norm_eps, self.weight)
        return None
