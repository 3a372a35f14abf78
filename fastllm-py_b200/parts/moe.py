"""Routed experts: a feed-forward that sends each token to a few of many small
gated feed-forwards and adds their outputs up with the router's weights.

Router: logits z = W_r h in float; scores s = sigmoid(z) (`score`: "sigmoid" or
"softmax" over the experts); the `top` experts with the largest s + bias are
chosen, where the bias (`correction`, a stored vector) steers the choice only;
the weights are the chosen experts' s, divided by their sum (+ `renormalise_eps`)
only if `renormalise` says so.  With `groups`, the experts form that many equal
groups of neighbours, a group's score is the sum of the `group_top` largest s + bias
in it (1: the largest), and only experts of the `keep_groups` best groups can be
chosen.  The weights are multiplied by `weight_scale` at the end.  Expert e:
W_down,e f(W_gate,e h, W_up,e h) with f = act(g) * u or the clamped swish unit
(`native.ops.ACTIVATIONS`), no biases; without a gate (`gated` False) W_down,e f(W_up,e h, 1).
The experts' matrices are stacked at load into [experts, 2 ff, hidden]
(gate rows, then up rows; [experts, ff, hidden] without a gate) and [experts, hidden, ff].
A `shared` feed-forward part runs for every token and is added to the experts' sum.

Two ways through the experts.  Few tokens (decode steps): one launch over
(token, choice) pairs, each streaming its expert's rows; the matrices are read
about once and the step is bound by that.  Many tokens in bfloat16: the pairs
are ordered by expert on the device and two tensor-core products run over tiles
of 64 rows that share an expert (`GROUP_FROM` pairs and up).  Neither path asks
the host anything, so steps with this part can be captured.
"""
from __future__ import annotations

import torch

from ..native import ops, scratch
from .base import Part
from .linear import Linear
from .registry import build_part, register_part


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    """params: hidden_size, experts, top, expert_ff, activation ("silu"), activation_params ((0, 0)), score ("sigmoid"),
    renormalise (False), renormalise_eps (0), groups (None), keep_groups (None: all), group_top (1),
    weight_scale (1), gated (True), shared (None | PartSpec of a feed-forward),
    choice_bias (True: a `correction` tensor is added to the scores for the choice).
    tensors: router [experts, hidden], correction [experts] (if choice_bias), and per expert i
    gate.i (if gated), up.i [ff, hidden], down.i [hidden, ff]."""
    category = "feed_forward"
    native_libraries = ("moe",)
    GROUP_FROM = 128                 # (token, choice) pairs from which the grouped path is taken
    SCRATCH = "routed experts"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden, self.experts, self.top = int(p["hidden_size"]), int(p["experts"]), int(p["top"])
        self.ff = int(p["expert_ff"])
        self.activation = p.get("activation", "silu")
        ops.activation_code(self.activation)
        self.activation_params = tuple(float(v) for v in p.get("activation_params", (0.0, 0.0)))
        self.groups = p.get("groups")
        self.keep_groups = p.get("keep_groups") or self.groups
        self.renormalise_eps = float(p.get("renormalise_eps", 0.0))
        self.group_top = int(p.get("group_top", 1))
        self.weight_scale = float(p.get("weight_scale", 1.0))
        self.gated = bool(p.get("gated", True))
        self.shared = build_part("feed_forward", p["shared"], ctx) if p.get("shared") is not None else None
        self.score = p.get("score", "sigmoid")
        if self.score not in ("sigmoid", "softmax"):
            raise ValueError(f"routed_experts: score {self.score!r} is not 'sigmoid' or 'softmax'")
        self.renormalise = bool(p.get("renormalise", False))
        self.choice_bias = bool(p.get("choice_bias", True))
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"routed_experts: top {self.top} of {self.experts} experts")
        if self.groups is not None and (self.experts % self.groups or not 1 <= self.keep_groups <= self.groups or
                                        self.keep_groups * (self.experts // self.groups) < self.top):
            raise ValueError(f"routed_experts: {self.keep_groups} of {self.groups} groups over {self.experts} experts "
                             f"cannot give {self.top} choices")
        if self.hidden * 4 > 48 * 1024:
            raise ValueError(f"routed_experts: hidden size {self.hidden} exceeds the kernels' 12288")

    def children(self):
        return [self.shared] if self.shared is not None else []

    def weight_shapes(self):
        shapes = {"router": (self.experts, self.hidden)}
        if self.choice_bias:
            shapes["correction"] = (self.experts,)
        for e in range(self.experts):
            if self.gated:
                shapes[f"gate.{e}"] = (self.ff, self.hidden)
            shapes[f"up.{e}"] = (self.ff, self.hidden)
            shapes[f"down.{e}"] = (self.hidden, self.ff)
        return shapes

    def load(self, tensors):
        self.router = Linear([tensors["router"]])
        self.correction = tensors["correction"].contiguous() if self.choice_bias else None
        first = tensors["up.0"]
        rows = 2 * self.ff if self.gated else self.ff
        self.gate_up = torch.empty((self.experts, rows, self.hidden), dtype=first.dtype, device=first.device)
        self.down = torch.empty((self.experts, self.hidden, self.ff), dtype=first.dtype, device=first.device)
        for e in range(self.experts):                    # expert by expert: no second copy of all of them
            if self.gated:
                self.gate_up[e, :self.ff] = tensors[f"gate.{e}"]
            self.gate_up[e, rows - self.ff:] = tensors[f"up.{e}"]
            self.down[e] = tensors[f"down.{e}"]

    def _grouped(self, dtype) -> bool:
        return ops.moe_group_takes(dtype, self.gate_up.dtype, self.hidden, self.ff)

    def _group_buffers(self, n, device):
        """(ints, act, y) of the grouped path for n tokens, carved out of one scratch buffer."""
        rows = ops.moe_group_rows(n, self.top, self.experts)
        n_ints = -(-(rows + n * self.top + rows // 64 + 1) // 4) * 4
        n_act = rows * self.ff // 2
        buf = scratch.get(device, self.SCRATCH, n_ints + n_act + rows * self.hidden)
        ints = buf[:n_ints].view(torch.int32)
        act = buf[n_ints:n_ints + n_act].view(torch.bfloat16).view(rows, self.ff)
        y = buf[n_ints + n_act:n_ints + n_act + rows * self.hidden].view(rows, self.hidden)
        return ints, act, y

    def reserve(self, limits):
        self.router.reserve(self.ctx.dtype, limits.max_tokens)

        if self.ctx.device.type == "cuda" and self._grouped(self.ctx.dtype):
            self._group_buffers(limits.max_tokens, self.ctx.device)       # sized now: nothing grows under a graph

    def forward(self, h, out, step):
        n = h.shape[0]
        ws = step.workspace
        # [n, top] without gaps between rows (the workspace pads rows to 16 bytes; whole padded rows are dense)
        padded = -(-self.top // 4) * 4
        chosen = ws.rows("moe_chosen", n, padded, torch.int32).view(-1)[:n * self.top].view(n, self.top)
        weights = ws.rows("moe_weights", n, padded, torch.float32).view(-1)[:n * self.top].view(n, self.top)
        logits = ws.rows("moe_logits", n, self.experts, torch.float32)
        self.router.forward(h, logits)                       # float accumulation, float logits
        ops.moe_pick(logits, self.correction, chosen, weights, self.top, self.score == "softmax", self.renormalise,
                     self.groups, self.keep_groups, self.renormalise_eps, self.group_top, self.weight_scale)
        shared = self.shared is not None
        if shared:                                           # the shared unit first: the experts' sum is added to it
            left = self.shared.forward(h, out, step)
            if left is not None:
                left.reduce_into(out)
        if n * self.top >= self.GROUP_FROM and self._grouped(h.dtype):
            ints, act, y = self._group_buffers(n, h.device)
            ops.moe_experts_grouped(h, self.gate_up, self.down, chosen, weights, ints, act, y, out, self.activation,
                                    self.activation_params, self.gated, accumulate=shared)
        else:
            act = ws.rows("moe_act", n, self.top * self.ff, torch.float32)
            ops.moe_experts(h, self.gate_up, self.down, chosen, weights, act, out, self.activation, self.activation_params,
                            self.gated, accumulate=shared)
        return None
