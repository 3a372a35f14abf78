"""Gated feed-forward: down( f(gate(h), up(h)) ), no biases; f = act(g) * u, SwiGLU when act is silu,
or the clamped swish unit (`native.ops.ACTIVATIONS`), whose two constants are `activation_params`.

fastllm_py/model.py:432-435 with the activation of
fastllm_py/kernels/ops.py:157-163: g / (1 + exp(-g)) * u in float.  gate and up
are stacked into one matrix so that one product serves both, with the activation
(`activation`: "silu", "relu", "gelu_tanh", "clamped_swish") in the product's epilogue where the
tensor-core kernel takes the problem, else product and one activation kernel."""
from __future__ import annotations

from ..native import ops
from .base import Part
from .linear import Linear
from .registry import register_part


@register_part("feed_forward", "glu")
@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """params: hidden_size, intermediate_size, activation ("silu"), activation_params ((0, 0)).  tensors: gate, up [I, hidden], down [hidden, I]."""
    category = "feed_forward"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = spec.params.get("activation", "silu")
        ops.activation_code(self.activation)
        self.activation_params = tuple(float(v) for v in spec.params.get("activation_params", (0.0, 0.0)))
        self.gate_up = None
        self.down = None

    def weight_shapes(self):
        return {"gate": (self.inter, self.hidden), "up": (self.inter, self.hidden),
                "down": (self.hidden, self.inter)}

    def load(self, tensors):
        if tensors["gate"].dtype != tensors["up"].dtype:
            raise ValueError("swiglu: gate and up matrices must be stored in one dtype")
        self.gate_up = Linear([tensors["gate"], tensors["up"]])
        self.down = Linear([tensors["down"]])

    def reserve(self, limits):
        for lin in (self.gate_up, self.down):
            if lin is not None:
                lin.reserve(self.ctx.dtype, limits.max_tokens)

    def forward(self, h, out, step):
        n = h.shape[0]
        dt = self.ctx.dtype
        act = step.workspace.rows("ffn_act", n, self.inter, dt)
        silu = self.activation == "silu"
        if self.gate_up.forward_gated(h, act, self.activation, self.activation_params):   # product and activation in one kernel
            return self.down.forward(act, out, defer=True)
        gu = step.workspace.rows("gate_up", n, 2 * self.inter, dt)
        partial = self.gate_up.forward(h, gu, defer=silu)
        if not silu:
            ops.glu(gu, act, self.activation, self.activation_params)
        elif partial is None:
            ops.swiglu(gu, act)
        else:
            ops.swiglu_partial(partial, act)
        return self.down.forward(act, out, defer=True)


@register_part("feed_forward", "mlp")
class PlainMLP(Part):
    """A feed-forward without a gate: down(act(up(h))), no biases; act is the gated units' f(x, 1)
    (`native.ops.ACTIVATIONS`: "relu_squared" is relu(x)^2).
    params: hidden_size, intermediate_size, activation ("relu_squared"), activation_params ((0, 0)).
    tensors: up [I, hidden], down [hidden, I]."""
    category = "feed_forward"
    native_libraries = ("norm_mix",)

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = spec.params.get("activation", "relu_squared")
        ops.activation_code(self.activation)
        self.activation_params = tuple(float(v) for v in spec.params.get("activation_params", (0.0, 0.0)))
        self.up = self.down = None

    def weight_shapes(self):
        return {"up": (self.inter, self.hidden), "down": (self.hidden, self.inter)}

    def load(self, tensors):
        self.up = Linear([tensors["up"]])
        self.down = Linear([tensors["down"]])

    def reserve(self, limits):
        for lin in (self.up, self.down):
            if lin is not None:
                lin.reserve(self.ctx.dtype, limits.max_tokens)

    def forward(self, h, out, step):
        n = h.shape[0]
        act = step.workspace.rows("mlp_act", n, self.inter, self.ctx.dtype)
        self.up.forward(h, act)
        ops.activation(act, act, self.activation, self.activation_params)
        return self.down.forward(act, out, defer=True)
