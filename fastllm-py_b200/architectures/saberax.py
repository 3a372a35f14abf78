"""Saberax as a plan of parts: a decoder of pre-norm layers whose mixer is one softmax attention, or
two mixers side by side.

Layer i (tensors `l<i>.*`, or those of layer `weights_of` with a cache and state of its own):
    x <- x + m * mixer(norm1(x));   x <- x + m * ff(norm2(x))          (layer norms with bias; m = residual_mult)
mixer "attention" (`mix.{q,k,sink,g,o}`): softmax attention whose keys serve as values, rotary pairs
(i, i + dims/2) with frequencies scaled by bands of wavelength, unit norms of q and k after the rotation, a
query seeing its own chunk of positions only, a sink in the denominator and a sigmoid gate per head.
mixer "parallel": `mix.left.*` softmax attention over every earlier token with weighted norms of q and k and
a query scale that grows with the logarithm of the position, beside `mix.right.*` a gated linear recurrence
per channel behind a short convolution; "parallel_2": `mix.left.*` sliding-window softmax attention with biased
projections, rotary pairs (2i, 2i + 1) with blended frequencies and unit norms after the rotation, beside
`mix.right.*` gated linear attention.  Both results are normed (`mix.left.out`, `mix.right.out`) and averaged.
Feed-forward "dense": `mlp.{gate,up,down}` with silu; "moe": `mlp.router`, `mlp.correction`,
`mlp.e<j>.{up,down}` (squared relu, no gate), sigmoid scores, the choice limited to the best groups of
neighbouring experts by the sum of a group's two best, weights renormalised and scaled, plus `mlp.shared.*` for
every token.  Then `final.norm` and `head`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.saberax import (AttentionConfig, DenseConfig, ExpertsConfig, GatedLinearAttentionConfig, PairConfig,
                              RecurrentUnitConfig, SaberaxConfig)
from ..parts.plan import LayerRun, LayerSpec, ModelPlan, PartSpec

DEFAULT_MAX_POSITIONS = 32768        # config.json gives no limit; the engine's max_model_len overrides this
RENORM_EPS = 1e-20                   # added to the sum of the chosen experts' scores
GROUP_TOP = 2                        # a group of experts is scored by the sum of its two best
DECAY_RATE = 8.0                     # the recurrent unit's a = exp(-8 r softplus(lam))
MIX_WEIGHT = 0.5                     # two mixers side by side are averaged


def _attention(m: AttentionConfig, width: int, eps: float, at: str) -> PartSpec:
    """The three softmax attentions of the design differ in what `role` fixes; sizes and constants are `m`'s."""
    role = m.role
    position = None
    if m.rot is not None:
        position = PartSpec("rotary", dict(rot_dim=m.rot.dims, theta=m.rot.base, scaling=m.rot.scaling, exact=True))
    params = dict(hidden_size=width, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale,
                  norm_eps=eps, position=position, q_temp=m.q_temp)
    tensors = {s: at + s for s in ("q", "k", "o")}
    if role == "chunked":
        params.update(qk_norm="unit", pairing="half", chunk=m.mask, sink=True, values_from_keys=True, head_gate=True)
        tensors.update(sink=at + "sink", gate=at + "g")
    elif role == "normed":
        params.update(qk_norm="weighted", window=m.mask)
        tensors.update(v=at + "v", q_norm=at + "q.norm", k_norm=at + "k.norm")
    elif role == "windowed":
        params.update(qk_norm="unit", pairing="interleaved", window=m.mask, biases=True)
        tensors.update(v=at + "v", q_bias=at + "q.b", k_bias=at + "k.b", v_bias=at + "v.b")
    else:
        raise ValueError(f"unknown attention role {role!r}")
    return PartSpec("normed_attention", params, tensors)


def _right(m, width: int, eps: float, at: str, shapes) -> PartSpec:
    if isinstance(m, RecurrentUnitConfig):
        names = {"y": "y", "x": "x", "y_bias": "y.b", "x_bias": "x.b", "conv": "conv", "conv_bias": "conv.b",
                 "gate_a": "ra", "gate_a_bias": "ra.b", "gate_i": "ri", "gate_i_bias": "ri.b", "lam": "lam", "o": "o"}
        return PartSpec("gated_recurrence", dict(hidden_size=width, width=m.width, blocks=m.blocks, taps=m.conv,
                                                 rate=DECAY_RATE), {slot: at + n for slot, n in names.items()})
    if isinstance(m, GatedLinearAttentionConfig):
        rank = m.rank                                    # the decay's inner size is the shape of its first matrix
        if shapes is not None and at + "a1" in shapes:
            rank = int(shapes[at + "a1"][0])
        names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2_bias": "a2.b"}
        return PartSpec("gated_linear_attention", dict(hidden_size=width, heads=m.heads, dim=m.dim, vdim=m.vdim, tau=m.tau,
                                                       rank=rank, norm_eps=eps),
                        {slot: at + n for slot, n in names.items()})
    raise ValueError(f"unknown mixer configuration {m!r}")


def make_plan(cfg: SaberaxConfig, tensor_names=None, tensor_shapes=None) -> ModelPlan:
    width, eps = cfg.width, cfg.norm_eps

    def norm(name):
        return PartSpec("layernorm", dict(size=width, eps=eps), {"weight": name, "bias": name + ".b"})

    def layer_spec(i, layer, base):
        """The parts of one layer whose tensors are named from `base` (its own `l<i>.`, or another layer's)."""
        m = layer.mixer
        mx = base + "mix."
        if isinstance(m, PairConfig):
            mixer = PartSpec("side_by_side",
                             dict(hidden_size=width, norm_eps=eps, weight=MIX_WEIGHT,
                                  left=_attention(m.left, width, eps, mx + "left."),
                                  right=_right(m.right, width, eps, mx + "right.", tensor_shapes)),
                             {"left_out": mx + "left.out", "right_out": mx + "right.out"})
        elif isinstance(m, AttentionConfig):
            mixer = _attention(m, width, eps, mx)
        else:
            raise ValueError(f"layer {i}: unknown mixer configuration {m!r}")
        norms = {"mixer": norm(base + "norm1")}
        f = layer.mlp
        ff = None
        if f is not None:
            fm = base + "mlp."
            if isinstance(f, DenseConfig):
                ff = PartSpec("glu", dict(hidden_size=width, intermediate_size=f.ff, activation="silu"),
                              {s: fm + s for s in ("gate", "up", "down")})
            elif isinstance(f, ExpertsConfig):
                tensors = {"router": fm + "router", "correction": fm + "correction"}
                for e in range(f.experts):
                    tensors.update({f"{s}.{e}": f"{fm}e{e}.{s}" for s in ("up", "down")})
                shared = None
                if f.shared_ff is not None:
                    shared = PartSpec("mlp", dict(hidden_size=width, intermediate_size=f.shared_ff,
                                                  activation="relu_squared"),
                                      {"up": fm + "shared.up", "down": fm + "shared.down"})
                ff = PartSpec("routed_experts",
                              dict(hidden_size=width, experts=f.experts, top=f.top, expert_ff=f.ff, gated=False,
                                   activation="relu_squared", score="sigmoid", renormalise=True,
                                   renormalise_eps=RENORM_EPS, weight_scale=f.scale, choice_bias=True, groups=f.groups,
                                   keep_groups=f.keep, group_top=GROUP_TOP, shared=shared), tensors)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward configuration {f!r}")
            norms["feed_forward"] = norm(base + "norm2")
        return LayerSpec("prenorm", mixer, ff, norms, params=dict(residual_scale=cfg.residual_mult))

    def same(a, b):
        return (a.type, a.mixer, a.mlp) == (b.type, b.mixer, b.mlp)

    layers, order, plan_index = [], [], {}
    for i, layer in enumerate(cfg.layers):
        source = layer.weights_of
        if source is not None and same(layer, cfg.layers[source]):
            continue                                     # runs the source's parts again, with a cache of its own
        # a layer with tensors of its own; or one on another layer's tensors whose constants (a window, say) differ
        # from that layer's: parts of its own over the same tensors
        plan_index[i] = len(layers)
        layers.append(layer_spec(i, layer, f"l{i if source is None else source}."))
    for i, layer in enumerate(cfg.layers):
        order.append(LayerRun(plan_index[i] if i in plan_index else plan_index[layer.weights_of]))
    io = dict(vocab_size=cfg.vocab, hidden_size=width)
    return ModelPlan(
        hidden_size=width, vocab_size=cfg.vocab, max_positions=DEFAULT_MAX_POSITIONS,
        embedding=PartSpec("table", io, {"weight": "embed"}),
        layers=layers, order=order, final_norm=norm("final.norm"),
        head=PartSpec("linear", io, {"weight": "head"}))


register_architecture("Saberax", SaberaxConfig, make_plan, model_types=("saberax",))
