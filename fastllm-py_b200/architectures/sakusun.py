"""Sakusun as a plan of parts: a decoder of windowed sink-attention layers and latent-attention layers whose
sublayers read the residual stream through a short causal convolution and are gated and normed on their output.

Embedding: `embed[token] * scale` plus a row of the hashed token-pair table `bigram` (block "table_pairs").
Layer i (tensors `l<i>.*`), block "gated_postnorm":
    h = x;  hc = h + conv(h; canon1);  x <- x + ls1 * norm1(mixer(hc) * sigmoid(rg1 h + rg1.b))
    the same with canon2, rg2, norm2, ls2 around the feed-forward (no second half without an `mlp`)
norm1 / norm2 are single numbers; each is folded with its layer scale into one weight vector (norm "rmsnorm_scalar").
mixer "attention" -> part "sink_attention": `mix.{q,k,v}` with `.b` biases, `mix.{q,k}.norm`, `mix.rel` (its rows give
the number of distance buckets), `mix.sink`, `mix.vmix`, `mix.o`; the first layer with `v_mix` is the blend's source
(its own `mix.vmix` is stored and unused).
mixer "latent_attention": `mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}`: queries through a latent of their own, an
output gate, rotary pairs (2i, 2i + 1) on the rotated parts, no window.
Feed-forward "dense": `mlp.{gate,up,down}` with the tanh form of gelu as the gate's activation.
Then `final.norm` (a single number) and `head`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sakusun import QueryLatentAttentionConfig, SakusunConfig, SinkAttentionConfig
from ..parts.plan import LayerRun, LayerSpec, ModelPlan, PartSpec

DEFAULT_MAX_POSITIONS = 32768        # config.json gives no limit; the engine's max_model_len overrides this
DEFAULT_BIAS_ROWS = 32               # rows of a distance-bias table when no checkpoint is there to give them


def make_plan(cfg: SakusunConfig, tensor_names=None, tensor_shapes=None) -> ModelPlan:
    """`tensor_shapes` (name -> shape of the checkpoint's tensors, when there is a checkpoint) gives the sizes that
    config.json leaves to the tensors."""
    width, eps = cfg.width, cfg.norm_eps
    layers, order = [], []
    first_blend = True
    for i, layer in enumerate(cfg.layers):
        base, m = f"l{i}.", layer.mixer
        mx = base + "mix."
        if isinstance(m, SinkAttentionConfig):
            tensors = {s: mx + s for s in ("q", "k", "v", "o", "sink")}
            tensors.update({f"{s}_bias": f"{mx}{s}.b" for s in ("q", "k", "v")})
            tensors.update({f"{s}_norm": f"{mx}{s}.norm" for s in ("q", "k")})
            bias_rows = None
            if m.bias_max is not None:
                tensors["rel"] = mx + "rel"
                shape = (tensor_shapes or {}).get(mx + "rel")
                bias_rows = int(shape[0]) if shape is not None else DEFAULT_BIAS_ROWS
            v_mix = None
            if m.v_mix:
                v_mix = "source" if first_blend else "blend"
                first_blend = False
                if v_mix == "blend":
                    tensors["v_mix"] = mx + "vmix"
            mixer = PartSpec("sink_attention",
                             dict(hidden_size=width, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                                  scale=m.scale, norm_eps=eps, window=m.window, keep_first=m.keep_first,
                                  softcap=m.softcap, bias_rows=bias_rows, bias_max=m.bias_max, sink=True, qk_norm=True,
                                  biases=True, v_mix=v_mix, v_mix_buffer="first_values"), tensors)
        elif isinstance(m, QueryLatentAttentionConfig):
            tensors = {s: mx + s for s in ("dq", "uq", "dkv", "uk", "uv", "g", "o")}
            tensors.update({"dq_norm": mx + "dq.norm", "dkv_norm": mx + "dkv.norm"})
            position = PartSpec("rotary", dict(rot_dim=m.rot_dim, theta=m.rot_base, scaling=None, exact=True))
            mixer = PartSpec("latent_attention",
                             dict(hidden_size=width, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim,
                                  kv_rank=m.kv_rank, q_rank=m.q_rank, scale=m.scale, window=None, norm_eps=eps,
                                  position=position, shares_cache=False, out_gate=True, pairing="interleaved"), tensors)
        else:
            raise ValueError(f"layer {i}: unknown mixer configuration {m!r}")
        order.append(LayerRun(i))

        def out_norm(n):
            return PartSpec("rmsnorm_scalar", dict(size=width, eps=eps), {"weight": f"{base}norm{n}", "scale": f"{base}ls{n}"})

        norms = {"mixer_out": out_norm(1)}
        block_tensors = {"gate_mixer": base + "rg1", "gate_mixer_bias": base + "rg1.b"}
        if cfg.taps:
            block_tensors["conv_mixer"] = base + "canon1"
        ff = None
        if layer.mlp is not None:
            ff = PartSpec("glu", dict(hidden_size=width, intermediate_size=layer.mlp.ff, activation="gelu_tanh"),
                          {s: f"{base}mlp.{s}" for s in ("gate", "up", "down")})
            norms["ff_out"] = out_norm(2)
            block_tensors.update({"gate_ff": base + "rg2", "gate_ff_bias": base + "rg2.b"})
            if cfg.taps:
                block_tensors["conv_ff"] = base + "canon2"
        layers.append(LayerSpec("gated_postnorm", mixer, ff, norms, params=dict(hidden_size=width, taps=cfg.taps, gate=True),
                                tensors=block_tensors))
    io = dict(vocab_size=cfg.vocab, hidden_size=width)
    if cfg.bigram_buckets is not None:
        embedding = PartSpec("table_pairs", dict(io, scale=cfg.embedding_scale, buckets=cfg.bigram_buckets,
                                                 mul_prev=cfg.bigram_mul_prev, mul_cur=cfg.bigram_mul_cur),
                             {"weight": "embed", "pairs": "bigram"})
    else:
        embedding = PartSpec("table", dict(io, scale=cfg.embedding_scale), {"weight": "embed"})
    # the blend's source stores a `vmix` number too; nothing reads it
    ignorable = tuple(f"l{i}.mix.vmix" for i, layer in enumerate(cfg.layers) if getattr(layer.mixer, "v_mix", False))
    return ModelPlan(
        hidden_size=width, vocab_size=cfg.vocab, max_positions=DEFAULT_MAX_POSITIONS, embedding=embedding,
        layers=layers, order=order, final_norm=PartSpec("rmsnorm_scalar", dict(size=width, eps=eps), {"weight": "final.norm"}),
        head=PartSpec("linear", dict(io, softcap=None), {"weight": "head"}), ignorable=ignorable)


register_architecture("Sakusun", SakusunConfig, make_plan, model_types=("sakusun",))
