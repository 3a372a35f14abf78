"""Grouped-query softmax attention whose queries and keys are normed head by head.

Per token: q = W_q h (+ b_q), k = W_k h (+ b_k), v = W_v h (+ b_v), one stacked product; query head h reads
key/value head h // (heads / kv_heads); keys have `dim`, values `vdim` elements.  Each query and key head passes an
RMS norm over its `dim` elements: `qk_norm` "weighted" norms before the rotation with a weight [dim] that the heads
share, "unit" after the rotation without a weight.  The rotation (a `position` part's tables) turns a head's first
`rot_dim` dimensions in pairs (2i, 2i + 1) (`pairing` "interleaved") or (i, i + rot_dim / 2) ("half").  With
`q_temp` = (coef, every) a query at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1).

    s_ij = q_i . k_j * scale;    p_ij = exp(s_ij) / ([exp(sink_head) +] sum over visible j' of exp(s_ij'))
    visible: j <= i, and with `window` w: i - j < w; with `chunk` c: floor(i / c) = floor(j / c)

The sink is one learned number per head in the denominator, without key or value.  With `values_from_keys` there
is no W_v: a token's value is its key as projected, before norm and rotation.  With `head_gate` head h's result is
multiplied by sigmoid(W_g h)_h, one number per head and token (W_g rides in the stacked product).

The attention itself is the sink-attention kernels' (CUDA cores in 32-bit; tensor cores for prompt portions and
split keys for single tokens in bfloat16), which take the chunk beside the window.
"""
from __future__ import annotations

import torch

from ..cache.needs import PagedKeysValues
from ..native import ops, scratch
from .base import Part
from .linear import Linear
from .registry import build_part, register_part


@register_part("mixer", "normed_attention")
class NormedAttention(Part):
    """params: hidden_size, heads, kv_heads, dim, vdim, scale, norm_eps, qk_norm (None | "weighted" | "unit"),
    position (PartSpec | None), pairing ("half" | "interleaved"), q_temp (None | (coef, every)), window (None | int),
    chunk (None | int), sink (bool), biases (bool), values_from_keys (bool), head_gate (bool).
    tensors: q [heads * dim, hidden], k [kv_heads * dim, hidden], o [hidden, heads * vdim]; v [kv_heads * vdim, hidden]
    unless values_from_keys; with biases q_bias, k_bias (and v_bias); for "weighted" q_norm, k_norm [dim]; with sink
    sink [heads]; with head_gate gate [heads, hidden]."""
    category = "mixer"
    native_libraries = ("sink_attention",)
    SCRATCH = "sink attention splits"
    honours_partial_side = True          # with `partial_side` set, the last product's partial sums go to the second scratch
    partial_side = False

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.scale = float(p["scale"])
        self.norm_eps = float(p.get("norm_eps", 1e-6))
        self.qk_norm = p.get("qk_norm")
        self.pairing = p.get("pairing", "half")
        self.q_temp = tuple(p["q_temp"]) if p.get("q_temp") else None
        self.window = int(p["window"]) if p.get("window") else None
        self.chunk = int(p["chunk"]) if p.get("chunk") else None
        self.has_sink = bool(p.get("sink", False))
        self.biases = bool(p.get("biases", False))
        self.v_from_k = bool(p.get("values_from_keys", False))
        self.gated = bool(p.get("head_gate", False))
        if self.heads % self.kv_heads:
            raise ValueError(f"normed_attention: {self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        if self.qk_norm not in (None, "weighted", "unit"):
            raise ValueError(f"normed_attention: qk_norm {self.qk_norm!r} is none of None, 'weighted', 'unit'")
        if self.pairing not in ("half", "interleaved"):
            raise ValueError(f"normed_attention: pairing {self.pairing!r} is neither 'half' nor 'interleaved'")
        if self.v_from_k and self.vdim != self.dim:
            raise ValueError("normed_attention: keys that serve as values have the values' size")
        if self.vdim > 256:
            raise ValueError(f"normed_attention: value size {self.vdim} is beyond the kernels' limit of 256")
        self.position = build_part("position", p["position"], ctx) if p.get("position") else None
        if self.position is not None and self.position.rot_dim > self.dim:
            raise ValueError("normed_attention: the position encoding turns more dimensions than a head has")
        self.q_cols, self.k_cols = self.heads * self.dim, self.kv_heads * self.dim
        self.v_cols = 0 if self.v_from_k else self.kv_heads * self.vdim
        self.gate_cols = self.heads if self.gated else 0
        self.proj = self.o = self.bias = self.q_w = self.k_w = self.sink = None

    def children(self):
        return [self.position] if self.position is not None else []

    def cache_need(self):
        # behind a chunk's start nothing is seen again: at most `chunk` tokens back, like a window of that size
        reach = min(x for x in (self.window, self.chunk) if x) if (self.window or self.chunk) else None
        return PagedKeysValues(self.kv_heads, self.dim, self.vdim, reach, 0)

    def weight_shapes(self):
        shapes = {"q": (self.q_cols, self.hidden), "k": (self.k_cols, self.hidden), "o": (self.hidden, self.heads * self.vdim)}
        if not self.v_from_k:
            shapes["v"] = (self.v_cols, self.hidden)
        if self.biases:
            shapes.update({"q_bias": (self.q_cols,), "k_bias": (self.k_cols,)})
            if not self.v_from_k:
                shapes["v_bias"] = (self.v_cols,)
        if self.qk_norm == "weighted":
            shapes.update({"q_norm": (self.dim,), "k_norm": (self.dim,)})
        if self.has_sink:
            shapes["sink"] = (self.heads,)
        if self.gated:
            shapes["gate"] = (self.heads, self.hidden)
        return shapes

    def load(self, tensors):
        names = ["q", "k"] + ([] if self.v_from_k else ["v"]) + (["gate"] if self.gated else [])
        mats = [tensors[s] for s in names]
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("normed_attention: the projections must be stored in one dtype")
        self.proj = Linear(mats)
        self.o = Linear([tensors["o"]])
        if self.biases:
            parts = [tensors["q_bias"], tensors["k_bias"]] + ([] if self.v_from_k else [tensors["v_bias"]])
            self.bias = torch.cat([t.float() for t in parts]).contiguous()
        if self.qk_norm == "weighted":
            self.q_w = tensors["q_norm"].float().contiguous()
            self.k_w = tensors["k_norm"].float().contiguous()
        if self.has_sink:
            self.sink = tensors["sink"].float().contiguous()

    def _tc(self) -> bool:
        return self.ctx.device.type == "cuda" and ops.sink_tc_takes(self.ctx.dtype, self.dim, self.vdim)

    def native_builds(self):
        """(library, defines) pairs compiled for this part's sizes, so that a model's first load builds them beside
        its other libraries."""
        return [ops.sink_tc_library(self.dim, self.vdim)] if self._tc() else []

    def reserve(self, limits):
        if self.proj is not None:
            self.proj.reserve(self.ctx.dtype, limits.max_tokens)
        if self.o is not None:
            self.o.reserve(self.ctx.dtype, limits.max_tokens, side=self.partial_side)
        if self._tc():
            from ..native.build import load_library
            load_library(*ops.sink_tc_library(self.dim, self.vdim))        # built now, not inside the first step
        if self.ctx.device.type == "cuda" and self._splits_single_tokens():
            longest = -(-limits.max_model_len // 1024) * 1024
            self._partials(min(limits.max_tokens, limits.max_requests),
                           ops.sink_decode_splits(self.window, 0, longest, self.chunk)[0])   # nothing grows under a graph

    # ---- what the host decides per step: how many blocks share a single token's keys
    @property
    def plan_key(self):
        return ("normed_attention", self.heads, self.kv_heads, self.dim, self.vdim, self.window, self.chunk)

    def _splits_single_tokens(self) -> bool:
        """bfloat16 steps give their single tokens to the split-key kernels (the 32-bit path keeps one kernel for every
        token, so that its sums do not depend on how a sequence was cut)."""
        return self.ctx.dtype == torch.bfloat16 and ops.sink_decode_takes(self.heads, self.kv_heads, self.dim, self.vdim)

    def plan_step(self, step):
        if not self._splits_single_tokens() or step.n_decode_tokens == 0:
            step.plans[self.plan_key] = (1, 0)
            return
        longest = step.max_seq_len
        if step.for_graph:                                    # a captured step serves many: cover the length rounded up
            longest = -(-longest // 1024) * 1024
        step.plans[self.plan_key] = ops.sink_decode_splits(self.window, 0, longest, self.chunk)

    def graph_key(self, step):
        return step.plans.get(self.plan_key)

    def _partials(self, n_tokens: int, n_splits: int):
        return scratch.get(self.ctx.device, self.SCRATCH, n_tokens * self.heads * n_splits * (self.vdim + 2))

    def forward(self, h, out, step, cache):
        n = h.shape[0]
        dt = self.ctx.dtype
        ws = step.workspace
        cols = self.q_cols + self.k_cols + self.v_cols + self.gate_cols
        proj = ws.rows("normed_attention_proj", n, cols, dt)
        self.proj.forward(h, proj)
        q = ws.rows("normed_attention_q", n, self.q_cols, dt)
        if self.position is not None:
            cos, sin = self.position.tables()
            rot = self.position.rot_dim
        else:
            cos = sin = None
            rot = 0
        ops.head_prep(proj, self.bias, self.q_w, self.k_w, {None: 0, "weighted": 1, "unit": 2}[self.qk_norm], self.norm_eps,
                      rot, self.pairing == "interleaved", cos, sin, step.positions, self.q_temp, self.v_from_k, q,
                      self.heads, self.kv_heads, self.dim, self.vdim, cache.slots, cache.tensor, cache.page_size)
        ctx = ws.rows("normed_attention_ctx", n, self.heads * self.vdim, dt)
        tc = self._tc()
        # (where only the CUDA-core kernel serves prompt rows, a mixed step gives it every row)
        single = step.n_decode_tokens if self._splits_single_tokens() and (tc or step.n_decode_tokens == n) else 0
        if single:                                            # single tokens: their keys split over blocks
            if self.plan_key not in step.plans:               # a step built by hand, not by the engine
                self.plan_step(step)
            n_splits, kept_splits = step.plans[self.plan_key]
            ops.sink_decode(q, ctx, cache.tensor, cache.block_table, step.tok_req, step.positions, step.decode_tokens,
                            self._partials(single, n_splits), n_splits, kept_splits, self.heads, self.kv_heads,
                            self.dim, self.vdim, self.window, 0, self.scale, None, None, None, self.sink, cache.page_size,
                            chunk=self.chunk)
        if single == n:
            pass
        elif tc:
            ops.sink_attention_tc(q, ctx, cache.tensor, cache.block_table, step, self.heads, self.kv_heads, self.dim,
                                  self.vdim, self.window, 0, self.scale, None, None, None, self.sink, cache.page_size,
                                  include_single=not single, chunk=self.chunk)
        else:
            ops.sink_attention_simt(q, ctx, cache.tensor, cache.block_table, step.tok_req, step.positions, self.heads,
                                    self.kv_heads, self.dim, self.vdim, self.window, 0, self.scale, None, None, None,
                                    self.sink, cache.page_size, chunk=self.chunk)
        if self.gated:
            ops.head_gate(ctx, proj[:, self.q_cols + self.k_cols + self.v_cols:], self.heads, self.vdim)
        return self.o.forward(ctx, out, defer=True, side=self.partial_side)
