"""Sink attention mixer: grouped-query attention without rotation, with capped and biased scores, a window that
keeps a sequence's first tokens, a sink in the softmax and values blended across layers.

Per token: q = W_q h + b_q, k = W_k h + b_k, v = W_v h + b_v (one stacked product; the biases are added by the
kernel that follows it).  q and k are each RMS-normed over the WHOLE projection (all heads at once) with a weight
per coordinate.  Query head h reads key/value head h // (heads / kv_heads); keys have `dim`, values `vdim` elements.

    s_ij = cap * tanh(q_i . k_j * scale / cap) + rel[bucket(i - j), head]
    p_ij = exp(s_ij) / (exp(sink_head) + sum over visible j' of exp(s_ij'))
    visible: j <= i and (i - j < window or j < keep_first)

bucket(n) maps a distance to one of the B rows of `rel`: n itself below B/2, then logarithmic steps up to
`bias_max`: min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(bias_max / (B/2)) * (B - B/2))).  The map is made once on the
host in float64, as a table by distance that ends where it saturates (at `bias_max`); the kernels look it up.
The sink is one learned number per head: a term of the denominator without key or value.

Value blending (`v_mix`): among the layers of a model that blend, the first ("source") keeps the values it made
for the step's tokens in a buffer named by `v_mix_buffer`; every later one ("blend") replaces its own by
(1 - lambda) v + lambda v_first, with its stored number lambda, before they are cached.

Each of cap, bias, sink, window, keep_first, the norms, the biases and the blend is optional by parameter.
"""
from __future__ import annotations

import math

import torch

from ..cache.needs import PagedKeysValues
from ..native import ops, scratch
from .base import Part
from .linear import Linear
from .registry import register_part


def distance_buckets(rows: int, bias_max: float) -> list:
    """bucket(n) for n = 0 .. ceil(bias_max): the row of a `rows`-row bias table that distance n takes.  Every larger
    distance takes the last entry's row (rows - 1)."""
    half = rows // 2
    if not bias_max > half or half < 1:
        raise ValueError(f"distance bias: bias_max {bias_max} must exceed half the table's {rows} rows")
    out = []
    for n in range(int(math.ceil(bias_max)) + 1):
        if n < half:
            out.append(n)
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(bias_max / half) * (rows - half)))))
    out[-1] = rows - 1                       # at and beyond bias_max the formula gives at least `rows`
    return out


@register_part("mixer", "sink_attention")
class SinkAttention(Part):
    """params: hidden_size, heads, kv_heads, dim, vdim, scale, norm_eps, window (None | int), keep_first (0),
    softcap (None | c), bias_rows (None | B), bias_max, sink (bool), qk_norm (bool), biases (bool),
    v_mix (None | "source" | "blend"), v_mix_buffer (name).
    tensors: q [heads * dim, hidden], k [kv_heads * dim, hidden], v [kv_heads * vdim, hidden], o [hidden, heads * vdim];
    with biases q_bias, k_bias, v_bias; with qk_norm q_norm [heads * dim], k_norm [kv_heads * dim]; with bias_rows
    rel [B, heads]; with sink sink [heads]; for "blend" v_mix []."""
    category = "mixer"
    native_libraries = ("sink_attention",)
    SCRATCH = "sink attention splits"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.scale = float(p["scale"])
        self.norm_eps = float(p.get("norm_eps", 1e-6))
        self.window = p.get("window")
        self.keep_first = int(p.get("keep_first") or 0) if self.window is not None else 0
        self.softcap = float(p["softcap"]) if p.get("softcap") else None
        self.bias_rows = int(p["bias_rows"]) if p.get("bias_rows") else None
        self.bias_max = float(p["bias_max"]) if self.bias_rows else None
        self.has_sink = bool(p.get("sink", False))
        self.qk_norm = bool(p.get("qk_norm", False))
        self.biases = bool(p.get("biases", False))
        self.v_mix = p.get("v_mix")
        self.v_mix_buffer = p.get("v_mix_buffer", "first_values")
        if self.heads % self.kv_heads:
            raise ValueError(f"sink_attention: {self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        if self.v_mix not in (None, "source", "blend"):
            raise ValueError(f"sink_attention: v_mix {self.v_mix!r} is none of None, 'source', 'blend'")
        if self.vdim > 256:
            raise ValueError(f"sink_attention: value size {self.vdim} is beyond the kernels' limit of 256")
        self.q_cols, self.k_cols, self.v_cols = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim
        self.qkv = self.o = self.bias = self.q_w = self.k_w = self.rel = self.sink = self.bucket_of = None
        self.lam = 0.0

    def cache_need(self):
        return PagedKeysValues(self.kv_heads, self.dim, self.vdim, self.window, self.keep_first)

    def weight_shapes(self):
        shapes = {"q": (self.q_cols, self.hidden), "k": (self.k_cols, self.hidden), "v": (self.v_cols, self.hidden),
                  "o": (self.hidden, self.heads * self.vdim)}
        if self.biases:
            shapes.update({"q_bias": (self.q_cols,), "k_bias": (self.k_cols,), "v_bias": (self.v_cols,)})
        if self.qk_norm:
            shapes.update({"q_norm": (self.q_cols,), "k_norm": (self.k_cols,)})
        if self.bias_rows:
            shapes["rel"] = (self.bias_rows, self.heads)
        if self.has_sink:
            shapes["sink"] = (self.heads,)
        if self.v_mix == "blend":
            shapes["v_mix"] = ()
        return shapes

    def load(self, tensors):
        mats = [tensors["q"], tensors["k"], tensors["v"]]
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("sink_attention: q, k and v matrices must be stored in one dtype")
        self.qkv = Linear(mats)
        self.o = Linear([tensors["o"]])
        if self.biases:
            self.bias = torch.cat([tensors[s].float() for s in ("q_bias", "k_bias", "v_bias")]).contiguous()
        if self.qk_norm:
            self.q_w = tensors["q_norm"].float().contiguous()
            self.k_w = tensors["k_norm"].float().contiguous()
        if self.bias_rows:
            self.rel = tensors["rel"].float().contiguous()
            self.bucket_of = torch.tensor(distance_buckets(self.bias_rows, self.bias_max), dtype=torch.int32,
                                          device=self.rel.device)
        if self.has_sink:
            self.sink = tensors["sink"].float().contiguous()
        if self.v_mix == "blend":
            self.lam = float(tensors["v_mix"].float().item())

    def native_builds(self):
        """(library, defines) pairs compiled for this part's sizes, so that a model's first load builds them beside
        its other libraries."""
        takes = self.ctx.device.type == "cuda" and ops.sink_tc_takes(self.ctx.dtype, self.dim, self.vdim)
        return [ops.sink_tc_library(self.dim, self.vdim)] if takes else []

    def reserve(self, limits):
        for lin in (self.qkv, self.o):
            if lin is not None:
                lin.reserve(self.ctx.dtype, limits.max_tokens)
        if self.ctx.device.type == "cuda" and ops.sink_tc_takes(self.ctx.dtype, self.dim, self.vdim):
            from ..native.build import load_library
            load_library(*ops.sink_tc_library(self.dim, self.vdim))        # built now, not inside the first step
        if self.ctx.device.type == "cuda" and self._splits_single_tokens():
            longest = -(-limits.max_model_len // 1024) * 1024
            self._partials(min(limits.max_tokens, limits.max_requests),
                           ops.sink_decode_splits(self.window, self.keep_first, longest)[0])   # nothing grows under a graph

    # ---- what the host decides per step: how many blocks share a single token's keys
    @property
    def plan_key(self):
        return ("sink_attention", self.heads, self.kv_heads, self.dim, self.vdim, self.window, self.keep_first)

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
        step.plans[self.plan_key] = ops.sink_decode_splits(self.window, self.keep_first, longest)

    def graph_key(self, step):
        return step.plans.get(self.plan_key)

    def _partials(self, n_tokens: int, n_splits: int):
        return scratch.get(self.ctx.device, self.SCRATCH, n_tokens * self.heads * n_splits * (self.vdim + 2))

    def forward(self, h, out, step, cache):
        n = h.shape[0]
        dt = self.ctx.dtype
        ws = step.workspace
        proj = ws.rows("sink_qkv", n, self.q_cols + self.k_cols + self.v_cols, dt)
        self.qkv.forward(h, proj)
        q = ws.rows("sink_q", n, self.q_cols, dt)
        v_first = None
        if self.v_mix is not None:
            v_first = ws.rows(self.v_mix_buffer, n, self.v_cols, torch.float32)
        ops.sink_prep(proj, self.bias, self.q_w, self.k_w, self.norm_eps, q, self.heads, self.kv_heads, self.dim,
                      self.vdim, {None: 0, "source": 1, "blend": 2}[self.v_mix], self.lam, v_first, cache.slots,
                      cache.tensor, cache.page_size)
        ctx = ws.rows("sink_ctx", n, self.heads * self.vdim, dt)
        tc = ops.sink_tc_takes(dt, self.dim, self.vdim)       # bfloat16 and sizes the tensor-core kernel is built for
        # (where only the CUDA-core kernel serves prompt rows, a mixed step gives it every row)
        single = step.n_decode_tokens if self._splits_single_tokens() and (tc or step.n_decode_tokens == n) else 0
        if single:                                            # single tokens: their keys split over blocks
            if self.plan_key not in step.plans:               # a step built by hand, not by the engine
                self.plan_step(step)
            n_splits, kept_splits = step.plans[self.plan_key]
            ops.sink_decode(q, ctx, cache.tensor, cache.block_table, step.tok_req, step.positions, step.decode_tokens,
                            self._partials(single, n_splits), n_splits, kept_splits, self.heads, self.kv_heads,
                            self.dim, self.vdim, self.window, self.keep_first, self.scale, self.softcap, self.bucket_of,
                            self.rel, self.sink, cache.page_size)
        if single == n:
            pass
        elif tc:
            ops.sink_attention_tc(q, ctx, cache.tensor, cache.block_table, step, self.heads, self.kv_heads, self.dim,
                                  self.vdim, self.window, self.keep_first, self.scale, self.softcap, self.bucket_of,
                                  self.rel, self.sink, cache.page_size, include_single=not single)
        else:
            ops.sink_attention_simt(q, ctx, cache.tensor, cache.block_table, step.tok_req, step.positions, self.heads,
                                    self.kv_heads, self.dim, self.vdim, self.window, self.keep_first, self.scale,
                                    self.softcap, self.bucket_of, self.rel, self.sink, cache.page_size)
        return self.o.forward(ctx, out, defer=True)
