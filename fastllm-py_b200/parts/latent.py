"""Latent attention mixer: attention over a compressed per-token cache.

Per token the layer caches one latent vector c (`kv_rank` elements: the first
rows of W_dkv h, RMS-normed with a weight) and one rotated key part (`rot_dim`
elements: the last rows of W_dkv h after rotary encoding) that all heads share.
Head h's key is [W_uk,h c | rotated part], its value W_uv,h c, its query
[q_plain | rotary(q_rot)] from W_q h laid out head by head; the score is their
dot product times `scale`, over the keys at or before the query and within
`window` if the layer has one; softmax in float; W_o on the concatenated heads.

Keys and values are never made.  The query's plain part is carried through
W_uk,h^T into latent space (q~ = [W_uk,h^T q_plain | q_rot], `kv_rank + rot_dim`
elements), attention runs on the cache rows themselves, and the weighted sum of
latents goes through W_uv,h: the same sums in another order, and the cache is
read once for all heads.  The per-head products take W_uk and W_uv re-laid at
load as [heads, kv_rank, dim] and [heads, vdim, kv_rank]; in bfloat16, with sizes
that are multiples of 32, they and the attention itself run on the tensor cores
(one batched launch each), else on the CUDA cores.

A layer with `shares_cache` has no W_dkv: it reads the rows another layer's run
wrote, with its own queries, W_uk, W_uv, window and scale.  The cache keeps what
the widest window among the layers that read it needs (`keep`).

Two variants by parameter.  `q_rank`: the queries go through a latent of their
own, c_q = RMSnorm(W_dq h) * w, q = W_uq c_q, instead of one matrix W_q; W_dq
is then stacked with W_dkv (and the gate) into the layer's first product.
`out_gate`: the concatenated heads are multiplied by sigmoid(W_g h) before W_o.
`pairing` names the rotary pairs: "halves" (i, i + rot_dim/2) or "interleaved"
(2i, 2i + 1); pair i turns by the position table's column i either way.
"""
from __future__ import annotations

import torch

from ..cache.needs import PagedRows
from ..native import ops, scratch
from .base import Part
from .linear import Linear
from .registry import build_part, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """params: hidden_size, heads, dim, rot_dim, vdim, kv_rank, scale, window (None | int), keep (None | int: what the
    cache keeps; absent: `window`), norm_eps, position (PartSpec of rot_dim dims), shares_cache (bool),
    q_rank (None | int), out_gate (bool), pairing ("halves" | "interleaved").
    tensors: q [heads * (dim + rot_dim), hidden] (with q_rank instead: dq [q_rank, hidden], dq_norm [q_rank],
    uq [heads * (dim + rot_dim), q_rank]), uk [heads * dim, kv_rank], uv [heads * vdim, kv_rank],
    o [hidden, heads * vdim], with out_gate g [heads * vdim, hidden], and, unless shares_cache,
    dkv [kv_rank + rot_dim, hidden], dkv_norm [kv_rank]."""
    category = "mixer"
    native_libraries = ("latent_attention", "gemm_mma", "gated_block")
    SPLIT_BELOW = 64                 # blocks (tokens x groups of 16 heads) under which a step's keys are split
    SCRATCH = "latent attention splits"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim, self.rot = int(p["heads"]), int(p["dim"]), int(p["rot_dim"])
        self.vdim, self.rank = int(p["vdim"]), int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.window = p.get("window")
        self.keep = p["keep"] if "keep" in p else self.window
        self.norm_eps = float(p["norm_eps"])
        self.shares_cache = bool(p.get("shares_cache", False))
        self.q_rank = int(p["q_rank"]) if p.get("q_rank") else None
        self.out_gate = bool(p.get("out_gate", False))
        if p.get("pairing", "halves") not in ("halves", "interleaved"):
            raise ValueError(f"latent_attention: pairing {p.get('pairing')!r} is neither 'halves' nor 'interleaved'")
        self.interleaved = p.get("pairing", "halves") == "interleaved"
        if self.rank > 1024:
            raise ValueError(f"latent_attention: kv_rank {self.rank} is beyond the kernel's limit of 1024")
        if self.window is not None and self.keep is not None and self.keep < self.window:
            raise ValueError("latent_attention: the cache keeps fewer tokens than the window sees")
        self.position = build_part("position", p["position"], ctx)
        if self.position.rot_dim != self.rot:
            raise ValueError("latent_attention: the position encoding must turn exactly rot_dim dimensions")
        self.q_cols = self.heads * (self.dim + self.rot)
        self.width = self.rank + self.rot                               # a cache row
        self.proj = self.o = self.uq = self.dq_norm = None

    def children(self):
        return [self.position]

    def cache_need(self):
        return None if self.shares_cache else PagedRows(self.width, self.keep)

    def weight_shapes(self):
        shapes = {"uk": (self.heads * self.dim, self.rank),
                  "uv": (self.heads * self.vdim, self.rank), "o": (self.hidden, self.heads * self.vdim)}
        if self.q_rank is None:
            shapes["q"] = (self.q_cols, self.hidden)
        else:
            shapes.update({"dq": (self.q_rank, self.hidden), "dq_norm": (self.q_rank,),
                           "uq": (self.q_cols, self.q_rank)})
        if self.out_gate:
            shapes["g"] = (self.heads * self.vdim, self.hidden)
        if not self.shares_cache:
            shapes["dkv"] = (self.width, self.hidden)
            shapes["dkv_norm"] = (self.rank,)
        return shapes

    def load(self, tensors):
        # the layer's first product: [q or dq | dkv | g], everything that reads h
        mats = [tensors["q"] if self.q_rank is None else tensors["dq"]]
        if not self.shares_cache:
            mats.append(tensors["dkv"])
        if self.out_gate:
            mats.append(tensors["g"])
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("latent_attention: the matrices that read the layer's input must be stored in one dtype")
        self.proj = Linear(mats)
        if self.q_rank is not None:
            self.uq = Linear([tensors["uq"]])
            self.dq_norm = tensors["dq_norm"].contiguous()
        self.dkv_norm = None if self.shares_cache else tensors["dkv_norm"].contiguous()
        self.uk_t = tensors["uk"].view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.uv = tensors["uv"].view(self.heads, self.vdim, self.rank).contiguous()
        self.o = Linear([tensors["o"]])

    def native_builds(self):
        """(library, defines) pairs compiled for this part's sizes, so that a model's first load builds them beside
        its other libraries."""
        takes = self.ctx.device.type == "cuda" and ops.latent_tc_takes(self.ctx.dtype, self.rank, self.rot)
        return [ops.latent_tc_library(self.rank, self.rot)] if takes else []

    def reserve(self, limits):
        for lin in (self.proj, self.o, self.uq):
            if lin is not None:
                lin.reserve(self.ctx.dtype, limits.max_tokens)
        if self.ctx.device.type == "cuda" and ops.latent_tc_takes(self.ctx.dtype, self.rank, self.rot):
            from ..native.build import load_library
            load_library(*ops.latent_tc_library(self.rank, self.rot))      # built now, not inside the first step
            most = max(1, (self.SPLIT_BELOW - 1) // -(-self.heads // 16))   # tokens of the largest step that splits
            longest = -(-limits.max_model_len // 1024) * 1024
            self._partials(min(most, limits.max_tokens), self._split(1, longest)[1])   # nothing grows under a graph

    # ---- what the host decides per step: whether and how the tensor-core kernel splits the keys
    @property
    def plan_key(self):
        return ("latent_attention", self.heads, self.rank, self.rot, self.window)

    def _split(self, n_tokens: int, longest: int):
        """(keys per split, splits) for a step of n_tokens whose longest sequence is `longest`; (0, 1): no split."""
        if not ops.latent_tc_takes(self.ctx.dtype, self.rank, self.rot) or \
                n_tokens * -(-self.heads // 16) >= self.SPLIT_BELOW:
            return 0, 1
        span = longest if self.window is None else min(self.window, longest)
        keys = max(128, -(-span // (30 * 32)) * 32)           # at most 32 splits
        return keys, (span - 1) // keys + 2

    def plan_step(self, step):
        longest = step.max_seq_len
        if step.for_graph:                                    # a captured step serves many: cover the length rounded up
            longest = -(-longest // 1024) * 1024
        step.plans[self.plan_key] = self._split(step.n_tokens, longest)

    def graph_key(self, step):
        return step.plans.get(self.plan_key)

    def _partials(self, n_tokens: int, n_splits: int):
        return scratch.get(self.ctx.device, self.SCRATCH, n_tokens * self.heads * n_splits * (self.rank + 2))

    def forward(self, h, out, step, cache):
        n = h.shape[0]
        dt = self.ctx.dtype
        ws = step.workspace
        if cache.writes == self.shares_cache:
            raise RuntimeError("latent_attention: the run's cache and the layer's shares_cache disagree")
        first = self.q_cols if self.q_rank is None else self.q_rank
        kv_cols = 0 if self.shares_cache else self.width
        cols = first + kv_cols + (self.heads * self.vdim if self.out_gate else 0)
        proj = ws.rows("latent_proj", n, cols, dt)
        self.proj.forward(h, proj)
        kv = None
        if self.q_rank is not None or self.out_gate:          # the latent's rows do not directly follow the queries
            kv = None if self.shares_cache else proj[:, first:first + kv_cols]
        queries = proj
        if self.q_rank is not None:
            cq = ws.rows("latent_cq", n, self.q_rank, dt)
            ops.rmsnorm(proj[:, :self.q_rank], self.dq_norm, cq, self.norm_eps)
            queries = ws.rows("latent_queries", n, self.q_cols, dt)
            self.uq.forward(cq, queries)
        tc = ops.latent_tc_takes(dt, self.rank, self.rot)     # bfloat16 and sizes the tensor-core kernel is built for
        q = ws.rows("latent_q", n, self.heads * self.width, dt if tc else torch.float32)
        cos, sin = self.position.tables()
        ops.latent_prep(queries, q, self.heads, self.dim, self.rot, self.rank, self.dkv_norm, self.norm_eps, cos, sin,
                        step.positions, cache.slots, cache.tensor if cache.writes else None, kv=kv,
                        interleaved=self.interleaved)
        proj = queries
        ops.gemm_batched(proj, self.dim + self.rot, self.uk_t, q, self.width)
        mix = ws.rows("latent_mix", n, self.heads * self.rank, dt if tc else torch.float32)
        if tc:
            if self.plan_key not in step.plans:               # a step built by hand, not by the engine
                self.plan_step(step)
            keys, splits = step.plans[self.plan_key]
            ops.latent_attention_tc(q, mix, cache.tensor, cache.block_table, step.tok_req, step.positions, self.heads,
                                    self.rank, self.rot, self.window, self.scale, cache.page_size, keys, splits,
                                    self._partials(n, splits) if keys else None)
        else:
            ops.latent_attention(q, mix, cache.tensor, cache.block_table, step.tok_req, step.positions, self.heads,
                                 self.rank, self.rot, self.window, self.scale, cache.page_size)
        ctx = ws.rows("latent_ctx", n, self.heads * self.vdim, dt)
        ops.gemm_batched(mix, self.rank, self.uv, ctx, self.vdim,
                         gate=ws.rows("latent_proj", n, cols, dt)[:, first + kv_cols:] if self.out_gate else None)
        return self.o.forward(ctx, out, defer=True)
