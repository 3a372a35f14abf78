"""Embedding and output head.

Embedding: x = table[ids] (fastllm_py/model.py:447), times `scale` for designs that scale it.  Head:
logits = x @ W^T in float, no bias (model.py:476), then, for a head with a
`softcap` c, logits <- c * tanh(logits / c); with tied
embeddings the head's matrix is the embedding table itself (model.py:228-231),
which the loader expresses by giving both parts the same tensor."""
from __future__ import annotations

from ..native import ops
from .base import Part
from .linear import Linear
from .registry import register_part


@register_part("embedding", "table")
class Embedding(Part):
    """params: vocab_size, hidden_size, scale (1: none).  tensors: weight [vocab, hidden]."""
    category = "embedding"
    takes_fed_tokens = True              # an id -1 - r is taken from row r of step.token_feed

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.scale = float(spec.params.get("scale", 1.0))
        self.table = None

    def weight_shapes(self):
        return {"weight": (self.vocab, self.hidden)}

    def load(self, tensors):
        self.table = tensors["weight"]

    def forward(self, step, out):
        ops.embed(self.table, step.token_ids, out, step.status, getattr(step, "token_feed", None), self.scale)


@register_part("embedding", "table_pairs")
class PairEmbedding(Embedding):
    """x = table[id] * scale + pairs[(previous id * mul_prev + id * mul_cur) mod buckets]: a second, hashed table
    indexed by the token and the one before it; a sequence's first token takes the table's last row (`buckets`).
    The token before a step's first one is per-request state (one int32 per request slot).
    params: vocab_size, hidden_size, scale, buckets, mul_prev, mul_cur.  tensors: weight [vocab, hidden],
    pairs [buckets + 1, hidden]."""
    native_libraries = ("gated_block",)

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.buckets = int(spec.params["buckets"])
        self.mul_prev = int(spec.params["mul_prev"])
        self.mul_cur = int(spec.params["mul_cur"])
        if self.buckets < 1:
            raise ValueError("table_pairs: buckets must be at least 1")
        self.pairs = None

    def weight_shapes(self):
        return {"weight": (self.vocab, self.hidden), "pairs": (self.buckets + 1, self.hidden)}

    def state_need(self):
        from ..cache.needs import FixedState
        return FixedState((1,), "int32")

    def load(self, tensors):
        self.table = tensors["weight"]
        self.pairs = tensors["pairs"]
        if self.pairs.dtype != self.table.dtype:
            raise ValueError("table_pairs: both tables must be stored in one dtype")

    def forward(self, step, out, state):
        ops.pair_embed(self.table, self.pairs, out, step, state.tensor, self.buckets, self.mul_prev, self.mul_cur,
                       self.scale)


@register_part("head", "linear")
class LinearHead(Part):
    """params: vocab_size, hidden_size, softcap (None | c > 0).  tensors: weight [vocab, hidden]."""
    category = "head"

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.softcap = spec.params.get("softcap")
        self.linear = None

    def weight_shapes(self):
        return {"weight": (self.vocab, self.hidden)}

    def load(self, tensors):
        # a table that the embedding part reads too stays row-major; a matrix of its own may be packed
        w = tensors["weight"]
        self.linear = Linear.sharing(w) if "weight" in self.shared_slots else Linear([w])

    def reserve(self, limits):
        if self.linear is not None:
            self.linear.reserve(self.ctx.dtype, min(limits.max_tokens, limits.max_requests))

    def forward(self, h, out):
        self.linear.forward(h, out)
        if self.softcap:
            ops.softcap(out, self.softcap)
