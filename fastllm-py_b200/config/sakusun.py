"""SakusunConfig: the typed configuration of the Sakusun decoder.

A Sakusun model is a list of layers, each with one of two attention mixers and an optional
feed-forward, normed on the sublayers' outputs only.  Its config.json is nested:

    architecture   "Sakusun"
    vocab, width   sizes of the embedding table and the residual stream
    norm.eps       the epsilon of every RMS norm
    embedding      {"scale": s, "bigram": {"buckets", "mul_prev", "mul_cur"}}   (bigram absent: one table only)
    canon.taps     taps of the causal convolution in front of every sublayer
    layers[i]      {"type": "attention" | "latent_attention", "mixer": {...}, "mlp": {...} | null}

    mixer of "attention":         heads, kv_heads, dim, vdim, scale, softcap, bias_max, mask {size, keep_first},
                                  v_mix (true: the layer's values are blended with those of the first such layer)
    mixer of "latent_attention":  heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot {base, dims}
    mlp "dense":                  ff

Every size and constant above is read here and nowhere else; the parts get them as parameters from the
plan (architectures/sakusun.py).  Sizes that only a tensor's shape gives (the rows of an attention layer's
distance-bias table) come from the checkpoint's tensor table when the plan is made.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float | None
    bias_max: float | None
    window: int | None
    keep_first: int
    v_mix: bool

    def to_raw(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.softcap is not None:
            out["softcap"] = self.softcap
        if self.bias_max is not None:
            out["bias_max"] = self.bias_max
        if self.window is not None:
            out["mask"] = {"keep_first": self.keep_first, "size": self.window}
        if self.v_mix:
            out["v_mix"] = True
        return out


@dataclass(frozen=True)
class QueryLatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float

    def to_raw(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank,
                "rot": {"base": self.rot_base, "dims": self.rot_dim}, "rot_dim": self.rot_dim, "scale": self.scale,
                "vdim": self.vdim}


@dataclass(frozen=True)
class DenseConfig:
    ff: int

    def to_raw(self) -> dict:
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class SakusunLayerConfig:
    type: str                        # "attention" | "latent_attention"
    mixer: object                    # SinkAttentionConfig | QueryLatentAttentionConfig
    mlp: object                      # DenseConfig | None

    def to_raw(self) -> dict:
        return {"mixer": self.mixer.to_raw(), "mlp": None if self.mlp is None else self.mlp.to_raw(), "type": self.type}


def _sub(raw: dict, key: str, where: str) -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}.{key} must be an object, got {v!r}")
    return v


def _mixer(kind: str, raw: dict, i: int):
    where = f"layers[{i}].mixer"
    r = KeyReader(raw)
    try:
        if kind == "attention":
            heads, kv_heads = r.integer("heads"), r.integer("kv_heads")
            if heads % kv_heads:
                raise ConfigError(f"heads {heads} is not a multiple of kv_heads {kv_heads}")
            mask = r.mapping("mask")
            window = keep = None
            if mask is not None:
                window = KeyReader(mask).integer("size")
                keep = KeyReader(mask).integer("keep_first", default=0, minimum=0)
            return SinkAttentionConfig(heads, kv_heads, r.integer("dim"), r.integer("vdim"), r.number("scale"),
                                       r.number("softcap", default=None) if raw.get("softcap") is not None else None,
                                       r.number("bias_max", default=None) if raw.get("bias_max") is not None else None,
                                       window, keep or 0, r.boolean("v_mix"))
        if kind == "latent_attention":
            rot_dim = r.integer("rot_dim")
            rot = KeyReader(_sub(raw, "rot", where))
            if rot.integer("dims") != rot_dim:
                raise ConfigError(f"rot.dims {rot.integer('dims')} differs from rot_dim {rot_dim}")
            if rot_dim % 2:
                raise ConfigError(f"rot_dim {rot_dim} must be even for rotary pairs")
            return QueryLatentAttentionConfig(r.integer("heads"), r.integer("dim"), rot_dim, r.integer("vdim"),
                                              r.integer("kv_rank"), r.integer("q_rank"), r.number("scale"),
                                              rot.number("base"))
    except ConfigError as e:
        raise ConfigError(f"{e} (in {where})") from None
    raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not a mixer of this architecture "
                      f"('attention', 'latent_attention')")


def _mlp(raw, i: int):
    if raw is None:
        return None
    where = f"layers[{i}].mlp"
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where} must be an object or null, got {raw!r}")
    if raw.get("kind") != "dense":
        raise ConfigError(f"config.json: {where}.kind {raw.get('kind')!r} is not supported ('dense')")
    try:
        return DenseConfig(KeyReader(raw).integer("ff"))
    except ConfigError as e:
        raise ConfigError(f"{e} (in {where})") from None


@dataclass(frozen=True)
class SakusunConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    bigram_buckets: int | None       # None: no second table
    bigram_mul_prev: int
    bigram_mul_cur: int
    taps: int                        # 0: no input convolution
    layers: tuple

    @classmethod
    def from_hf(cls, raw: dict) -> "SakusunConfig":
        r = KeyReader(raw)
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        layers = []
        for i, lr in enumerate(layers_raw):
            if not isinstance(lr, dict) or not isinstance(lr.get("type"), str):
                raise ConfigError(f"config.json: layers[{i}] must be an object with a 'type'")
            layers.append(SakusunLayerConfig(lr["type"], _mixer(lr["type"], _sub(lr, "mixer", f"layers[{i}]"), i),
                                             _mlp(lr.get("mlp"), i)))
        blenders = [layer.mixer for layer in layers if getattr(layer.mixer, "v_mix", False)]
        if len({m.kv_heads * m.vdim for m in blenders}) > 1:
            raise ConfigError("config.json: layers with v_mix must agree in kv_heads * vdim (they blend their values)")
        norm = KeyReader(_sub(raw, "norm", "config"))
        emb = r.mapping("embedding") or {}
        bigram = KeyReader(emb).mapping("bigram")
        buckets = mul_prev = mul_cur = None
        if bigram is not None:
            b = KeyReader(bigram)
            buckets, mul_prev, mul_cur = b.integer("buckets"), b.integer("mul_prev", minimum=0), b.integer("mul_cur", minimum=0)
        canon = r.mapping("canon")
        return cls(vocab=r.integer("vocab"), width=r.integer("width"), norm_eps=norm.number("eps"),
                   embedding_scale=KeyReader(emb).number("scale", default=1.0), bigram_buckets=buckets,
                   bigram_mul_prev=mul_prev or 0, bigram_mul_cur=mul_cur or 0,
                   taps=0 if canon is None else KeyReader(canon).integer("taps"), layers=tuple(layers))

    def summary(self) -> str:
        """One line for a load message."""
        kinds = [layer.type for layer in self.layers]
        return (f"Sakusun: {len(kinds)}L width={self.width} ({kinds.count('attention')} windowed attention with sink, "
                f"{kinds.count('latent_attention')} latent attention; input convolution of {self.taps} taps)")

    def to_hf(self) -> dict:
        """The config.json that reads back as this configuration."""
        emb = {"scale": self.embedding_scale}
        if self.bigram_buckets is not None:
            emb["bigram"] = {"buckets": self.bigram_buckets, "mul_cur": self.bigram_mul_cur,
                             "mul_prev": self.bigram_mul_prev}
        out = {"architecture": "Sakusun", "embedding": emb, "layers": [layer.to_raw() for layer in self.layers],
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.taps:
            out["canon"] = {"taps": self.taps}
        return out
