"""SaberaxConfig: the typed configuration of the Saberax decoder.

A Saberax model is a list of pre-norm layers (layer norms with weight and bias; every
sublayer's result is multiplied by one number before it is added).  A layer's mixer is one
softmax attention, or two mixers side by side (a softmax attention beside a recurrent one)
whose results are normed and averaged.  A layer may use another layer's tensors.  Its
config.json is nested:

    architecture     "Saberax"
    vocab, width     sizes of the embedding table and the residual stream
    norm.eps         the epsilon of every norm
    residual_mult    the factor on every sublayer's result (absent: 1)
    layers[i]        {"type": "parallel" | "parallel_2" | "attention", "mixer": {...}, "mlp": {...} | null,
                      "weights_of": j (absent: tensors of its own)}

    mixer of "attention" (keys serve as values; a query sees its own chunk of positions; a sink; a gate per head):
        heads, kv_heads, dim, vdim, scale, mask {size} (absent: every earlier token),
        rot {base, dims, scaling {factor, low, high, original} (absent: none)} (absent: no rotation)
    mixer of "parallel":  left  {heads, kv_heads, dim, vdim, scale, q_temp {coef, every} (absent: none),
                                 mask {size} (a window; absent: every earlier token)}
                          right {width, blocks, conv}
    mixer of "parallel_2": left {heads, kv_heads, dim, vdim, scale, mask {size} (absent: every earlier token),
                                 rot {base, dims, scaling {factor, original, fast, slow} (absent: none)}}
                           right {heads, dim, vdim, tau}
    mlp "dense":  ff
    mlp "moe":    expert {ff}, router {experts, top, scale (absent: 1), groups {count, keep} (absent: no groups)},
                  shared {ff} (absent: no shared expert)

Every size and constant above is read here and nowhere else; the parts get them
as parameters from the plan (architectures/saberax.py).
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    scaling: tuple | None     # None | ("yarn", factor, original, fast, slow) | ("bands", factor, original, low, high)

    def to_raw(self) -> dict:
        out = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            kind, factor, original, a, b = self.scaling
            names = ("fast", "slow") if kind == "yarn" else ("low", "high")
            out["scaling"] = {"factor": factor, "original": original, names[0]: a, names[1]: b}
        return out


@dataclass(frozen=True)
class AttentionConfig:
    """One softmax attention.  `role` says which of the design's three it is: "chunked" (the lone mixer),
    "normed" (beside the recurrent unit) or "windowed" (beside the gated linear attention)."""
    role: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask: int | None                 # chunk or window size
    rot: RotationConfig | None
    q_temp: tuple | None             # (coef, every)

    def to_raw(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.mask is not None:
            out["mask"] = {"size": self.mask}
        if self.rot is not None:
            out["rot"] = self.rot.to_raw()
        if self.q_temp is not None:
            out["q_temp"] = {"coef": self.q_temp[0], "every": self.q_temp[1]}
        return out


@dataclass(frozen=True)
class RecurrentUnitConfig:
    width: int
    blocks: int
    conv: int

    def to_raw(self) -> dict:
        return {"blocks": self.blocks, "conv": self.conv, "width": self.width}


@dataclass(frozen=True)
class GatedLinearAttentionConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int = 16                   # inner size of the decay's two matrices: a checkpoint's tensor shapes give it;
                                     # this number serves only where there is no checkpoint (random weights)

    def to_raw(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "tau": self.tau, "vdim": self.vdim}


@dataclass(frozen=True)
class PairConfig:
    left: AttentionConfig
    right: object                    # RecurrentUnitConfig | GatedLinearAttentionConfig

    def to_raw(self) -> dict:
        return {"left": self.left.to_raw(), "right": self.right.to_raw()}


@dataclass(frozen=True)
class DenseConfig:
    ff: int

    def to_raw(self) -> dict:
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    scale: float
    groups: int | None               # None: every expert can be chosen
    keep: int | None
    ff: int
    shared_ff: int | None

    def to_raw(self) -> dict:
        router = {"experts": self.experts, "scale": self.scale, "top": self.top}
        if self.groups is not None:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        out = {"expert": {"ff": self.ff}, "kind": "moe", "router": router}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class SaberaxLayerConfig:
    type: str                        # "parallel" | "parallel_2" | "attention"
    mixer: object                    # PairConfig | AttentionConfig
    mlp: object                      # DenseConfig | ExpertsConfig | None
    weights_of: int | None           # the layer whose tensors this one uses

    def to_raw(self) -> dict:
        out = {"mixer": self.mixer.to_raw(), "mlp": None if self.mlp is None else self.mlp.to_raw(), "type": self.type}
        if self.weights_of is not None:
            out["weights_of"] = self.weights_of
        return out


MIXER_TYPES = ("parallel", "parallel_2", "attention")


def _sub(raw: dict, key: str, where: str) -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}.{key} must be an object, got {v!r}")
    return v


def _rotation(raw: dict, dim: int, kind: str):
    rot = KeyReader(raw).mapping("rot")
    if rot is None:
        return None
    r = KeyReader(rot)
    dims = r.integer("dims", minimum=0)
    if dims % 2 or dims > dim:
        raise ConfigError(f"rot.dims {dims} must be even and at most dim {dim}")
    if dims == 0:
        return None
    scaling = r.mapping("scaling")
    if scaling is not None:
        s = KeyReader(scaling)
        if kind == "yarn":
            scaling = ("yarn", s.number("factor"), s.number("original"), s.number("fast"), s.number("slow"))
        else:
            low, high = s.number("low"), s.number("high")
            if low == high:
                raise ConfigError("rot.scaling: low and high must differ")
            scaling = ("bands", s.number("factor"), s.number("original"), low, high)
    return RotationConfig(r.number("base"), dims, scaling)


def _attention(raw: dict, role: str) -> AttentionConfig:
    r = KeyReader(raw)
    heads, kv_heads, dim = r.integer("heads"), r.integer("kv_heads"), r.integer("dim")
    if heads % kv_heads:
        raise ConfigError(f"heads {heads} is not a multiple of kv_heads {kv_heads}")
    vdim = r.integer("vdim")
    if role == "chunked" and vdim != dim:
        raise ConfigError(f"vdim {vdim} must equal dim {dim} where the keys serve as values")
    mask = r.mapping("mask")
    size = None if mask is None else KeyReader(mask).integer("size")
    temp = r.mapping("q_temp")
    if temp is not None:
        t = KeyReader(temp)
        temp = (t.number("coef", positive=False), t.integer("every"))
    rot = None if role == "normed" else _rotation(raw, dim, "yarn" if role == "windowed" else "bands")
    return AttentionConfig(role, heads, kv_heads, dim, vdim, r.number("scale"), size, rot, temp)


def _mixer(kind: str, raw: dict, i: int):
    where = f"layers[{i}].mixer"
    try:
        if kind == "attention":
            return _attention(raw, "chunked")
        if kind == "parallel":
            right = KeyReader(_sub(raw, "right", where))
            width, blocks = right.integer("width"), right.integer("blocks")
            if width % blocks:
                raise ConfigError(f"right.width {width} is not a multiple of right.blocks {blocks}")
            return PairConfig(_attention(_sub(raw, "left", where), "normed"),
                              RecurrentUnitConfig(width, blocks, right.integer("conv")))
        if kind == "parallel_2":
            right = KeyReader(_sub(raw, "right", where))
            return PairConfig(_attention(_sub(raw, "left", where), "windowed"),
                              GatedLinearAttentionConfig(right.integer("heads"), right.integer("dim"),
                                                         right.integer("vdim"), right.number("tau")))
    except ConfigError as e:
        raise ConfigError(f"{e} (in {where})") from None
    raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not a mixer of this architecture {MIXER_TYPES}")


def _mlp(raw, i: int):
    if raw is None:
        return None
    where = f"layers[{i}].mlp"
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where} must be an object or null, got {raw!r}")
    kind = raw.get("kind")
    try:
        if kind == "dense":
            return DenseConfig(KeyReader(raw).integer("ff"))
        if kind == "moe":
            router = KeyReader(_sub(raw, "router", where))
            experts, top = router.integer("experts"), router.integer("top")
            if top > experts:
                raise ConfigError(f"router.top {top} exceeds router.experts {experts}")
            groups = router.mapping("groups")
            count = keep = None
            if groups is not None:
                g = KeyReader(groups)
                count, keep = g.integer("count"), g.integer("keep")
                if experts % count or keep > count:
                    raise ConfigError(f"router.groups: {count} groups must divide {experts} experts, and keep "
                                      f"{keep} of them")
                if keep * (experts // count) < top:
                    raise ConfigError(f"router.groups: {keep} groups of {experts // count} experts cannot "
                                      f"give {top} choices")
            shared = KeyReader(raw).mapping("shared")
            return ExpertsConfig(experts, top, router.number("scale", default=1.0), count, keep,
                                 KeyReader(_sub(raw, "expert", where)).integer("ff"),
                                 None if shared is None else KeyReader(shared).integer("ff"))
    except ConfigError as e:
        raise ConfigError(f"{e} (in {where})") from None
    raise ConfigError(f"config.json: {where}.kind {kind!r} is not supported ('dense', 'moe')")


@dataclass(frozen=True)
class SaberaxConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: tuple

    @classmethod
    def from_hf(cls, raw: dict) -> "SaberaxConfig":
        r = KeyReader(raw)
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        layers = []
        for i, lr in enumerate(layers_raw):
            if not isinstance(lr, dict) or not isinstance(lr.get("type"), str):
                raise ConfigError(f"config.json: layers[{i}] must be an object with a 'type'")
            mixer = _mixer(lr["type"], _sub(lr, "mixer", f"layers[{i}]"), i)
            source = KeyReader(lr).integer("weights_of", default=None, minimum=0)
            layers.append(SaberaxLayerConfig(lr["type"], mixer, _mlp(lr.get("mlp"), i), source))
        for i, layer in enumerate(layers):
            j = layer.weights_of
            if j is None:
                continue
            if j >= len(layers) or j == i or layers[j].weights_of is not None:
                raise ConfigError(f"config.json: layers[{i}].weights_of {j} must name another layer with tensors "
                                  f"of its own")
            if layers[j].type != layer.type or (layers[j].mlp is None) != (layer.mlp is None):
                raise ConfigError(f"config.json: layers[{i}] uses the tensors of layers[{j}] but is a layer of another "
                                  f"kind")
        norm = KeyReader(_sub(raw, "norm", "config"))
        return cls(vocab=r.integer("vocab"), width=r.integer("width"), norm_eps=norm.number("eps"),
                   residual_mult=r.number("residual_mult", default=1.0, positive=False), layers=tuple(layers))

    def summary(self) -> str:
        """One line for a load message."""
        kinds = [layer.type for layer in self.layers]
        routed = sum(isinstance(layer.mlp, ExpertsConfig) for layer in self.layers)
        shared = sum(layer.weights_of is not None for layer in self.layers)
        return (f"Saberax: {len(kinds)}L width={self.width} ({kinds.count('attention')} chunked attention, "
                f"{kinds.count('parallel')} attention beside a recurrent unit, {kinds.count('parallel_2')} windowed "
                f"attention beside gated linear attention; {routed} with routed experts; {shared} on another "
                f"layer's tensors)")

    def to_hf(self) -> dict:
        """The config.json that reads back as this configuration."""
        return {"architecture": "Saberax", "layers": [layer.to_raw() for layer in self.layers],
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab,
                "width": self.width}
