"""Small Saberax configurations and weights for the tests.

`config(...)` builds the raw config.json dict from layer descriptions, `weights(raw, seed)` draws
every tensor (bfloat16, like a stored model), `write(raw, tensors, folder)` makes a model folder.
The spread of each kind of tensor is chosen so that every mechanism matters: norm weights away
from 1 and biases away from 0, sinks and gates of both signs, decays between 0.3 and 1, router rows
and corrections large enough that groups and choices differ from token to token.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _softmax(heads, kv_heads, dim, vdim, scale):
    return {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale if scale is not None else dim ** -0.5,
            "vdim": vdim}


def normed(heads=4, kv_heads=2, dim=16, vdim=24, q_temp=(0.3, 8), scale=None):
    """The attention beside the recurrent unit: every earlier token, weighted norms, a query scale by position."""
    m = _softmax(heads, kv_heads, dim, vdim, scale)
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def recurrent(width=24, blocks=3, conv=4):
    return {"blocks": blocks, "conv": conv, "width": width}


def windowed(heads=4, kv_heads=2, dim=16, vdim=16, window=11, rot=8, base=10000.0, scaling=None, scale=None):
    """The attention beside the gated linear attention: biases, interleaved rotary pairs, unit norms, a window."""
    m = _softmax(heads, kv_heads, dim, vdim, scale)
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot}
        if scaling is not None:
            factor, original, fast, slow = scaling
            m["rot"]["scaling"] = {"factor": factor, "fast": fast, "original": original, "slow": slow}
    return m


def linear_attention(heads=2, dim=8, vdim=12, tau=8.0):
    return {"dim": dim, "heads": heads, "tau": tau, "vdim": vdim}


def pair(left, right):
    kind = "parallel" if "width" in right else "parallel_2"
    return {"type": kind, "mixer": {"left": left, "right": right}}


def chunked(heads=4, kv_heads=2, dim=16, chunk=13, rot=8, base=10000.0, scaling=None, scale=None):
    """The lone attention: keys as values, rotate-half pairs, unit norms, chunks, a sink, a gate per head."""
    m = _softmax(heads, kv_heads, dim, dim, scale)
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot}
        if scaling is not None:
            factor, original, low, high = scaling
            m["rot"]["scaling"] = {"factor": factor, "high": high, "low": low, "original": original}
    return {"type": "attention", "mixer": m}


def dense(ff=48):
    return {"ff": ff, "kind": "dense"}


def moe(experts=6, top=2, ff=24, scale=2.0, groups=None, shared=16):
    router = {"experts": experts, "scale": scale, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"expert": {"ff": ff}, "kind": "moe", "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def config(layers, vocab=97, width=40, eps=1e-5, mult=0.7):
    """`layers`: (mixer entry, mlp) pairs, or an int j for a layer that uses layer j's tensors."""
    out = []
    for entry in layers:
        if isinstance(entry, int):
            out.append(dict(json.loads(json.dumps(out[entry])), weights_of=entry))
        else:
            mixer, mlp = entry
            out.append({"mixer": mixer["mixer"], "mlp": mlp, "type": mixer["type"]})
    return {"architecture": "Saberax", "layers": out, "norm": {"eps": eps}, "residual_mult": mult, "vocab": vocab,
            "width": width}


def _attention_shapes(out, p, m, w, kind):
    out[p + "q"] = (m["heads"] * m["dim"], w)
    out[p + "k"] = (m["kv_heads"] * m["dim"], w)
    out[p + "o"] = (w, m["heads"] * m["vdim"])
    if kind == "chunked":
        out[p + "sink"] = (m["heads"],)
        out[p + "g"] = (m["heads"], w)
        return
    out[p + "v"] = (m["kv_heads"] * m["vdim"], w)
    if kind == "normed":
        out[p + "q.norm"] = out[p + "k.norm"] = (m["dim"],)
    else:
        out[p + "q.b"], out[p + "k.b"], out[p + "v.b"] = (out[p + "q"][0],), (out[p + "k"][0],), (out[p + "v"][0],)


def tensor_shapes(raw, rank=6) -> dict:
    """`rank`: the inner size of the gated linear attention's decay matrices (config.json does not hold it)."""
    w = raw["width"]
    out = {"embed": (raw["vocab"], w), "final.norm": (w,), "final.norm.b": (w,), "head": (raw["vocab"], w)}
    for i, layer in enumerate(raw["layers"]):
        if "weights_of" in layer:
            continue
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = out[p + "norm1.b"] = (w,)
        if layer["type"] == "attention":
            _attention_shapes(out, p + "mix.", m, w, "chunked")
        else:
            _attention_shapes(out, p + "mix.left.", m["left"], w, "normed" if layer["type"] == "parallel" else "windowed")
            out[p + "mix.left.out"] = out[p + "mix.right.out"] = (w,)
            r, q = m["right"], p + "mix.right."
            if layer["type"] == "parallel":
                n, bw = r["width"], r["width"] // r["blocks"]
                out[q + "y"] = out[q + "x"] = (n, w)
                out[q + "y.b"] = out[q + "x.b"] = out[q + "conv.b"] = out[q + "lam"] = (n,)
                out[q + "conv"] = (n, r["conv"])
                out[q + "ra"] = out[q + "ri"] = (r["blocks"], bw, bw)
                out[q + "ra.b"] = out[q + "ri.b"] = (r["blocks"], bw)
                out[q + "o"] = (w, n)
            else:
                hd, hv = r["heads"] * r["dim"], r["heads"] * r["vdim"]
                out[q + "q"] = out[q + "k"] = (hd, w)
                out[q + "v"] = out[q + "g"] = (hv, w)
                out[q + "o"] = (w, hv)
                out[q + "norm"] = (r["vdim"],)
                out[q + "a1"], out[q + "a2"], out[q + "a2.b"] = (rank, w), (hd, rank), (hd,)
        f = layer["mlp"]
        if f is None:
            continue
        out[p + "norm2"] = out[p + "norm2.b"] = (w,)
        if f["kind"] == "dense":
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (f["ff"], w)
            out[p + "mlp.down"] = (w, f["ff"])
        else:
            e_ff = f["expert"]["ff"]
            out[p + "mlp.router"] = (f["router"]["experts"], w)
            out[p + "mlp.correction"] = (f["router"]["experts"],)
            for e in range(f["router"]["experts"]):
                out[f"{p}mlp.e{e}.up"] = (e_ff, w)
                out[f"{p}mlp.e{e}.down"] = (w, e_ff)
            if f.get("shared") is not None:
                out[p + "mlp.shared.up"] = (f["shared"]["ff"], w)
                out[p + "mlp.shared.down"] = (w, f["shared"]["ff"])
    return out


def weights(raw, seed=0, gain=1.0, rank=6, slow=False) -> dict:
    """`gain` scales all matrices; `slow`: decays close to one (the recurrent unit's and the linear attention's), so
    that far tokens still count."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(raw, rank).items():
        leaf = name.split(".")[-1]
        tail2 = ".".join(name.split(".")[-2:])

        def randn(std):
            return torch.randn(shape, generator=gen) * std

        if tail2 in ("q.norm", "k.norm") or leaf in ("norm1", "norm2", "out") or name == "final.norm" or \
                (leaf == "norm" and "right" in name):
            t = 1.0 + randn(0.3)
        elif tail2 in ("norm1.b", "norm2.b", "norm.b"):
            t = randn(0.2)
        elif tail2 == "a2.b":
            t = (4.0 if slow else 1.0) + randn(1.0)          # sigmoid(z)^(1/tau): decays near one
        elif tail2 in ("ra.b", "ri.b", "y.b", "x.b", "conv.b", "q.b", "k.b", "v.b"):
            t = randn(0.3)
        elif leaf == "lam":
            t = (-6.0 if slow else -2.0) + randn(1.0)        # a = exp(-8 r softplus(lam))
        elif leaf == "conv":
            t = randn(0.5)
        elif leaf in ("ra", "ri"):
            t = randn(1.5 / shape[-1] ** 0.5)
        elif leaf == "sink":
            t = randn(1.5)
        elif leaf == "correction":
            t = randn(0.3)
        elif name == "embed":
            t = randn(0.6)
        elif leaf == "router":
            t = randn(3.0 / shape[1] ** 0.5)
        elif leaf == "a2":
            t = randn(2.0 / shape[1] ** 0.5)
        else:
            t = randn(gain * 1.5 / shape[1] ** 0.5)
        out[name] = t.to(torch.bfloat16)
    return out


def write(raw, tensors, folder):
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw, indent=1))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
