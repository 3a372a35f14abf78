"""Small Sakusun configurations and weights for the tests.

`config(...)` builds the raw config.json dict from layer descriptions, `weights(raw, seed)` draws
every tensor (bfloat16, like a stored model), `write(raw, tensors, folder)` makes a model folder.
The spread of each kind of tensor is chosen so that every mechanism matters: norm numbers and layer
scales away from 1, taps of the input convolution of the size of the signal, gate biases that open and
close channels, distance biases and sinks of the size of the scores, blend weights well inside (0, 1).
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def attention(heads=4, kv_heads=2, dim=16, vdim=24, window=11, keep_first=3, softcap=30.0, bias_max=40, v_mix=False,
              scale=None, bias_rows=8):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale if scale is not None else dim ** -0.5,
         "vdim": vdim, "_bias_rows": bias_rows}
    if bias_max is not None:
        m["bias_max"] = bias_max
    if softcap is not None:
        m["softcap"] = softcap
    if window is not None:
        m["mask"] = {"keep_first": keep_first, "size": window}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m}


def latent(heads=3, dim=16, rot=8, vdim=12, kv_rank=20, q_rank=28, base=10000.0, scale=None):
    return {"type": "latent_attention",
            "mixer": {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "rot": {"base": base, "dims": rot},
                      "rot_dim": rot, "scale": scale if scale is not None else (dim + rot) ** -0.5, "vdim": vdim}}


def dense(ff=48):
    return {"ff": ff, "kind": "dense"}


def config(layers, vocab=97, width=40, eps=1e-5, embed_scale=0.7, bigram=(53, 31, 5), taps=3):
    """layers: list of (mixer description, mlp description | None).  Returns (raw config, rows of each layer's
    distance-bias table): the rows are a size that only the tensor gives."""
    raw = {"architecture": "Sakusun", "embedding": {"scale": embed_scale}, "layers": [], "norm": {"eps": eps},
           "vocab": vocab, "width": width}
    if bigram is not None:
        raw["embedding"]["bigram"] = {"buckets": bigram[0], "mul_cur": bigram[2], "mul_prev": bigram[1]}
    if taps:
        raw["canon"] = {"taps": taps}
    rows = {}
    for i, (m, f) in enumerate(layers):
        mixer = dict(m["mixer"])
        if "_bias_rows" in mixer:
            rows[i] = mixer.pop("_bias_rows")
        raw["layers"].append({"type": m["type"], "mixer": mixer, "mlp": f})
    return raw, rows


def tensor_shapes(raw, rows) -> dict:
    w = raw["width"]
    out = {"embed": (raw["vocab"], w), "final.norm": (), "head": (raw["vocab"], w)}
    bg = raw["embedding"].get("bigram")
    if bg is not None:
        out["bigram"] = (bg["buckets"] + 1, w)
    taps = raw.get("canon", {}).get("taps", 0)
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        subs = (1,) if layer["mlp"] is None else (1, 2)
        for n in subs:
            out[f"{p}norm{n}"] = ()
            out[f"{p}ls{n}"] = (w,)
            out[f"{p}rg{n}"] = (w, w)
            out[f"{p}rg{n}.b"] = (w,)
            if taps:
                out[f"{p}canon{n}"] = (w, taps)
        if layer["type"] == "attention":
            q, k, v = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            out.update({p + "mix.q": (q, w), p + "mix.k": (k, w), p + "mix.v": (v, w), p + "mix.q.b": (q,),
                        p + "mix.k.b": (k,), p + "mix.v.b": (v,), p + "mix.q.norm": (q,), p + "mix.k.norm": (k,),
                        p + "mix.sink": (m["heads"],), p + "mix.o": (w, m["heads"] * m["vdim"])})
            if m.get("bias_max") is not None:
                out[p + "mix.rel"] = (rows[i], m["heads"])
            if m.get("v_mix"):
                out[p + "mix.vmix"] = ()
        else:
            qk = m["heads"] * (m["dim"] + m["rot_dim"])
            out.update({p + "mix.dq": (m["q_rank"], w), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (qk, m["q_rank"]),
                        p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], w), p + "mix.dkv.norm": (m["kv_rank"],),
                        p + "mix.uk": (m["heads"] * m["dim"], m["kv_rank"]), p + "mix.uv": (m["heads"] * m["vdim"], m["kv_rank"]),
                        p + "mix.g": (m["heads"] * m["vdim"], w), p + "mix.o": (w, m["heads"] * m["vdim"])})
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (ff, w)
            out[p + "mlp.down"] = (w, ff)
    return out


def weights(raw, rows, seed=0, sharp=1.0) -> dict:
    """`sharp` scales the query norms of the attention layers and the query up-projections of the latent layers
    (larger: peakier softmax, so single keys decide outputs)."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(raw, rows).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        r = torch.randn(shape, generator=gen)
        if leaf in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + 0.3 * r
        elif leaf in ("ls1", "ls2"):
            t = 0.6 + 0.25 * r
        elif leaf in ("canon1", "canon2"):
            t = 0.4 * r
        elif leaf in ("rg1.b", "rg2.b"):
            t = 0.8 * r
        elif leaf in ("mix.q.b", "mix.k.b", "mix.v.b"):
            t = 0.3 * r
        elif leaf in ("mix.q.norm",):
            t = (1.0 + 0.3 * r) * sharp
        elif leaf in ("mix.k.norm", "mix.dq.norm", "mix.dkv.norm"):
            t = 1.0 + 0.3 * r
        elif leaf == "mix.rel":
            t = 1.2 * r
        elif leaf == "mix.sink":
            t = 1.0 * r
        elif leaf == "mix.vmix":
            t = 0.5 + 0.15 * r.clamp(-2, 2)
        elif name in ("embed", "bigram"):
            t = 0.5 * r
        else:
            t = r * (1.5 / shape[1] ** 0.5)
            if leaf == "mix.uq":
                t = t * sharp
        out[name] = t.to(torch.bfloat16)
    return out


def write(raw, tensors, folder):
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw, indent=1))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
