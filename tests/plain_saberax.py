"""A plain, slow Saberax: whole sequences, float64, one function per mechanism.

Nothing here is shared with the engine: it reads a raw config dict (the nested
config.json form) and a dict of tensors by checkpoint name, and walks the
tokens of ONE sequence with loops and dense matrices.  It is the oracle of
tests/test_saberax_*.py.

Notation: h is a layer's normed input [T, width]; W x means x @ W^T.  `alter` (a set of words)
changes one reading at a time, for the tests that must tell a right engine from a nearly right one.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x, w, b, eps):
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(dims, base, scaling=None):
    """(f [dims / 2], gain).  scaling with `fast`/`slow`: a ramp over the pair index blends f towards f / factor and
    both tables gain 0.1 ln(factor) + 1.  scaling with `low`/`high`: by wavelength l = 2 pi / f against
    `original`: kept below original / high, divided by factor above original / low, blended between."""
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    gain = 1.0
    if scaling is not None and "fast" in scaling:
        factor, orig = float(scaling["factor"]), float(scaling["original"])

        def turn_dim(turns):
            return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

        lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
        f = f / factor * ramp + f * (1 - ramp)
        gain = 0.1 * math.log(factor) + 1.0
    elif scaling is not None:
        factor, orig = float(scaling["factor"]), float(scaling["original"])
        low, high = float(scaling["low"]), float(scaling["high"])
        out = []
        for fi in f.tolist():
            wave = 2 * math.pi / fi
            if wave < orig / high:
                out.append(fi)
            elif wave > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wave - low) / (high - low)
                out.append((1 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=F)
    return f, gain


def rotate(x, positions, rot, pairing):
    """x [T, heads, d]: the first rot["dims"] dimensions of every head turn by the position's angles;
    pairing "interleaved": (2i, 2i + 1); "half": (i, i + dims / 2)."""
    dims = rot["dims"]
    f, gain = rotary_frequencies(dims, rot["base"], rot.get("scaling"))
    ang = positions.to(F)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * gain)[:, None, :], (torch.sin(ang) * gain)[:, None, :]
    out = x.clone()
    if pairing == "interleaved":
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        half = dims // 2
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    return out


def softmax_attention(q, k, v, scale, visible, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; visible(i, j) -> bool; sink [H] or None: exp(sink) joins
    the denominator only."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j)]
            s = torch.stack([(q[i, hd] * k[j, g]).sum() * scale for j in js])
            top = s.max() if sink is None else torch.maximum(s.max(), sink[hd])
            e = torch.exp(s - top)
            den = e.sum() + (torch.exp(sink[hd] - top) if sink is not None else 0.0)
            out[i, hd] = (e[:, None] * torch.stack([v[j, g] for j in js])).sum(0) / den
    return out


def qk_normed_attention(h, t, m, eps, alter=()):
    """Causal softmax attention without rotation (over every earlier token unless a window is given); q and k normed
    per head with a weight; q grows with the logarithm of the position in steps of `every`."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms((h @ t["q"].T).view(T, H, d), eps) * t["q.norm"]
    k = rms((h @ t["k"].T).view(T, G, d), eps) * t["k.norm"]
    v = (h @ t["v"].T).view(T, G, dv)
    qt = m.get("q_temp")
    if qt is not None and "no_temp" not in alter:
        p = torch.arange(T, dtype=F)
        q = q * (1.0 + qt["coef"] * torch.log(torch.floor((p + 1) / qt["every"]) + 1.0))[:, None, None]
    size = None if m.get("mask") is None else m["mask"]["size"] + ("wider" in alter) - ("narrower" in alter)
    o = softmax_attention(q, k, v, m["scale"], lambda i, j: size is None or i - j < size)
    return o.reshape(T, H * dv) @ t["o"].T


def window_attention(h, t, m, eps, alter=()):
    """Biased projections, interleaved rotary pairs, unit norms after the rotation, a sliding window."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ t["q"].T + t["q.b"]).view(T, H, d)
    k = (h @ t["k"].T + t["k.b"]).view(T, G, d)
    v = (h @ t["v"].T + t["v.b"]).view(T, G, dv)
    if m.get("rot") is not None:
        pairing = "half" if "other_pairing" in alter else "interleaved"
        q, k = rotate(q, pos, m["rot"], pairing), rotate(k, pos, m["rot"], pairing)
    q, k = rms(q, eps), rms(k, eps)
    size = None if m.get("mask") is None else m["mask"]["size"] + ("wider" in alter) - ("narrower" in alter)
    o = softmax_attention(q, k, v, m["scale"], lambda i, j: size is None or i - j < size)
    return o.reshape(T, H * dv) @ t["o"].T


def chunked_attention(h, t, m, eps, alter=()):
    """Values are the keys as projected; rotate-half pairs; unit norms after the rotation; a query sees its own
    chunk of `mask.size` positions only; a sink per head; a sigmoid gate per head on the output."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T)
    q = (h @ t["q"].T).view(T, H, d)
    k = (h @ t["k"].T).view(T, G, d)
    v = k.clone()
    if m.get("rot") is not None:
        pairing = "interleaved" if "other_pairing" in alter else "half"
        q, k = rotate(q, pos, m["rot"], pairing), rotate(k, pos, m["rot"], pairing)
    q, k = rms(q, eps), rms(k, eps)
    size = None if m.get("mask") is None else m["mask"]["size"] + ("wider" in alter) - ("narrower" in alter)
    sink = None if "no_sink" in alter else t["sink"]
    o = softmax_attention(q, k, v, m["scale"], lambda i, j: size is None or i // size == j // size, sink)
    if "no_gate" not in alter:
        o = o * torch.sigmoid(h @ t["g"].T)[:, :, None]
    return o.reshape(T, H * d) @ t["o"].T


def gated_recurrence(h, t, m, state=None):
    """The real-gated linear recurrent unit between two branches.  state: None or (S [width], the last
    taps - 1 inputs of the convolution [taps - 1, width]); returns (output, new state)."""
    T = h.shape[0]
    W, B, taps = m["width"], m["blocks"], m["conv"]
    y = gelu_tanh(h @ t["y"].T + t["y.b"])
    x = h @ t["x"].T + t["x.b"]
    S, tail = (torch.zeros(W, dtype=F), torch.zeros(taps - 1, W, dtype=F)) if state is None else state
    xs = torch.cat([tail, x], dim=0)                     # row i + taps - 1 is token i
    u = torch.stack([(xs[i:i + taps] * t["conv"].T).sum(0) for i in range(T)]) + t["conv.b"]
    ub = u.view(T, B, W // B)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", t["ra"], ub) + t["ra.b"]).reshape(T, W)
    g = torch.sigmoid(torch.einsum("boi,tbi->tbo", t["ri"], ub) + t["ri.b"]).reshape(T, W)
    log_a = -8.0 * r * torch.nn.functional.softplus(t["lam"])
    a = torch.exp(log_a)
    out = torch.zeros(T, W, dtype=F)
    for i in range(T):
        S = a[i] * S + torch.sqrt(1.0 - a[i] ** 2) * g[i] * u[i]
        out[i] = S
    return (out * y) @ t["o"].T, (S, xs[T:])


def gated_linear_attention(h, t, m, eps, state=None):
    """A matrix state per head whose rows (one per key channel) decay by a number made from the token.
    state: None or S [heads, dim, vdim]; returns (output, S)."""
    T = h.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (h @ t["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ t["k"].T).view(T, H, d)
    v = (h @ t["v"].T).view(T, H, dv)
    z = (h @ t["a1"].T) @ t["a2"].T + t["a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F) if state is None else state
    o = torch.zeros(T, H, dv, dtype=F)
    for i in range(T):
        S = alpha[i][:, :, None] * S + k[i][:, :, None] * v[i][:, None, :]
        o[i] = torch.einsum("hdv,hd->hv", S, q[i])
    o = rms(o, eps) * t["norm"]
    g = h @ t["g"].T
    return (o.reshape(T, H * dv) * (g * torch.sigmoid(g))) @ t["o"].T, S


def side_by_side(left, right, t, eps):
    """Half the sum of the two mixers' outputs, each normed over the width with a weight of its own."""
    return 0.5 * (rms(left, eps) * t["left.out"] + rms(right, eps) * t["right.out"])


def dense_unit(h, t):
    g = h @ t["gate"].T
    return (g * torch.sigmoid(g) * (h @ t["up"].T)) @ t["down"].T


def squared_relu_unit(h, up, down):
    return torch.relu(h @ up.T) ** 2 @ down.T


def route(h, router, correction, r):
    """(chosen [T, top], weights [T, top]).  r: experts, top, scale, groups {count, keep} or absent."""
    s = torch.sigmoid(h @ router.T)
    pick = s + correction
    E, top = r["experts"], r["top"]
    groups = r.get("groups")
    if groups is not None:
        per = E // groups["count"]
        score = pick.view(-1, groups["count"], per).topk(min(2, per), dim=-1).values.sum(-1)
        keep = score.topk(groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter(1, keep, True)
        pick = pick.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    chosen = pick.topk(top, dim=-1).indices
    w = s.gather(1, chosen)
    return chosen, w / (w.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)


def experts(h, t, f):
    chosen, w = route(h, t["router"], t["correction"], f["router"])
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for c, wt in zip(chosen[i].tolist(), w[i]):
            out[i] += wt * squared_relu_unit(h[i:i + 1], t[f"e{c}.up"], t[f"e{c}.down"])[0]
    if f.get("shared") is not None:
        out = out + squared_relu_unit(h, t["shared.up"], t["shared.down"])
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v.to(F) for k, v in tensors.items() if k.startswith(prefix)}


def mixer(kind, h, t, m, eps, alter=()):
    if kind == "parallel":
        left = qk_normed_attention(h, sub(t, "left."), m["left"], eps, alter)
        right, _ = gated_recurrence(h, sub(t, "right."), m["right"])
        return side_by_side(left, right, t, eps)
    if kind == "parallel_2":
        left = window_attention(h, sub(t, "left."), m["left"], eps, alter)
        right, _ = gated_linear_attention(h, sub(t, "right."), m["right"], eps)
        return side_by_side(left, right, t, eps)
    if kind == "attention":
        return chunked_attention(h, t, m, eps, alter)
    raise ValueError(kind)


def forward(cfg, tensors, tokens, layers_out=None, alter=()):
    """Logits [T, vocab] of one whole sequence.  `layers_out`: a list that receives the residual stream after
    every layer run."""
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = tensors["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        t = sub(tensors, f"l{src}.")
        h = layer_norm(x, t["norm1"], t["norm1.b"], eps)
        x = x + mult * mixer(layer["type"], h, sub(t, "mix."), layer["mixer"], eps, alter)
        f = layer.get("mlp")
        if f is not None:
            h = layer_norm(x, t["norm2"], t["norm2.b"], eps)
            ft = sub(t, "mlp.")
            x = x + mult * (dense_unit(h, ft) if f["kind"] == "dense" else experts(h, ft, f))
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, tensors["final.norm"].to(F), tensors["final.norm.b"].to(F), eps)
    return x @ tensors["head"].to(F).T
