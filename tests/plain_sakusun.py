"""Sakusun written out plainly: whole sequences, float64, one function per mechanism.

Nothing here is shared with the engine.  `forward(raw, weights, tokens)` gives the logits at every
position of one sequence from the raw config.json dict and the tensors by name.  Notation: T tokens,
C channels (the width), x the residual stream [T, C].

`alter` changes the reading on purpose, for tests that must tell a right engine from a nearly
right one: {"window": +1} widens every window by a token, {"keep_first": -1} keeps one token
fewer, {"no_sink": True} drops the sink, {"no_bias": True} the distance bias, {"no_cap": True}
the cap, {"pairing": "halves"} turns the pairs (i, i + n/2), {"no_conv": True} / {"no_gate": True}
/ {"no_blend": True} / {"no_pairs": True} drop one mechanism each.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms_div(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_taps(h, w):
    """sum_j w[:, j] h[t - taps + 1 + j], rows before the start are zero.  h [T, C], w [C, taps]."""
    T, C = h.shape
    taps = w.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def pair_rows(tokens, buckets, mul_prev, mul_cur):
    rows = [buckets]
    for a, b in zip(tokens[:-1], tokens[1:]):
        rows.append((a * mul_prev + b * mul_cur) % buckets)
    return rows


def embed(raw, W, tokens, alter):
    e = raw.get("embedding", {})
    x = W["embed"].to(F)[tokens] * float(e.get("scale", 1.0))
    bg = e.get("bigram")
    if bg is not None and not alter.get("no_pairs"):
        x = x + W["bigram"].to(F)[pair_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])]
    return x


def distance_row(n, rows, far):
    """Which row of a `rows`-row table a distance n >= 0 takes."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def sink_attention(h, W, p, m, eps, first_values, alter):
    """h [T, C] -> [T, C].  `first_values`: a one-element list holding the values of the first blending layer."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ W[p + "q"].to(F).T + W[p + "q.b"].to(F)
    k = h @ W[p + "k"].to(F).T + W[p + "k.b"].to(F)
    v = h @ W[p + "v"].to(F).T + W[p + "v.b"].to(F)
    q = rms_div(q, eps) * W[p + "q.norm"].to(F)                # over all heads at once
    k = rms_div(k, eps) * W[p + "k.norm"].to(F)
    if m.get("v_mix"):
        if first_values[0] is None:
            first_values[0] = v.clone()
        elif not alter.get("no_blend"):
            lam = float(W[p + "vmix"].to(F))
            v = (1.0 - lam) * v + lam * first_values[0]
    q, k, v = q.view(T, H, dk), k.view(T, G, dk), v.view(T, G, dv)
    mask = m.get("mask")
    size = None if mask is None else mask["size"] + alter.get("window", 0)
    keep = 0 if mask is None else max(0, mask.get("keep_first", 0) + alter.get("keep_first", 0))
    cap = None if alter.get("no_cap") else m.get("softcap")
    rel = None if (alter.get("no_bias") or m.get("bias_max") is None) else W[p + "rel"].to(F)
    sink = None if alter.get("no_sink") else W[p + "sink"].to(F)
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    seen = j <= i
    if size is not None:
        seen = seen & ((i - j < size) | (j < keep))
    if rel is not None:
        row_of = torch.tensor([distance_row(n, rel.shape[0], m["bias_max"]) for n in range(T)])
        rows = row_of[(i - j).clamp(min=0)]                                    # [T, T]
    out = torch.zeros(T, H, dv, dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        if rel is not None:
            s = s + rel[:, hd][rows]
        s = s.masked_fill(~seen, float("-inf"))
        top = s.max(-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[hd])
        e = torch.exp(s - top)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[hd] - top)                           # a term without key or value
        out[:, hd] = (e / den) @ v[:, g]
    return out.reshape(T, H * dv) @ W[p + "o"].to(F).T


def turn_pairs(x, positions, base, dims, pairing="interleaved"):
    """Rotates the first `dims` entries of the last axis of x [T, ..., n] at the given positions."""
    out = x.clone()
    for i in range(dims // 2):
        a, b = (2 * i, 2 * i + 1) if pairing == "interleaved" else (i, i + dims // 2)
        ang = positions.to(F) * base ** (-2.0 * i / dims)
        shape = [-1] + [1] * (x.dim() - 2)
        c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
        out[..., a] = x[..., a] * c - x[..., b] * s
        out[..., b] = x[..., b] * c + x[..., a] * s
    return out


def latent_attention(h, W, p, m, eps, alter):
    T = h.shape[0]
    H, dk, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    pairing = alter.get("pairing", "interleaved")
    cq = rms_div(h @ W[p + "dq"].to(F).T, eps) * W[p + "dq.norm"].to(F)
    q = (cq @ W[p + "uq"].to(F).T).view(T, H, dk + dr)
    q_plain, q_rot = q[..., :dk], turn_pairs(q[..., dk:], pos, m["rot"]["base"], m["rot"]["dims"], pairing)
    down = h @ W[p + "dkv"].to(F).T
    c = rms_div(down[:, :rank], eps) * W[p + "dkv.norm"].to(F)
    k_rot = turn_pairs(down[:, rank:], pos, m["rot"]["base"], m["rot"]["dims"], pairing)      # one for all heads
    k_plain = (c @ W[p + "uk"].to(F).T).view(T, H, dk)
    v = (c @ W[p + "uv"].to(F).T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ v[:, hd]
    merged = out.reshape(T, H * dv) * torch.sigmoid(h @ W[p + "g"].to(F).T)
    return merged @ W[p + "o"].to(F).T


def gelu_unit(h, W, p):
    g = h @ W[p + "gate"].to(F).T
    act = 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3)))
    return (act * (h @ W[p + "up"].to(F).T)) @ W[p + "down"].to(F).T


def sublayer(x, W, base, n, run, raw, alter):
    """x + ls * norm(run(h + conv(h)) * sigmoid(rg h + b)), h = x."""
    eps = raw["norm"]["eps"]
    h = x
    hc = h
    if raw.get("canon") and not alter.get("no_conv"):
        hc = h + causal_taps(h, W[f"{base}canon{n}"].to(F))
    y = run(hc)
    if not alter.get("no_gate"):
        y = y * torch.sigmoid(h @ W[f"{base}rg{n}"].to(F).T + W[f"{base}rg{n}.b"].to(F))
    y = rms_div(y, eps) * float(W[f"{base}norm{n}"].to(F)) * W[f"{base}ls{n}"].to(F)
    return x + y


def forward(raw, W, tokens, alter=None, layers_out=None):
    alter = alter or {}
    eps = raw["norm"]["eps"]
    x = embed(raw, W, list(tokens), alter)
    first_values = [None]
    for i, layer in enumerate(raw["layers"]):
        base, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            x = sublayer(x, W, base, 1, lambda hc: sink_attention(hc, W, base + "mix.", m, eps, first_values, alter), raw, alter)
        else:
            x = sublayer(x, W, base, 1, lambda hc: latent_attention(hc, W, base + "mix.", m, eps, alter), raw, alter)
        if layer["mlp"] is not None:
            x = sublayer(x, W, base, 2, lambda hc: gelu_unit(hc, W, base + "mlp."), raw, alter)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms_div(x, eps) * float(W["final.norm"].to(F))
    return x @ W["head"].to(F).T


def greedy(raw, W, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(raw, W, toks)[-1].argmax()))
    return toks[len(prompt):]
