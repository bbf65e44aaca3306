"""Plain, slow implementation of the Kogonex decoder for whole sequences.

No cache, no batching, no kernels: one function per mechanism, written from the equations, in
the dtype of the tensors it is given (float64 in the tests).  It shares no code with the engine
under ``acorninfer_b200/``: it takes the raw ``config.json`` dictionary and a dict of tensors by
checkpoint name.

The model, in this file's notation (x is the residual stream, one row per token):

  x = embed[t] + bigram[row(prev, t)]
  for every layer:  x += norm1(mixer(x));  x += norm2(ff(x))      (norms on the outputs only)
  logits = head . norm_final(x)

with two mixers (attention through a shared low-rank latent with a sliding window and a per-head
sink; a gated delta rule with one decay per key channel) and a routed mixture of small SwiGLU
experts of which some are the identity.
"""

from __future__ import annotations

import math

import torch


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last dimension."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------ embedding


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every token: a hash of (previous token, token) into ``buckets``
    rows; a sequence's first token has no previous one and takes the extra row ``buckets``."""
    rows = [buckets]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((int(prev) * mul_prev + int(cur) * mul_cur) % buckets)
    return rows


def embed(cfg, w, tokens):
    x = w["embed"][torch.as_tensor(tokens)]
    b = cfg["embedding"].get("bigram") if cfg.get("embedding") else None
    if b:
        x = x + w["bigram"][torch.as_tensor(bigram_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"]))]
    return x


# ------------------------------------------------------------------ rotary positions


def rotary_frequencies(rot):
    """(frequency of every rotated pair, factor on cos and sin).  Plain: f_i = base^(-2i/dims).
    With ``scaling``: pairs that turn fast keep f_i, pairs that turn slowly get f_i / factor, a linear
    ramp over the pair index between, and cos/sin are stretched by 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def pair_of(turns):
        return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, rot):
    """Rotates the pairs (2i, 2i+1) of the first ``dims`` entries of the last dimension by
    position * frequency_i; the rest passes.  x: [tokens, ..., n]."""
    f, mag = rotary_frequencies(rot)
    dims = rot["dims"]
    ang = torch.as_tensor(positions, dtype=torch.float64)[:, None] * torch.tensor(f, dtype=torch.float64)[None]
    cos, sin = (ang.cos() * mag).to(x.dtype), (ang.sin() * mag).to(x.dtype)
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ------------------------------------------------------------------ latent attention


def latent_and_key(m, w, p, h, eps):
    """What a layer keeps of every token: the normed latent c [T, rank] and the rotated key part
    shared by all heads [T, rot_dim]."""
    T = h.shape[0]
    d = h @ w[p + "dkv"].T
    c = rms_norm(d[:, :m["kv_rank"]], w[p + "dkv.norm"], eps)
    kr = rotate(d[:, m["kv_rank"]:], range(T), m["rot"])
    return c, kr


def windowed_sink_softmax(scores, sink, window):
    """scores [T, T] of one head (query, key).  Query i sees key j if 0 <= i - j < window (no
    window: j <= i).  The denominator holds exp(sink) besides the seen keys' terms."""
    T = scores.shape[0]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) if window is None else ((j <= i) & (i - j < window))
    s = scores.masked_fill(~seen, float("-inf"))
    top = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))


def latent_attention(m, w, p, h, eps, shared=None):
    """Returns (output [T, width], (c, kr)).  ``shared``: another layer's (c, kr) to read instead of
    making its own."""
    T = h.shape[0]
    H, dim, rd, vd = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, dim + rd)
    qu, qr = q[..., :dim], rotate(q[..., dim:], range(T), m["rot"])
    c, kr = shared if shared is not None else latent_and_key(m, w, p, h, eps)
    ku = (c @ w[p + "uk"].T).view(T, H, dim)
    v = (c @ w[p + "uv"].T).view(T, H, vd)
    window = m["mask"]["size"] if m.get("mask") else None
    heads = []
    for a in range(H):
        s = (qu[:, a] @ ku[:, a].T + qr[:, a] @ kr.T) * m["scale"]
        heads.append(windowed_sink_softmax(s, w[p + "sink"][a], window) @ v[:, a])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T, (c, kr)


# ------------------------------------------------------------------ gated delta rule


def short_conv(x, taps_w):
    """Causal convolution over time per channel: y[t, c] = sum_j w[c, j] x[t - (taps-1) + j, c],
    zeros before the start (the last column weighs the current token)."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + T] * taps_w[:, j][None]
    return y


def channel_delta(m, w, p, h, eps):
    """Per head: a matrix S [dim, vdim], zero at the start.  For every token, with unit-length q and
    k (q further times dim^-1/2), a write strength beta in (0, 1) and a decay g in (0, 1) per key
    channel:  S = g[:, None] * S;  u = beta * (v - S^T k);  S += k u^T;  o = S^T q."""
    T = h.shape[0]
    H, KH, dim, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, KH, dim)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, KH, dim)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, vd)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                   # [T, H]
    step = torch.nn.functional.softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(T, H, dim)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * step)          # [T, H, dim]
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, vd)
    rep = H // KH
    out = torch.zeros(T, H, vd, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(dim, vd, dtype=h.dtype)
        for t in range(T):
            kt, qt = k[t, a // rep], q[t, a // rep]
            S = g[t, a][:, None] * S
            u = beta[t, a] * (v[t, a] - S.T @ kt)
            S = S + torch.outer(kt, u)
            out[t, a] = S.T @ qt
    out = rms_norm(out, w[p + "norm"], eps) * gate
    return out.reshape(T, H * vd) @ w[p + "o"].T


# ------------------------------------------------------------------ mixture of experts


def route(r, z, correction):
    """z: router logits of one token over experts + identity experts.  Returns [(expert, weight)]:
    the ``top`` largest of softmax(z) + correction among the experts of the ``keep`` groups whose
    largest such score is largest; the weight is softmax(z) itself, not renormalized."""
    s = torch.softmax(z, -1)
    choice = s + correction
    n = choice.numel()
    groups = r.get("groups")
    if groups:
        per = n // groups["count"]
        best = choice.view(groups["count"], per).max(-1).values
        kept = torch.topk(best, groups["keep"]).indices.tolist()
        allowed = torch.zeros(n, dtype=torch.bool)
        for gi in kept:
            allowed[gi * per:(gi + 1) * per] = True
        choice = choice.masked_fill(~allowed, float("-inf"))
    picked = torch.topk(choice, r["top"]).indices.tolist()
    return [(e, s[e]) for e in picked]


def moe(f, w, p, h):
    r = f["router"]
    z = h @ w[p + "router"].T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in route(r, z[t], w[p + "correction"]):
            if e >= r["experts"]:                                    # an identity expert
                y = h[t]
            else:
                ep = f"{p}e{e}."
                y = (silu(h[t] @ w[ep + "gate"].T) * (h[t] @ w[ep + "up"].T)) @ w[ep + "down"].T
            out[t] = out[t] + weight * y
    return out


# ------------------------------------------------------------------ the model


def forward(cfg, weights, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of a whole sequence (and the residual stream after every layer)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = embed(cfg, w, tokens)
    kept, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "latent_attention":
            y, kept[i] = latent_attention(m, w, p, x, eps, kept[m["kv_from"]] if m.get("kv_from") is not None else None)
        elif layer["type"] == "channel_delta":
            y = channel_delta(m, w, p, x, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp"):
            x = x + rms_norm(moe(layer["mlp"], w, f"l{i}.mlp.", x), w[f"l{i}.norm2"], eps)
        after.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
