"""Plain implementation of Vagulorn: whole sequences, no cache, float64, one function per mechanism.

It shares no code with the package: it takes the ``config.json`` dictionary and the checkpoint's
tensors by name, and every recurrence is a loop over tokens.  Notation: T tokens, W the width, a head
has ``dim`` query/key entries and ``vdim`` value entries.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + z.clamp(min=0)


def rotate(x, base, dims, interleaved):
    """x [T, heads, dim]: the first ``dims`` entries of every head are turned by position * base^(-2i/dims),
    pair i being entries (i, i + dims/2), or (2i, 2i+1) if ``interleaved``."""
    if dims == 0:
        return x
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=F64)
    ang = torch.arange(T, dtype=F64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    ia = 2 * torch.arange(dims // 2) if interleaved else torch.arange(dims // 2)
    ib = ia + 1 if interleaved else ia + dims // 2
    out = x.clone()
    u, v = x[..., ia], x[..., ib]
    out[..., ia] = u * c - v * s
    out[..., ib] = v * c + u * s
    return out


def visible(T, rule, size, keep_first=0):
    """[T, T] bool: may query i read key j.  rule None: every j <= i; "blocks": j <= i in i's block of
    ``size`` positions; "window": j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if rule == "blocks":
        ok = ok & (i // size == j // size)
    elif rule == "window":
        ok = ok & ((i - j < size) | (j < keep_first))
    return ok


def softmax_attention(q, k, v, scale, ok):
    """q [T, H, dim], k [T, G, dim], v [T, G, vdim]; query head h reads key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~ok, -math.inf)
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return out


def attention(w, p, m, h, eps, beside):
    """The attention mixer from its input rows h [T, W].  ``beside``: the form that stands beside the linear
    attention (values = keys as projected, interleaved rotary pairs, window with kept first keys, a gate per head)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = k.clone() if beside else (h @ w[p + "v"].T).view(T, G, dv)
    q = rms_norm(q, eps) * w[p + "q.norm"]
    k = rms_norm(k, eps) * w[p + "k.norm"]
    rot = m.get("rot")
    if rot:
        q = rotate(q, rot["base"], rot["dims"], beside)
        k = rotate(k, rot["base"], rot["dims"], beside)
    mask = m.get("mask")
    if mask is None:
        ok = visible(T, None, 0)
    elif beside:
        ok = visible(T, "window", mask["size"], mask.get("keep_first", 0))
    else:
        ok = visible(T, "blocks", mask["size"])
    o = softmax_attention(q, k, v, m["scale"], ok)
    if beside:
        o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, -1) @ w[p + "o"].T


def decay_recurrence(decay, k, v, q):
    """Per head S <- decay S + k v^T, o = S^T q.  decay [H]; k, q [T, H, dim]; v [T, H, vdim]."""
    T, H, d = k.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=F64)
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def linear_attention(w, p, m, h, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    o = decay_recurrence(torch.tensor(m["decay"], dtype=F64), k, v, q).reshape(T, H * dv)
    y = rms_norm(o, eps) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def causal_conv(x, taps_w, bias):
    """x [T, C]; taps_w [C, K], column K-1 for the current token; zeros before the first token."""
    T, K = x.shape[0], taps_w.shape[1]
    padded = torch.cat([torch.zeros(K - 1, x.shape[1], dtype=F64), x], 0)
    out = bias[None, :].expand(T, -1).clone()
    for j in range(K):
        out = out + padded[j:j + T] * taps_w[:, j][None, :]
    return out


def selective_recurrence(a, dt, B, C, x, D):
    """Per head S <- a_t S + dt_t B_t x_t^T (S [N, vdim]), y_t = S^T C_t + D x_t.  a, dt [T, H];
    B, C [T, H, N] (already spread from their groups to the heads); x [T, H, vdim]; D [H]."""
    T, H, N = B.shape
    S = torch.zeros(H, N, x.shape[-1], dtype=F64)
    y = torch.zeros_like(x)
    for t in range(T):
        S = a[t][:, None, None] * S + dt[t][:, None, None] * B[t][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnv,hn->hv", S, C[t]) + D[:, None] * x[t]
    return y


def state_space(w, p, m, h, eps):
    T = h.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, V)
    head_group = torch.arange(H) // (H // G)
    B = xbc[:, inner:inner + G * N].view(T, G, N)[:, head_group]
    C = xbc[:, inner + G * N:].view(T, G, N)[:, head_group]
    dt = softplus(dt + w[p + "dt_bias"])
    a = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    y = selective_recurrence(a, dt, B, C, x, w[p + "D"]).reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_norm(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def feed_forward(w, p, h):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def mixer(w, p, layer, h, eps):
    m, kind = layer["mixer"], layer["type"]
    if kind == "attention":
        return attention(w, p, m, h, eps, beside=False)
    if kind == "parallel":
        return (m["left_scale"] * attention(w, p + "left.", m["left"], h, eps, beside=True)
                + m["right_scale"] * linear_attention(w, p + "right.", m["right"], h, eps))
    if kind == "mamba2":
        return state_space(w, p, m, h, eps)
    raise ValueError(kind)


def forward(cfg: dict, weights: dict, tokens, stream_after_layers: list | None = None):
    """Logits [T, vocab] of one sequence (float64)."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        y = mixer(w, p + "mix.", layer, h, eps)
        if layer.get("mlp"):
            y = y + feed_forward(w, p + "mlp.", h)
        x = x + y
        if stream_after_layers is not None:
            stream_after_layers.append(x.clone())
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["embed"].T
