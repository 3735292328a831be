"""A plain, slow, whole-sequence implementation of the Ravapel design, one function per mechanism.

Written from the design's equations only; it shares no code with the package.  Everything runs
in the dtype of the weights it is given (the tests pass 64-bit copies).  ``forward`` returns the
logits of every position of one sequence.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm with a weight stored around zero."""
    return rms(x, eps) * (1 + w)


def embed(tokens, W, cfg):
    """Token rows, hashed bigram rows (the last row for the first token), learned positions."""
    ids = torch.tensor(tokens)
    x = W["embed"][ids]
    big = (cfg.get("embedding") or {}).get("bigram")
    if big:
        rows = [big["buckets"]] + [(tokens[i - 1] * big["mul_prev"] + tokens[i] * big["mul_cur"]) % big["buckets"]
                                   for i in range(1, len(tokens))]
        x = x + W["bigram"][torch.tensor(rows)]
    return x + W["pos"][: len(tokens)]


def causal_conv(h, w):
    """conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j), zeros before the start; h: [T, C], w: [C, taps]."""
    T, taps = h.shape[0], w.shape[1]
    padded = torch.cat([h.new_zeros(taps - 1, h.shape[1]), h])
    return sum(w[:, j] * padded[j: j + T] for j in range(taps))


def hgrn2_recurrence(q, f, v):
    """q, f: [T, H, d]; v: [T, H, dv].  S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T; o_t = S_t^T q_t."""
    T, H, d = q.shape
    S = q.new_zeros(H, d, v.shape[-1])
    out = []
    for t in range(T):
        S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out)


def hgrn2(h, W, p, m, eps):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = F.silu(h @ W[p + ".q"].T).view(T, H, d)
    v = (h @ W[p + ".v"].T).view(T, H, dv)
    lower = W[p + ".lower"]
    f = (lower + (1 - lower) * torch.sigmoid(h @ W[p + ".f"].T + W[p + ".f.b"])).view(T, H, d)
    o = rms(hgrn2_recurrence(q, f, v), eps) * W[p + ".norm"]
    return o.reshape(T, H * dv) @ W[p + ".o"].T


def rotate_halves(x, positions, dims, base):
    """The first `dims` entries of each head: entry i pairs with entry i + dims / 2."""
    if not dims:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = angle.cos()[:, None, :], angle.sin()[:, None, :]
    u, w = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - w * s, w * c + u * s, x[..., dims:]], dim=-1)


def sigmoid_chunk_attention(q, k, v, scale, head_bias, chunk):
    """q: [T, H, d]; k: [T, G, d]; v: [T, G, dv].  Weight of a visible key: sigmoid(score + bias[h]),
    not normalised; position i sees j <= i in the same chunk (counted from position 0)."""
    T, H, _ = q.shape
    G = k.shape[1]
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if chunk:
        visible = visible & ((pos[None, :] // chunk) == (pos[:, None] // chunk))
    out = q.new_zeros(T, H, v.shape[-1])
    for h in range(H):
        g = h // (H // G)
        w = torch.sigmoid((q[:, h] @ k[:, g].T) * scale + head_bias[h]) * visible
        out[:, h] = w @ v[:, g]
    return out


def left_attention(h, W, p, m, eps):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms((h @ W[p + ".q"].T).view(T, H, d), eps) * W[p + ".q.norm"]
    k = rms((h @ W[p + ".k"].T).view(T, G, d), eps) * W[p + ".k.norm"]
    v = (h @ W[p + ".v"].T).view(T, G, dv)
    rot = m.get("rot") or {}
    pos = torch.arange(T)
    q = rotate_halves(q, pos, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_halves(k, pos, rot.get("dims", 0), rot.get("base", 1.0))
    chunk = (m.get("mask") or {}).get("size")
    o = sigmoid_chunk_attention(q, k, v, m["scale"], W[p + ".pb"], chunk)
    return o.reshape(T, H * dv) @ W[p + ".o"].T


def mlstm_recurrence(q, k, v, logi, logf):
    """q, k: [T, H, d]; v: [T, H, dv]; logi, logf: [T, H].  Returns o [T, H, dv]."""
    T, H, d = q.shape
    S, n, m = q.new_zeros(H, d, v.shape[-1]), q.new_zeros(H, d), q.new_zeros(H)
    out = []
    for t in range(T):
        m_new = torch.maximum(logf[t] + m, logi[t])
        a, b = torch.exp(logf[t] + m - m_new), torch.exp(logi[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out.append(torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None])
    return torch.stack(out)


def mlstm(h, W, p, m, eps):
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    T = h.shape[0]
    q = (h @ W[p + ".q"].T).view(T, H, d) * d ** -0.5
    k = (h @ W[p + ".k"].T).view(T, H, d)
    v = (h @ W[p + ".v"].T).view(T, H, dv)
    logi = cap * torch.tanh((h @ W[p + ".i"].T + W[p + ".i.b"]) / cap)
    logf = F.logsigmoid(cap * torch.tanh((h @ W[p + ".f"].T + W[p + ".f.b"]) / cap))
    o = rms(mlstm_recurrence(q, k, v, logi, logf), eps).reshape(T, H * dv) * W[p + ".norm"]
    return (o * torch.sigmoid(h @ W[p + ".g"].T)) @ W[p + ".o"].T


def feed_forward(h, W, p):
    g = h @ W[p + ".gate"].T + W[p + ".gate.b"]
    u = h @ W[p + ".up"].T + W[p + ".up.b"]
    return (F.silu(g) * u) @ W[p + ".down"].T + W[p + ".down.b"]


def layer(i, x, cfg, W):
    spec, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}"
    h = norm_one_plus(x, W[p + ".norm1"], eps)
    if cfg.get("canon"):
        h = h + causal_conv(h, W[p + ".canon1"])
    if spec["type"] == "hgrn2":
        y = hgrn2(h, W, p + ".mix", spec["mixer"], eps)
    else:
        mx = spec["mixer"]
        y = (mx["left_scale"] * left_attention(h, W, p + ".mix.left", mx["left"], eps)
             + mx["right_scale"] * mlstm(h, W, p + ".mix.right", mx["right"], eps))
    x = x + norm_one_plus(y, W[p + ".norm1b"], eps)
    if spec.get("mlp") is not None:
        y = feed_forward(norm_one_plus(x, W[p + ".norm2"], eps), W, p + ".mlp")
        x = x + norm_one_plus(y, W[p + ".norm2b"], eps)
    return x


def forward(cfg, weights, tokens, dtype=torch.float64, streams=None):
    W = {k: v.to(dtype) for k, v in weights.items()}
    x = embed(tokens, W, cfg)
    x0 = x
    loop, n = cfg.get("loop"), len(cfg["layers"])
    if loop:
        order = list(range(loop["start"]))
        for _ in range(loop["times"]):
            order += ["in"] + list(range(loop["start"], loop["stop"])) if loop["stop"] > loop["start"] else []
        order += list(range(loop["stop"], n))
    else:
        order = list(range(n))
    for step in order:
        if step == "in":
            x = torch.cat([x, x0], dim=-1) @ W["loop.in"].T
        else:
            x = layer(step, x, cfg, W)
            if streams is not None:
                streams.append(x)
    x = norm_one_plus(x, W["final.norm"], cfg["norm"]["eps"])
    return x @ W["head"].T
