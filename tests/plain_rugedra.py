"""A plain, slow, whole-sequence implementation of the Rugedra design, one function per
mechanism, written from the design's equations.  It is the oracle the engine's Rugedra parts
are compared with; it shares no code with the package (it reads the same ``config.json``
dictionary and the same tensor names, nothing else).  Everything is computed in the dtype of
the tensors it is given (tests pass 32- or 64-bit floats).

Notation: ``T`` tokens of one sequence, positions ``0 .. T-1``; ``x`` is ``[T, width]``.
"""

from __future__ import annotations

import math

import torch


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate_interleaved(x, positions, base, dims):
    """``x``: [T, ..., D].  The first ``dims`` entries of the last axis are rotated in pairs
    (2i, 2i+1) by the angle ``p * base^(-2i/dims)``; the rest pass unchanged."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]  # [T, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = ang.cos().view(shape), ang.sin().view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_attention(h, w, p, cfg, eps, positions=None):
    """``w``: the mixer's tensors by short name (q, dkv, dkv.norm, uk, uv, g, o)."""
    T = h.shape[0]
    H, dim, rot, vdim, rank = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"], cfg["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    q = (h @ w["q"].T).view(T, H, dim + rot)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    dkv = h @ w["dkv"].T
    c = rms_unit(dkv[:, :rank], eps) * w["dkv.norm"]
    k_rot = dkv[:, rank:]
    q_rot = rotate_interleaved(q_rot, pos, cfg["rot"]["base"], cfg["rot"]["dims"])
    k_rot = rotate_interleaved(k_rot, pos, cfg["rot"]["base"], cfg["rot"]["dims"])
    k_plain = (c @ w["uk"].T).view(T, H, dim)
    v = (c @ w["uv"].T).view(T, H, vdim)
    scores = torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thd,sd->hts", q_rot, k_rot)
    scores = scores * cfg["scale"]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, float("-inf"))
    probs = scores.softmax(-1)
    out = torch.einsum("hts,shd->thd", probs, v)
    gate = torch.sigmoid(h @ w["g"].T)  # [T, H]
    out = out * gate[..., None]
    return out.reshape(T, H * vdim) @ w["o"].T


def short_conv_silu(x, taps_w):
    """``x``: [T, C]; ``taps_w``: [C, taps], the last column weighs the current token; zeros
    before the start.  Then silu."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x])
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j: j + T] * taps_w[:, j]
    return y * torch.sigmoid(y)


def channel_delta(h, w, cfg, eps):
    """Gated delta rule with one decay per head and key channel.  ``w``: the mixer's tensors by
    short name."""
    T = h.shape[0]
    H, KH, dim, vdim = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = short_conv_silu(h @ w["q"].T, w["q.conv"]).view(T, KH, dim)
    k = short_conv_silu(h @ w["k"].T, w["k.conv"]).view(T, KH, dim)
    v = short_conv_silu(h @ w["v"].T, w["v.conv"]).view(T, H, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)  # [T, H]
    a = (h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]
    decay = torch.exp(-torch.exp(w["A_log"])[None, :, None] * torch.nn.functional.softplus(a.view(T, H, dim)))
    rep = H // KH
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        kh = hd // rep
        for t in range(T):
            S = decay[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            out[t, hd] = S.T @ q[t, kh]
    out = rms_unit(out, eps) * w["norm"]
    gate = torch.sigmoid((h @ w["g1"].T) @ w["g2"].T).view(T, H, vdim)
    return (out * gate).reshape(T, H * vdim) @ w["o"].T


def dense_ff(h, w):
    z = torch.relu(h @ w["up"].T)
    return (z * z) @ w["down"].T


def expert_ff(h, gate_w, up_w, down_w, limit):
    g = torch.clamp(h @ gate_w.T, max=limit)
    u = torch.clamp(h @ up_w.T, min=-limit, max=limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1)
    return y @ down_w.T


def route(h, router_w, cfg):
    """Returns (chosen experts [T, top], their weights [T, top])."""
    r = cfg["router"]
    E, top = r["experts"], r["top"]
    groups, keep = r["groups"]["count"], r["groups"]["keep"]
    s = (h @ router_w.T).softmax(-1)  # [T, E]
    per = E // groups
    group_score = s.view(-1, groups, per).max(-1).values  # [T, groups]
    kept = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros(s.shape[0], groups, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    allowed = allowed[:, :, None].expand(-1, -1, per).reshape(-1, E)
    masked = s.masked_fill(~allowed, -1.0)
    chosen = masked.topk(top, dim=-1).indices
    weights = s.gather(1, chosen)
    return chosen, weights / (weights.sum(-1, keepdim=True) + 1e-20)


def moe_ff(h, w, cfg):
    chosen, weights = route(h, w["router"], cfg)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t].tolist(), weights[t]):
            out[t] += wt * expert_ff(h[t: t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"],
                                     cfg["expert"]["limit"])[0]
    return out


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, ids: list[int], dtype=torch.float32, return_layers=False):
    """Logits ``[T, vocab]`` of one sequence; with ``return_layers`` also the residual stream
    after every layer ``[layers, T, width]``."""
    w = {k: v.to(dtype) for k, v in tensors.items()}
    eps, m = config["norm"]["eps"], config["residual_mult"]
    T = len(ids)
    x = w["embed"][torch.tensor(ids)] + w["pos"][:T]
    layers = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], eps)
        mix = _sub(w, p + "mix.")
        if layer["type"] == "latent_attention":
            y = latent_attention(h, mix, p, layer["mixer"], eps)
        elif layer["type"] == "channel_delta":
            y = channel_delta(h, mix, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + m * y
        if layer.get("mlp") is not None:
            h = layer_norm(x, w[p + "norm2"], eps)
            mlp = _sub(w, p + "mlp.")
            y = dense_ff(h, mlp) if layer["mlp"]["kind"] == "dense" else moe_ff(h, mlp, layer["mlp"])
            x = x + m * y
        layers.append(x)
    logits = (layer_norm(x, w["final.norm"], eps) @ w["head"].T) * config["logit_scale"]
    return (logits, torch.stack(layers)) if return_layers else logits
