"""A plain, slow implementation of the Galupel design in float64, one function per mechanism, whole sequences only.

It shares nothing with the engine: it reads config.json and the safetensors file itself, keeps no cache, and computes every
position of a sequence from all of its tokens with dense masks.

    norm in groups      a row is cut into n equal consecutive parts, each divided by sqrt(mean(part^2) + eps); times a weight
    a layer             x <- x + norm1(mixer(x));  x <- x + norm2(ff(x))          (the sub-layers read x itself)
    attention           q, k RMS-normed per head (weights shared by the heads), no positions; score q.k * scale * temp[head];
                        query i sees j with 0 <= i - j < w, and the mean key / mean value of every block b of P tokens with
                        b P + P - 1 <= i - w; one softmax over both; kv_from: another layer's keys and values
    latent attention    c = rms_norm(first kv_rank rows of W_dkv h) * weight; the last rot_dim rows are a rotated key part
                        shared by the heads; keys W_uk c, values W_uv c; rotation of neighbouring pairs; a window
    feed-forward        experts W_down gelu(W_up h); s = sigmoid(W_router h); choice by s + correction inside the best groups
                        (a group's score: its two largest choice scores); weights s, not renormalised
    output              norm, the embedding matrix, a scale, a cap c tanh(z / c)
"""
from __future__ import annotations

import json
import math
import os

import torch
from safetensors import safe_open

F64 = torch.float64


def load_folder(folder: str):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt", device="cpu") as f:
        for name in f.keys():
            w[name] = f.get_tensor(name).to(F64)
    return cfg, w


def group_norm(x, weight, groups: int, eps: float):
    T, W = x.shape
    parts = x.reshape(T, groups, W // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(T, W) * weight


def rms_norm(x, weight, eps: float):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def pooled_window_weights(scores_tokens, scores_blocks, window: int, block: int):
    """Softmax over the tokens of the window and the blocks wholly in front of it.  ``scores_tokens`` [T, T],
    ``scores_blocks`` [T, n_blocks]; returns the two parts of the weights."""
    T, nb = scores_tokens.shape[0], scores_blocks.shape[1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    b = torch.arange(nb)[None, :]
    st = scores_tokens.masked_fill(~((i - j >= 0) & (i - j < window)), -math.inf)
    sb = scores_blocks.masked_fill(~(b * block + block - 1 <= i - window), -math.inf)
    a = torch.softmax(torch.cat([st, sb], 1), -1)
    return a[:, :T], a[:, T:]


def attention(m: dict, w: dict, pre: str, h, eps: float, kv_of_layer: dict, layer: int):
    T = h.shape[0]
    H, G, Dk, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ w[pre + "q"].T).reshape(T, H, Dk), w[pre + "q.norm"], eps)
    if m.get("kv_from") is not None:
        k, v = kv_of_layer[m["kv_from"]]
    else:
        k = rms_norm((h @ w[pre + "k"].T).reshape(T, G, Dk), w[pre + "k.norm"], eps)
        v = (h @ w[pre + "v"].T).reshape(T, G, Dv)
        kv_of_layer[layer] = (k, v)
    window, P = m["mask"]["size"], m["mask"].get("pool")
    nb = T // P if P else 0
    kp = k[:nb * P].reshape(nb, P, G, Dk).mean(1) if nb else k.new_zeros(0, G, Dk)
    vp = v[:nb * P].reshape(nb, P, G, Dv).mean(1) if nb else v.new_zeros(0, G, Dv)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        f = m["scale"] * w[pre + "temp"][hd]
        at, ab = pooled_window_weights(q[:, hd] @ k[:, g].T * f, q[:, hd] @ kp[:, g].T * f, window, P or 1)
        out[:, hd] = at @ v[:, g] + ab @ vp[:, g]
    return out.reshape(T, H * Dv) @ w[pre + "o"].T


def rotate_pairs(x, dims: int, base: float):
    """x [T, ..., R]: the pair (x[2i], x[2i+1]), i < dims / 2, turned by position * base^(-2i / dims)."""
    if not dims:
        return x
    T = x.shape[0]
    x = x.clone()
    a = torch.arange(T, dtype=F64)[:, None] * base ** (-2 * torch.arange(dims // 2, dtype=F64) / dims)[None, :]
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    u, v = x[..., 0:dims:2].clone(), x[..., 1:dims:2].clone()
    x[..., 0:dims:2] = u * torch.cos(a) - v * torch.sin(a)
    x[..., 1:dims:2] = v * torch.cos(a) + u * torch.sin(a)
    return x


def latent_attention(m: dict, w: dict, pre: str, h, eps: float):
    T = h.shape[0]
    H, Dk, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[pre + "q"].T).reshape(T, H, Dk + R)
    d = h @ w[pre + "dkv"].T
    c = rms_norm(d[:, :C], w[pre + "dkv.norm"], eps)
    k_plain = (c @ w[pre + "uk"].T).reshape(T, H, Dk)
    v = (c @ w[pre + "uv"].T).reshape(T, H, Dv)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q_rot, k_rot = rotate_pairs(q[:, :, Dk:], rot["dims"], rot["base"]), rotate_pairs(d[:, C:], rot["dims"], rot["base"])
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = i - j >= 0
    if m.get("mask"):
        seen = seen & (i - j < m["mask"]["size"])
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        s = (q[:, hd, :Dk] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        out[:, hd] = torch.softmax(s.masked_fill(~seen, -math.inf), -1) @ v[:, hd]
    return out.reshape(T, H * Dv) @ w[pre + "o"].T


def route(z, correction, top: int, count: int, keep: int):
    """-> (chosen experts [T, top], their weights)."""
    T, E = z.shape
    s = torch.sigmoid(z)
    choice = s + correction
    per = E // count
    grouped = choice.reshape(T, count, per)
    group_score = grouped.topk(min(2, per), -1).values.sum(-1)
    kept = torch.zeros(T, count, dtype=torch.bool)
    kept.scatter_(1, group_score.topk(keep, -1).indices, True)
    choice = choice.masked_fill(~kept[:, :, None].expand(T, count, per).reshape(T, E), -math.inf)
    idx = choice.topk(top, -1).indices
    return idx, s.gather(1, idx)


def experts(mlp: dict, w: dict, pre: str, h):
    r = mlp["router"]
    g = r.get("groups") or {"count": 1, "keep": 1}
    idx, wgt = route(h @ w[pre + "router"].T, w[pre + "correction"], r["top"], g["count"], g["keep"])
    out = torch.zeros_like(h)
    for e in range(r["experts"]):
        y = torch.nn.functional.gelu(h @ w[pre + f"e{e}.up"].T) @ w[pre + f"e{e}.down"].T
        share = (wgt * (idx == e)).sum(-1, keepdim=True)
        out += share * y
    return out


def forward(cfg: dict, w: dict, tokens, streams_out: list | None = None):
    """Logits [T, vocab] of every position.  ``streams_out`` collects the residual stream after every layer."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    x = group_norm(w["embed"][torch.as_tensor(tokens)], w["embed.norm"], groups, eps)
    kv_of_layer: dict = {}
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        if layer["type"] == "attention":
            y = attention(layer["mixer"], w, pre + "mix.", x, eps, kv_of_layer, i)
        else:
            y = latent_attention(layer["mixer"], w, pre + "mix.", x, eps)
        x = x + group_norm(y, w[pre + "norm1"], groups, eps)
        if layer["mlp"] is not None:
            x = x + group_norm(experts(layer["mlp"], w, pre + "mlp.", x), w[pre + "norm2"], groups, eps)
        if streams_out is not None:
            streams_out.append(x.clone())
    z = group_norm(x, w["final.norm"], groups, eps) @ w["embed"].T * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z
