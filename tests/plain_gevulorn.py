"""A plain, slow Gevulorn in float64 torch on the CPU: one function per mechanism, written from the design's equations.

It shares no code with the engine: weights are a dict from disk names to tensors, a sequence is processed whole, the
attention is a loop over queries and the recurrence a loop over tokens.  Notation: T tokens, W the model width, H query
heads, G key/value heads, D the size of a query or key head, Dv of a value head.
"""
from __future__ import annotations

import json
import math
import os

import torch
from safetensors import safe_open


def load_folder(folder: str, dtype=torch.float64):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt", device="cpu") as f:
        for name in f.keys():
            t = f.get_tensor(name)
            w[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, w


# ---- small pieces ---------------------------------------------------------------------------------
def layer_norm(x, weight, bias, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis, var the mean of the squared deviations."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight + bias


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def soft_cap(z, cap):
    return cap * torch.tanh(z / cap)


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims) for i < dims/2; with ``scaling`` {factor, low, high, original}: a frequency whose wavelength
    l = 2 pi / f is shorter than original/high stays, one longer than original/low is divided by factor, and between the
    two the divided and the plain frequency are blended by s = (original/l - low) / (high - low)."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling:
        fac, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for x in f:
            l = 2 * math.pi / x
            if l < orig / high:
                out.append(x)
            elif l > orig / low:
                out.append(x / fac)
            else:
                s = (orig / l - low) / (high - low)
                out.append((1 - s) * x / fac + s * x)
        f = out
    return f


def rotate_halves(x, positions, freqs):
    """Rotary positions on the first 2 * len(freqs) elements of the last axis: element i is paired with element
    i + len(freqs).  x [T, heads, D]; positions [T]."""
    out = x.clone()
    half = len(freqs)
    for i, f in enumerate(freqs):
        a = positions.to(x.dtype) * f
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


# ---- masks ----------------------------------------------------------------------------------------
def sees_window(i, j, size, keep_first):
    """A sliding window that also keeps the sequence's first tokens."""
    return j <= i and (i - j < size or j < keep_first)


def sees_chunk(i, j, size):
    """Only keys of the query's own chunk; chunks are counted from position 0."""
    return j <= i and i // size == j // size


# ---- attention ------------------------------------------------------------------------------------
def sink_softmax_attention(q, k, v, scale, sees, sinks, cap=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv].  ``sees(i, j)`` says which keys a query sees; the weights
    are exp(s_j) / (exp(sink_h) + sum exp(s_j)): the sink has neither key nor value and is neither scaled nor capped.
    ``cap``: s <- cap tanh(s / cap) after scaling."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for i in range(T):
        js = [j for j in range(i + 1) if sees(i, j)]
        for h in range(H):
            g = h // (H // G)
            s = (k[js, g] @ q[i, h]) * scale
            if cap is not None:
                s = soft_cap(s, cap)
            m = torch.maximum(s.max(), sinks[h])
            e = torch.exp(s - m)
            out[i, h] = (e[:, None] * v[js, g]).sum(0) / (e.sum() + torch.exp(sinks[h] - m))
    return out


def attention_mixer(h, w, p, m, eps):
    """Mixer 'attention': no biases; rotation, then q and k divided by their root mean square (no weight); a window that
    keeps the first tokens; a learned sink per head."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, Dv)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot and rot["dims"]:
        f = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate_halves(q, pos, f), rotate_halves(k, pos, f)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    mask = m.get("mask") or {}
    size, keep = mask.get("size"), mask.get("keep_first", 0)
    sees = (lambda i, j: sees_window(i, j, size, keep)) if size is not None else (lambda i, j: j <= i)
    o = sink_softmax_attention(q, k, v, m["scale"], sees, w[p + "sink"])
    return o.reshape(T, H * Dv) @ w[p + "o"].T


def attention_2_mixer(h, w, p, m, eps):
    """Mixer 'attention_2': biased projections; weighted RMS norm of q and k before the rotation; scaled frequencies;
    capped scores; chunked mask; a learned sink per head."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, D)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, D)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, Dv)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot and rot["dims"]:
        f = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate_halves(q, pos, f), rotate_halves(k, pos, f)
    mask = m.get("mask") or {}
    size = mask.get("size")
    sees = (lambda i, j: sees_chunk(i, j, size)) if size is not None else (lambda i, j: j <= i)
    o = sink_softmax_attention(q, k, v, m["scale"], sees, w[p + "sink"], cap=m.get("softcap"))
    return o.reshape(T, H * Dv) @ w[p + "o"].T + w[p + "o.b"]


# ---- gated linear attention -----------------------------------------------------------------------
def gla_mixer(h, w, p, m, eps, state=None):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T and o_t = S_t^T q_t per head, alpha = sigmoid(z)^(1/tau) per key channel
    with z from a low-rank projection; each head's o is RMS-normed with a weight shared by the heads, the heads are
    multiplied by silu(W_g h) and projected.  Returns (output, final state [H, D, Dv])."""
    T = h.shape[0]
    H, D, Dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ w[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, Dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / tau)).view(T, H, D)
    S = torch.zeros(H, D, Dv, dtype=h.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit_rms(o, eps) * w[p + "norm"]
    return (o.reshape(T, H * Dv) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T, S


# ---- feed-forwards --------------------------------------------------------------------------------
def squared_relu_mlp(h, w, p):
    return (torch.relu(h @ w[p + "up"].T) ** 2) @ w[p + "down"].T


def gated_expert(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_experts(h, w, p, mlp, chosen_out=None):
    """Top-k routing: a token goes to the ``top`` experts of largest router logit, mixed by a softmax taken over those
    ``top`` logits alone; plus the shared expert, if the layer has one."""
    top = mlp["router"]["top"]
    z = h @ w[p + "router"].T
    val, idx = torch.topk(z, top, dim=-1)
    wgt = torch.softmax(val, -1)
    if chosen_out is not None:
        chosen_out.append((z, idx))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            out[t] += wgt[t, c] * gated_expert(h[t:t + 1], w, f"{p}e{int(idx[t, c])}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, w, p + "shared.")
    return out


def feed_forward(h, w, p, mlp):
    if mlp["kind"] == "dense":
        return squared_relu_mlp(h, w, p)
    return routed_experts(h, w, p, mlp)


# ---- the model ------------------------------------------------------------------------------------
def layer_runs(cfg):
    """The order in which layers run, as (layer, pass) pairs: the block of layers [start, stop) is repeated ``times`` times
    back to back.  ``pass`` numbers the repetition at its first layer (where that repetition's vector joins the stream) and is
    None everywhere else."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    after = []
    for i, step in layer_runs(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        if step is not None:
            x = x + w["loop.step"][step]
        h1 = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        kind, m = layer["type"], layer["mixer"]
        if kind == "gla":
            y, _ = gla_mixer(h1, w, p + "mix.", m, eps)
        elif kind == "attention":
            y = attention_mixer(h1, w, p + "mix.", m, eps)
        elif kind == "attention_2":
            y = attention_2_mixer(h1, w, p + "mix.", m, eps)
        else:
            raise ValueError(kind)
        if layer.get("mlp"):
            y = y + feed_forward(layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps), w, p + "mlp.", layer["mlp"])
        x = x + y
        after.append(x)
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    if cfg.get("logit_softcap"):
        logits = soft_cap(logits, cfg["logit_softcap"])
    return (logits, torch.stack(after)) if return_layers else logits
