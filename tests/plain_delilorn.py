"""A plain, slow Delilorn in float64 on the CPU: one function per mechanism, whole sequences only
(no cache, no state carried between calls, no batches).  It shares no code with the package;
the GPU tests hold the engine to it.

Notation: x [T, width] is the stream, h the normalised input of a sub-layer, W[name] the
checkpoint tensor of that name (linear weights [out, in], applied as h @ W.T)."""
from __future__ import annotations

import json
import math
import os

import torch
from safetensors.torch import load_file


def load_folder(folder):
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    weights = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return cfg, weights


# ----------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """The block norms and the final norm: their weight is stored as its distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    """The norms inside the mixers: their weight is the factor itself."""
    return unit_rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def frequencies(rot):
    """f_i = base^(-2i/dims), with the long waves stretched where ``rot`` has a "scaling"."""
    dims, base = rot["dims"], rot["base"]
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            wave = 2.0 * math.pi / f
            if wave > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif not wave < sc["original"] / sc["high"]:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


def rotate(x, positions, rot):
    """x [T, heads, n]: element i < dims/2 is paired with i + dims/2; the pair at position p turns
    by the angle p * f_i.  Elements from ``dims`` on pass."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    half = dims // 2
    ang = positions.double()[:, None] * frequencies(rot)[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def visible(i, j, mask):
    """May the query at position i see the key at position j?"""
    if j > i:
        return False
    if not mask:
        return True
    return i - j < mask["size"] or j < mask.get("keep_first", 0)


# ----------------------------------------------------------------------------- mixers
def window_attention(h, W, p, m):
    """Grouped-query softmax attention, rotary on the first rot.dims of every head, a window of
    mask.size keys beside the first mask.keep_first of the sequence."""
    T = h.shape[0]
    H, G, n, nv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate((h @ W[p + "q"].T).view(T, H, n), pos, m.get("rot"))
    k = rotate((h @ W[p + "k"].T).view(T, G, n), pos, m.get("rot"))
    v = (h @ W[p + "v"].T).view(T, G, nv)
    out = torch.zeros(T, H, nv, dtype=torch.float64)
    for a in range(H):
        g = a // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, m.get("mask"))]
            s = (k[js, g] @ q[i, a]) * m["scale"]
            out[i, a] = torch.softmax(s, 0) @ v[js, g]
    return out.reshape(T, H * nv) @ W[p + "o"].T


def latent_kv(h, W, p, m, eps):
    """What a latent-attention layer keeps per token: the normed latent and the one rotated key
    part that all heads share."""
    T = h.shape[0]
    r = m["kv_rank"]
    down = h @ W[p + "dkv"].T
    c = norm_plain(down[:, :r], W[p + "dkv.norm"], eps)
    k_rot = rotate(down[:, None, r:], torch.arange(T), m.get("rot"))[:, 0]
    return c, k_rot


def latent_attention(h, W, p, m, eps, kv):
    """Queries through a latent; keys and values expanded from the kept latent ``kv`` = (c, k_rot)
    (this layer's own or another's); a sink in the softmax's denominator; a sigmoid gate."""
    T = h.shape[0]
    H, n, nr, nv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, k_rot = kv
    cq = norm_plain(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).view(T, H, n + nr)
    q_plain = q[..., :n]
    q_rot = rotate(q[..., n:], torch.arange(T), m.get("rot"))
    k_plain = (c @ W[p + "uk"].T).view(T, H, n)
    v = (c @ W[p + "uv"].T).view(T, H, nv)
    out = torch.zeros(T, H, nv, dtype=torch.float64)
    for a in range(H):
        sink = W[p + "sink"][a]
        for i in range(T):
            s = (k_plain[: i + 1, a] @ q_plain[i, a] + k_rot[: i + 1] @ q_rot[i, a]) * m["scale"]
            top = torch.maximum(s.max(), sink)
            e = torch.exp(s - top)
            out[i, a] = (e @ v[: i + 1, a]) / (e.sum() + torch.exp(sink - top))
    gate = torch.sigmoid(h @ W[p + "g"].T)
    return (out.reshape(T, H * nv) * gate) @ W[p + "o"].T


def lightning(h, W, p, m, eps):
    """A matrix state per head with one constant decay; silu on q, k and v; the heads normed
    together; a sigmoid gate."""
    T = h.shape[0]
    H, n, nv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].T).view(T, H, n)
    k = silu(h @ W[p + "k"].T).view(T, H, n)
    v = silu(h @ W[p + "v"].T).view(T, H, nv)
    out = torch.zeros(T, H, nv, dtype=torch.float64)
    for a in range(H):
        S = torch.zeros(n, nv, dtype=torch.float64)
        for t in range(T):
            S = m["decay"][a] * S + torch.outer(k[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    y = norm_plain(out.reshape(T, H * nv), W[p + "norm"], eps)
    return (y * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


# ----------------------------------------------------------------------------- feed-forward
def route(h, W, p, r):
    """(expert numbers [T, top], their weights [T, top]): the largest entries of the softmax over
    all experts, as they are."""
    s = torch.softmax(h @ W[p + "router"].T, dim=-1)
    w, idx = torch.topk(s, r["top"], dim=-1)
    return idx, w


def experts(h, W, p, mlp):
    idx, w = route(h, W, p, mlp["router"])
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=torch.float64)
    for t in range(h.shape[0]):
        for e, g in zip(idx[t].tolist(), w[t]):
            a = torch.relu(W[p + f"e{e}.up"] @ h[t]).pow(2)
            out[t] += g * (W[p + f"e{e}.down"] @ a)
    return out


# ----------------------------------------------------------------------------- the model
def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and, on request, the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = norm_around_zero(x, W[p + "norm1"], eps)
        if layer["type"] == "lightning":
            y = lightning(h, W, p + "mix.", m, eps)
        elif layer["type"] == "attention":
            y = window_attention(h, W, p + "mix.", m)
        elif layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_kv(h, W, p + "mix.", m, eps)
            y = latent_attention(h, W, p + "mix.", m, eps, kept[m["kv_from"] if m.get("kv_from") is not None else i])
        else:
            raise ValueError(layer["type"])
        x = x + norm_around_zero(y, W[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = norm_around_zero(x, W[p + "norm2"], eps)
            x = x + norm_around_zero(experts(h, W, p + "mlp.", layer["mlp"]), W[p + "norm2b"], eps)
        streams.append(x)
    logits = norm_around_zero(x, W["final.norm"], eps) @ W["embed"].T
    return (logits, torch.stack(streams)) if return_layers else logits


def logits(cfg, W, tokens):
    return forward(cfg, W, tokens)


def greedy(cfg, W, prompt, n):
    """n greedy tokens after ``prompt``; with each, the gap between the best and the second logit."""
    ids, out, gaps = list(prompt), [], []
    for _ in range(n):
        row = forward(cfg, W, ids)[-1]
        best = torch.topk(row, 2)
        out.append(int(best.indices[0]))
        gaps.append(float(best.values[0] - best.values[1]))
        ids.append(out[-1])
    return out, gaps
