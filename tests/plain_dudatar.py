"""A plain, slow Dudatar in float64 on the CPU: one function per mechanism, whole sequences only
(no cache, no state carried between calls, no batches).  It shares no code with the package;
the GPU tests hold the engine to it.

Notation: x [T, width] is the stream, h the normalised input of a block's sub-layers, W[name]
the checkpoint tensor of that name (linear weights [out, in], applied as h @ W.T)."""
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


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = (x - mu).pow(2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def silu(z):
    return z * torch.sigmoid(z)


def rotate(x, positions, dims, base):
    """x [T, heads, n]: element i < dims/2 is paired with i + dims/2; the pair at position p turns
    by the angle p * base^(-2i/dims).  Elements from ``dims`` on pass."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    ang = positions.double()[:, None] * freq[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def soft_cap(y, cap):
    return cap * torch.tanh(y / cap) if cap else y


# ----------------------------------------------------------------------------- mixers
def softmax_attention(h, W, p, m, eps):
    """The left mixer: grouped-query causal softmax attention, unit-norm q and k after the
    rotation, one sigmoid gate per head."""
    T = h.shape[0]
    H, G, n, nv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate((h @ W[p + "q"].T).view(T, H, n), pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate((h @ W[p + "k"].T).view(T, G, n), pos, m["rot"]["dims"], m["rot"]["base"])
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    v = (h @ W[p + "v"].T).view(T, G, nv)
    gate = torch.sigmoid(h @ W[p + "g"].T)
    heads = []
    for a in range(H):
        g = a // (H // G)
        out = torch.zeros(T, nv, dtype=torch.float64)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, a]) * m["scale"]
            w = torch.softmax(s, 0)
            out[i] = w @ v[: i + 1, g]
        heads.append(out * gate[:, a:a + 1])
    return torch.cat(heads, -1) @ W[p + "o"].T


def matrix_state_scan(q, k, v, decay):
    """One head: S_t = diag(decay_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, n], v [T, nv],
    decay [T, n] (a constant per head is a row of equal numbers)."""
    T, n = q.shape
    S = torch.zeros(n, v.shape[1], dtype=torch.float64)
    out = []
    for t in range(T):
        S = decay[t][:, None] * S + torch.outer(k[t], v[t])
        out.append(S.T @ q[t])
    return torch.stack(out)


def retention(h, W, p, m, eps):
    """The right mixer: a constant decay per head, rotary q and k, k / sqrt(n)."""
    T = h.shape[0]
    H, n, nv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate((h @ W[p + "q"].T).view(T, H, n), pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate((h @ W[p + "k"].T).view(T, H, n), pos, m["rot"]["dims"], m["rot"]["base"]) * n ** -0.5
    v = (h @ W[p + "v"].T).view(T, H, nv)
    heads = [unit_rms(matrix_state_scan(q[:, a], k[:, a], v[:, a], torch.full((T, n), float(m["decay"][a]),
                                                                              dtype=torch.float64)), eps)
             for a in range(H)]
    return (torch.cat(heads, -1) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def gated_linear_attention(h, W, p, m, eps):
    T = h.shape[0]
    H, n, nv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, n) * n ** -0.5
    k = (h @ W[p + "k"].T).view(T, H, n)
    v = (h @ W[p + "v"].T).view(T, H, nv)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / m["tau"]).view(T, H, n)
    heads = [unit_rms(matrix_state_scan(q[:, a], k[:, a], v[:, a], alpha[:, a]), eps) * W[p + "norm"] for a in range(H)]
    return (torch.cat(heads, -1) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def two_mixers(h, W, p, m, eps):
    left = unit_rms(softmax_attention(h, W, p + "left.", m["left"], eps), eps) * W[p + "left.out"]
    right = unit_rms(retention(h, W, p + "right.", m["right"], eps), eps) * W[p + "right.out"]
    return 0.5 * (left + right)


def dense_ff(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


# ----------------------------------------------------------------------------- the stack
def block(x, cfg, W, i):
    layer, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    h = layer_norm(x, W[p + "norm1"], eps)
    mixer = gated_linear_attention if layer["type"] == "gla" else two_mixers
    y = mixer(h, W, p + "mix.", layer["mixer"], eps)
    if layer.get("mlp") is not None:
        y = y + dense_ff(h, W, p + "mlp.")
    return x + y


def run_order(cfg):
    """[(layer, pass number or None)]: the pass number stands at the first layer of a pass."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def logits(cfg, W, ids, streams=None):
    x0 = W["embed"][torch.tensor(ids)]
    x = x0
    for i, t in run_order(cfg):
        if t is not None:
            x = torch.cat([x, x0], -1) @ W["loop.in"].T + W["loop.step"][t]
        x = block(x, cfg, W, i)
        if streams is not None:
            streams.append(x)
    y = layer_norm(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T
    return soft_cap(y, cfg.get("logit_softcap") or 0.0)


def greedy(cfg, W, ids, n):
    """n tokens by argmax, and the gap between the best and the second logit at each."""
    ids, out, gaps = list(ids), [], []
    for _ in range(n):
        top = logits(cfg, W, ids)[-1].topk(2)
        out.append(int(top.indices[0]))
        gaps.append(float(top.values[0] - top.values[1]))
        ids.append(out[-1])
    return out, gaps
