"""A plain, slow implementation of the Safepel design: whole sequences, no cache, token-by-token recurrences,
one function per mechanism.  It is the yardstick the engine's Safepel model is measured against and shares no code
with the product path (it reads safetensors through the other plain implementation's reader).

Notation.  A layer is  x += post1(mixer(pre1(x)));  x += post2(ff(pre2(x)))  where every norm is a weighted layer
norm without bias.  Mixers:

* ``delta``: per head a matrix state S [dim, vdim];  S = g S;  u = beta (v - S^T k);  S += k u^T;  o = S^T q,
  after short causal convolutions + SiLU on q, k, v and unit-length q (times dim^-1/2) and k.
* ``parallel``: left_scale * (windowed soft-capped attention whose values are the unrotated keys)
  + right_scale * (decayed linear attention  S = d S + k v^T, o = S^T q  with a gated RMS norm over all heads).

Everything runs in the dtype given (float32 by default; float64 to arbitrate).  Run on the CPU.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- small pieces
def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def short_conv(x, taps_w):
    """x [T, C]; taps_w [C, taps], the last column multiplies the current token; zeros before the start."""
    T, C = x.shape
    n = taps_w.shape[1]
    padded = torch.cat([x.new_zeros(n - 1, C), x], 0)
    out = x.new_zeros(T, C)
    for j in range(n):
        out = out + padded[j:j + T] * taps_w[:, j]
    return out


def rotate_adjacent(x, positions, base, dims):
    """x [T, heads, dim]: pairs (2i, 2i+1) of the first ``dims`` elements turn by p * base^(-2i/dims)."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = (float(base) ** (-2.0 * i / dims)).to(x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]            # [T, dims/2]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# --------------------------------------------------------------------------- mixers
def delta_mixer(h, w, p, m, eps):
    """Gated delta rule, one token after the other.  ``p``: tensor prefix '<layer>.mix.'; ``m``: the mixer's sizes."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = F.silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, D)
    k = F.silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, D)
    v = F.silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                          # [T, H]
    g = torch.exp(-torch.exp(w[p + "A_log"]) * F.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    out = h.new_zeros(T, H, V)
    for hd in range(H):
        kv = hd // (H // G)
        S = h.new_zeros(D, V)
        for t in range(T):
            S = g[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, hd] = S.T @ q[t, kv]
    out = rms(out, eps) * w[p + "norm"]
    gate = F.silu(h @ w[p + "g"].T).view(T, H, V)
    return (out * gate).reshape(T, H * V) @ w[p + "o"].T


def capped_window_attention(h, w, p, m, positions):
    """The left half of the parallel mixer: values are the keys as projected (before rotation)."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = k
    q = rotate_adjacent(q, positions, m["rot"]["base"], m["rot"]["dims"])
    kr = rotate_adjacent(k, positions, m["rot"]["base"], m["rot"]["dims"])
    cap, W = m["softcap"], m["mask"]["size"]
    i, j = positions[:, None], positions[None, :]
    visible = (i - j >= 0) & (i - j < W)
    out = h.new_zeros(T, H, D)
    for hd in range(H):
        kv = hd // (H // G)
        s = (q[:, hd] @ kr[:, kv].T) * m["scale"]
        s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~visible, float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ v[:, kv]
    return out.reshape(T, H * D) @ w[p + "o"].T


def decayed_linear_attention(h, w, p, m, eps):
    """The right half of the parallel mixer, one token after the other."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = F.silu(h @ w[p + "q"].T).view(T, H, D)
    k = F.silu(h @ w[p + "k"].T).view(T, H, D)
    v = F.silu(h @ w[p + "v"].T).view(T, H, V)
    out = h.new_zeros(T, H, V)
    for hd in range(H):
        S = h.new_zeros(D, V)
        d = float(m["decay"][hd])
        for t in range(T):
            S = d * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    o = rms(out.reshape(T, H * V), eps) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps, positions):
    left = capped_window_attention(h, w, p + "left.", m["left"], positions)
    right = decayed_linear_attention(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def feed_forward(h, w, p):
    return (torch.relu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# --------------------------------------------------------------------------- the model
def forward(cfg, w: Dict[str, torch.Tensor], tokens: List[int], return_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and the residual stream after every layer)."""
    eps = cfg["norm"]["eps"]
    positions = torch.arange(len(tokens))
    x = w["embed"][torch.as_tensor(tokens)]
    x = layer_norm(x, w["embed.norm"], eps)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "delta":
            y = delta_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps, positions)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + layer_norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            y = feed_forward(layer_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
            x = x + layer_norm(y, w[p + "norm2b"], eps)
        after.append(x)
    logits = (layer_norm(x, w["final.norm"], eps) @ w["head"].T) * cfg["logit_scale"]
    return (logits, torch.stack(after)) if return_layers else logits


def greedy(cfg, w, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
