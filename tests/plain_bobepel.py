"""A plain, slow statement of the Bobepel design in 32-bit torch on the CPU: one function per mechanism, whole
sequences at a time, no cache.  It shares no code with the engine; the tests compare the engine with it.

``cfg`` is the parsed ``config.json`` (a dict), ``W`` maps tensor names to float32 tensors.
"""
from __future__ import annotations


import torch

F = torch.float32


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """The layers' and the model's norm: the stored weight lies around zero."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def visible(n, window=None):
    """[n, n] bool: query i (rows) sees key j (columns): j <= i, and with a window i - j < window."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & (i - j < window)
    return ok


def masked_softmax(scores, ok):
    scores = scores.masked_fill(~ok, float("-inf"))
    return torch.softmax(scores, dim=-1)


def distance_slopes(n_heads):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / n_heads) for h in range(n_heads)], dtype=F)


def query_temperature(n, coef, every):
    p = torch.arange(n, dtype=torch.int64)
    return 1.0 + coef * torch.log((torch.div(p + 1, every, rounding_mode="floor") + 1).to(F))


def rotate_pairs(x, base, dims):
    """x [n, ..., d]: the first ``dims`` elements of the last axis, neighbours (2i, 2i+1) as pairs, pair i turned by
    position * base^(-2i/dims); position = index along axis 0."""
    n = x.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    ang = torch.arange(n, dtype=F)[:, None] * f.to(F)[None, :]      # positions and angles are 32-bit
    shape = [n] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def mixer_attention(h, m, W, p, eps):
    """Grouped-query attention with normed queries and keys, a query temperature and a distance bias; no rotation."""
    n = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(n, H, D)
    k = (h @ W[p + "k"].T).view(n, G, D)
    v = (h @ W[p + "v"].T).view(n, G, V)
    q = norm_plain(q, W[p + "q.norm"], eps)
    k = norm_plain(k, W[p + "k.norm"], eps)
    if m.get("q_temp"):
        q = q * query_temperature(n, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    dist = (torch.arange(n)[:, None] - torch.arange(n)[None, :]).to(F)
    s = s - distance_slopes(H)[:, None, None] * dist[None]
    w = masked_softmax(s, visible(n, (m.get("mask") or {}).get("size"))[None])
    o = torch.einsum("hij,jhv->ihv", w, vv).reshape(n, H * V)
    return o @ W[p + "o"].T


def mixer_latent_attention(h, m, W, p, eps, query_latent, gated):
    """Attention whose keys and values are read out of one latent vector a position, plus a rotated key part that
    all heads share."""
    n = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    if query_latent:
        cq = norm_plain(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
        q = cq @ W[p + "uq"].T
    else:
        q = h @ W[p + "q"].T
    q = q.view(n, H, D + R)
    q_plain, q_rot = q[..., :D], q[..., D:]
    dkv = h @ W[p + "dkv"].T
    c = norm_plain(dkv[:, :C], W[p + "dkv.norm"], eps)
    k_rot = dkv[:, C:]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q_rot = rotate_pairs(q_rot, base, dims)
    k_rot = rotate_pairs(k_rot, base, dims)
    k_plain = (c @ W[p + "uk"].T).view(n, H, D)
    v = (c @ W[p + "uv"].T).view(n, H, V)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    w = masked_softmax(s, visible(n, (m.get("mask") or {}).get("size"))[None])
    o = torch.einsum("hij,jhv->ihv", w, v).reshape(n, H * V)
    if gated:
        o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def expert(x, W, p, limit):
    g = torch.clamp(x @ W[p + "gate"].T, max=limit)
    u = torch.clamp(x @ W[p + "up"].T, min=-limit, max=limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return y @ W[p + "down"].T


def router(h, W, p, top):
    """(chosen experts [n, top], their weights [n, top], all scores [n, E])."""
    s = torch.sigmoid(h @ W[p + "router"].T)
    w, idx = torch.topk(s, top, dim=-1)
    return idx, w, s


def feed_forward(h, f, W, p):
    n = h.shape[0]
    out = torch.zeros(n, h.shape[1], dtype=F)
    if f.get("router"):
        idx, w, _ = router(h, W, p, f["router"]["top"])
        for t in range(n):
            for r in range(idx.shape[1]):
                e = int(idx[t, r])
                out[t] += expert(w[t, r] * h[t:t + 1], W, f"{p}e{e}.", f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + expert(h, W, p + "shared.", f["shared"]["limit"])
    return out


def layer(x, entry, W, src, eps):
    """One layer on the whole sequence: x [n, width] -> x + mixer(h) + ff(h), h the one norm of x."""
    p = f"l{src}."
    h = norm_one_plus(x, W[p + "norm1"], eps)
    m, t = entry["mixer"], entry["type"]
    if t == "attention":
        y = mixer_attention(h, m, W, p + "mix.", eps)
    elif t == "latent_attention":
        y = mixer_latent_attention(h, m, W, p + "mix.", eps, query_latent=False, gated=True)
    elif t == "latent_attention_2":
        y = mixer_latent_attention(h, m, W, p + "mix.", eps, query_latent=True, gated=False)
    else:
        raise ValueError(t)
    if entry.get("mlp") is not None:
        y = y + feed_forward(h, entry["mlp"], W, p + "mlp.")
    return x + y


def forward(cfg, W, tokens, return_layers=False):
    """Logits [n, vocab] of one sequence (and, on request, the stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)].to(F)
    after = []
    for i, entry in enumerate(cfg["layers"]):
        x = layer(x, entry, W, entry.get("weights_of", i), eps)
        after.append(x.clone())
    logits = norm_one_plus(x, W["final.norm"], eps) @ W["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
