"""A plain, slow implementation of the Kuzipel decoder: whole sequences, no cache, one function per mechanism.

Kuzipel is a pre-norm decoder.  Every layer holds one token mixer and, optionally, a routed feed-forward:

  x += m * s1 * mixer(ln1(x));  x += m * s2 * ffn(ln2(x))

with a layer norm that has a weight and no bias, learned per-channel scales s1, s2 and one constant m.
The mixers:

  latent_attention  causal softmax attention whose keys and values are expanded from a small latent
                    per token (plus one short rotated key part shared by all heads); queries pass a
                    latent of their own.
  wkv               a linear recurrence with a matrix state per head, a per-channel decay made from the
                    input, a bonus for the current token, and inputs mixed with the previous token's.

A run of layers may be repeated with the same weights; before every pass the stream is re-made from
itself and the embedding output by one linear map over their concatenation.

Nothing here is shared with the engine; everything is computed on the CPU in float64 unless the
caller's tensors say otherwise.  Weights are a dictionary by checkpoint tensor name; sizes and
constants come from the configuration dictionary (the keys of config.json).
"""
from __future__ import annotations

import math

import torch


def silu(z):
    return z * torch.sigmoid(z)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w, population variance, no bias."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w


# ------------------------------------------------------------------ rotation
def rotate_half_pairs(x, positions, base, dims):
    """Rotate the first `dims` entries of the last axis: entry i pairs with i + dims/2, angle p * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]          # [T, half]
    cos, sin = torch.cos(ang).to(x.dtype), torch.sin(ang).to(x.dtype)
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, rest], dim=-1)


# ------------------------------------------------------------------ latent attention
def latent_attention(h, W, pre, c, eps, positions=None):
    """h [T, width] -> [T, width].  c: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot{base, dims}."""
    T = h.shape[0]
    H, D, R, Dv, C = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    cq = unit_rms(h @ W[pre + "dq"].T, eps) * W[pre + "dq.norm"]
    q = (cq @ W[pre + "uq"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], q[..., D:]
    kv = h @ W[pre + "dkv"].T
    lat = unit_rms(kv[:, :C], eps) * W[pre + "dkv.norm"]
    k_rot = kv[:, C:]                                                   # [T, R], one for all heads
    k_plain = (lat @ W[pre + "uk"].T).view(T, H, D)
    v = (lat @ W[pre + "uv"].T).view(T, H, Dv)
    base, dims = c["rot"]["base"], c["rot"]["dims"]
    q_rot = rotate_half_pairs(q_rot, pos, base, dims)
    k_rot = rotate_half_pairs(k_rot, pos, base, dims)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * c["scale"]
        s = s.masked_fill(~causal, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, hd] = p @ v[:, hd]
    return out.reshape(T, H * Dv) @ W[pre + "o"].T


# ------------------------------------------------------------------ wkv
def wkv_decay(mix_w, W, pre):
    """exp(-exp(W2 tanh(W1 x) + w0)): per head and key channel, in (0, 1)."""
    return torch.exp(-torch.exp(torch.tanh(mix_w @ W[pre + "w1"].T) @ W[pre + "w2"].T + W[pre + "w0"]))


def wkv_recurrence(r, k, v, w, u):
    """r, k, v, w [T, H, D], u [H, D] -> o [T, H, D].  S [D(key), D(value)] per head starts at zero."""
    T, H, D = r.shape
    S = torch.zeros(H, D, D, dtype=r.dtype)
    o = torch.zeros(T, H, D, dtype=r.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]                        # [H, D, D]
        o[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = w[t][:, :, None] * S + kv
    return o


def wkv(h, W, pre, c, eps):
    T, width = h.shape
    H, D = c["heads"], c["dim"]
    prev = torch.cat([torch.zeros(1, width, dtype=h.dtype), h[:-1]], dim=0)
    mix = {s: h + (prev - h) * W[pre + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ W[pre + "r"].T).view(T, H, D)
    k = (mix["k"] @ W[pre + "k"].T).view(T, H, D)
    v = (mix["v"] @ W[pre + "v"].T).view(T, H, D)
    gate = silu(mix["g"] @ W[pre + "g"].T)
    w = wkv_decay(mix["w"], W, pre).view(T, H, D)
    o = wkv_recurrence(r, k, v, w, W[pre + "u"])
    y = unit_rms(o, eps).reshape(T, H * D) * W[pre + "norm"] * gate
    return y @ W[pre + "o"].T


# ------------------------------------------------------------------ feed-forward
def gated_expert(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def route(h, W, pre, top):
    """-> (chosen experts [T, top], their weights [T, top]): largest logits, softmax over the chosen only."""
    z = h @ W[pre + "router"].T + W[pre + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def route_margin(h, W, pre, top):
    """Per token, how far the last chosen logit lies above the first refused one (infinite when every expert is chosen)."""
    z = h @ W[pre + "router"].T + W[pre + "router.b"]
    if top >= z.shape[-1]:
        return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    val = torch.topk(z, top + 1, dim=-1).values
    return val[:, top - 1] - val[:, top]


def moe(h, W, pre, c, margins=None):
    T = h.shape[0]
    out = torch.zeros(T, W[pre + "e0.down"].shape[0], dtype=h.dtype)
    idx, wt = route(h, W, pre, c["router"]["top"])
    if margins is not None:
        margins.append(route_margin(h, W, pre, c["router"]["top"]))
    for t in range(T):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * gated_expert(h[t:t + 1], W, f"{pre}e{e}.")[0]
    if c.get("shared"):
        out = out + torch.sigmoid(h @ W[pre + "shared.sg"].T) * gated_expert(h, W, pre + "shared.")
    return out


# ------------------------------------------------------------------ the model
def run_order(cfg):
    """Layer indices in the order they run, and which of these runs start a pass of the repeated part."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(L)), set()
    a, b, n = loop["start"], loop["stop"], loop["times"]
    order = list(range(a))
    starts = set()
    for _ in range(n):
        starts.add(len(order))
        order += list(range(a, b))
    order += list(range(b, L))
    return order, starts


def forward(tokens, W, cfg, streams=None, margins=None):
    """tokens [T] -> logits [T, vocab].  With `streams` (a list), the residual stream after every layer run is appended;
    with `margins` (a list), every router's margin per token (see route_margin)."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x0 = W["embed"][torch.as_tensor(tokens)]
    x = x0
    order, starts = run_order(cfg)
    for j, i in enumerate(order):
        if j in starts:
            x = torch.cat([x, x0], dim=-1) @ W["loop.in"].T
        layer, pre = cfg["layers"][i], f"l{i}."
        hin = layer_norm(x, W[pre + "norm1"], eps)
        if layer["type"] == "latent_attention":
            y = latent_attention(hin, W, pre + "mix.", layer["mixer"], eps)
        elif layer["type"] == "wkv":
            y = wkv(hin, W, pre + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + m * W[pre + "ls1"] * y
        if layer.get("mlp"):
            x = x + m * W[pre + "ls2"] * moe(layer_norm(x, W[pre + "norm2"], eps), W, pre + "mlp.", layer["mlp"], margins)
        if streams is not None:
            streams.append(x.clone())
    return layer_norm(x, W["final.norm"], eps) @ W["head"].T
