"""A plain, slow implementation of the Kazedra decoder: whole sequences, no cache, one function per mechanism.

Kazedra is a pre-norm decoder whose layers hold two token mixers that read the same normalised
input and whose outputs are added with fixed weights:

  left   softmax attention without rotation.  Keys double as values (the value of a token is its key
         projection before the key norm).  q and k are normalised over the whole projection (all heads
         at once).  q grows with the logarithm of the position in steps of `every` tokens.  A learned
         bias by bucketed distance is added to the scaled score, and the softmax denominator holds one
         extra term exp(sink) per head.
  right  the gated delta rule: a matrix state per head that decays, is corrected towards the new value
         along the new key, and is read with the query, after short causal convolutions.

Nothing here is shared with the engine; everything is computed on the CPU in float64 unless a dtype is
given.  Weights are a dictionary by checkpoint tensor name.
"""
from __future__ import annotations

import math

import torch


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


# ------------------------------------------------------------------ left mixer
def distance_bucket(n: int, n_buckets: int, max_distance: int) -> int:
    """Exact buckets for the first half of the table, logarithmic ones up to max_distance, then the last."""
    half = n_buckets // 2
    if n < half:
        return n
    r = math.log(n / half) / math.log(max_distance / half) * (n_buckets - half)
    return min(n_buckets - 1, half + int(math.floor(r)))


def query_temperature(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((p + 1) // every + 1)


def sink_bias_attention(h, W, pre, c, eps):
    """h [T, width] -> [T, width].  W: weights, pre: tensor name prefix, c: the mixer's sizes and constants."""
    T = h.shape[0]
    H, G, D = c["heads"], c["kv_heads"], c["dim"]
    q = h @ W[pre + "q"].T + W[pre + "q.b"]
    k = h @ W[pre + "k"].T + W[pre + "k.b"]
    v = k.clone()                                            # values: the key projection as it is
    q = unit_rms(q, eps) * W[pre + "q.norm"]                 # over all heads at once
    k = unit_rms(k, eps) * W[pre + "k.norm"]
    temp = torch.tensor([query_temperature(p, c["q_temp"]["coef"], c["q_temp"]["every"]) for p in range(T)], dtype=h.dtype)
    q = q * temp[:, None]
    q = q.view(T, H, D)
    k = k.view(T, G, D)
    v = v.view(T, G, D)
    rel = W[pre + "rel"]
    B = rel.shape[0]
    bucket = torch.tensor([[distance_bucket(i - j, B, c["bias_max"]) if j <= i else 0 for j in range(T)] for i in range(T)])
    out = torch.zeros(T, H, D, dtype=h.dtype)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * c["scale"] + rel[bucket, hd]
        s = s.masked_fill(~causal, float("-inf"))
        sink = W[pre + "sink"][hd]
        m = torch.maximum(s.max(dim=-1, keepdim=True).values, sink)
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True) + torch.exp(sink - m)
        out[:, hd] = (e / den) @ v[:, g]
    return out.reshape(T, H * D) @ W[pre + "o"].T + W[pre + "o.b"]


# ----------------------------------------------------------------- right mixer
def short_conv(x, w):
    """Causal per-channel convolution over time; x [T, C], w [C, taps], last tap on the current token."""
    T, C = x.shape
    taps = w.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + xp[j:j + T] * w[:, j]
    return y


def unit_vector(x):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def gated_delta_rule(h, W, pre, c, eps, state=None):
    """h [T, width] -> [T, width].  `state` (optional): list per head of [dim, vdim] matrices, updated in place."""
    T = h.shape[0]
    H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = silu(short_conv(h @ W[pre + "q"].T, W[pre + "q.conv"])).view(T, G, D)
    k = silu(short_conv(h @ W[pre + "k"].T, W[pre + "k.conv"])).view(T, G, D)
    v = silu(short_conv(h @ W[pre + "v"].T, W[pre + "v.conv"])).view(T, H, Dv)
    q = unit_vector(q) * D ** -0.5
    k = unit_vector(k)
    beta = torch.sigmoid(h @ W[pre + "b"].T)                                      # [T, H]
    decay = torch.exp(-torch.exp(W[pre + "A_log"]) * torch.nn.functional.softplus(h @ W[pre + "a"].T + W[pre + "dt_bias"]))
    gate = silu(h @ W[pre + "g"].T).view(T, H, Dv)
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(D, Dv, dtype=h.dtype) if state is None else state[hd]
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
        if state is not None:
            state[hd] = S
    out = unit_rms(out, eps) * W[pre + "norm"] * gate
    return out.reshape(T, H * Dv) @ W[pre + "o"].T


# ---------------------------------------------------------------- feed-forward
def dense_ff(x, W, pre):
    return (silu(x @ W[pre + "gate"].T) * (x @ W[pre + "up"].T)) @ W[pre + "down"].T


# ----------------------------------------------------------------------- model
def parallel_mixer(x, W, pre, m, eps):
    left = sink_bias_attention(x, W, pre + "left.", m["left"], eps)
    right = gated_delta_rule(x, W, pre + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def forward(config, weights, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    layers = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        if layer["type"] != "parallel":
            raise ValueError(f"unknown layer type {layer['type']}")
        x = x + parallel_mixer(norm_one_plus(x, W[p + "norm1"], eps), W, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError("unknown feed-forward kind")
            x = x + dense_ff(norm_one_plus(x, W[p + "norm2"], eps), W, p + "mlp.")
        layers.append(x)
    logits = norm_one_plus(x, W["final.norm"], eps) @ W["head"].T * config["logit_scale"]
    return (logits, torch.stack(layers)) if return_layers else logits
