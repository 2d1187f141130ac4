"""The Fikizen decoder in plain, slow arithmetic: one function per mechanism, float64, no cache.

A whole sequence goes in; where a mechanism carries something from one token to the next it is
walked token by token.  Nothing here is shared with the engine's parts or kernels.  ``cfg`` is the
dictionary that config.json holds, ``W`` maps tensor names to float64 tensors.

Notation: ``x`` is the residual stream [T, width]; ``h`` is what a sublayer reads; a linear map
stored [out, in] is applied as ``h @ M.T``; ``pos`` are the tokens' places in their sequence.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------ small functions
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def unit_length(x, eps=1e-6):
    """x / sqrt(sum(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + eps)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def silu(z):
    return z * torch.sigmoid(z)


def bent_square(z, p, q):
    """The feed-forward's activation with its two learnt numbers: a parabola on the right,
    ``softplus(p) z^2 + z/2``, and a saturating branch on the left,
    ``(1/2 + softplus(q)) (e^z - 1 - z) + z/2``."""
    right = softplus(p) * z * z + 0.5 * z
    left = (0.5 + softplus(q)) * (torch.expm1(z) - z) + 0.5 * z
    return torch.where(z > 0, right, left)


def turn_halves(v, pos, dims, base):
    """Dim i of the last axis turns together with dim i + dims/2 by ``pos * base^(-2i/dims)``,
    i < dims/2; the dims from ``dims`` on stay.  ``v``: [T, heads, n]."""
    out = v.clone()
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    ang = pos.to(F64)[:, None] * torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def in_window(pos, size):
    """[T, T] truth table: query i sees key j if 0 <= pos_i - pos_j < size."""
    d = pos[:, None] - pos[None, :]
    return (d >= 0) & (d < size)


def sink_softmax_heads(q, k, v, scale, ok):
    """q [T, H, D], k [T, G, D], v [T, G, V]; head h reads key/value head h // (H / G).  The weights
    of a row are exp(s_j) / (1 + sum_j exp(s_j)): one more place with score 0 and no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~ok, float("-inf"))
        top = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - top)
        out[:, h] = (e / (torch.exp(-top) + e.sum(dim=-1, keepdim=True))) @ v[:, g]
    return out


def short_conv(z, taps):
    """Causal convolution over time, one filter per channel: z [T, C], taps [C, n] whose last
    column meets the current token; zeros stand before the start."""
    T, C = z.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, C, dtype=F64), z], dim=0)
    out = torch.zeros(T, C, dtype=F64)
    for j in range(n):
        out += padded[j:j + T] * taps[:, j][None, :]
    return out


# ------------------------------------------------------------------------- mixers
def gated_window_attention(h, W, p, m, pos):
    """Windowed attention with a sink, partly turned heads and one gate number per head."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, D)
    k = (h @ W[p + "k"].T).reshape(T, G, D)
    v = (h @ W[p + "v"].T).reshape(T, G, V)
    rot = m["rot"]
    q, k = turn_halves(q, pos, rot["dims"], rot["base"]), turn_halves(k, pos, rot["dims"], rot["base"])
    o = sink_softmax_heads(q, k, v, m["scale"], in_window(pos, m["mask"]["size"]))
    o = o * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * V) @ W[p + "o"].T


def normed_window_attention(h, W, p, m, pos, eps):
    """The left mixer of a pair: biased projections, q and k normed over all their heads at once,
    each value head brought to unit rms, window and sink, no gate."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms(h @ W[p + "q"].T + W[p + "q.b"], eps) * W[p + "q.norm"]
    k = unit_rms(h @ W[p + "k"].T + W[p + "k.b"], eps) * W[p + "k.norm"]
    v = unit_rms((h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, V), eps)
    rot = m["rot"]
    q = turn_halves(q.reshape(T, H, D), pos, rot["dims"], rot["base"])
    k = turn_halves(k.reshape(T, G, D), pos, rot["dims"], rot["base"])
    o = sink_softmax_heads(q, k, v, m["scale"], in_window(pos, m["mask"]["size"]))
    return o.reshape(T, H * V) @ W[p + "o"].T


def channel_delta_memory(h, W, p, m, eps):
    """The right mixer of a pair: a matrix S [D, D] per head with a decay per key channel and a
    removal along the unit key; both read the state the token found:
    S <- diag(w) S - (a * u) (u^T S) + k v^T, o = S^T r."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    r = (h @ W[p + "r"].T).reshape(T, H, D)
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, D)
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"]))
    a = torch.sigmoid(h @ W[p + "a"].T + W[p + "a.b"])
    w, a = w.reshape(T, H, D), a.reshape(T, H, D)
    u = unit_length(k)
    S = torch.zeros(H, D, D, dtype=F64)                          # [head, key channel, value channel]
    o = torch.zeros(T, H, D, dtype=F64)
    for t in range(T):
        seen = torch.einsum("hk,hkv->hv", u[t], S)
        S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * seen[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, r[t])
    o = unit_rms(o, eps).reshape(T, H * D) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def side_by_side(h, W, p, m, pos, eps):
    left = normed_window_attention(h, W, p + "left.", m["left"], pos, eps)
    right = channel_delta_memory(h, W, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def gated_delta_memory(h, W, p, m, eps):
    """A matrix S [D, V] per head: it fades by one number per head, then the key's old answer is
    replaced by a share beta of the new value, and the read-out sees the write."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, D)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, D)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, V)
    q = unit_length(q) * D ** -0.5
    k = unit_length(k)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                           # [T, H]
    fade = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    S = torch.zeros(H, D, V, dtype=F64)
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        for n in range(H):
            g = n // (H // G)
            S[n] = fade[t, n] * S[n]
            u = beta[t, n] * (v[t, n] - S[n].T @ k[t, g])
            S[n] = S[n] + torch.outer(k[t, g], u)
            o[t, n] = S[n].T @ q[t, g]
    o = unit_rms(o, eps) * W[p + "norm"] * silu(h @ W[p + "g"].T).reshape(T, H, V)
    return o.reshape(T, H * V) @ W[p + "o"].T


# ------------------------------------------------------------------- feed-forward
def feed_forward(h, W, p):
    act = W[p + "act"]
    return bent_square(h @ W[p + "up"].T, act[0], act[1]) @ W[p + "down"].T


# -------------------------------------------------------------------------- model
def weight_layer(cfg, i):
    """The layer whose tensors layer i uses."""
    return cfg["layers"][i].get("weights_of", i)


def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of a whole sequence.  ``layers_out``: a list that receives the stream
    after every layer."""
    W = {n: t.to(F64) for n, t in W.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(tok))
    x = W["embed"][tok]
    for i, layer in enumerate(cfg["layers"]):
        lp = f"l{weight_layer(cfg, i)}."
        h = unit_rms(x, eps) * W[lp + "norm1"]
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            y = gated_window_attention(h, W, lp + "mix.", m, pos)
        elif kind == "parallel":
            y = side_by_side(h, W, lp + "mix.", m, pos, eps)
        elif kind == "delta":
            y = gated_delta_memory(h, W, lp + "mix.", m, eps)
        else:
            raise ValueError(f"layer {i}: unknown type {kind!r}")
        x = x + y
        if layer.get("mlp") is not None:
            x = x + feed_forward(unit_rms(x, eps) * W[lp + "norm2"], W, lp + "mlp.")
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = (unit_rms(x, eps) * W["final.norm"]) @ W["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
