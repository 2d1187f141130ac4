"""The Zinizen decoder in plain, slow arithmetic: one function per mechanism, float64, no cache.

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


def centred_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis, var the mean squared deviation."""
    d = x - x.mean(dim=-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(dim=-1, keepdim=True) + eps) * w + b


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


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


def causal_softmax(scores):
    """Softmax over the keys j <= i of every row i; ``scores`` [heads, T, T]."""
    T = scores.shape[-1]
    seen = torch.tril(torch.ones(T, T, dtype=torch.bool))
    return torch.softmax(scores.masked_fill(~seen, float("-inf")), dim=-1)


# ------------------------------------------------------------------ embedding
def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every token: a hash of the token and the one before it; the
    first token of a sequence takes the table's last row."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets)
    return rows


def embed(cfg, W, tokens):
    x = W["embed"][tokens]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + W["bigram"][bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])]
    return x


# ------------------------------------------------------------------ mixers
def biased_attention(h, W, p, m, pos, eps, v_first):
    """Grouped attention without rotation: q and k normed over the whole projection, a query
    temperature, capped scores and a bias that grows with the distance, per head.  ``v_first``: the
    values of the first value-mixing layer (None in that layer itself and in layers that do not
    mix).  Returns the output and this layer's values."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms(h @ W[p + "q"].T, eps) * W[p + "q.norm"]
    k = unit_rms(h @ W[p + "k"].T, eps) * W[p + "k.norm"]
    v = h @ W[p + "v"].T
    if m.get("v_mix") and v_first is not None:
        lam = W[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    temp = m.get("q_temp")
    if temp:
        q = q * (1.0 + temp["coef"] * torch.log(torch.floor((pos.to(F64) + 1.0) / temp["every"]) + 1.0))[:, None]
    q = q.view(T, H, D).transpose(0, 1)
    kk = k.view(T, G, D).transpose(0, 1).repeat_interleave(H // G, dim=0)
    vv = v.view(T, G, V).transpose(0, 1).repeat_interleave(H // G, dim=0)
    s = q @ kk.transpose(1, 2) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / H) for i in range(H)], dtype=F64)
    dist = (pos[:, None] - pos[None, :]).to(F64)
    s = s - slopes[:, None, None] * dist[None]
    o = causal_softmax(s) @ vv
    return o.transpose(0, 1).reshape(T, H * V) @ W[p + "o"].T, v


def latent_attention(h, W, p, m, pos, eps):
    """Keys and values made per head from one normed latent per token, one rotated key part shared by
    the heads, queries through a latent of their own, a sigmoid gate of one number per head."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = unit_rms(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).view(T, H, D + R)
    down = h @ W[p + "dkv"].T
    c = unit_rms(down[:, :C], eps) * W[p + "dkv.norm"]
    rot = m["rot"]
    k_rot = turn_halves(down[:, None, C:], pos, rot["dims"], rot["base"])            # [T, 1, R]
    q_rot = turn_halves(q[:, :, D:], pos, rot["dims"], rot["base"])
    k_plain = (c @ W[p + "uk"].T).view(T, H, D)
    v = (c @ W[p + "uv"].T).view(T, H, V)
    s = torch.einsum("ihd,jhd->hij", q[:, :, :D], k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])
    o = torch.einsum("hij,jhv->ihv", causal_softmax(s * m["scale"]), v)
    gate = torch.sigmoid(h @ W[p + "g"].T)                                           # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * V) @ W[p + "o"].T


def short_conv(z, taps, bias):
    """Per channel: out[t] = bias + sum_k taps[:, k] * z[t - (K - 1 - k)], zeros before the start."""
    T, K = z.shape[0], taps.shape[1]
    out = bias.expand(T, -1).clone()
    for k in range(K):
        back = K - 1 - k
        if back < T:
            out[back:] += z[:T - back] * taps[:, k]
    return out


def gated_linear_unit(h, W, p, m):
    """Two branches of ``width``: one through gelu, one through a short convolution into a
    recurrence per channel whose decay and input gate come from block-diagonal maps."""
    T, N, B = h.shape[0], m["width"], m["blocks"]
    y = gelu_tanh(h @ W[p + "y"].T + W[p + "y.b"])
    u = short_conv(h @ W[p + "x"].T + W[p + "x.b"], W[p + "conv"], W[p + "conv.b"])
    ub = u.view(T, B, N // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, W[p + "ra"]) + W[p + "ra.b"]).reshape(T, N)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, W[p + "ri"]) + W[p + "ri.b"]).reshape(T, N)
    log_a = -8.0 * r * softplus(W[p + "lam"])
    a = torch.exp(log_a)
    S = torch.zeros(N, dtype=F64)
    out = torch.empty(T, N, dtype=F64)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] * a[t]) * i[t] * u[t]
        out[t] = S
    return (out * y) @ W[p + "o"].T


# ------------------------------------------------------------------ feed-forwards
def capped_expert(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def route(h, W, p, router):
    """(chosen experts [T, top], their weights [T, top])."""
    s = torch.softmax(h @ W[p + "router"].T, dim=-1)
    choice = s + W[p + "correction"]
    idx = torch.topk(choice, router["top"], dim=-1).indices
    w = torch.gather(s, 1, idx)
    return idx, w / (w.sum(dim=-1, keepdim=True) + 1e-20) * router["scale"]


def routed_feed_forward(h, W, p, mlp):
    idx, w = route(h, W, p, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(idx[t].tolist(), w[t]):
            out[t] += we * capped_expert(h[t:t + 1], W, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + capped_expert(h, W, p + "shared.", mlp["shared"]["limit"])
    return out


def feed_forward(h, W, p, mlp):
    if mlp["kind"] == "dense":
        return gelu_tanh(h @ W[p + "up"].T) @ W[p + "down"].T
    return routed_feed_forward(h, W, p, mlp)


# ------------------------------------------------------------------ the model
def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of a whole sequence; ``layers_out``: a list that gets the stream after every layer."""
    W = {n: t.to(F64) for n, t in W.items()}
    eps = cfg["norm"]["eps"]
    pos = torch.arange(len(tokens))
    x = embed(cfg, W, list(tokens))

    def norm(name, z):
        return centred_norm(z, W[name], W[name + ".b"], eps)

    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        h = norm(f"l{i}.norm1", x)
        if layer["type"] == "attention":
            y, v = biased_attention(h, W, p, m, pos, eps, v_first)
            if m.get("v_mix") and v_first is None:
                v_first = v
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, W, p, m, pos, eps)
        elif layer["type"] == "rglru":
            y = gated_linear_unit(h, W, p, m)
        else:
            raise ValueError(layer["type"])
        x = x + norm(f"l{i}.norm1b", y)
        if layer.get("mlp") is not None:
            x = x + norm(f"l{i}.norm2b", feed_forward(norm(f"l{i}.norm2", x), W, f"l{i}.mlp.", layer["mlp"]))
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm("final.norm", x) @ W["head"].T
