"""Delta-rule memories: a matrix state per head and request that every token first lets fade, then
corrects along its key, then reads.

``gated_delta`` (one fade and one write strength per head; the gated delta rule).  q and k have
``num_key_heads`` heads of ``key_dim`` channels that ``num_heads`` value heads of ``value_dim`` share in
groups.  Each of q, k and v passes a short causal convolution over time per channel and silu; q and k
become unit vectors per head, q also times ``key_dim^-1/2``; ``beta = sigmoid(W_b x)``,
``g = exp(-exp(A_log) * softplus(W_a x + dt_bias))``:

    S <- g S;  e = beta (v - S^T k);  S <- S + k e^T;  o = S^T q

and each head's o, divided by its root mean square, times a weight of ``value_dim`` and silu(W_g x),
goes through W_o.  The last ``conv_taps - 1`` inputs of the convolutions are state too.

``channel_delta`` (a decay and a removal rate per key channel; the generalized delta rule).  r, k and
v have ``num_heads`` heads of ``key_dim``.  With ``u = k / |k|``, ``w = exp(-rate * sigmoid(W_w2 tanh(W_w1 x)
+ w0))`` and ``a = sigmoid(W_a x + a_bias)``:

    S <- diag(w) S - (a * u) (u^T S) + k v^T;  o = S^T r

and each head's o, divided by its root mean square, times a weight over all heads and sigmoid(W_g x),
goes through W_o.

Both: one product makes the wide projections of a step, a second, small one whose output stays
32-bit makes the gates'; a kernel forms what enters the walk in 32-bit; one kernel walks every
request's tokens in order from its slot's state (prompt portions and single tokens alike); one
kernel norms and gates.  The states start at zero when a request takes a slot and live in
``StateSpec`` rows, 32-bit.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import CompositeCacheSpec, ParamSpec, Part, StateSpec, register_mixer


@register_mixer("gated_delta")
class GatedDelta(Part):
    graph_safe = True
    kernels = ("gemm", "delta_rule")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if s.num_key_heads <= 0 or s.num_heads % s.num_key_heads:
            raise ValueError(f"{s.num_heads} heads cannot share {s.num_key_heads} key heads")
        if s.conv_taps < 1:
            raise ValueError(f"conv_taps must be at least 1, got {s.conv_taps}")
        self.qk = s.num_key_heads * s.key_dim
        self.vv = s.num_heads * s.value_dim

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        H, n = spec.hidden_size, spec.num_heads
        qk, vv = spec.num_key_heads * spec.key_dim, n * spec.value_dim
        return {"q": ParamSpec((qk, H)), "k": ParamSpec((qk, H)), "v": ParamSpec((vv, H)), "g": ParamSpec((vv, H)),
                "o": ParamSpec((H, vv)), "b": ParamSpec((n, H)), "a": ParamSpec((n, H)),
                "q_conv": ParamSpec((qk, spec.conv_taps), role="vector", init="normal"),
                "k_conv": ParamSpec((qk, spec.conv_taps), role="vector", init="normal"),
                "v_conv": ParamSpec((vv, spec.conv_taps), role="vector", init="normal"),
                "A_log": ParamSpec((n,), role="vector", init="normal"),
                "dt_bias": ParamSpec((n,), role="vector", init="normal"),
                "norm": ParamSpec((spec.value_dim,), role="vector", init="ones")}

    def load(self, tensors):
        self.w_in = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0).contiguous()
        self.w_gates = torch.cat([tensors["b"], tensors["a"]], dim=0).contiguous()
        self.w_out = tensors["o"].contiguous()
        self.taps = tuple(tensors[n].contiguous() for n in ("q_conv", "k_conv", "v_conv"))
        self.a_log, self.dt_bias, self.norm = tensors["A_log"], tensors["dt_bias"], tensors["norm"]

    def cache_spec(self):
        s = self.spec
        parts = [StateSpec((s.num_heads, s.value_dim, s.key_dim))]             # S, key channels contiguous
        if s.conv_taps > 1:
            parts.append(StateSpec((s.conv_taps - 1, 2 * self.qk + self.vv)))   # the convolutions' last inputs
        return CompositeCacheSpec(tuple(parts))

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        s, ops = self.spec, self.rt.ops
        T, n = x.shape[0], s.num_heads
        proj = ops.linear(x, self.w_in)                                     # [T, q | k | v | g]
        raw = ops.linear(x, self.w_gates, out_dtype=torch.float32)          # [T, b | a]
        qk = self.rt.empty(T, 2 * self.qk, dtype=torch.float32)
        v = self.rt.empty(T, self.vv, dtype=torch.float32)
        scal = self.rt.empty(T, 2 * n, dtype=torch.float32)
        conv_state = cache[1].state if s.conv_taps > 1 else None
        ops.gated_delta_prep(proj, 0, self.qk, 2 * self.qk, s.num_key_heads, n, s.key_dim, s.value_dim, self.taps,
                             conv_state, raw, self.a_log, self.dt_bias, ctx, qk, v, scal, s.unit_eps)
        o = self.rt.empty(T, self.vv, dtype=torch.float32)
        ops.delta_scan("scalar", qk, scal, v, cache[0].state, ctx, o, n, s.num_key_heads, s.key_dim, s.value_dim)
        y = self.rt.empty(T, self.vv)
        ops.delta_output(o, self.norm, n, s.eps, proj[:, 2 * self.qk + self.vv:], "silu", y)
        return ops.linear(y, self.w_out)


@register_mixer("channel_delta")
class ChannelDelta(Part):
    graph_safe = True
    kernels = ("gemm", "delta_rule")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if spec.decay_rank < 1:
            raise ValueError(f"decay_rank must be at least 1, got {spec.decay_rank}")
        self.hd = spec.num_heads * spec.key_dim

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        H, hd = spec.hidden_size, spec.num_heads * spec.key_dim
        return {"r": ParamSpec((hd, H)), "k": ParamSpec((hd, H)), "v": ParamSpec((hd, H)), "g": ParamSpec((hd, H)),
                "o": ParamSpec((H, hd)), "a": ParamSpec((hd, H)),
                "a_bias": ParamSpec((hd,), role="vector", init="normal"),
                "w1": ParamSpec((spec.decay_rank, H)), "w2": ParamSpec((hd, spec.decay_rank)),
                "w0": ParamSpec((hd,), role="vector", init="normal"),
                "norm": ParamSpec((hd,), role="vector", init="ones")}

    def load(self, tensors):
        self.w_in = torch.cat([tensors["r"], tensors["k"], tensors["v"], tensors["g"]], dim=0).contiguous()
        self.w_gates = torch.cat([tensors["a"], tensors["w1"]], dim=0).contiguous()
        self.w_decay = tensors["w2"].contiguous()
        self.w_out = tensors["o"].contiguous()
        self.a_bias, self.w0, self.norm = tensors["a_bias"], tensors["w0"], tensors["norm"]

    def cache_spec(self):
        s = self.spec
        return StateSpec((s.num_heads, s.key_dim, s.key_dim))

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        s, ops, hd = self.spec, self.rt.ops, self.hd
        T, n, D = x.shape[0], s.num_heads, s.key_dim
        proj = ops.linear(x, self.w_in)                                     # [T, r | k | v | g]
        raw = ops.linear(x, self.w_gates, out_dtype=torch.float32)          # [T, a | w1]
        hidden = self.rt.empty(T, s.decay_rank)
        ops.tanh_rows(raw[:, hd:], hidden)
        decay_raw = ops.linear(hidden, self.w_decay, out_dtype=torch.float32)
        vecs = self.rt.empty(T, n, 5, D, dtype=torch.float32)
        v = self.rt.empty(T, hd, dtype=torch.float32)
        ops.channel_delta_prep(proj, 0, hd, 2 * hd, n, D, D, decay_raw, self.w0, raw[:, :hd], self.a_bias,
                               s.decay_rate, vecs, v, s.unit_eps)
        o = self.rt.empty(T, hd, dtype=torch.float32)
        ops.delta_scan("channel", vecs, None, v, cache.state, ctx, o, n, n, D, D)
        y = self.rt.empty(T, hd)
        ops.delta_output(o, self.norm, n, s.eps, proj[:, 3 * hd:], "sigmoid", y)
        return ops.linear(y, self.w_out)
