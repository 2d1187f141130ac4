"""A recurrent block with a real-gated linear recurrent unit (RG-LRU).

Two branches of ``width`` channels leave one product: ``y = gelu_tanh(W_y x + b_y)`` and the input of
a short causal convolution per channel, ``u = conv(W_x x + b_x)``.  u is cut into ``blocks`` equal
parts; in each, two square matrices give the recurrence's gates, ``r = sigmoid(R_b u_b + b_r)`` and
``i = sigmoid(I_b u_b + b_i)``.  Every channel then carries one number from token to token:

    a = exp(-rate * r * softplus(lam));   S <- a S + sqrt(1 - a^2) * i * u

and ``W_o (S * y)`` is the block's result.  S starts at zero when a request takes a slot, and so do
the convolution's last ``conv_taps - 1`` inputs, which are state too; both live in ``StateSpec`` rows,
32-bit.  The product of the two branches leaves in 32-bit, and the convolution, the gates' products,
sigmoid, softplus, the exponential, the square root, the state and the product with y are all formed
in 32-bit; only what enters W_o is rounded to the compute dtype.  The gates' products: in 32-bit
storage multiply-adds on u as it is; with bfloat16 maps u enters the tensor cores as the sum of two
bfloat16 numbers (the rounded value and the rounded rest, 16 bits of mantissa) against the maps
repeated along k, so that the 32-bit sums carry u's digits and nothing is rounded to bfloat16's 8.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import CompositeCacheSpec, ParamSpec, Part, StateSpec, register_mixer


@register_mixer("rglru")
class RGLRU(Part):
    graph_safe = True
    kernels = ("gemm", "latent", "rglru")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if s.blocks < 1 or s.width % s.blocks:
            raise ValueError(f"{s.blocks} blocks do not divide a width of {s.width}")
        if s.conv_taps < 1:
            raise ValueError(f"conv_taps must be at least 1, got {s.conv_taps}")
        if rt.dtype == torch.bfloat16:
            self.kernels = self.kernels + ("latent_tc",)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        H, N, B = spec.hidden_size, spec.width, spec.blocks
        vec = dict(role="vector", init="normal")
        return {"y": ParamSpec((N, H)), "y_bias": ParamSpec((N,), **vec),
                "x": ParamSpec((N, H)), "x_bias": ParamSpec((N,), **vec),
                "conv": ParamSpec((N, spec.conv_taps), **vec), "conv_bias": ParamSpec((N,), **vec),
                "ra": ParamSpec((B, N // B, N // B)), "ra_bias": ParamSpec((B, N // B), **vec),
                "ri": ParamSpec((B, N // B, N // B)), "ri_bias": ParamSpec((B, N // B), **vec),
                "lam": ParamSpec((N,), **vec), "o": ParamSpec((H, N))}

    def load(self, tensors):
        self.w_in = torch.cat([tensors["y"], tensors["x"]], dim=0).contiguous()          # rows: y, then x
        # per block the rows of R_b, then those of I_b: one product makes both gates' inputs
        self.w_gates = torch.cat([tensors["ra"], tensors["ri"]], dim=1).contiguous()     # [B, 2 bw, bw]
        self.split = self.w_gates.dtype == torch.bfloat16
        if self.split:                                  # the same maps for the rounded u and for its rest
            self.w_gates = torch.cat([self.w_gates, self.w_gates], dim=2).contiguous()   # [B, 2 bw, 2 bw]
        self.w_out = tensors["o"].contiguous()
        self.taps = tensors["conv"].contiguous()
        self.vecs = {n: tensors[n].reshape(-1).contiguous() for n in ("y_bias", "x_bias", "conv_bias", "ra_bias",
                                                                       "ri_bias", "lam")}

    def cache_spec(self):
        s = self.spec
        return CompositeCacheSpec((StateSpec((s.width,)), StateSpec((max(s.conv_taps - 1, 1), s.width))))

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        s, ops, v = self.spec, self.rt.ops, self.vecs
        T, N, B = x.shape[0], s.width, s.blocks
        f32 = torch.float32
        proj = ops.linear(x, self.w_in, out_dtype=f32)                     # [T, y | x]
        state, conv_state = cache[0].state, cache[1].state
        u = self.rt.empty(T, N, dtype=f32)
        gates = self.rt.empty(T, 2 * N, dtype=f32)
        if self.split:
            halves = self.rt.empty(T, 2 * N, dtype=torch.bfloat16)
            ops.rglru_conv(proj, N, v["x_bias"], self.taps, v["conv_bias"], conv_state, ctx, u, split=halves, blocks=B)
            ops.batched_nt(halves.view(T, B, 2 * (N // B)), self.w_gates, gates.view(T, B, 2 * (N // B)))
        else:
            ops.rglru_conv(proj, N, v["x_bias"], self.taps, v["conv_bias"], conv_state, ctx, u)
            ops.batched_nt(u.view(T, B, N // B), self.w_gates, gates.view(T, B, 2 * (N // B)), exact=True)
        ops.rglru_gates(gates, v["ra_bias"], v["ri_bias"], v["lam"], s.rate, u, proj, 0, v["y_bias"], B)
        out = self.rt.empty(T, N)
        ops.rglru_walk(gates, proj, N, 0, v["x_bias"], s.conv_taps, state, conv_state, ctx, out, B)
        return ops.linear(out, self.w_out)
