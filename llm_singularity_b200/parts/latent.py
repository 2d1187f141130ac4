"""Causal softmax attention over a cached latent.

A token leaves one row in the cache: ``c = rmsnorm(W_dkv x)[:kv_rank] * w`` and, behind it, the
last ``rot_dim`` outputs of W_dkv rotated by the token's position (one key part shared by all
heads, not normed).  Head h's unrotated key is ``W_uk[h] c``, its value ``W_uv[h] c``.  Queries
come through a latent of their own, ``q = W_uq (rmsnorm(W_dq x) * w_q)``, per head ``[plain_dim
unrotated | rot_dim rotated]``; the score is ``(q_plain . k_plain + q_rot . k_rot) * scale``.

Keys and values are never formed.  Since ``q_plain . (W_uk[h] c) = (W_uk[h]^T q_plain) . c``, the
query is carried into the latent's space once per step (a product per head), attention runs over
the cache rows themselves (every head reads the same rows, whose first ``kv_rank`` values are
also the values), and ``W_uv[h]`` is applied to the weighted sum of latents afterwards.  A layer
with ``reads_only`` has no W_dkv and attends over the rows another layer's call wrote in the same
step (the run order names that cache).  ``gate_per_head``: W_g (one row a head) rides in the same
product as the down projections and ``sigmoid(W_g x)_h`` multiplies head h's output.  Norms, angles, scores, softmax and weighted sums are
32-bit.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import POSITIONS, LatentPagesSpec, ParamSpec, Part, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Part):
    graph_safe = True
    kernels = ("gemm", "latent")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        self.position = POSITIONS.build(s.position, rt)
        table = self.position.rotary_table()
        if table is None:
            self.inv_freq, self.rot_dims, self.pairing = None, 0, "half"
        else:
            self.inv_freq, self.rot_dims = table
            self.pairing = getattr(s.position, "pairing", "half")
            if self.rot_dims > s.rot_dim:
                raise ValueError(f"{self.rot_dims} rotating dims in a rotated part of {s.rot_dim}")
        self.width = s.kv_rank + s.rot_dim
        if rt.dtype == torch.bfloat16:
            self.kernels = self.kernels + ("latent_tc",)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        s, H = spec, spec.hidden_size
        p = {"dq": ParamSpec((s.q_rank, H)),
             "dq_norm": ParamSpec((s.q_rank,), role="vector", init="ones"),
             "uq": ParamSpec((s.num_heads * (s.plain_dim + s.rot_dim), s.q_rank)),
             "uk": ParamSpec((s.num_heads * s.plain_dim, s.kv_rank)),
             "uv": ParamSpec((s.num_heads * s.value_dim, s.kv_rank)),
             "o": ParamSpec((H, s.num_heads * s.value_dim))}
        if getattr(s, "gate_per_head", False):
            p["g"] = ParamSpec((s.num_heads, H))
        if not s.reads_only:
            p["dkv"] = ParamSpec((s.kv_rank + s.rot_dim, H))
            p["dkv_norm"] = ParamSpec((s.kv_rank,), role="vector", init="ones")
        return p

    def children(self):
        return {"position": self.position}

    def load(self, tensors):
        s = self.spec
        # one product for both down projections: rows of W_dq, then W_dkv
        rows = [tensors["dq"]] + ([] if s.reads_only else [tensors["dkv"]]) + ([tensors["g"]] if "g" in tensors else [])
        self.w_down = torch.cat(rows, dim=0).contiguous()
        self.gate_off = self.w_down.shape[0] - s.num_heads if "g" in tensors else None
        self.q_norm = tensors["dq_norm"]
        self.kv_norm = tensors.get("dkv_norm")
        self.w_uq = tensors["uq"].contiguous()
        # W_uk per head, transposed: [heads, kv_rank, plain_dim], the operand that carries a query
        # into the latent's space
        self.w_uk_t = tensors["uk"].reshape(s.num_heads, s.plain_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv"].reshape(s.num_heads, s.value_dim, s.kv_rank).contiguous()
        self.w_out = tensors["o"].contiguous()

    def cache_spec(self):
        return LatentPagesSpec(self.width)

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        s, ops, T = self.spec, self.rt.ops, x.shape[0]
        if writes_cache and s.reads_only:
            raise ValueError("a latent-attention layer without a latent projection cannot write a cache")
        down = ops.linear(x, self.w_down, out_dtype=torch.float32)
        cq = self.rt.empty(T, s.q_rank)
        ops.latent_prep(down, s.q_rank, s.kv_rank, s.rot_dim, self.q_norm, self.kv_norm, s.eps, self.inv_freq,
                        self.rot_dims, self.pairing, ctx, cache, cq, writes_cache)
        q = ops.linear(cq, self.w_uq, out_dtype=torch.float32)      # [T, heads * (plain + rot)]
        qf = self.rt.empty(T, s.num_heads, self.width, dtype=torch.float32)
        q3 = q.view(T, s.num_heads, s.plain_dim + s.rot_dim)
        ops.batched_nt(q3[:, :, :s.plain_dim], self.w_uk_t, qf[:, :, :s.kv_rank])
        ops.latent_query_rot(q, qf, s.num_heads, s.plain_dim, s.rot_dim, s.kv_rank, self.inv_freq,
                             self.rot_dims, self.pairing, ctx)
        mixed = self.rt.empty(T, s.num_heads, s.kv_rank)
        ops.latent_attention(qf, ctx, cache, s.kv_rank, s.rot_dim, s.scale, mixed)
        heads_out = self.rt.empty(T, s.num_heads, s.value_dim)
        ops.batched_nt(mixed, self.w_uv, heads_out)
        if self.gate_off is not None:
            ops.head_gate(heads_out, down[:, self.gate_off:self.gate_off + s.num_heads])
        return ops.linear(heads_out.view(T, s.num_heads * s.value_dim), self.w_out)
