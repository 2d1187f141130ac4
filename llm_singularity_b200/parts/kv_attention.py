"""Softmax attention over a paged cache whose keys and values have sizes of their own.

Per layer call: one product against the row-wise concatenation ``[Wq; Wk; Wv; Wg]`` -> one kernel
that adds the biases, norms every head of q and k (RMS over the head, one weight of head size for
all heads), applies the query temperature and the rotation, and writes queries to a buffer and
keys and values to this step's cache places -> every query row attends the cached keys not after
it, within its window and its chunk, query head ``h`` reading kv head ``h // (heads / kv_heads)``
-> the heads' outputs times ``sigmoid(Wg x)`` -> output projection.  Each of bias, norm,
temperature, rotation, window, chunk and gate is there only if the spec asks for it.  Scores,
softmax, norms, positions and angles are 32-bit.  Further options of the spec: the norm of q and k
taken over all heads at once (``qk_norm_span`` "all"), value heads brought to unit rms before they
are cached (``v_unit_norm``), one more place with score 0 and no value in every softmax (``sink``),
and a gate of one number per head (``gate_per_head``); scores capped by ``cap * tanh(s / cap)``
(``logit_softcap``) and lowered in proportion to the key's distance with a slope per head
(``linear_bias``); and values shared within a token among the layers of a model that name the same
``value_mix_key``: the "source" layer lends the rows of its value projection to the step
(``ctx.lent``), a "mixed" layer caches ``(1 - lambda) v + lambda v_source``.

Where the spec is what the framework's grouped attention already covers after the preparation (keys
and values of one size, no chunks, no gate), the same attention kernels run (tensor cores for
bfloat16 heads of 64 or 128); everything else runs the kernels of ``csrc/attention_dv.cu``.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import POSITIONS, PagedKVSpec, ParamSpec, Part, register_mixer


@register_mixer("kv_attention")
class KVAttention(Part):
    graph_safe = True
    kernels = ("gemm", "attention_prep", "attention_dv")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads {s.num_heads} is not a multiple of num_kv_heads {s.num_kv_heads}")
        for name, v in (("window", s.window), ("chunk", s.chunk)):
            if v is not None and v < 1:
                raise ValueError(f"{name} must be at least 1, got {v}")
        if s.temp_every < 0:
            raise ValueError(f"temp_every must not be negative, got {s.temp_every}")
        self.norm_all = getattr(s, "qk_norm_span", "head") == "all"
        if getattr(s, "qk_norm_span", "head") not in ("head", "all"):
            raise ValueError(f"qk_norm_span '{s.qk_norm_span}' is not known (head, all)")
        self.v_unit = bool(getattr(s, "v_unit_norm", False))
        self.sink = bool(getattr(s, "sink", False))
        self.gate_per_head = bool(getattr(s, "gate_per_head", False))
        self.softcap = float(getattr(s, "logit_softcap", None) or 0.0)
        self.linear_bias = bool(getattr(s, "linear_bias", False))
        self.value_mix = getattr(s, "value_mix", None)
        if self.value_mix not in (None, "source", "mixed"):
            raise ValueError(f"value_mix '{self.value_mix}' is not known (source, mixed)")
        if self.value_mix and (s.qkv_bias or self.v_unit):
            raise ValueError("values that layers share are neither biased nor normed")
        self.position = POSITIONS.build(s.position, rt)
        self.table = self.position.rotary_table()
        if self.table is None and s.position.kind != "none":
            raise ValueError(f"a position encoding of kind '{s.position.kind}' is not a rotation this mixer can fuse")
        self.pairing = getattr(s.position, "pairing", "half")
        self.q_size = s.num_heads * s.key_dim
        self.k_size = s.num_kv_heads * s.key_dim
        self.v_size = s.num_kv_heads * s.value_dim
        self.o_size = s.num_heads * s.value_dim
        # the framework's grouped attention takes over where nothing here is beyond it
        self.plain = (s.key_dim == s.value_dim and s.chunk is None and not s.out_gate and s.key_dim % 16 == 0
                      and 16 <= s.key_dim <= 256 and not self.sink and not self.softcap and not self.linear_bias)
        if self.plain:
            self.kernels = self.kernels + ("attention",)
            if rt.dtype == torch.bfloat16 and s.key_dim in (64, 128):
                self.kernels = self.kernels + ("attention_tc", "attention_tc5")
        elif (rt.dtype == torch.bfloat16 and s.key_dim == s.value_dim and s.key_dim in (64, 128) and s.chunk is None
              and (not s.out_gate or self.gate_per_head)):
            # steps of prompt portions only go to the tcgen05 prompt kernel, sink and gate per head included
            self.kernels = self.kernels + ("attention_tc5",)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        s, H = spec, spec.hidden_size
        q, k, v, o = s.num_heads * s.key_dim, s.num_kv_heads * s.key_dim, s.num_kv_heads * s.value_dim, \
            s.num_heads * s.value_dim
        p = {"q": ParamSpec((q, H)), "k": ParamSpec((k, H)), "v": ParamSpec((v, H)), "o": ParamSpec((H, o))}
        if s.qkv_bias:
            p.update(q_bias=ParamSpec((q,), role="vector", init="normal"),
                     k_bias=ParamSpec((k,), role="vector", init="normal"),
                     v_bias=ParamSpec((v,), role="vector", init="normal"))
        if s.qk_norm:
            whole = getattr(s, "qk_norm_span", "head") == "all"
            p.update(q_norm=ParamSpec((q if whole else s.key_dim,), role="vector", init="ones"),
                     k_norm=ParamSpec((k if whole else s.key_dim,), role="vector", init="ones"))
        if s.out_gate:
            p["g"] = ParamSpec((s.num_heads if getattr(s, "gate_per_head", False) else o, H))
        if getattr(s, "value_mix", None) == "mixed":
            p["vmix"] = ParamSpec((), role="vector", init="normal")
        return p

    def children(self):
        return {"position": self.position}

    def load(self, tensors):
        rows = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if self.spec.out_gate else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_out = tensors["o"].contiguous()
        self.extras = {n: tensors[n].contiguous() for n in ("q_bias", "k_bias", "v_bias", "q_norm", "k_norm")
                       if n in tensors}
        self.v_lambda = tensors["vmix"].reshape(1).contiguous() if "vmix" in tensors else None

    def cache_spec(self):
        s = self.spec
        return PagedKVSpec(s.num_kv_heads, s.key_dim, s.window, None if s.value_dim == s.key_dim else s.value_dim)

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        s, ops = self.spec, self.rt.ops
        T = x.shape[0]
        proj = ops.linear(x, self.w_in)                                   # [T, q | k | v | g]
        q = self.rt.empty(T, self.q_size)
        inv_freq, rotary_dim = self.table if self.table is not None else (None, 0)
        v_off = self.q_size + self.k_size
        if self.value_mix:
            # what the layers of a step lend one another lives with the step: here the rows of the
            # source layer's value projection (the tensor stays alive as long as the step does)
            lent = ctx.__dict__.setdefault("lent", {})
            if self.value_mix == "source":
                lent[s.value_mix_key] = proj[:, v_off:v_off + self.v_size]
            elif s.value_mix_key not in lent:
                raise ValueError(f"no layer before this one lent '{s.value_mix_key}' to the step")
        ops.attention_prep(proj, 0, self.q_size, self.q_size + self.k_size, s.num_heads, s.num_kv_heads,
                           s.key_dim, s.value_dim, ctx, cache, q, norm_eps=s.eps, temp_coef=s.temp_coef,
                           temp_every=s.temp_every, inv_freq=inv_freq, rotary_dim=rotary_dim, pairing=self.pairing,
                           store=writes_cache, **self.extras, **self._prep_options(ctx))
        out = self.rt.empty(T, self.o_size)
        if self.plain:
            ops.paged_attention(q, s.num_heads, s.num_kv_heads, s.key_dim, ctx, cache, s.scale, s.window or 0, out)
        else:
            gate = proj[:, self.q_size + self.k_size + self.v_size:] if s.out_gate else None
            ops.attention_dv(q, s.num_heads, s.num_kv_heads, s.key_dim, s.value_dim, ctx, cache, s.scale,
                             s.window or 0, s.chunk or 0, gate, out, **self._softmax_options())
        return ops.linear(out, self.w_out)

    def _prep_options(self, ctx=None) -> dict:
        """Keyword arguments of the preparation kernel that only some specs need."""
        opts = {}
        if self.value_mix == "mixed":
            opts.update(v_first=ctx.lent[self.spec.value_mix_key], v_lambda=self.v_lambda)
        if self.norm_all:
            opts["norm_all"] = True
        if self.v_unit:
            opts["v_unit"] = True
        return opts

    def _softmax_options(self) -> dict:
        opts = {}
        if self.sink:
            opts["sink"] = True
        if self.gate_per_head and self.spec.out_gate:
            opts["gate_per_head"] = True
        if self.softcap:
            opts["softcap"] = self.softcap
        if self.linear_bias:
            opts["linear_bias"] = True
        return opts
