"""Routed feed-forward: every token is sent through ``top`` of ``num_experts`` small gated
feed-forwards, ``down_e(act(gate_e u) * up_e u)``, no bias.

The router is one product with 32-bit output; its logits become scores (sigmoid, or softmax
over all experts), the ``top`` largest are chosen (the lower index wins a tie) and, if the spec
says so, divided by their sum.  A score multiplies what the spec names: the expert's input
(``u = s x``; with a gated expert that is not the same as scaling its output) or its output.
With ``choice_bias`` a learnt number per expert joins the scores for the choice only; the chosen
scores are divided by their sum + ``renorm_eps`` and multiplied by ``weight_scale``.  ``shared``: a
gated feed-forward that every token passes besides its chosen experts; its rows join the 32-bit sum
over the chosen experts' rows in the combining kernel.

The experts' matrices are stacked (``[E, 2F, H]`` with rows alternating gate_i, up_i, and
``[E, H, F]``); a step's (token, choice) pairs are sorted by expert on the device into row
tiles that belong to one expert each, two grouped products run over the used tiles, and the
rows are summed back per token in the order of the token's choices.  Nothing is read back to the
host, so a decode step launches the same kernels whatever the router decides.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import FEED_FORWARDS, ParamSpec, Part, register_feed_forward


@register_feed_forward("moe")
class RoutedExperts(Part):
    graph_safe = True
    kernels = ("gemm", "moe")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if not 0 < s.top <= s.num_experts:
            raise ValueError(f"top {s.top} of {s.num_experts} experts")
        if s.score not in ("sigmoid", "softmax") or s.weight_on not in ("input", "output"):
            raise ValueError(f"score '{s.score}' / weight_on '{s.weight_on}' is not known")
        known = getattr(rt.ops, "ACTIVATIONS", None)
        if known is not None and s.activation not in known:
            raise ValueError(f"activation '{s.activation}' is not implemented")
        shared = getattr(s, "shared", None)
        self.shared = FEED_FORWARDS.build(shared, rt) if shared is not None else None
        if self.shared is not None:
            self.kernels = self.kernels + ("activation",)

    def children(self) -> Dict[str, Part]:
        return {"shared": self.shared} if self.shared is not None else {}

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        H, F = spec.hidden_size, spec.expert_size
        p = {"router": ParamSpec((spec.num_experts, H))}
        if getattr(spec, "choice_bias", False):
            p["choice_bias"] = ParamSpec((spec.num_experts,), role="vector", init="normal")
        for e in range(spec.num_experts):
            p[f"e{e}.gate"] = ParamSpec((F, H))
            p[f"e{e}.up"] = ParamSpec((F, H))
            p[f"e{e}.down"] = ParamSpec((H, F))
        return p

    def load(self, tensors):
        s = self.spec
        E, F, H = s.num_experts, s.expert_size, s.hidden_size
        self.w_router = tensors["router"].contiguous()
        self.choice_bias = tensors["choice_bias"].contiguous() if "choice_bias" in tensors else None
        # rows 2i, 2i + 1 of an expert = gate_i, up_i
        self.w_gate_up = torch.stack(
            [torch.stack([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=1).reshape(2 * F, H) for e in range(E)]
        ).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(E)]).contiguous()

    def forward(self, x, ctx):
        s, ops, T = self.spec, self.rt.ops, x.shape[0]
        logits = ops.linear(x, self.w_router, out_dtype=torch.float32)
        out = self.rt.empty(T, s.hidden_size)
        extra = {}
        if self.choice_bias is not None:
            extra["choice_bias"] = self.choice_bias
        for name, default in (("weight_scale", 1.0), ("renorm_eps", 0.0), ("limit", 0.0)):
            if getattr(s, name, default) != default:
                extra[name] = float(getattr(s, name))
        if self.shared is not None:                 # its rows join the sum over the chosen experts
            extra["add"] = lambda: self.shared.forward(x, ctx)
        ops.moe_routed_experts(x, logits, s.top, s.score, s.renormalize, self.w_gate_up, self.w_down,
                               s.activation, s.weight_on, out, **extra)
        return out
