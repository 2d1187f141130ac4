"""RMSNorm, fused with the residual addition that precedes it.

``y = x * rsqrt(mean(x^2) + eps) * w`` with eps inside the square root and the
weight applied after normalisation (reference: kernels/src/rmsnorm.cu:42-72, used
at models/llama/llama_model.cpp:506-508,629-631,658-660).  The residual stream is
32-bit; sum of squares, rsqrt and the product are 32-bit; the result is rounded
to the compute dtype only on the way out.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import ParamSpec, Part, register_norm


class NormedDelta:
    """A sublayer's output that a norm behind the sublayer still has to take before it joins the
    stream: ``stream += mult * unit(values) * weight``.  Handed on in place of a plain delta, so
    that this norm, the sum and the norm in front of the next sublayer are one kernel."""

    __slots__ = ("values", "weight", "eps", "mult")

    def __init__(self, values: torch.Tensor, weight: torch.Tensor, eps: float, mult: float):
        self.values, self.weight, self.eps, self.mult = values, weight, float(eps), float(mult)


@register_norm("rmsnorm")
class RMSNorm(Part):
    """``unit_offset`` in the spec: the checkpoint stores the weight's distance from one; one is added
    (in 32-bit) when the weight is loaded, and the kernels see an ordinary weight."""

    graph_safe = True
    replayable = True
    foldable = True
    kernels = ("norm",)

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if getattr(spec, "unit_offset", False):
            self.kernels = self.kernels + ("sandwich",)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        init = "normal" if getattr(spec, "unit_offset", False) else "ones"
        return {"weight": ParamSpec((spec.size,), role="vector", init=init)}

    def load(self, tensors):
        self.weight = tensors["weight"]
        if getattr(self.spec, "unit_offset", False):
            self.weight = (self.weight.float() + 1.0).contiguous()

    def pending(self, values: torch.Tensor, mult: float = 1.0) -> NormedDelta:
        """``values`` as something this norm takes before it is added to the stream ``mult`` times."""
        return NormedDelta(values, self.weight, self.spec.eps, mult)

    def _stream(self, residual, delta, step, rows):
        """The sum and this norm through the kernel that also takes a norm behind the sublayer and a
        step vector."""
        y = w = None
        eps, mult = 0.0, 1.0
        if isinstance(delta, NormedDelta):
            y, w, eps, mult = delta.values, delta.weight, delta.eps, delta.mult
        elif isinstance(delta, torch.Tensor):
            y = delta
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = self.rt.empty(n, residual.shape[1])
        self.rt.ops.stream_norm(residual, y, w, eps, mult, step, rows, self.weight, self.spec.eps, out)
        return out

    def fold(self):
        """What a product needs to take this norm upon itself: the weight and eps."""
        return self.weight, self.spec.eps

    def add_norm(self, residual: torch.Tensor, delta, step: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``delta``: a tensor, None, a ``NormedDelta`` or a ``StreamCopy`` (nothing pending).  ``step``: a
        vector added to every row of the stream with the sum."""
        if isinstance(delta, StreamCopy):
            delta = None
        if isinstance(delta, NormedDelta) or step is not None:
            return self._stream(residual, delta, step, None)
        out = self.rt.empty(*residual.shape)
        self.rt.ops.add_rmsnorm(residual, delta, self.weight, self.spec.eps, out)
        return out

    def gather_add_norm(self, residual: torch.Tensor, delta, rows: torch.Tensor) -> torch.Tensor:
        if isinstance(delta, StreamCopy):
            delta = None
        if isinstance(delta, NormedDelta):
            return self._stream(residual, delta, None, rows)
        out = self.rt.empty(rows.shape[0], residual.shape[1])
        self.rt.ops.gather_add_rmsnorm(residual, delta, rows, self.weight, self.spec.eps, out)
        return out


class CentredDelta:
    """A sublayer's output that a centred norm with weight and bias behind the sublayer still has to take
    before it joins the stream: ``stream += mult * (centred(values) * weight + bias)``."""

    __slots__ = ("values", "weight", "bias", "eps", "mult")

    def __init__(self, values: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float, mult: float):
        self.values, self.weight, self.bias, self.eps, self.mult = values, weight, bias, float(eps), float(mult)


@register_norm("layernorm")
class LayerNorm(Part):
    """``(x - mean) / sqrt(var + eps) * w + b`` over the model width, all in 32-bit, fused with the sum
    into the stream that precedes it and, where a norm of this kind stands behind the sublayer whose
    output is summed (``pending``), with that norm too."""

    graph_safe = True
    replayable = True
    kernels = ("sandwich",)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.size,), role="vector", init="ones"),
                "bias": ParamSpec((spec.size,), role="vector", init="normal")}

    def load(self, tensors):
        self.weight, self.bias = tensors["weight"].contiguous(), tensors["bias"].contiguous()

    def pending(self, values: torch.Tensor, mult: float = 1.0) -> CentredDelta:
        """``values`` as something this norm takes before it is added to the stream ``mult`` times."""
        return CentredDelta(values, self.weight, self.bias, self.spec.eps, mult)

    def _run(self, residual, delta, rows):
        y = w = b = None
        eps, mult = 0.0, 1.0
        if isinstance(delta, CentredDelta):
            y, w, b, eps, mult = delta.values, delta.weight, delta.bias, delta.eps, delta.mult
        elif isinstance(delta, torch.Tensor):
            y = delta
        elif delta is not None and not isinstance(delta, StreamCopy):
            raise ValueError(f"a centred norm cannot take a pending {type(delta).__name__}")
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = self.rt.empty(n, residual.shape[1])
        self.rt.ops.stream_centred_norm(residual, y, w, b, eps, mult, rows, self.weight, self.bias, self.spec.eps, out)
        return out

    def add_norm(self, residual: torch.Tensor, delta) -> torch.Tensor:
        return self._run(residual, delta, None)

    def gather_add_norm(self, residual: torch.Tensor, delta, rows: torch.Tensor) -> torch.Tensor:
        return self._run(residual, delta, rows)


class StreamCopy:
    """What a block that norms after the sum hands to the next block in place of a pending delta:
    nothing is left to add, and ``values`` is the residual stream rounded to the compute dtype
    (the stream itself where the compute dtype is 32-bit), ready to be a product's operand."""

    __slots__ = ("values",)

    def __init__(self, values: torch.Tensor):
        self.values = values


@register_norm("group_rmsnorm")
class GroupRMSNorm(Part):
    """RMS norm in ``groups`` equal consecutive parts of the vector, one weight over the whole:
    ``y[g] = x[g] / sqrt(mean(x[g]^2) + eps) * w[g]``, all in 32-bit.

    Besides the interface of every norm (``add_norm``: the sum stays in the stream, for
    arrangements that norm before a sublayer) it has ``scale_add_norm`` for arrangements that norm
    after the sum: the stream itself becomes ``norm(alpha * x + gate * delta)``."""

    graph_safe = True
    kernels = ("rownorm",)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.size,), role="vector", init="ones")}

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if spec.groups <= 0 or spec.size % spec.groups:
            raise ValueError(f"{spec.groups} groups do not divide a vector of {spec.size}")

    def load(self, tensors):
        self.weight = tensors["weight"]

    def _copy(self, residual):
        return None if self.rt.dtype == torch.float32 else self.rt.empty(*residual.shape)

    def add_norm(self, residual: torch.Tensor, delta) -> torch.Tensor:
        if isinstance(delta, StreamCopy):
            delta = None
        out = self.rt.empty(*residual.shape)
        self.rt.ops.post_group_norm(residual, delta, self.weight, self.spec.eps, self.spec.groups, 1.0, out,
                                    keep_sum=True)
        return out

    def scale_add_norm(self, residual: torch.Tensor, alpha: float, delta: torch.Tensor,
                       gate: Optional[torch.Tensor] = None, gate_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """residual <- norm(alpha * residual + delta * sigmoid(gate + gate_bias)) in place; returns the
        stream as a product's operand (a rounded copy, or the stream itself in 32-bit)."""
        out = self._copy(residual)
        self.rt.ops.post_group_norm(residual, delta, self.weight, self.spec.eps, self.spec.groups, alpha, out,
                                    gate=gate, gate_bias=gate_bias, dtype=self.rt.dtype)
        return residual if out is None else out

    def gather_add_norm(self, residual: torch.Tensor, delta, rows: torch.Tensor) -> torch.Tensor:
        if delta is not None and not isinstance(delta, StreamCopy):
            raise ValueError("the group norm gathers rows of a stream that has nothing pending")
        out = self.rt.empty(rows.shape[0], residual.shape[1])
        self.rt.ops.gather_group_norm(residual, rows, self.weight, self.spec.eps, self.spec.groups, out)
        return out
