"""Block arrangements: how norms, mixer and feed-forward sit on the residual stream.

``pre_norm`` is the reference's order (models/llama/llama_model.cpp:502-655):
``x += mixer(norm1(x)); x += ffn(norm2(x))``.  The residual stream is a 32-bit
tensor updated in place.  Each addition is fused with the norm that follows it,
so a block hands its feed-forward output back as ``pending`` (not yet added) and
the next block's first norm, or the head's final norm, adds it.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FEED_FORWARDS, MIXERS, NORMS, ParamSpec, Part, register_block
from .norm import StreamCopy


@register_block("pre_norm")
class PreNormBlock(Part):
    graph_safe = True
    replayable = True
    folds_next = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mixer_norm = NORMS.build(spec.mixer_norm, rt)
        self.mixer = MIXERS.build(spec.mixer, rt)
        self.ffn_norm = NORMS.build(spec.ffn_norm, rt) if spec.ffn is not None else None
        self.ffn = FEED_FORWARDS.build(spec.ffn, rt) if spec.ffn is not None else None

    def children(self) -> Dict[str, Part]:
        c = {"mixer_norm": self.mixer_norm, "mixer": self.mixer}
        if self.ffn is not None:
            c.update(ffn_norm=self.ffn_norm, ffn=self.ffn)
        return c

    def first_norm(self):
        """The norm this block's input meets first, if the block before may fold it into its last
        product."""
        return self.mixer_norm if self.mixer_norm.foldable else None

    def _input(self, h, part):
        """``h`` as ``part`` can take it: a norm's output with the rows' scale still owed only if the
        part says so."""
        if isinstance(h, torch.Tensor) or part.takes_unnormed:
            return h
        return self.rt.ops.finish_norm(h)

    def forward(self, residual: torch.Tensor, pending, ctx, cache, writes_cache: bool = True,
                next_norm=None):
        """``pending`` is the output of the block before, not yet added to the residual stream; or,
        if that block was given this block's ``first_norm()`` as its ``next_norm`` and folded it,
        an ``ops.NormOut``: added already, and what the mixer takes.  What comes back is the one or
        the other in the same way."""
        ops = self.rt.ops
        fold = getattr(ops, "folds_norm", None)
        fold = fold is not None and fold(residual.shape[0], self.rt.dtype)
        if isinstance(pending, getattr(ops, "NormOut", ())):
            h = pending
        else:
            h = self.mixer_norm.add_norm(residual, pending)
        if self.ffn is None:
            # the mixer's result is the block's: the norm it meets next is the next block's or the head's
            if fold and next_norm is not None and self.mixer.folds_norm:
                return self.mixer.forward(self._input(h, self.mixer), ctx, cache, writes_cache,
                                          into=(residual, *next_norm.fold()))
            return self.mixer.forward(self._input(h, self.mixer), ctx, cache, writes_cache)
        if fold and self.mixer.folds_norm and self.ffn_norm.foldable:
            h = self.mixer.forward(self._input(h, self.mixer), ctx, cache, writes_cache,
                                   into=(residual, *self.ffn_norm.fold()))
        else:
            a = self.mixer.forward(self._input(h, self.mixer), ctx, cache, writes_cache)
            h = self.ffn_norm.add_norm(residual, a)
        if fold and next_norm is not None and self.ffn.folds_norm:
            return self.ffn.forward(self._input(h, self.ffn), ctx, into=(residual, *next_norm.fold()))
        return self.ffn.forward(self._input(h, self.ffn), ctx)


class TokenSide(Part):
    """A narrow second embedding of the token, added to the stream at the end of a block:
    ``x += unit(W_proj (act(W_gate x) * e)) * w``, where ``e`` is this block's ``dim`` columns of the
    table the embedding holds beside its own and ``unit`` divides by the root mean square."""

    graph_safe = True
    kernels = ("gemm", "rownorm")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.table = None

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        return {"gate": ParamSpec((spec.dim, spec.hidden_size)), "proj": ParamSpec((spec.hidden_size, spec.dim)),
                "norm": ParamSpec((spec.hidden_size,), role="vector", init="ones")}

    def load(self, tensors):
        self.w_gate = tensors["gate"].contiguous()
        self.w_proj = tensors["proj"].contiguous()
        self.norm = tensors["norm"]

    def bind_embedding(self, embedding) -> None:
        table = getattr(embedding, "side_weight", None)
        if table is None or table.shape[1] < self.spec.offset + self.spec.dim:
            raise ValueError("the embedding has no table of per-token inputs wide enough for this block")
        self.table = table

    def forward(self, residual: torch.Tensor, h: torch.Tensor, ctx) -> torch.Tensor:
        s, ops = self.spec, self.rt.ops
        g = ops.linear(h, self.w_gate)
        ge = self.rt.empty(*g.shape)
        ops.token_side_gate(g, self.table, ctx.token_ids, s.offset, s.activation, ge)
        y = ops.linear(ge, self.w_proj)
        out = None if self.rt.dtype == torch.float32 else self.rt.empty(*residual.shape)
        ops.unit_add(residual, y, self.norm, s.eps, out)
        return residual if out is None else out


@register_block("post_norm")
class PostNormBlock(Part):
    """``x <- norm1(alpha x + g1 * mixer(x)); x <- norm2(alpha x + g2 * ffn(x))``, then the per-token
    side input if the spec has one.  The sublayers read the stream itself; with ``gated_residual``
    ``g = sigmoid(W x + b)`` of the sublayer's input multiplies its result, else g = 1.  The stream
    is 32-bit and updated in place; each sum, its gate and the norm behind it are one kernel, which
    also leaves the rounded copy that the next products read.  ``ffn`` None: no second step.

    What it hands on is a ``StreamCopy``: nothing pending, and the copy for whoever reads next."""

    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mixer_norm = NORMS.build(spec.mixer_norm, rt)
        self.mixer = MIXERS.build(spec.mixer, rt)
        self.ffn = FEED_FORWARDS.build(spec.ffn, rt) if spec.ffn is not None else None
        self.ffn_norm = NORMS.build(spec.ffn_norm, rt) if spec.ffn is not None else None
        self.side = TokenSide(spec.side, rt) if spec.side is not None else None
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and not hasattr(n, "scale_add_norm"):
                raise ValueError(f"a norm of kind '{n.spec.kind}' cannot follow the sum (no scale_add_norm)")

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        p, H = {}, spec.hidden_size
        if spec.gated_residual:
            p["mixer_gate"] = ParamSpec((H, H))
            p["mixer_gate_bias"] = ParamSpec((H,), role="vector", init="normal")
            if spec.ffn is not None:
                p["ffn_gate"] = ParamSpec((H, H))
                p["ffn_gate_bias"] = ParamSpec((H,), role="vector", init="normal")
        return p

    def load(self, tensors):
        self.gates = {k: v.contiguous() for k, v in tensors.items()}

    def children(self) -> Dict[str, Part]:
        c = {"mixer_norm": self.mixer_norm, "mixer": self.mixer}
        if self.ffn is not None:
            c.update(ffn_norm=self.ffn_norm, ffn=self.ffn)
        if self.side is not None:
            c["side"] = self.side
        return c

    def bind_embedding(self, embedding) -> None:
        if self.side is not None:
            self.side.bind_embedding(embedding)

    def _sublayer(self, residual, h, y, norm, which):
        gate = bias = None
        if self.spec.gated_residual:
            gate = self.rt.ops.linear(h, self.gates[which + "_gate"])
            bias = self.gates[which + "_gate_bias"]
        return norm.scale_add_norm(residual, self.spec.alpha, y, gate, bias)

    def forward(self, residual: torch.Tensor, pending, ctx, cache, writes_cache: bool = True):
        ops = self.rt.ops
        if isinstance(pending, StreamCopy):
            h = pending.values
        elif pending is not None:
            raise ValueError("a block that norms after the sum cannot take a pending delta")
        elif self.rt.dtype == torch.float32:
            h = residual
        else:
            h = self.rt.empty(*residual.shape)
            ops.cast_rows(residual, h)
        y = self.mixer.forward(h, ctx, cache, writes_cache)
        h = self._sublayer(residual, h, y, self.mixer_norm, "mixer")
        if self.ffn is not None:
            y = self.ffn.forward(h, ctx)
            h = self._sublayer(residual, h, y, self.ffn_norm, "ffn")
        if self.side is not None:
            h = self.side.forward(residual, h, ctx)
        return StreamCopy(h)


@register_block("sandwich_norm")
class SandwichBlock(Part):
    """``x += mult * post1(mixer(norm1(x))); x += mult * post2(ffn(norm2(x)))``: a norm in front of and
    behind every sublayer.  The stream is 32-bit and updated in place.  The norm behind a sublayer,
    the sum and the norm in front of the next sublayer are one kernel, so the block hands its last
    sublayer's output on as a ``NormedDelta`` that the next block's first norm, or the head's, takes.
    ``step``: a vector that joins the stream before the block's first norm (a pass through looped
    layers begins here)."""

    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mixer_norm = NORMS.build(spec.mixer_norm, rt)
        self.mixer = MIXERS.build(spec.mixer, rt)
        self.mixer_post_norm = NORMS.build(spec.mixer_post_norm, rt)
        self.ffn = FEED_FORWARDS.build(spec.ffn, rt) if spec.ffn is not None else None
        self.ffn_norm = NORMS.build(spec.ffn_norm, rt) if spec.ffn is not None else None
        self.ffn_post_norm = NORMS.build(spec.ffn_post_norm, rt) if spec.ffn is not None else None
        for n in (self.mixer_post_norm, self.ffn_post_norm):
            if n is not None and not hasattr(n, "pending"):
                raise ValueError(f"a norm of kind '{n.spec.kind}' cannot stand behind a sublayer (no pending)")

    def children(self) -> Dict[str, Part]:
        c = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_post_norm": self.mixer_post_norm}
        if self.ffn is not None:
            c.update(ffn_norm=self.ffn_norm, ffn=self.ffn, ffn_post_norm=self.ffn_post_norm)
        return c

    def forward(self, residual: torch.Tensor, pending, ctx, cache, writes_cache: bool = True, step=None):
        mult = self.spec.residual_mult
        h = self.mixer_norm.add_norm(residual, pending, step) if step is not None \
            else self.mixer_norm.add_norm(residual, pending)
        y = self.mixer.forward(h, ctx, cache, writes_cache)
        if self.ffn is None:
            return self.mixer_post_norm.pending(y, mult)
        h = self.ffn_norm.add_norm(residual, self.mixer_post_norm.pending(y, mult))
        return self.ffn_post_norm.pending(self.ffn.forward(h, ctx), mult)
