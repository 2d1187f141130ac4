"""Token embedding and output head.

Embedding: ``h0[t, :] = E[id_t, :]`` (times the spec's ``scale``, 1 in the reference) with no position term
(reference: kernels/src/embedding.cu:12-26, models/llama/llama_model.cpp:424-425);
the rows are widened into the 32-bit residual stream.

Head: final norm, then ``logits = x W^T`` with no bias, scale or soft cap; with
tied embeddings ``W`` is the embedding table (llama_model.cpp:257-261,658-666).
The reference multiplies every token's row by the vocabulary matrix and copies
one row out (llama_model.cpp:663-698); here only the rows whose logits are
wanted are gathered, before the norm, so the large product has as many rows as
answers.  Logits are 32-bit.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import NORMS, ParamSpec, Part, StateSpec


class Embedding(Part):
    graph_safe = True
    kernels = ("embedding",)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        p = {"weight": ParamSpec((spec.vocab_size, spec.hidden_size), role="table")}
        if getattr(spec, "side_size", 0):
            # a second table of per-token inputs that blocks pick their columns from
            p["side_weight"] = ParamSpec((spec.vocab_size, spec.side_size), role="table")
        if getattr(spec, "pair_buckets", 0):
            # a table indexed by a hash of the token and the one before it, added to the token's row
            p["pair_weight"] = ParamSpec((spec.pair_buckets + 1, spec.hidden_size), role="table")
        return p

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()
        if "side_weight" in tensors:
            self.side_weight = tensors["side_weight"].contiguous()
        if "pair_weight" in tensors:
            self.pair_weight = tensors["pair_weight"].contiguous()

    def cache_spec(self):
        """What the embedding keeps per request between steps: with a table of token pairs, the last
        token of the step before (one int per slot); else nothing."""
        return StateSpec((), dtype=torch.int32) if getattr(self.spec, "pair_buckets", 0) else None

    def forward(self, token_ids: torch.Tensor, ctx=None, cache=None) -> torch.Tensor:
        out = self.rt.empty(token_ids.shape[0], self.spec.hidden_size, dtype=torch.float32)
        scale = float(getattr(self.spec, "scale", 1.0))
        if getattr(self.spec, "pair_buckets", 0):
            if ctx is None or cache is None:
                raise ValueError("an embedding with a table of token pairs needs the step and its state")
            s = self.spec
            self.rt.ops.embedding_pair(self.weight, self.pair_weight, ctx, cache.state, s.pair_buckets, s.pair_mul_prev,
                                       s.pair_mul_cur, out, scale)
        elif scale != 1.0:
            self.rt.ops.embedding(self.weight, token_ids, out, scale)
        else:
            self.rt.ops.embedding(self.weight, token_ids, out)
        return out


class StepVectors(Part):
    """A table of vectors of model width, one of which the run order may add to the stream before
    a layer call (the number of the pass through a looped stretch of layers).  32-bit."""

    graph_safe = True

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        rows, width = spec
        return {"table": ParamSpec((rows, width), role="vector", init="normal")}

    def load(self, tensors):
        self.table = tensors["table"].contiguous()

    def row(self, i: int) -> torch.Tensor:
        return self.table[i]


class LMHead(Part):
    graph_safe = True
    kernels = ("gemm", "norm")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.norm = NORMS.build(spec.norm, rt)
        self.weight: Optional[torch.Tensor] = None
        if getattr(spec, "logit_softcap", None):
            self.kernels = self.kernels + ("activation",)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        if spec.tied:
            return {}
        return {"weight": ParamSpec((spec.vocab_size, spec.hidden_size))}

    def children(self) -> Dict[str, Part]:
        return {"norm": self.norm}

    def load(self, tensors):
        if not self.spec.tied:
            self.weight = tensors["weight"].contiguous()

    def tie(self, embedding: Embedding) -> None:
        self.weight = embedding.weight

    def forward(self, residual: torch.Tensor, pending: Optional[torch.Tensor],
                rows: torch.Tensor) -> torch.Tensor:
        h = self.norm.gather_add_norm(residual, pending, rows)
        logits = self.rt.ops.linear(h, self.weight, out_dtype=torch.float32)
        cap = getattr(self.spec, "logit_softcap", None)
        if cap:
            self.rt.ops.softcap(logits, float(cap))           # cap * tanh(logits / cap), in place
        return logits
