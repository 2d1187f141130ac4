"""Mixers side by side on one input.

Every branch is a mixer of any registered kind and reads the same rows.  How the results meet is
the spec's ``combine``: each branch's result RMS-normed over the model width with a weight of its
own and the mean of those taken ("normed_mean"), or the results added with fixed factors
("weighted_sum"); one kernel either way.  The branches' caches travel under one cache id as a ``CompositeCacheSpec``:
pages for the branches that keep keys and values, the request's slot row for those with state.
"""
from __future__ import annotations

from typing import Dict

from .base import MIXERS, CompositeCacheSpec, ParamSpec, Part, register_mixer


@register_mixer("parallel")
class ParallelMixer(Part):
    kernels = ("sandwich",)

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if not spec.branches or len(spec.names) != len(spec.branches) or len(set(spec.names)) != len(spec.names):
            raise ValueError("a parallel mixer needs branches, each with a name of its own")
        self.combine = getattr(spec, "combine", "normed_mean")
        if self.combine not in ("normed_mean", "weighted_sum"):
            raise ValueError(f"combine '{self.combine}' is not known (normed_mean, weighted_sum)")
        if self.combine == "weighted_sum" and len(spec.scales) != len(spec.branches):
            raise ValueError("a weighted sum needs one factor per branch")
        self.branches = [MIXERS.build(b, rt) for b in spec.branches]
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.branches)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        if getattr(spec, "combine", "normed_mean") == "weighted_sum":
            return {}
        return {f"{n}_out": ParamSpec((spec.hidden_size,), role="vector", init="ones") for n in spec.names}

    def children(self) -> Dict[str, Part]:
        return dict(zip(self.spec.names, self.branches))

    def load(self, tensors):
        self.weights = [tensors[f"{n}_out"] for n in self.spec.names] if self.combine == "normed_mean" else []

    def cache_spec(self):
        return CompositeCacheSpec(tuple(b.cache_spec() for b in self.branches))

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        ys = [b.forward(x, ctx, cache[i], writes_cache) for i, b in enumerate(self.branches)]
        out = self.rt.empty(*ys[0].shape)
        if self.combine == "weighted_sum":
            self.rt.ops.branch_sum(ys, self.spec.scales, out)
        else:
            self.rt.ops.branch_mean(ys, self.weights, self.spec.eps, out)
        return out
