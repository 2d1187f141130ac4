"""FikizenConfig: the Fikizen decoder's configuration, read from config.json keys.

A Fikizen model is a list of layers in pre-norm arrangement (``x += mixer(norm1(x))``, then
``x += ff(norm2(x))`` where the layer has a feed-forward), each with one of three mixers.
``attention``: grouped softmax attention over a sliding window with a sink in the softmax, heads
partly rotated (halves paired) and one sigmoid gate number per head.  ``parallel``: two mixers on
the same input whose results are added with fixed factors; ``left`` is windowed sink attention with
biased projections, q and k normed over all their heads at once and value heads of unit rms,
``right`` a delta-rule memory with a decay and a removal rate per key channel.  ``delta``: a
delta-rule memory with one fade and one write strength per head, behind short convolutions.  The
feed-forward is dense and ungated with a two-branch activation that has two learnt numbers.  A
layer may use another layer's weights (``weights_of``) with a cache or state of its own.  The
logits pass a soft cap.  Every size and constant below comes from config.json; the tensor names are
those of the checkpoint.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Mapping, Optional, Tuple

from .llama import ConfigError
from .specs import (BlockSpec, ChannelDeltaSpec, DenseMLPSpec, EmbeddingSpec, GatedDeltaSpec, HeadSpec, KVAttentionSpec,
                    LayerCall, ModelSpec, ParallelMixerSpec, RMSNormSpec, RotarySpec)

MIXER_KINDS = ("attention", "parallel", "delta")


def _get(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _pos_int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where} '{key}' must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class FikizenAttention:
    """Windowed sink attention as either mixer has it."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class FikizenChannelMemory:
    heads: int
    dim: int
    # hidden size of the low-rank decay projection: no key of config.json gives it, the shape of the
    # stored tensor does (``FikizenConfig.with_checkpoint_shapes``)
    decay_rank: int = 16


@dataclass(frozen=True)
class FikizenGatedMemory:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class FikizenLayer:
    kind: str
    attention: Optional[FikizenAttention] = None            # the mixer itself, or the left one of a pair
    channel: Optional[FikizenChannelMemory] = None           # the right one of a pair
    gated: Optional[FikizenGatedMemory] = None               # the ``delta`` mixer
    left_scale: float = 1.0
    right_scale: float = 1.0
    ff: Optional[int] = None                                 # None: no feed-forward
    weights_of: Optional[int] = None                         # the layer whose tensors this one uses


@dataclass(frozen=True)
class FikizenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[FikizenLayer, ...]
    logit_softcap: Optional[float] = None

    architecture = "Fikizen"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "FikizenConfig":
        norm = _get(d, "norm", "the model")
        raw_layers = _get(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        cap = d.get("logit_softcap")
        cfg = cls(vocab=_pos_int(d, "vocab", "the model"), width=_pos_int(d, "width", "the model"),
                  norm_eps=float(_get(norm, "eps", "'norm'")),
                  layers=tuple(cls._parse_layer(i, e) for i, e in enumerate(raw_layers)),
                  logit_softcap=None if cap is None else float(cap))
        cfg.validate()
        return cfg

    @staticmethod
    def _parse_attention(m: Mapping[str, Any], where: str) -> FikizenAttention:
        heads = _pos_int(m, "heads", where)
        rot, mask = _get(m, "rot", where), _get(m, "mask", where)
        return FikizenAttention(
            heads=heads, kv_heads=_pos_int(m, "kv_heads", where) if m.get("kv_heads") is not None else heads,
            dim=_pos_int(m, "dim", where), vdim=_pos_int(m, "vdim", where), scale=float(_get(m, "scale", where)),
            window=_pos_int(mask, "size", where + " mask"), rot_dims=_pos_int(rot, "dims", where + " rot"),
            rot_base=float(_get(rot, "base", where + " rot")))

    @classmethod
    def _parse_layer(cls, i: int, entry: Mapping[str, Any]) -> FikizenLayer:
        where = f"layer {i}"
        kind = _get(entry, "type", where)
        if kind not in MIXER_KINDS:
            raise ConfigError(f"config.json: {where} has type '{kind}' (known: {', '.join(MIXER_KINDS)})")
        m = _get(entry, "mixer", where)
        mlp, ff = entry.get("mlp"), None
        if mlp is not None:
            if mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"config.json: {where} has a feed-forward of kind '{mlp.get('kind')}' (known: dense)")
            ff = _pos_int(mlp, "ff", where + " mlp")
        of = entry.get("weights_of")
        if of is not None and (isinstance(of, bool) or not isinstance(of, int)):
            raise ConfigError(f"config.json: {where} 'weights_of' must name a layer by its number, got {of!r}")
        common = dict(ff=ff, weights_of=of)
        if kind == "attention":
            return FikizenLayer(kind, attention=cls._parse_attention(m, where), **common)
        if kind == "delta":
            heads = _pos_int(m, "heads", where)
            gated = FikizenGatedMemory(
                heads=heads, kv_heads=_pos_int(m, "kv_heads", where) if m.get("kv_heads") is not None else heads,
                dim=_pos_int(m, "dim", where), vdim=_pos_int(m, "vdim", where), conv=_pos_int(m, "conv", where))
            return FikizenLayer(kind, gated=gated, **common)
        right = _get(m, "right", where)
        channel = FikizenChannelMemory(heads=_pos_int(right, "heads", where + " right"),
                                       dim=_pos_int(right, "dim", where + " right"))
        return FikizenLayer(kind, attention=cls._parse_attention(_get(m, "left", where), where + " left"), channel=channel,
                            left_scale=float(_get(m, "left_scale", where)), right_scale=float(_get(m, "right_scale", where)),
                            **common)

    def validate(self) -> None:
        if self.norm_eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if self.logit_softcap is not None and self.logit_softcap <= 0:
            raise ConfigError(f"logit_softcap must be positive, got {self.logit_softcap}")
        for i, l in enumerate(self.layers):
            a = l.attention
            if a is not None:
                if a.heads % a.kv_heads:
                    raise ConfigError(f"layer {i}: {a.heads} heads cannot share {a.kv_heads} kv heads")
                if a.rot_dims % 2 or a.rot_dims > a.dim:
                    raise ConfigError(f"layer {i}: rot.dims {a.rot_dims} must be even and at most dim {a.dim}")
                if a.rot_base <= 0:
                    raise ConfigError(f"layer {i}: rot.base must be positive")
            if l.gated is not None and l.gated.heads % l.gated.kv_heads:
                raise ConfigError(f"layer {i}: {l.gated.heads} heads cannot share {l.gated.kv_heads} kv heads")
            if l.weights_of is not None:
                j = l.weights_of
                if not 0 <= j < len(self.layers) or j == i or self.layers[j].weights_of is not None:
                    raise ConfigError(f"layer {i}: weights_of {j} must name another layer that has weights of its own")
                o = self.layers[j]
                if (o.kind, o.attention, o.channel, o.gated, o.left_scale, o.right_scale, o.ff) != \
                        (l.kind, l.attention, l.channel, l.gated, l.left_scale, l.right_scale, l.ff):
                    raise ConfigError(f"layer {i}: uses the weights of layer {j} but is described differently")

    # ------------------------------------------------------------------ writing
    @staticmethod
    def _attention_dict(a: FikizenAttention) -> dict:
        return {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale,
                "mask": {"size": a.window}, "rot": {"base": a.rot_base, "dims": a.rot_dims}}

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            if l.kind == "attention":
                m = self._attention_dict(l.attention)
            elif l.kind == "delta":
                g = l.gated
                m = {"heads": g.heads, "kv_heads": g.kv_heads, "dim": g.dim, "vdim": g.vdim, "conv": g.conv}
            else:
                m = {"left": self._attention_dict(l.attention), "right": {"heads": l.channel.heads, "dim": l.channel.dim},
                     "left_scale": l.left_scale, "right_scale": l.right_scale}
            e = {"type": l.kind, "mixer": m, "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}}
            if l.weights_of is not None:
                e["weights_of"] = l.weights_of
            layers.append(e)
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d

    # -------------------------------------------------------------- translation
    def _attention_spec(self, a: FikizenAttention, left: bool) -> KVAttentionSpec:
        position = RotarySpec(head_dim=a.dim, rotary_dim=a.rot_dims, theta=a.rot_base, pairing="half")
        return KVAttentionSpec(hidden_size=self.width, num_heads=a.heads, num_kv_heads=a.kv_heads, key_dim=a.dim,
                               value_dim=a.vdim, scale=a.scale, window=a.window, qkv_bias=left, qk_norm=left,
                               qk_norm_span="all" if left else "head", v_unit_norm=left, eps=self.norm_eps, sink=True,
                               out_gate=not left, gate_per_head=not left, position=position)

    def _mixer_spec(self, l: FikizenLayer):
        if l.kind == "attention":
            return self._attention_spec(l.attention, left=False)
        if l.kind == "delta":
            g = l.gated
            return GatedDeltaSpec(hidden_size=self.width, num_heads=g.heads, num_key_heads=g.kv_heads, key_dim=g.dim,
                                  value_dim=g.vdim, conv_taps=g.conv, eps=self.norm_eps)
        c = l.channel
        right = ChannelDeltaSpec(hidden_size=self.width, num_heads=c.heads, key_dim=c.dim, decay_rank=c.decay_rank,
                                 eps=self.norm_eps)
        return ParallelMixerSpec(hidden_size=self.width, branches=(self._attention_spec(l.attention, left=True), right),
                                 names=("left", "right"), eps=self.norm_eps, combine="weighted_sum",
                                 scales=(l.left_scale, l.right_scale))

    @staticmethod
    def _mixer_names(l: FikizenLayer, p: str, b: str):
        """(checkpoint name, (owner path, the part's parameter)) of a layer's mixer."""
        if l.kind == "attention":
            pairs = [("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o")]
            return [(p + ck, (b, local)) for ck, local in pairs]
        if l.kind == "delta":
            pairs = [("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("b", "b"), ("a", "a"),
                     ("q.conv", "q_conv"), ("k.conv", "k_conv"), ("v.conv", "v_conv"), ("A_log", "A_log"),
                     ("dt_bias", "dt_bias"), ("norm", "norm")]
            return [(p + ck, (b, local)) for ck, local in pairs]
        left = [("q", "q"), ("q.b", "q_bias"), ("k", "k"), ("k.b", "k_bias"), ("v", "v"), ("v.b", "v_bias"), ("o", "o"),
                ("q.norm", "q_norm"), ("k.norm", "k_norm")]
        right = [("r", "r"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("a", "a"), ("a.b", "a_bias"), ("w1", "w1"),
                 ("w2", "w2"), ("w0", "w0"), ("norm", "norm")]
        return ([(p + "left." + ck, (b + ".left", local)) for ck, local in left] +
                [(p + "right." + ck, (b + ".right", local)) for ck, local in right])

    def to_model_spec(self) -> ModelSpec:
        W = self.width
        norm = RMSNormSpec(size=W, eps=self.norm_eps)
        names = [("embed", ("embedding", "weight")), ("final.norm", ("head.norm", "weight")), ("head", ("head", "weight"))]
        blocks, block_of = [], {}
        for i, l in enumerate(self.layers):
            if l.weights_of is not None:
                continue
            p, b = f"l{i}.", f"blocks.{len(blocks)}"
            block_of[i] = len(blocks)
            ffn = None if l.ff is None else DenseMLPSpec(hidden_size=W, intermediate_size=l.ff, activation="bent_square")
            blocks.append(BlockSpec(mixer=self._mixer_spec(l), ffn=ffn, mixer_norm=norm,
                                    ffn_norm=norm if ffn is not None else None))
            names.append((p + "norm1", (b + ".mixer_norm", "weight")))
            names += self._mixer_names(l, p + "mix.", b + ".mixer")
            if ffn is not None:
                names += [(p + "norm2", (b + ".ffn_norm", "weight")), (p + "mlp.up", (b + ".ffn", "up_proj")),
                          (p + "mlp.down", (b + ".ffn", "down_proj")), (p + "mlp.act", (b + ".ffn", "act"))]
        # every layer has a cache of its own, also one that borrows its weights
        order = tuple(LayerCall(block=block_of[i if l.weights_of is None else l.weights_of], cache=i)
                      for i, l in enumerate(self.layers))
        return ModelSpec(
            architecture=self.architecture,
            embedding=EmbeddingSpec(vocab_size=self.vocab, hidden_size=W),
            blocks=tuple(blocks), order=order,
            head=HeadSpec(vocab_size=self.vocab, hidden_size=W, tied=False, norm=norm, logit_softcap=self.logit_softcap),
            tensor_names=tuple(names))

    def with_checkpoint_shapes(self, shapes: Mapping[str, Tuple[int, ...]]) -> "FikizenConfig":
        """The configuration with what only the checkpoint's shapes tell filled in: the hidden size of
        each decay projection, ``l<i>.mix.right.w1`` [rank, width]."""
        layers = list(self.layers)
        for i, l in enumerate(layers):
            src = i if l.weights_of is None else l.weights_of
            shape = shapes.get(f"l{src}.mix.right.w1")
            if l.kind == "parallel" and shape is not None and len(shape) == 2:
                layers[i] = replace(l, channel=replace(l.channel, decay_rank=int(shape[0])))
        return replace(self, layers=tuple(layers))
