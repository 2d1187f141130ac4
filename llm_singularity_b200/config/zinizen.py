"""ZinizenConfig: the Zinizen decoder's configuration, read from config.json keys.

A Zinizen model is a list of layers, each with one of three mixers and a feed-forward of one of two
kinds (or none).  ``attention``: grouped softmax attention over all earlier tokens, no rotation; q
and k are each normed over the whole projection, the query grows with the logarithm of its position
in steps, scaled scores are capped by ``cap * tanh(s / cap)`` and lowered in proportion to the key's
distance with a slope per head; the layers that say ``v_mix`` blend their values with those the
first such layer made of the same token.  ``latent_attention``: keys and values made per head from
one cached latent per token plus a rotated key part shared by the heads, queries through a latent of
their own, a sigmoid gate of one number per head.  ``rglru``: a recurrent block with a real-gated
linear recurrent unit behind a short convolution.  Feed-forwards: ``dense`` (two products around the
tanh form of gelu) or ``moe`` (softmax router whose choice takes a learnt correction per expert,
capped gated experts, an optional shared expert).  Every sublayer has a centred norm with weight and
bias in front and behind (``x += norm_b(sublayer(norm(x)))``).  The embedding adds a row of a second
table chosen by a hash of the token and the one before it.  Every size and constant below comes
from config.json; the tensor names are those of the checkpoint.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .llama import ConfigError
from .specs import (DenseMLPSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, KVAttentionSpec, LatentAttentionSpec, LayerCall,
                    LayerNormSpec, ModelSpec, MoESpec, RGLRUSpec, RotarySpec, SandwichBlockSpec)

MIXER_KINDS = ("attention", "latent_attention", "rglru")
MLP_KINDS = ("dense", "moe")
RGLRU_RATE = 8.0             # log a = -RGLRU_RATE * r * softplus(lam)
RENORM_EPS = 1e-20           # joins the sum of the chosen scores before the division
EXPERT_ACTIVATION = "capped_glu"


def _get(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _pos_int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where} '{key}' must be a positive integer, got {v!r}")
    return v


def _pos_float(d: Mapping[str, Any], key: str, where: str) -> float:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not v > 0:
        raise ConfigError(f"config.json: {where} '{key}' must be a positive number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class ZinizenAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float] = None
    temp_coef: float = 0.0
    temp_every: int = 0               # 0: no query temperature
    v_mix: bool = False


@dataclass(frozen=True)
class ZinizenLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class ZinizenRecurrent:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class ZinizenMLP:
    kind: str
    ff: int = 0                       # dense: hidden size; moe: an expert's
    limit: float = 0.0                # moe: the experts' cap
    experts: int = 0
    top: int = 0
    scale: float = 1.0                # moe: multiplies the renormalised weights
    shared_ff: int = 0                # 0: no shared expert
    shared_limit: float = 0.0


@dataclass(frozen=True)
class ZinizenLayer:
    kind: str
    mixer: Any                        # ZinizenAttention | ZinizenLatent | ZinizenRecurrent
    mlp: Optional[ZinizenMLP] = None


@dataclass(frozen=True)
class ZinizenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[ZinizenLayer, ...]
    bigram_buckets: int = 0           # 0: no table of token pairs
    bigram_mul_prev: int = 0
    bigram_mul_cur: int = 0

    architecture = "Zinizen"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ZinizenConfig":
        norm = _get(d, "norm", "the model")
        raw_layers = _get(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = tuple(cls._parse_layer(i, e) for i, e in enumerate(raw_layers))
        kw = {}
        bigram = (d.get("embedding") or {}).get("bigram")
        if bigram:
            kw = dict(bigram_buckets=_pos_int(bigram, "buckets", "embedding.bigram"),
                      bigram_mul_prev=int(_get(bigram, "mul_prev", "embedding.bigram")),
                      bigram_mul_cur=int(_get(bigram, "mul_cur", "embedding.bigram")))
        cfg = cls(vocab=_pos_int(d, "vocab", "the model"), width=_pos_int(d, "width", "the model"),
                  norm_eps=_pos_float(norm, "eps", "'norm'"), layers=layers, **kw)
        cfg.validate()
        return cfg

    @staticmethod
    def _parse_mixer(kind: str, m: Mapping[str, Any], where: str):
        if kind == "attention":
            heads = _pos_int(m, "heads", where)
            kw = dict(heads=heads, kv_heads=_pos_int(m, "kv_heads", where) if m.get("kv_heads") is not None else heads,
                      dim=_pos_int(m, "dim", where), vdim=_pos_int(m, "vdim", where),
                      scale=float(_get(m, "scale", where)), v_mix=bool(m.get("v_mix", False)))
            if m.get("softcap"):
                kw["softcap"] = _pos_float(m, "softcap", where)
            temp = m.get("q_temp")
            if temp:
                kw.update(temp_coef=float(_get(temp, "coef", where + " q_temp")),
                          temp_every=_pos_int(temp, "every", where + " q_temp"))
            return ZinizenAttention(**kw)
        if kind == "latent_attention":
            rot = _get(m, "rot", where)
            return ZinizenLatent(heads=_pos_int(m, "heads", where), dim=_pos_int(m, "dim", where),
                                 rot_dim=_pos_int(m, "rot_dim", where), vdim=_pos_int(m, "vdim", where),
                                 q_rank=_pos_int(m, "q_rank", where), kv_rank=_pos_int(m, "kv_rank", where),
                                 scale=float(_get(m, "scale", where)), rot_dims=_pos_int(rot, "dims", where + " rot"),
                                 rot_base=_pos_float(rot, "base", where + " rot"))
        return ZinizenRecurrent(width=_pos_int(m, "width", where), blocks=_pos_int(m, "blocks", where),
                                conv=_pos_int(m, "conv", where))

    @staticmethod
    def _parse_mlp(mlp: Mapping[str, Any], where: str) -> ZinizenMLP:
        kind = mlp.get("kind", "dense")
        if kind not in MLP_KINDS:
            raise ConfigError(f"config.json: {where} has a feed-forward of kind '{kind}' (known: {', '.join(MLP_KINDS)})")
        if kind == "dense":
            return ZinizenMLP("dense", ff=_pos_int(mlp, "ff", where + " mlp"))
        expert, router = _get(mlp, "expert", where + " mlp"), _get(mlp, "router", where + " mlp")
        kw = dict(ff=_pos_int(expert, "ff", where + " expert"), limit=_pos_float(expert, "limit", where + " expert"),
                  experts=_pos_int(router, "experts", where + " router"), top=_pos_int(router, "top", where + " router"),
                  scale=float(router.get("scale", 1.0)))
        shared = mlp.get("shared")
        if shared:
            kw.update(shared_ff=_pos_int(shared, "ff", where + " shared"),
                      shared_limit=_pos_float(shared, "limit", where + " shared"))
        return ZinizenMLP("moe", **kw)

    @classmethod
    def _parse_layer(cls, i: int, entry: Mapping[str, Any]) -> ZinizenLayer:
        where = f"layer {i}"
        kind = _get(entry, "type", where)
        if kind not in MIXER_KINDS:
            raise ConfigError(f"config.json: {where} has type '{kind}' (known: {', '.join(MIXER_KINDS)})")
        mlp = entry.get("mlp")
        return ZinizenLayer(kind, cls._parse_mixer(kind, _get(entry, "mixer", where), where),
                            None if mlp is None else cls._parse_mlp(mlp, where))

    def validate(self) -> None:
        shared_values = None
        for i, l in enumerate(self.layers):
            m = l.mixer
            if l.kind == "attention":
                if m.heads % m.kv_heads:
                    raise ConfigError(f"layer {i}: {m.heads} heads cannot share {m.kv_heads} kv heads")
                if m.v_mix:
                    if shared_values is None:
                        shared_values = m.kv_heads * m.vdim
                    elif shared_values != m.kv_heads * m.vdim:
                        raise ConfigError(f"layer {i}: v_mix layers must make values of one size, "
                                          f"{m.kv_heads * m.vdim} here and {shared_values} in the first")
            elif l.kind == "latent_attention":
                if m.rot_dims % 2 or m.rot_dims > m.rot_dim:
                    raise ConfigError(f"layer {i}: rot.dims {m.rot_dims} must be even and at most rot_dim {m.rot_dim}")
            elif m.width % m.blocks:
                raise ConfigError(f"layer {i}: {m.blocks} blocks do not divide a width of {m.width}")
            if l.mlp is not None and l.mlp.kind == "moe" and l.mlp.top > l.mlp.experts:
                raise ConfigError(f"layer {i}: top {l.mlp.top} of {l.mlp.experts} experts")

    # ------------------------------------------------------------------ writing
    @staticmethod
    def _mixer_dict(l: ZinizenLayer) -> dict:
        m = l.mixer
        if l.kind == "attention":
            d = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
            if m.softcap:
                d["softcap"] = m.softcap
            if m.temp_every:
                d["q_temp"] = {"coef": m.temp_coef, "every": m.temp_every}
            if m.v_mix:
                d["v_mix"] = True
            return d
        if l.kind == "latent_attention":
            return {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "q_rank": m.q_rank,
                    "kv_rank": m.kv_rank, "scale": m.scale, "rot": {"base": m.rot_base, "dims": m.rot_dims}}
        return {"width": m.width, "blocks": m.blocks, "conv": m.conv}

    @staticmethod
    def _mlp_dict(f: Optional[ZinizenMLP]):
        if f is None:
            return None
        if f.kind == "dense":
            return {"kind": "dense", "ff": f.ff}
        d = {"kind": "moe", "expert": {"ff": f.ff, "limit": f.limit},
             "router": {"experts": f.experts, "top": f.top, "scale": f.scale}}
        if f.shared_ff:
            d["shared"] = {"ff": f.shared_ff, "limit": f.shared_limit}
        return d

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": [{"type": l.kind, "mixer": self._mixer_dict(l), "mlp": self._mlp_dict(l.mlp)} for l in self.layers]}
        if self.bigram_buckets:
            d["embedding"] = {"bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev,
                                         "mul_cur": self.bigram_mul_cur}}
        return d

    # -------------------------------------------------------------- translation
    def _mixer_spec(self, l: ZinizenLayer, first_mix: Optional[int], i: int):
        W, m = self.width, l.mixer
        if l.kind == "attention":
            return KVAttentionSpec(hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, key_dim=m.dim,
                                   value_dim=m.vdim, scale=m.scale, qk_norm=True, qk_norm_span="all", eps=self.norm_eps,
                                   temp_coef=m.temp_coef, temp_every=m.temp_every, logit_softcap=m.softcap,
                                   linear_bias=True,
                                   value_mix=None if not m.v_mix else ("source" if i == first_mix else "mixed"))
        if l.kind == "latent_attention":
            return LatentAttentionSpec(hidden_size=W, num_heads=m.heads, plain_dim=m.dim, rot_dim=m.rot_dim,
                                       value_dim=m.vdim, q_rank=m.q_rank, kv_rank=m.kv_rank, scale=m.scale,
                                       eps=self.norm_eps, gate_per_head=True,
                                       position=RotarySpec(head_dim=m.rot_dim, rotary_dim=m.rot_dims, theta=m.rot_base,
                                                           pairing="half"))
        return RGLRUSpec(hidden_size=W, width=m.width, blocks=m.blocks, conv_taps=m.conv, rate=RGLRU_RATE)

    def _ffn_spec(self, f: Optional[ZinizenMLP]):
        if f is None:
            return None
        W = self.width
        if f.kind == "dense":
            return DenseMLPSpec(hidden_size=W, intermediate_size=f.ff, activation="gelu_tanh")
        shared = None
        if f.shared_ff:
            shared = GatedMLPSpec(hidden_size=W, intermediate_size=f.shared_ff, activation=EXPERT_ACTIVATION,
                                  limit=f.shared_limit)
        return MoESpec(hidden_size=W, expert_size=f.ff, num_experts=f.experts, top=f.top, activation=EXPERT_ACTIVATION,
                       score="softmax", renormalize=True, weight_on="output", choice_bias=True, weight_scale=f.scale,
                       renorm_eps=RENORM_EPS, limit=f.limit, shared=shared)

    @staticmethod
    def _mixer_names(l: ZinizenLayer, p: str, b: str, source: bool):
        """(checkpoint name, (owner path, the part's parameter)) of a layer's mixer."""
        if l.kind == "attention":
            pairs = [("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q.norm", "q_norm"), ("k.norm", "k_norm")]
            if l.mixer.v_mix and not source:
                pairs.append(("vmix", "vmix"))
        elif l.kind == "latent_attention":
            pairs = [("dq", "dq"), ("dq.norm", "dq_norm"), ("uq", "uq"), ("dkv", "dkv"), ("dkv.norm", "dkv_norm"),
                     ("uk", "uk"), ("uv", "uv"), ("g", "g"), ("o", "o")]
        else:
            pairs = [("y", "y"), ("y.b", "y_bias"), ("x", "x"), ("x.b", "x_bias"), ("conv", "conv"),
                     ("conv.b", "conv_bias"), ("ra", "ra"), ("ra.b", "ra_bias"), ("ri", "ri"), ("ri.b", "ri_bias"),
                     ("lam", "lam"), ("o", "o")]
        return [(p + ck, (b, local)) for ck, local in pairs]

    @staticmethod
    def _mlp_names(f: ZinizenMLP, p: str, b: str):
        if f.kind == "dense":
            return [(p + "up", (b, "up_proj")), (p + "down", (b, "down_proj"))]
        names = [(p + "router", (b, "router")), (p + "correction", (b, "choice_bias"))]
        for e in range(f.experts):
            names += [(f"{p}e{e}.{w}", (b, f"e{e}.{w}")) for w in ("gate", "up", "down")]
        if f.shared_ff:
            names += [(f"{p}shared.{w}", (b + ".shared", w + "_proj")) for w in ("gate", "up", "down")]
        return names

    def to_model_spec(self) -> ModelSpec:
        W = self.width
        norm = LayerNormSpec(size=W, eps=self.norm_eps)
        names = [("embed", ("embedding", "weight")), ("final.norm", ("head.norm", "weight")),
                 ("final.norm.b", ("head.norm", "bias")), ("head", ("head", "weight"))]
        if self.bigram_buckets:
            names.append(("bigram", ("embedding", "pair_weight")))
        first_mix = next((i for i, l in enumerate(self.layers) if l.kind == "attention" and l.mixer.v_mix), None)
        blocks, ignorable = [], []
        for i, l in enumerate(self.layers):
            p, b = f"l{i}.", f"blocks.{i}"
            ffn = self._ffn_spec(l.mlp)
            blocks.append(SandwichBlockSpec(mixer=self._mixer_spec(l, first_mix, i), ffn=ffn, mixer_norm=norm,
                                            mixer_post_norm=norm, ffn_norm=norm if ffn is not None else None,
                                            ffn_post_norm=norm if ffn is not None else None))
            for ck, owner in (("norm1", "mixer_norm"), ("norm1b", "mixer_post_norm"), ("norm2", "ffn_norm"),
                              ("norm2b", "ffn_post_norm")):
                if ffn is None and ck.startswith("norm2"):
                    ignorable += [p + ck, p + ck + ".b"]
                else:
                    names += [(p + ck, (f"{b}.{owner}", "weight")), (p + ck + ".b", (f"{b}.{owner}", "bias"))]
            names += self._mixer_names(l, p + "mix.", b + ".mixer", source=i == first_mix)
            if i == first_mix:
                ignorable.append(p + "mix.vmix")          # (the first value-mixing layer has nothing to mix with)
            if l.mlp is not None:
                names += self._mlp_names(l.mlp, p + "mlp.", b + ".ffn")
        order = tuple(LayerCall(block=i, cache=i) for i in range(len(self.layers)))
        return ModelSpec(
            architecture=self.architecture,
            embedding=EmbeddingSpec(vocab_size=self.vocab, hidden_size=W, pair_buckets=self.bigram_buckets,
                                    pair_mul_prev=self.bigram_mul_prev, pair_mul_cur=self.bigram_mul_cur),
            blocks=tuple(blocks), order=order,
            head=HeadSpec(vocab_size=self.vocab, hidden_size=W, tied=False, norm=norm),
            tensor_names=tuple(names), ignorable=tuple(ignorable))
