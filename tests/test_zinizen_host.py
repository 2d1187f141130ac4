"""The Zinizen design on the host: its configuration (reading, refusals, writing back), the model
spec it becomes (parts, tensor names, what every layer and the embedding keep per request), and
properties of the plain model that the GPU tests rely on."""
import copy

import pytest
import torch

import plain_zinizen as P
import zinizen_util as U
from llm_singularity_b200.config.llama import ConfigError
from llm_singularity_b200.config.zinizen import ZinizenConfig
from llm_singularity_b200.engine.runner import expected_tensors_of
from llm_singularity_b200.models.decoder import DecoderModel
from llm_singularity_b200.parts import CompositeCacheSpec, LatentPagesSpec, PagedKVSpec, Runtime, StateSpec
from llm_singularity_b200.registry import architecture_of

F64 = torch.float64


@pytest.mark.parametrize("name", sorted(U.CONFIGS))
def test_configuration_reads_and_writes_back(name):
    cfg = U.CONFIGS[name]
    assert architecture_of(cfg).config_cls is ZinizenConfig
    typed = ZinizenConfig.from_dict(cfg)
    assert typed.to_dict() == cfg
    assert ZinizenConfig.from_dict(typed.to_dict()) == typed


def test_refusals_name_the_layer():
    base = U.CONFIGS["mix_a"]
    def broken(change):
        cfg = copy.deepcopy(base)
        change(cfg)
        return cfg
    cases = [(lambda c: c["layers"][0].update(type="conv"), "layer 0"),
             (lambda c: c["layers"][3]["mixer"].update(kv_heads=3, heads=5), "layer 3"),
             (lambda c: c["layers"][1]["mixer"].update(blocks=7), "layer 1"),
             (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=14), "layer 2"),
             (lambda c: c["layers"][4]["mixer"].update(vdim=35), "layer 4"),          # shared values of another size
             (lambda c: c["layers"][3]["mlp"]["router"].update(top=9), "layer 3"),
             (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "layer 0"),
             (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "layer 0"),
             (lambda c: c["norm"].pop("eps"), "norm"),
             (lambda c: c.pop("width"), "width")]
    for change, where in cases:
        with pytest.raises(ConfigError) as e:
            ZinizenConfig.from_dict(broken(change))
        assert where in str(e.value)


def test_spec_parts_names_and_caches():
    cfg = U.CONFIGS["mix_a"]
    spec = ZinizenConfig.from_dict(cfg).to_model_spec()
    kinds = [b.mixer.kind for b in spec.blocks]
    assert kinds == ["kv_attention", "rglru", "latent_attention", "kv_attention", "kv_attention"]
    assert [b.kind for b in spec.blocks] == ["sandwich_norm"] * 5
    assert [b.mixer.value_mix for b in spec.blocks if b.mixer.kind == "kv_attention"] == ["source", "mixed", "mixed"]
    assert spec.blocks[2].ffn is None and spec.blocks[1].ffn.kind == "dense_mlp"
    moe = spec.blocks[0].ffn
    assert (moe.kind, moe.score, moe.renormalize, moe.weight_on, moe.choice_bias) == ("moe", "softmax", True, "output", True)
    assert moe.shared.intermediate_size == 40 and moe.shared.limit == 0.8 and spec.blocks[3].ffn.shared is None
    assert spec.embedding.pair_buckets == 97 and not spec.head.tied
    names = expected_tensors_of(spec)
    assert names["bigram"][0] == (98, 72) and names["head"][0] == (211, 72)
    assert names["l0.mix.q.norm"][0] == (120,) and names["l0.mix.k.norm"][0] == (60,)
    assert "l0.mix.vmix" not in names and "l0.mix.vmix" in spec.ignorable and names["l3.mix.vmix"][0] == ()
    assert names["l1.mix.ra"][0] == (3, 20, 20) and names["l1.mix.conv"][0] == (60, 3)
    assert names["l2.mix.dkv"][0] == (56, 72) and names["l2.mix.g"][0] == (3, 72) and names["l2.mix.uq"][0] == (96, 36)
    assert names["l0.mlp.correction"][0] == (5,) and names["l0.mlp.shared.down"][0] == (72, 40)
    assert "l2.norm2" not in names and "l2.norm2" in spec.ignorable and names["l2.norm1b.b"][0] == (72,)
    model = DecoderModel(spec, Runtime("cpu", torch.float32, ops=object()))
    caches = model.cache_specs()
    assert len(caches) == 6                                       # five layers and the embedding's last token
    assert caches[0] == PagedKVSpec(3, 20, None, 12) and caches[2] == LatentPagesSpec(56)
    assert isinstance(caches[1], CompositeCacheSpec) and [p.shape for p in caches[1].parts] == [(60,), (2, 60)]
    assert caches[5] == StateSpec((), dtype=torch.int32)
    # a model without the table of token pairs keeps nothing for the embedding
    plain = DecoderModel(ZinizenConfig.from_dict(U.CONFIGS["mix_c"]).to_model_spec(), Runtime("cpu", torch.float32, ops=object()))
    assert len(plain.cache_specs()) == 4


def test_plain_token_pairs():
    assert P.bigram_rows([5, 9, 9, 0], 17, 13, 5) == [17, (5 * 13 + 9 * 5) % 17, (9 * 13 + 9 * 5) % 17, (9 * 13) % 17]


def test_plain_router_correction_changes_the_choice_not_the_weights():
    W = {"r.router": torch.tensor([[1.0], [0.9], [0.0]], dtype=F64), "r.correction": torch.tensor([0.0, 0.5, 0.0], dtype=F64)}
    idx, w = P.route(torch.ones(1, 1, dtype=F64), W, "r.", {"top": 1, "scale": 2.0})
    assert idx.tolist() == [[1]] and abs(w.item() - 2.0) < 1e-12            # one chosen: its renormalised weight is the scale
    idx, w = P.route(torch.ones(1, 1, dtype=F64), W, "r.", {"top": 2, "scale": 1.0})
    s = torch.softmax(torch.tensor([1.0, 0.9, 0.0], dtype=F64), 0)
    assert idx.tolist() == [[1, 0]] and torch.allclose(w[0], torch.stack([s[1], s[0]]) / (s[0] + s[1]))


def test_plain_expert_saturates_at_its_limit():
    W = {"e.gate": torch.tensor([[1.0]], dtype=F64), "e.up": torch.tensor([[1.0]], dtype=F64), "e.down": torch.tensor([[1.0]], dtype=F64)}
    big, small = P.capped_expert(torch.tensor([[50.0]], dtype=F64), W, "e.", 2.0), P.capped_expert(torch.tensor([[-50.0]], dtype=F64), W, "e.", 2.0)
    assert abs(big.item() - 2.0 * torch.sigmoid(torch.tensor(3.404, dtype=F64)).item() * 3.0) < 1e-12
    assert abs(small.item()) < 1e-12                                           # the gate is not capped from below: it vanishes


def test_plain_recurrence_first_token_and_convolution_zeros():
    g = torch.Generator().manual_seed(0)
    N, B, K = 6, 2, 3
    W = {"m.y": torch.randn(N, 4, generator=g), "m.y.b": torch.randn(N, generator=g), "m.x": torch.randn(N, 4, generator=g),
         "m.x.b": torch.randn(N, generator=g), "m.conv": torch.randn(N, K, generator=g), "m.conv.b": torch.randn(N, generator=g),
         "m.ra": torch.randn(B, 3, 3, generator=g), "m.ra.b": torch.randn(B, 3, generator=g), "m.ri": torch.randn(B, 3, 3, generator=g),
         "m.ri.b": torch.randn(B, 3, generator=g), "m.lam": torch.randn(N, generator=g), "m.o": torch.eye(N)}
    W = {n: t.double() for n, t in W.items()}
    h = torch.randn(5, 4, generator=g).double()
    out = P.gated_linear_unit(h, W, "m.", {"width": N, "blocks": B})
    # the first token alone gives the same first row (nothing before it enters), and a later token's row changes
    # when an earlier input does
    assert torch.allclose(out[:1], P.gated_linear_unit(h[:1], W, "m.", {"width": N, "blocks": B}))
    h2 = h.clone(); h2[0] += 1.0
    assert not torch.allclose(out[4], P.gated_linear_unit(h2, W, "m.", {"width": N, "blocks": B})[4])
    x0 = h[0] @ W["m.x"].T + W["m.x.b"]
    u0 = W["m.conv.b"] + W["m.conv"][:, K - 1] * x0                        # zeros before the start
    assert torch.allclose(P.short_conv(h @ W["m.x"].T + W["m.x.b"], W["m.conv"], W["m.conv.b"])[0], u0)


def test_plain_attention_shared_values_and_slopes():
    cfg = U.single("attention", mlp=None, heads=4, kv=2, dim=8, vdim=6)
    W = {n: t.double() for n, t in U.make_weights(cfg, 1).items()}
    m, pos = cfg["layers"][0]["mixer"], torch.arange(9)
    h = torch.randn(9, 56, generator=torch.Generator().manual_seed(2)).double()
    out, v = P.biased_attention(h, W, "l0.mix.", m, pos, 1e-5, None)
    assert v.shape == (9, 12) and torch.allclose(v, h @ W["l0.mix.v"].T)
    # mixing with other values changes the output; lambda 0 does not
    W["l0.mix.vmix"] = torch.tensor(0.0, dtype=F64)
    same, _ = P.biased_attention(h, W, "l0.mix.", dict(m, v_mix=True), pos, 1e-5, torch.ones(9, 12, dtype=F64))
    assert torch.allclose(same, out)
    W["l0.mix.vmix"] = torch.tensor(0.5, dtype=F64)
    mixed, v2 = P.biased_attention(h, W, "l0.mix.", dict(m, v_mix=True), pos, 1e-5, torch.ones(9, 12, dtype=F64))
    assert not torch.allclose(mixed, out) and torch.allclose(v2, 0.5 * v + 0.5)
