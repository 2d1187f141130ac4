"""The Fikizen design's host side: configuration, run order, parameter names, cache needs, and the
plain model's own consistency (each mechanism restated a second way).  No GPU."""
import copy
import math

import pytest
import torch

import fikizen_util as U
import plain_fikizen as P

F64 = torch.float64


def _rand(*shape, seed=0, scale=1.0):
    return scale * torch.randn(*shape, dtype=F64, generator=torch.Generator().manual_seed(seed))


# ------------------------------------------------------------------------------ configuration
@pytest.mark.parametrize("name", sorted(U.CONFIGS))
def test_configuration_round_trip_and_registry(name, tmp_path):
    from llm_singularity_b200.registry import load_config
    cfg = U.CONFIGS[name]
    c = U.typed(cfg, U.DECAY_RANKS[name])
    assert c.to_dict() == cfg
    W = U.make_weights(cfg, 1, rank=U.DECAY_RANKS[name])
    U.write_model(str(tmp_path), cfg, W)
    assert load_config(str(tmp_path)).to_dict() == cfg


@pytest.mark.parametrize("name", sorted(U.CONFIGS))
def test_run_order_borrowed_weights_and_caches(name):
    """Every layer is one call with a cache of its own; a layer that borrows weights runs the block
    of the layer it names and has no tensors."""
    from llm_singularity_b200.engine.runner import expected_tensors_of
    cfg = U.CONFIGS[name]
    spec = U.typed(cfg, U.DECAY_RANKS[name]).to_model_spec()
    own = [i for i, l in enumerate(cfg["layers"]) if "weights_of" not in l]
    assert len(spec.blocks) == len(own)
    assert [c.cache for c in spec.order] == list(range(len(cfg["layers"])))
    assert [own[c.block] for c in spec.order] == [P.weight_layer(cfg, i) for i in range(len(cfg["layers"]))]
    names = expected_tensors_of(spec)
    for i, l in enumerate(cfg["layers"]):
        mine = [n for n in names if n.startswith(f"l{i}.")]
        assert bool(mine) == ("weights_of" not in l)
        if mine:
            assert (f"l{i}.norm2" in names) == (l["mlp"] is not None) == (f"l{i}.mlp.act" in names)


def test_parameters_and_cache_kinds():
    from llm_singularity_b200.engine.runner import expected_tensors_of
    from llm_singularity_b200.models.decoder import DecoderModel
    from llm_singularity_b200.parts import CompositeCacheSpec, PagedKVSpec, Runtime, StateSpec
    cfg = U.CONFIGS["mix_a"]
    spec = U.typed(cfg, 5).to_model_spec()
    names = expected_tensors_of(spec)
    assert names["l0.mix.left.q.norm"][0] == (128,) and names["l0.mix.left.k.norm"][0] == (64,)
    assert names["l0.mix.left.v.b"][0] == (32,) and names["l0.mix.right.w1"][0] == (5, 72)
    assert names["l0.mix.right.w2"][0] == (48, 5) and names["l0.mix.right.a.b"][0] == (48,)
    assert names["l1.mix.q.conv"][0] == (32, 3) and names["l1.mix.v.conv"][0] == (96, 3)
    assert names["l1.mix.norm"][0] == (24,) and names["l1.mix.b"][0] == (4, 72) and names["l1.mix.A_log"][0] == (4,)
    assert names["l2.mix.g"][0] == (6, 72) and names["l2.mix.o"][0] == (72, 192) and names["l2.mlp.act"][0] == (2,)
    model = DecoderModel(spec, Runtime("cpu", torch.float32, ops=object()))
    caches = model.cache_specs()
    assert len(caches) == 4
    pair = caches[0]
    assert isinstance(pair, CompositeCacheSpec) and pair.paged and not pair.shareable and pair.window == 24
    assert pair.parts[0] == PagedKVSpec(2, 32, 24, 16) and pair.parts[1] == StateSpec((3, 16, 16))
    assert caches[3] == pair
    delta = caches[1]
    assert isinstance(delta, CompositeCacheSpec) and not delta.paged
    assert delta.parts == (StateSpec((4, 24, 16)), StateSpec((2, 2 * 32 + 96)))
    assert caches[2] == PagedKVSpec(3, 16, 20, 32)


def test_decay_rank_comes_from_the_checkpoint():
    from llm_singularity_b200.config.fikizen import FikizenConfig
    cfg = U.CONFIGS["mix_a"]
    c = FikizenConfig.from_dict(cfg).with_checkpoint_shapes({"l0.mix.right.w1": (9, 72)})
    assert c.layers[0].channel.decay_rank == 9 and c.layers[3].channel.decay_rank == 9   # the borrower follows


def test_bad_configurations_are_refused():
    from llm_singularity_b200.config.fikizen import FikizenConfig
    from llm_singularity_b200.config.llama import ConfigError
    for change in (lambda c: c["layers"][0].update(type="other"),
                   lambda c: c["layers"][2]["mixer"].update(kv_heads=4),
                   lambda c: c["layers"][2]["mixer"]["rot"].update(dims=7),
                   lambda c: c["layers"][2]["mixer"]["rot"].update(dims=18),
                   lambda c: c["layers"][2]["mixer"].pop("mask"),
                   lambda c: c["layers"][0]["mlp"].update(kind="moe"),
                   lambda c: c["layers"][3].update(weights_of=3),
                   lambda c: c["layers"][3].update(weights_of=1),
                   lambda c: c["layers"][1]["mixer"].update(kv_heads=3),
                   lambda c: c["layers"][0]["mixer"].pop("left_scale"),
                   lambda c: c.update(logit_softcap=0.0),
                   lambda c: c["norm"].pop("eps")):
        cfg = copy.deepcopy(U.CONFIGS["mix_a"])
        change(cfg)
        with pytest.raises(ConfigError):
            FikizenConfig.from_dict(cfg)


# ---------------------------------------------------- the plain model, each mechanism a second way
def test_plain_window_and_sink():
    ok = P.in_window(torch.arange(9), 4)
    assert ok[6].tolist() == [False, False, False, True, True, True, True, False, False]
    assert ok[2].tolist() == [True, True, True] + [False] * 6
    # one head, one key: the weight of the only visible key is e^s / (1 + e^s)
    q, k, v = torch.tensor([[[2.0]]], dtype=F64), torch.tensor([[[1.5]]], dtype=F64), torch.tensor([[[7.0]]], dtype=F64)
    o = P.sink_softmax_heads(q, k, v, 0.5, torch.ones(1, 1, dtype=torch.bool))
    assert abs(o.item() - 7.0 * math.exp(1.5) / (1 + math.exp(1.5))) < 1e-12
    # very negative scores: everything goes to the sink, nothing overflows
    o = P.sink_softmax_heads(-q * 500, k, v, 1.0, torch.ones(1, 1, dtype=torch.bool))
    assert 0 <= o.item() < 1e-100 or o.item() == 0.0
    # grouped heads read the right key head
    q, k, v = _rand(5, 4, 3, seed=1), _rand(5, 2, 3, seed=2), _rand(5, 2, 2, seed=3)
    ok = P.in_window(torch.arange(5), 3)
    o = P.sink_softmax_heads(q, k, v, 0.7, ok)
    for h in range(4):
        for i in range(5):
            js = [j for j in range(5) if 0 <= i - j < 3]
            e = torch.stack([torch.exp(0.7 * (q[i, h] @ k[j, h // 2])) for j in js])
            want = sum(w * v[j, h // 2] for w, j in zip(e, js)) / (1 + e.sum())
            assert (o[i, h] - want).abs().max() < 1e-12


def test_plain_turn_is_a_rotation_of_paired_dims():
    v = _rand(4, 2, 10, seed=4)
    pos = torch.tensor([0, 3, 17, 400])
    out = P.turn_halves(v, pos, 6, 100.0)
    assert torch.equal(out[0], v[0]) and torch.equal(out[..., 6:], v[..., 6:])
    for i in range(3):
        a = pos.to(F64) * 100.0 ** (-2.0 * i / 6)
        z = torch.complex(v[..., i], v[..., i + 3]) * torch.polar(torch.ones(4, dtype=F64), a)[:, None]
        assert (out[..., i] - z.real).abs().max() < 1e-12 and (out[..., i + 3] - z.imag).abs().max() < 1e-12
    # scores depend on the distance only
    q, k = _rand(1, 1, 6, seed=5), _rand(1, 1, 6, seed=6)
    s = lambda pq, pk: (P.turn_halves(q, torch.tensor([pq]), 6, 50.0) * P.turn_halves(k, torch.tensor([pk]), 6, 50.0)).sum()
    assert abs(s(9, 4) - s(105, 100)) < 1e-12


def test_plain_short_convolution():
    z, taps = _rand(7, 3, seed=7), _rand(3, 4, seed=8)
    out = P.short_conv(z, taps)
    for t in range(7):
        for c in range(3):
            want = sum(taps[c, 3 - d] * z[t - d, c] for d in range(4) if t - d >= 0)
            assert abs(out[t, c] - want) < 1e-12


def test_plain_activation_branches():
    p, q = torch.tensor(0.3, dtype=F64), torch.tensor(-0.2, dtype=F64)
    z = torch.tensor([-3.0, -1e-9, 0.0, 1e-9, 2.0], dtype=F64)
    y = P.bent_square(z, p, q)
    sp = lambda x: math.log1p(math.exp(x))
    assert abs(y[4] - (sp(0.3) * 4 + 1)) < 1e-12
    assert abs(y[0] - ((0.5 + sp(-0.2)) * (math.exp(-3) - 1 + 3) - 1.5)) < 1e-12
    assert y[2] == 0 and abs(y[1]) < 1e-9 and abs(y[3]) < 1e-9          # continuous, slope 1/2 at zero


def test_plain_memories_carry_their_state():
    """Each delta-rule memory against a restatement with explicit matrices, and walked in two halves
    (with the convolution's last inputs carried) against one walk."""
    H, D, V, T = 2, 5, 3, 11
    k, v, q = _rand(T, H, D, seed=9), _rand(T, H, V, seed=10), _rand(T, H, D, seed=11)
    k = P.unit_length(k)
    fade, beta = torch.rand(T, H, dtype=F64), torch.rand(T, H, dtype=F64)
    # gated: S_t = g S (I - beta k k^T applied on the key side) + beta k v^T
    for h in range(H):
        S = torch.zeros(D, V, dtype=F64)
        for t in range(T):
            S = fade[t, h] * S
            S = (torch.eye(D, dtype=F64) - beta[t, h] * torch.outer(k[t, h], k[t, h])) @ S + beta[t, h] * torch.outer(k[t, h], v[t, h])
        S2 = torch.zeros(D, V, dtype=F64)
        for t in range(T):
            S2 = fade[t, h] * S2
            u = beta[t, h] * (v[t, h] - S2.T @ k[t, h])
            S2 = S2 + torch.outer(k[t, h], u)
        assert (S - S2).abs().max() < 1e-12
    # whole models of one memory layer: a prefix's logits do not depend on what follows (nothing looks ahead)
    for kind in ("delta", "parallel"):
        cfg = U.single(kind)
        W = U.make_weights(cfg, 5)
        toks = U.tokens_for(cfg, 40, 2)
        whole = P.forward(cfg, W, toks)
        assert (P.forward(cfg, W, toks[:23]) - whole[:23]).abs().max() < 1e-10


def test_plain_channel_memory_reads_the_old_state_in_both_terms():
    """One head, two key channels, by hand."""
    cfg = U.single("parallel", rheads=1, rdim=2)
    m = cfg["layers"][0]["mixer"]["right"]
    width = cfg["width"]
    W = {n: t.double() for n, t in U.make_weights(cfg, 6).items()}
    h = _rand(3, width, seed=12)
    p = "l0.mix.right."
    out = P.channel_delta_memory(h, W, p, m, 1e-5)
    r, k, v = h @ W[p + "r"].T, h @ W[p + "k"].T, h @ W[p + "v"].T
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"]))
    a = torch.sigmoid(h @ W[p + "a"].T + W[p + "a.b"])
    S = torch.zeros(2, 2, dtype=F64)
    rows = []
    for t in range(3):
        u = k[t] / torch.sqrt((k[t] ** 2).sum() + 1e-6)
        S = torch.diag(w[t]) @ S - torch.outer(a[t] * u, u @ S) + torch.outer(k[t], v[t])
        o = S.T @ r[t]
        o = o / torch.sqrt((o ** 2).mean() + 1e-5) * W[p + "norm"] * torch.sigmoid(h[t] @ W[p + "g"].T)
        rows.append(o @ W[p + "o"].T)
    assert (torch.stack(rows) - out).abs().max() < 1e-12
