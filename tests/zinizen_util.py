"""Small Zinizen models for the tests: configurations that differ in every size, random weights made
here (not by the engine), and helpers that step the engine and compare with tests/plain_zinizen.py.

The sizes are chosen so that nothing passes by two sizes being equal or a count being one: key and
value sizes differ, kv heads are one, several or as many as the heads, the latent's rotated part is
rotated wholly or in part, convolutions have one to five taps, the recurrence has one to five blocks,
experts are chosen one, two or three at a time with and without a shared expert, layers come with
and without feed-forward, cap, temperature and shared values, and one model has no table of token
pairs.
"""
import json
import math
import os

import torch

import plain_zinizen


def att(heads, kv, dim, vdim, scale=None, cap=None, temp=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale or 1.0 / math.sqrt(dim)}
    if cap:
        m["softcap"] = cap
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    if v_mix:
        m["v_mix"] = True
    return m


def lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, rot=None, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
            "rot": {"dims": rot[0], "base": rot[1]} if rot else {"dims": rot_dim, "base": 10000.0},
            "scale": scale or 1.0 / math.sqrt(dim + rot_dim)}


def rec(width, blocks, conv):
    return {"width": width, "blocks": blocks, "conv": conv}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, scale=1.0, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def model(width, vocab, layers, eps=1e-5, bigram=None):
    cfg = {"architecture": "Zinizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if bigram:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return cfg


CONFIGS = {
    # nothing a multiple of eight; values shared by three attention layers with a latent layer between
    "mix_a": model(72, 211, [
        layer("attention", att(6, 3, 20, 12, cap=9.0, temp=(0.4, 7), v_mix=True), moe(5, 2, 24, 1.2, 1.7, shared=(40, 0.8))),
        layer("rglru", rec(60, 3, 3), dense(50)),
        layer("latent_attention", lat(3, 20, 12, 28, 36, 44, rot=(8, 300.0)), None),
        layer("attention", att(9, 3, 10, 12, scale=0.4, v_mix=True), moe(7, 3, 16, 2.0, 0.8)),
        layer("attention", att(3, 1, 24, 36, cap=30.0, v_mix=True), dense(30)),
    ], eps=2e-5, bigram=(97, 13, 5)),
    # sizes that fill whole tiles (the tensor-core paths in bfloat16)
    "mix_b": model(128, 160, [
        layer("rglru", rec(256, 2, 3), moe(8, 2, 64, 1.25, 2.0, shared=(96, 0.9))),
        layer("attention", att(4, 2, 64, 64, cap=40.0, temp=(0.2, 32), v_mix=True), dense(256)),
        layer("latent_attention", lat(2, 64, 32, 64, 96, 128), moe(8, 2, 64, 1.25, 2.0, shared=(96, 0.9))),
        layer("attention", att(8, 2, 128, 64, v_mix=True), moe(16, 4, 32, 3.0, 2.0)),
        layer("rglru", rec(128, 1, 2), None),
    ], eps=1e-6, bigram=(1009, 29, 11)),
    # counts that are one, sizes that are equal, no table of token pairs
    "mix_c": model(48, 53, [
        layer("latent_attention", lat(1, 16, 16, 16, 16, 16, rot=(16, 50.0)), moe(3, 1, 48, 0.7)),
        layer("rglru", rec(48, 1, 1), None),
        layer("attention", att(2, 2, 16, 16, temp=(1.0, 1)), moe(2, 2, 8, 5.0, 1.0, shared=(8, 5.0))),
        layer("rglru", rec(40, 5, 5), dense(48)),
    ]),
}


def single(kind, mlp="dense", **kw):
    """A one-layer model of one mixer kind."""
    if kind == "attention":
        mixer = att(kw.get("heads", 6), kw.get("kv", 2), kw.get("dim", 24), kw.get("vdim", 40), kw.get("scale"),
                    kw.get("cap", 20.0), kw.get("temp", (0.3, 16)))
    elif kind == "latent_attention":
        mixer = lat(kw.get("heads", 3), kw.get("dim", 24), kw.get("rot_dim", 8), kw.get("vdim", 20), kw.get("q_rank", 30),
                    kw.get("kv_rank", 36), kw.get("rot"))
    else:
        mixer = rec(kw.get("width", 64), kw.get("blocks", 4), kw.get("conv", 4))
    ff = {"dense": dense(44), "moe": moe(kw.get("experts", 6), kw.get("top", 2), 20, kw.get("limit", 1.0), kw.get("rscale", 1.3),
                                           shared=kw.get("shared", (28, 0.9))), None: None}[mlp]
    return model(56, 97, [layer(kind, mixer, ff)], bigram=kw.get("bigram", (89, 11, 3)))


def typed(cfg):
    from llm_singularity_b200.config.zinizen import ZinizenConfig
    return ZinizenConfig.from_dict(cfg)


def make_weights(cfg, seed, sharpen=3.0):
    """Random bfloat16-representable weights, name -> float32 tensor.  The weights of the query norms are
    scaled up so that the softmax is peaked and one wrong or missing key shows; routers are scaled up
    and their corrections are as large as the scores, so that the correction changes choices; the
    recurrence's gate maps and decay parameters move its decay over its whole range; the experts' maps
    are large enough that their caps are met."""
    from llm_singularity_b200.engine.runner import expected_tensors_of
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, role, init) in expected_tensors_of(typed(cfg).to_model_spec()).items():
        if name.endswith((".q.norm", ".dq.norm")):
            t = sharpen * (1.0 + 0.2 * torch.randn(shape, generator=g))
        elif init == "ones":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(".vmix"):
            t = 0.35 + 0.2 * torch.rand(shape, generator=g)
        elif name.endswith(".correction"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name.endswith(".conv"):
            t = 0.6 * torch.randn(shape, generator=g)
        elif name.endswith(".lam"):
            t = -2.0 + 1.5 * torch.randn(shape, generator=g)
        elif name.endswith((".ra", ".ri")):
            t = 2.5 * torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        elif len(shape) <= 1 or name.endswith((".ra.b", ".ri.b")):
            t = 0.5 * torch.randn(shape, generator=g)
        elif name in ("embed", "bigram"):
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if name.endswith(".router"):
                t = t * 3.0
            if ".mlp.e" in name or ".mlp.shared" in name:
                t = t * 1.5
        out[name] = t.to(torch.bfloat16).float()
    # In a model of several layers the routed feed-forwards speak softly (the norm behind them has a small
    # weight): bfloat16 rounding turns a router's close call the other way now and then, which changes that
    # position and, through the recurrent states of later layers, those after it; with a small weight what
    # such a flip changes stays within rounding.  One-layer models keep the full weight, and in 32-bit
    # nothing flips.
    if len(cfg["layers"]) > 1:
        for i, l in enumerate(cfg["layers"]):
            if l["mlp"] is not None and l["mlp"]["kind"] == "moe":
                for name in (f"l{i}.norm2b", f"l{i}.norm2b.b"):
                    out[name] = (0.2 * out[name]).to(torch.bfloat16).float()
    return out


def write_model(path, cfg, weights, dtype=torch.bfloat16):
    from llm_singularity_b200.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    write_safetensors(os.path.join(path, "model.safetensors"), {n: t.to(dtype) for n, t in weights.items()})
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    return path


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def plain_logits(cfg, weights, tokens):
    return plain_zinizen.forward(cfg, weights, tokens).float()


def make_runner(path, dtype, pages=64, slots=4, page_size=16, max_len=None, **kw):
    from llm_singularity_b200.engine.runner import ModelRunner
    return ModelRunner(path, dtype=dtype, device="cuda:0", page_size=page_size, num_pages=pages,
                       max_requests=slots, max_model_len=max_len or pages * page_size, **kw)


def run_cuts(runner, rid, tokens, cuts):
    """One request alone, its tokens in portions of the given sizes, every place wanted."""
    from llm_singularity_b200.engine.batch import StepEntry
    assert sum(cuts) == len(tokens)
    assert runner.open(rid)
    at, rows = 0, []
    for c in cuts:
        rows.append(runner.step([StepEntry(rid, tokens[at:at + c], list(range(c)))]).float().cpu().clone())
        at += c
    runner.close(rid)
    runner.check_kernels()
    return torch.cat(rows)


def position_errors(got, want):
    """Per position: rms over the vocabulary of the difference (means taken off), over the rms of
    the wanted logits."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()


def rel_err(got, want):
    return position_errors(got, want).max().item()


TOLERANCE = {"float32": 2e-4, "bfloat16": 0.08}


def close(got, want, dtype):
    """32-bit: every position within the tolerance.  bfloat16: under a peaked softmax or a router's near
    tie rounding can move a position by more than rounding alone (another key takes most of a query's
    weight, another expert is chosen); so at most one position in twenty may be outside, and the median
    must lie far inside.  A fault of the cache, the state or the batch shows in 32-bit, where no such
    allowance is made."""
    e = position_errors(got, want)
    if dtype == "float32":
        return bool(e.max() < TOLERANCE[dtype])
    return bool((e > TOLERANCE[dtype]).float().mean() <= 0.05 and e.median() < TOLERANCE[dtype] / 3)
