"""Small Fikizen models for the tests: configurations that differ in every size, random weights made
here (not by the engine), and helpers that step the engine and compare with tests/plain_fikizen.py.

The sizes are chosen so that nothing passes by two sizes being equal or a count being one: key and
value sizes differ, kv heads are one, several or as many as the heads, fewer dims rotate than a head
has in one layer and all of them in another, windows are shorter than a page in one model and span
several pages in another, convolutions have two to five taps, the decay projections' hidden sizes
differ, layers borrow weights from attention, parallel and delta layers, and one model has no soft
cap.
"""
import json
import math
import os

import torch

import plain_fikizen


def _att(heads, kv, dim, vdim, window, rot, scale=None):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale or 1.0 / math.sqrt(dim),
            "mask": {"size": window}, "rot": {"dims": rot[0], "base": rot[1]}}


def _pair(left, right_heads, right_dim, left_scale, right_scale):
    return {"left": left, "right": {"heads": right_heads, "dim": right_dim}, "left_scale": left_scale,
            "right_scale": right_scale}


def _delta(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _layer(kind, mixer, ff, of=None):
    e = {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    if of is not None:
        e["weights_of"] = of
    return e


_A0 = _pair(_att(4, 2, 32, 16, 24, (16, 5000.0)), 3, 16, 0.7, 0.4)
_B0 = _att(4, 1, 64, 64, 40, (64, 10000.0))
_B1 = _delta(2, 2, 64, 32, 4)
_C0 = _delta(3, 3, 10, 6, 5)

CONFIGS = {
    # a pair first, borrowed later; a delta layer without feed-forward; key and value sizes differ
    "mix_a": {
        "architecture": "Fikizen", "vocab": 211, "width": 72, "norm": {"eps": 2e-5}, "logit_softcap": 12.0,
        "layers": [
            _layer("parallel", _A0, 40),
            _layer("delta", _delta(4, 2, 16, 24, 3), None),
            _layer("attention", _att(6, 3, 16, 32, 20, (8, 300.0), scale=0.3), 56),
            _layer("parallel", _A0, 40, of=0),
        ]},
    # sizes that fill whole tiles (the tensor-core paths in bfloat16); attention and delta layers borrowed
    "mix_b": {
        "architecture": "Fikizen", "vocab": 160, "width": 128, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
        "layers": [
            _layer("attention", _B0, 128),
            _layer("delta", _B1, 64),
            _layer("parallel", _pair(_att(4, 2, 64, 32, 33, (32, 100000.0)), 2, 64, 0.5, 1.0), 64),
            _layer("attention", _B0, 128, of=0),
            _layer("delta", _delta(4, 1, 128, 64, 2), None),
            _layer("delta", _B1, 64, of=1),
        ]},
    # nothing a multiple of eight, windows shorter than a page, no soft cap
    "mix_c": {
        "architecture": "Fikizen", "vocab": 53, "width": 100, "norm": {"eps": 1e-5},
        "layers": [
            _layer("delta", _C0, 30),
            _layer("parallel", _pair(_att(3, 1, 10, 14, 5, (6, 700.0)), 5, 6, 1.0, 0.25), None),
            _layer("attention", _att(5, 5, 12, 6, 7, (12, 50.0)), 18),
            _layer("delta", _C0, 30, of=0),
        ]},
}
DECAY_RANKS = {"mix_a": 5, "mix_b": 32, "mix_c": 3}


def single(kind, mlp=True, **kw):
    """A one-layer model of one mixer kind."""
    if kind == "attention":
        mixer = _att(kw.get("heads", 6), kw.get("kv", 2), kw.get("dim", 24), kw.get("vdim", 40), kw.get("window", 50),
                     kw.get("rot", (12, 2000.0)))
    elif kind == "delta":
        mixer = _delta(kw.get("heads", 6), kw.get("kv", 3), kw.get("dim", 20), kw.get("vdim", 12), kw.get("conv", 4))
    else:
        mixer = _pair(_att(kw.get("heads", 4), kw.get("kv", 2), kw.get("dim", 24), kw.get("vdim", 40), kw.get("window", 50),
                           kw.get("rot", (12, 2000.0))), kw.get("rheads", 3), kw.get("rdim", 20),
                      kw.get("left_scale", 0.6), kw.get("right_scale", 0.9))
    cfg = {"architecture": "Fikizen", "vocab": 97, "width": 56, "norm": {"eps": 1e-5},
           "layers": [_layer(kind, mixer, 44 if mlp else None)]}
    if kw.get("cap"):
        cfg["logit_softcap"] = kw["cap"]
    return cfg


def typed(cfg, rank=7):
    """The engine's configuration of ``cfg`` with decay projections of ``rank`` hidden values."""
    from llm_singularity_b200.config.fikizen import FikizenConfig
    shapes = {f"l{i}.mix.right.w1": (rank, cfg["width"]) for i in range(len(cfg["layers"]))}
    return FikizenConfig.from_dict(cfg).with_checkpoint_shapes(shapes)


def make_weights(cfg, seed, sharpen=3.0, rank=7):
    """Random bfloat16-representable weights, name -> float32 tensor.  Query and key maps of the
    attention mixers are scaled up so that the softmax is peaked and one wrong or missing key shows
    (but not so far that the sink's share vanishes); the gate maps of the memories are scaled up so
    that decays, removal rates and write strengths move over their whole range."""
    from llm_singularity_b200.engine.runner import expected_tensors_of
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, role, init) in expected_tensors_of(typed(cfg, rank).to_model_spec()).items():
        if init == "ones":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(".conv"):
            t = 0.6 * torch.randn(shape, generator=g)
        elif name.endswith("A_log"):
            t = -1.0 + 0.7 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if name.endswith((".mix.q", ".mix.k", ".left.q", ".left.k")):
                t = t * sharpen
            if name.endswith((".right.a", ".right.w2", ".mix.a", ".mix.b", ".mix.g", ".right.w1")):
                t = t * 2.5
        out[name] = t.to(torch.bfloat16).float()
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
    return plain_fikizen.forward(cfg, weights, tokens).float()


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
    """32-bit: every position within the tolerance.  bfloat16: under a peaked softmax rounding can
    move most of a query's weight from one key to another of nearly the same score, which changes
    that position by more than rounding; so at most one position in twenty may be outside, and the
    median must lie far inside.  A fault of the cache, the state or the batch shows in 32-bit, where
    no such allowance is made."""
    e = position_errors(got, want)
    if dtype == "float32":
        return bool(e.max() < TOLERANCE[dtype])
    return bool((e > TOLERANCE[dtype]).float().mean() <= 0.05 and e.median() < TOLERANCE[dtype] / 3)
