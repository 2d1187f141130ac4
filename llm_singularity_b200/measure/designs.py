"""Prefill and decode throughput of a design (Ridotar, Fogezen, Fikizen, Zinizen) beside the Llama decoder at equal size.

Zinizen: layers cycling through the RG-LRU block, biased capped attention that shares values between
its layers, gated latent attention and the biased attention once more; the first layer's feed-forward
is dense, the others route every token to ``top`` of ``experts`` capped gated experts beside a shared
one.  It is also run beside Ridotar, the design closest to it (routed experts, latent attention, a
recurrence walked token by token).

Fikizen: layers cycling through windowed sink attention with a gate per head, the gated
delta-rule memory behind short convolutions (no feed-forward), the parallel pair (normed windowed
attention beside the delta-rule memory with gates per key channel) and the first layer's weights
once more; dense ungated feed-forwards of the Llama model's width.  It is also run beside Fogezen,
the design closest to it (mixers side by side, a matrix memory, attention with sizes of its own).

Fogezen: layers alternating between biased attention with a query temperature and the parallel
pair (chunked, gated attention with normed and rotated heads beside a matrix memory), the second
layer run twice in a row as a loop (as many layer runs as the Llama model has layers), dense
feed-forwards of the Llama model's width.

For each size a Ridotar model (layers cycling through its three mixers, the fourth reading the
third's latent cache; routed experts whose active width equals the dense model's feed-forward)
and a Llama model of the same width, depth, vocabulary and active feed-forward width are built
with random weights (N(0, 0.02), norms 1) and stepped through ``ModelRunner.step``: one prompt of
``prefill_tokens`` in one step (logits for its last token), and decode steps of ``batch`` requests
whose contexts end at ``context`` tokens.  Times are CUDA events on the launching stream after
warm-up steps, the median of ``reps`` runs; inputs are random token ids.
"""
from __future__ import annotations

import math
import statistics
from typing import Dict

import torch

SIZES = {
    # width, layers, heads of 128, experts, top, expert width
    "w1024": dict(width=1024, layers=4, experts=16, top=2, ff=1024, kv_rank=256, vocab=32000),
    "w2048": dict(width=2048, layers=8, experts=32, top=4, ff=1024, kv_rank=512, vocab=32000),
}


def ridotar_config(width, layers, experts, top, ff, kv_rank, vocab) -> dict:
    heads = width // 128
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    latent = {"heads": heads, "dim": 128, "vdim": 128, "rot_dim": 64, "q_rank": 3 * width // 4,
              "kv_rank": kv_rank, "rot": {"base": 10000.0, "dims": 64}, "scale": 1.0 / math.sqrt(192)}
    out = []
    for i in range(layers):
        kind = i % 4
        if kind == 0:
            out.append({"type": "lightning", "mlp": mlp,
                        "mixer": {"heads": heads, "dim": 128, "vdim": 128,
                                  "decay": [1.0 - 2.0 ** (-5 - 3 * h / heads) for h in range(heads)]}})
        elif kind == 1:
            out.append({"type": "hgrn2", "mlp": mlp, "mixer": {"heads": heads, "dim": 128, "vdim": 128}})
        elif kind == 2:
            out.append({"type": "latent_attention", "mlp": mlp, "mixer": dict(latent)})
        else:
            out.append({"type": "latent_attention", "mlp": mlp, "mixer": dict(latent, kv_from=i - 1)})
    return {"architecture": "Ridotar", "vocab": vocab, "width": width, "norm": {"eps": 1e-6, "groups": 4},
            "postln_alpha": 1.5, "token_side": {"dim": 32}, "layers": out}


def fogezen_config(width, layers, experts, top, ff, kv_rank, vocab) -> dict:
    heads = width // 128
    mlp = {"kind": "dense", "ff": top * ff}
    attention = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                 "q_temp": {"coef": 0.1, "every": 512}}
    pair = {"left": {"heads": max(1, heads // 2), "kv_heads": max(1, heads // 8), "dim": 128, "vdim": 64,
                     "scale": 128 ** -0.5, "mask": {"size": 1024}, "rot": {"base": 10000.0, "dims": 64}},
            "right": {"heads": max(1, heads // 2), "dim": 64, "vdim": 128, "gate_cap": 15.0}}
    stored = max(2, layers - 1)                   # one layer is run twice
    out = [{"type": "parallel" if i % 2 else "attention", "mlp": mlp,
            "mixer": dict(pair) if i % 2 else dict(attention)} for i in range(stored)]
    return {"architecture": "Fogezen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "embedding": {"scale": float(width) ** 0.5}, "residual_mult": 0.5, "layers": out,
            "loop": {"start": 1, "stop": 2, "times": 2 if layers > 2 else 1}}


def fikizen_config(width, layers, experts, top, ff, kv_rank, vocab) -> dict:
    heads = width // 128
    mlp = {"kind": "dense", "ff": top * ff}
    attention = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                 "mask": {"size": 1024}, "rot": {"base": 1000000.0, "dims": 64}}
    delta = {"heads": heads, "kv_heads": max(1, heads // 2), "dim": 128, "vdim": 128, "conv": 4}
    pair = {"left": {"heads": max(1, heads // 2), "kv_heads": max(1, heads // 8), "dim": 128, "vdim": 64,
                     "scale": 128 ** -0.5, "mask": {"size": 1024}, "rot": {"base": 10000.0, "dims": 64}},
            "right": {"heads": max(1, heads // 2), "dim": 64}, "left_scale": 0.6, "right_scale": 0.5}
    out = []
    for i in range(layers):
        kind = i % 4
        if kind == 0:
            out.append({"type": "attention", "mixer": dict(attention), "mlp": mlp})
        elif kind == 1:
            out.append({"type": "delta", "mixer": dict(delta), "mlp": None})
        elif kind == 2:
            out.append({"type": "parallel", "mixer": dict(pair), "mlp": mlp})
        else:
            out.append({"type": "attention", "mixer": dict(attention), "mlp": mlp, "weights_of": 0})
    return {"architecture": "Fikizen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
            "layers": out}


def zinizen_config(width, layers, experts, top, ff, kv_rank, vocab) -> dict:
    heads = width // 128
    moe = {"kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "router": {"experts": experts, "top": top, "scale": 2.0},
           "shared": {"ff": ff, "limit": 5.0}}
    attention = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                 "softcap": 30.0, "q_temp": {"coef": 0.1, "every": 512}, "v_mix": True}
    latent = {"heads": heads, "dim": 128, "vdim": 128, "rot_dim": 64, "q_rank": 3 * width // 4, "kv_rank": kv_rank,
              "rot": {"base": 10000.0, "dims": 64}, "scale": 1.0 / math.sqrt(192)}
    recurrent = {"width": width, "blocks": heads, "conv": 4}
    out = []
    for i in range(layers):
        kind = i % 4
        mlp = {"kind": "dense", "ff": top * ff} if i == 0 else moe
        if kind == 0:
            out.append({"type": "rglru", "mixer": dict(recurrent), "mlp": mlp})
        elif kind == 2:
            out.append({"type": "latent_attention", "mixer": dict(latent), "mlp": mlp})
        else:
            out.append({"type": "attention", "mixer": dict(attention), "mlp": mlp})
    return {"architecture": "Zinizen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 33, "mul_cur": 5}}, "layers": out}


DESIGNS = {"ridotar": ridotar_config, "fogezen": fogezen_config, "fikizen": fikizen_config, "zinizen": zinizen_config}
# the designs each is also measured beside (Llama always is)
CLOSEST = {"fikizen": ("fogezen",), "zinizen": ("ridotar",)}


def llama_config(width, layers, experts, top, ff, kv_rank, vocab) -> dict:
    heads = width // 128
    return dict(architectures=["LlamaForCausalLM"], num_hidden_layers=layers, hidden_size=width,
                num_attention_heads=heads, num_key_value_heads=max(1, heads // 4), head_dim=128,
                intermediate_size=top * ff, vocab_size=vocab, rope_theta=10000.0, rope_scaling=None,
                rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072)


def _runner(cfg_dict, pages, slots, max_len, seed=0):
    from ..engine.runner import ModelRunner, expected_tensors_of
    from ..registry import architecture_of
    from ..weights.random_init import random_tensors
    config = architecture_of(cfg_dict).config_cls.from_dict(cfg_dict)
    tensors = random_tensors(expected_tensors_of(config.to_model_spec()), seed, dtype=torch.bfloat16, device="cuda:0")
    return ModelRunner(None, config=config, tensors=tensors, dtype="bfloat16", page_size=16, num_pages=pages,
                       max_requests=slots, max_tokens_per_step=max(2048, slots), max_model_len=max_len)


def _measure(cfg_dict, vocab, prefill_tokens, batch, context, steps, warmup, reps) -> Dict[str, float]:
    from .. import kernels
    from ..engine.batch import StepEntry
    per_request = -(-(context + 8) // 16)
    runner = _runner(cfg_dict, batch * per_request + -(-prefill_tokens // 16) + 8, batch + 1, max(context + 8, prefill_tokens))
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, vocab, (prefill_tokens,), generator=g).tolist()
    times = []
    for i in range(3 + reps):
        runner.open("p")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0 = kernels.launch_count()
        e0.record()
        runner.step([StepEntry("p", toks, [prefill_tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        prefill_launches = kernels.launch_count() - n0
        runner.close("p")
        if i >= 3:
            times.append(e0.elapsed_time(e1))
    prefill_ms = statistics.median(times)
    ids = [f"d{i}" for i in range(batch)]
    start = context - (steps + warmup + 2)
    for rid in ids:
        assert runner.open(rid)
        seq = torch.randint(0, vocab, (start,), generator=g).tolist()
        for s in range(0, start, 2048):
            runner.step([StepEntry(rid, seq[s:s + 2048], [])])
    feed = torch.randint(0, vocab, (batch,), generator=g).tolist()

    def decode(n):
        for _ in range(n):
            runner.step([StepEntry(rid, [t], [0]) for rid, t in zip(ids, feed)])

    runner.cuda_graphs, keep = False, runner.cuda_graphs
    n0 = kernels.launch_count()
    decode(1)
    decode_launches = kernels.launch_count() - n0
    runner.cuda_graphs = keep
    decode(warmup)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    decode(steps)
    e1.record()
    torch.cuda.synchronize()
    decode_ms = e0.elapsed_time(e1) / steps
    runner.check_kernels()
    return {"prefill_ms": round(prefill_ms, 3), "prefill_tok_s": round(prefill_tokens / prefill_ms * 1e3, 1),
            "decode_ms": round(decode_ms, 4), "decode_tok_s": round(batch / decode_ms * 1e3, 1),
            "prefill_launches": prefill_launches, "decode_launches": decode_launches,
            "graph_replays": runner.graph_replays}


def compare(sizes=("w1024", "w2048"), prefill_tokens=2048, batch=8, context=2048, steps=32, warmup=8, reps=5,
            layers=None, design="ridotar") -> Dict[str, dict]:
    import gc
    out = {}
    for name in sizes:
        size = dict(SIZES[name])
        if layers:
            size["layers"] = layers
        row = {"size": size}
        others = [(d, DESIGNS[d]) for d in CLOSEST.get(design, ())]
        for which, make in [(design, DESIGNS[design])] + others + [("llama", llama_config)]:
            row[which] = _measure(make(**size), size["vocab"], prefill_tokens, batch, context, steps, warmup, reps)
            gc.collect()
            torch.cuda.empty_cache()
        row[design + "_over_llama"] = {"prefill": round(row[design]["prefill_tok_s"] / row["llama"]["prefill_tok_s"], 3),
                                       "decode": round(row[design]["decode_tok_s"] / row["llama"]["decode_tok_s"], 3)}
        for d, _ in others:
            row[design + "_over_" + d] = {"prefill": round(row[design]["prefill_tok_s"] / row[d]["prefill_tok_s"], 3),
                                          "decode": round(row[design]["decode_tok_s"] / row[d]["decode_tok_s"], 3)}
        out[name] = row
    return out
