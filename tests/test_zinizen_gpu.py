"""The Zinizen design in the engine against tests/plain_zinizen.py (float64, whole sequences, one
function per mechanism, no cache).  Every test makes its own small model (tests/zinizen_util.py).

Covered: each mixer and each feed-forward alone; whole prompts against token-by-token stepping;
portions of changing size down to two tokens; batches of unequal requests against each alone; pages
and state slots given back and used again (the recurrence's state, the convolution's last inputs and
the embedding's last token are state of a slot); keys far back, at page borders and among the first
tokens with one score made to stand out, under the cap and the distance's slope of every head; long
portions on the tensor-memory attention kernel and in the segmented walk of the recurrence, beside
single tokens; long decoding; other sizes, also counts of one and sizes that are equal; the single
kernels against the plain functions; greedy generation through the engine's entry point and the
trace runner.
"""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_zinizen as P
import zinizen_util as U

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
F64 = torch.float64
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _setup(tmp_path, cfg, seed, **kw):
    W = U.make_weights(cfg, seed, **kw)
    return W, U.write_model(str(tmp_path / f"m{seed}"), cfg, W)


# ----------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", DTYPES)
def test_each_mechanism_alone(tmp_path, dtype):
    cases = [("attention", "dense", {}), ("latent_attention", "dense", {}), ("rglru", "dense", {}),
             ("attention", None, dict(heads=4, kv=4, dim=32, vdim=32, cap=None, temp=None, bigram=None)),
             ("attention", "moe", dict(heads=3, kv=1, dim=64, vdim=16, cap=3.0, temp=(2.0, 5))),
             ("latent_attention", "moe", dict(heads=2, dim=32, rot_dim=16, vdim=8, q_rank=12, kv_rank=20, rot=(4, 77.0),
                                              experts=9, top=3, shared=None)),
             ("latent_attention", None, dict(heads=5, dim=8, rot_dim=6, vdim=12, q_rank=40, kv_rank=10)),
             ("rglru", "moe", dict(width=96, blocks=1, conv=1, experts=4, top=1, limit=0.3)),
             ("rglru", None, dict(width=70, blocks=7, conv=6))]
    for n, (kind, mlp, kw) in enumerate(cases):
        cfg = U.single(kind, mlp, **kw)
        W, path = _setup(tmp_path, cfg, 100 + n)
        toks = U.tokens_for(cfg, 77, n)
        want = U.plain_logits(cfg, W, toks)
        r = U.make_runner(path, dtype, pages=8)
        whole = U.run_cuts(r, "w", toks, [77])
        assert U.close(whole, want, dtype), (kind, mlp, kw, U.rel_err(whole, want))
        stepped = U.run_cuts(r, "s", toks, [1] * 77)             # the same slot and pages once more
        assert U.close(stepped, want, dtype), (kind, mlp, kw, "token by token", U.rel_err(stepped, want))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix_a", "mix_b", "mix_c"])
def test_portions_of_any_size(tmp_path, dtype, name, n=150):
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 7)
    toks = U.tokens_for(cfg, n, 3)
    want = U.plain_logits(cfg, W, toks)
    r = U.make_runner(path, dtype, pages=12)
    ragged, pattern = [], [2, 15, 1, 16, 17, 31, 2, 2, 33, 5]
    while sum(ragged) < n:
        ragged.append(min(pattern[len(ragged) % len(pattern)], n - sum(ragged)))
    for cuts in ([n], [n - 40] + [1] * 40, ragged, [16] * (n // 16) + [n % 16], [2] * (n // 2), [3] * (n // 3)):
        cuts = [c for c in cuts if c]
        got = U.run_cuts(r, "p", toks, cuts)
        assert U.close(got, want, dtype), (cuts[:6], U.rel_err(got, want))
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix_a", "mix_c"])
def test_long_portions_walked_in_segments(tmp_path, dtype, name, monkeypatch, n=150):
    """The recurrence's long portions cut into segments of 16 and of 5 tokens that are walked side by
    side: a whole prompt, a long portion after a short one, and two long portions of unequal length in
    one batch, against the plain model."""
    from llm_singularity_b200 import kernels as K
    from llm_singularity_b200.engine.batch import StepEntry
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 11)
    toks, other = U.tokens_for(cfg, n, 4), U.tokens_for(cfg, 97, 5)
    want, want_other = U.plain_logits(cfg, W, toks), U.plain_logits(cfg, W, other)
    monkeypatch.setattr(K, "RGLRU_SEGMENT_FROM", 20)
    for seg in (16, 5):
        monkeypatch.setattr(K, "RGLRU_SEGMENT", seg)
        r = U.make_runner(path, dtype, pages=24)
        for cuts in ([n], [3, n - 4, 1], [70, 80], [n]):
            got = U.run_cuts(r, "p", toks, cuts)
            assert U.close(got, want, dtype), (seg, cuts, U.rel_err(got, want))
        assert r.open("x") and r.open("y")
        a = r.step([StepEntry("x", toks[:90], list(range(90))), StepEntry("y", other[:96], list(range(96)))]).float().cpu()
        b = r.step([StepEntry("y", other[96:], [0]), StepEntry("x", toks[90:], list(range(n - 90)))]).float().cpu()
        r.close("x"); r.close("y")
        r.check_kernels()
        assert U.close(torch.cat([a[:90], b[1:]]), want, dtype), seg
        assert U.close(torch.cat([a[90:], b[:1]]), want_other, dtype), seg
        r.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_portions_beside_single_tokens(tmp_path, dtype, name="mix_b"):
    """Portions of 140 to 300 tokens in one step with another request's single token, the single token
    before the portion and after it (attention layers with equal key and value sizes send such portions
    to another kernel than single tokens and short portions; the recurrence walks them in segments),
    against the plain model of each request alone."""
    from llm_singularity_b200.engine.batch import StepEntry
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 13)
    x, y = U.tokens_for(cfg, 450, 6), U.tokens_for(cfg, 170, 7)
    want_x, want_y = U.plain_logits(cfg, W, x), U.plain_logits(cfg, W, y)
    r = U.make_runner(path, dtype, pages=48)
    assert r.open("x") and r.open("y")
    every = lambda n: list(range(n))
    a = r.step([StepEntry("y", y[:139], every(139))]).float().cpu()
    b = r.step([StepEntry("y", y[139:140], [0]), StepEntry("x", x[:300], every(300))]).float().cpu()
    c = r.step([StepEntry("x", x[300:440], every(140)), StepEntry("y", y[140:141], [0])]).float().cpu()
    d = r.step([StepEntry("y", y[141:], every(29)), StepEntry("x", x[440:], every(10))]).float().cpu()
    r.close("x"); r.close("y")
    r.check_kernels()
    got_x = torch.cat([b[1:], c[:140], d[29:]])
    got_y = torch.cat([a, b[:1], c[140:], d[:29]])
    assert U.close(got_x, want_x, dtype), U.rel_err(got_x, want_x)
    assert U.close(got_y, want_y, dtype), U.rel_err(got_y, want_y)
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix_a", "mix_b", "mix_c"])
def test_mixed_batches_with_slots_and_pages_used_again(tmp_path, dtype, name):
    """Four requests of unequal length stepped together (portions beside single tokens, a request
    left out of some steps, ends at different times, a fifth request taking over a freed slot and
    freed pages: its recurrent state, its convolution's inputs and its last token start afresh)
    against the plain model of each alone."""
    from llm_singularity_b200.engine.batch import StepEntry
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 9)
    lens = {"a": 70, "b": 23, "c": 41, "d": 1, "e": 37}
    toks = {k: U.tokens_for(cfg, n, 20 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: U.plain_logits(cfg, W, t) for k, t in toks.items()}
    r = U.make_runner(path, dtype, pages=12, slots=4)      # 192 token places for 172 tokens
    plan = [[("a", 33), ("b", 2)], [("a", 1), ("b", 17), ("c", 5)], [("d", 1), ("c", 1), ("a", 1)],
            [("b", 1), ("c", 30), ("a", 20)], [("b", 1), ("a", 1), ("c", 1)], [("b", 1), ("c", 2)],
            [("b", 1), ("e", 3), ("a", 14), ("c", 2)], [("e", 33), ("b", 0)], [("e", 1)]]
    at = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    for step in plan:
        entries, who = [], []
        for k, n in step:
            n = min(n, lens[k] - at[k])
            if n <= 0:
                continue
            if not r.cache.has(k):
                assert r.open(k), f"no slot for {k}"
            entries.append(StepEntry(k, toks[k][at[k]:at[k] + n], list(range(n))))
            who.append((k, n))
        logits = r.step(entries).float().cpu()
        row = 0
        for k, n in who:
            got[k].append(logits[row:row + n].clone())
            row += n
            at[k] += n
            if at[k] == lens[k]:
                r.close(k)
    r.check_kernels()
    assert at == lens
    for k in lens:
        assert U.close(torch.cat(got[k]), want[k], dtype), (k, U.rel_err(torch.cat(got[k]), want[k]))
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_keys_page_borders_and_first_tokens(tmp_path, dtype):
    """A strongly peaked softmax against pages of 16: a key that is lost, one page or one place off, or
    a first token left out changes the logits by far more than the tolerance.  The attention's heads
    differ in how fast they forget (the distance's slope), so some look far back and some do not."""
    for kind, kw, seed in (("attention", dict(cap=60.0, temp=(0.25, 48)), 31), ("latent_attention", {}, 32),
                           ("attention", dict(heads=8, kv=8, dim=16, vdim=16, cap=None), 33)):
        cfg = U.single(kind, mlp=None, **kw)
        W, path = _setup(tmp_path, cfg, seed, sharpen=8.0)
        n = 300
        toks = U.tokens_for(cfg, n, 5)
        want = U.plain_logits(cfg, W, toks)
        r = U.make_runner(path, dtype, pages=20)
        for cuts in ([n], [255, 1, 1, 15, 17, 11], [n - 64] + [1] * 64, [49, 2, 48, 1, 1, 49, 50, 100], [129, 2, 130, 39]):
            got = U.run_cuts(r, "f", toks, cuts)
            assert U.close(got, want, dtype), (kind, cuts[:4], U.rel_err(got, want))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tmp_path, dtype, name="mix_b"):
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 13)
    n = 200
    toks = U.tokens_for(cfg, n, 8)
    want = U.plain_logits(cfg, W, toks)
    r = U.make_runner(path, dtype, pages=14)
    got = U.run_cuts(r, "l", toks, [3] + [1] * (n - 3))
    assert U.close(got, want, dtype), U.rel_err(got, want)
    assert r.graph_replays > 150                              # single tokens replay a captured step


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_engine(tmp_path, dtype, name="mix_a"):
    """Greedy generation through Engine (scheduler, portions of 16, three requests at once) gives
    the tokens the plain model picks, wherever its choice is not a near tie."""
    from llm_singularity_b200 import Engine
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 17)
    eng = Engine(path, dtype=dtype, kv_block_size=16, num_kv_blocks=24, max_batch_size=3,
                 max_tokens_per_batch=48, prefill_chunk=16)
    prompts = [U.tokens_for(cfg, n, 40 + n) for n in (5, 37, 18)]
    new = 12
    ids = [eng.add_request(p, max_new_tokens=new) for p in prompts]
    out = {i: [] for i in ids}
    while eng.has_work():
        for rid, tok, _ in eng.step():
            assert tok >= 0
            out[rid].append(tok)
    for rid, p in zip(ids, prompts):
        seq = list(p)
        for tok in out[rid]:
            logits = U.plain_logits(cfg, W, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if (top2[0] - top2[1]) > (0.05 if dtype == "float32" else 0.5):
                assert tok == int(logits.argmax()), (rid, len(seq))
            seq.append(tok)
        assert len(out[rid]) == new


def test_trace_replay_of_a_small_model(tmp_path):
    """bin/trace_run on a model made here: two requests in portions and single tokens through two
    slots' worth of pages, a third request on what they gave back; 32-bit."""
    cfg = U.CONFIGS["mix_c"]
    W, path = _setup(tmp_path, cfg, 21)
    a, b, c = (U.tokens_for(cfg, n, 60 + n) for n in (40, 9, 33))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[7:], "want": [0, 1]}, {"id": "a", "tokens": a[31:], "want": [8]}], "end": ["a", "b"]},
             {"step": 3, "entries": [{"id": "c", "tokens": c[:2], "want": []}], "end": []},
             {"step": 4, "entries": [{"id": "c", "tokens": c[2:], "want": [30]}], "end": ["c"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in (0, 1, 2, 3, 4)]
    assert not (out / "3.f32").exists()
    want = {k: U.plain_logits(cfg, W, t) for k, t in (("a", a), ("b", b), ("c", c))}
    read = lambda i: torch.frombuffer(bytearray((out / f"{i}.f32").read_bytes()), dtype=torch.float32).view(-1, cfg["vocab"])
    got = {"a": torch.cat([read(0), read(1)[:1], read(2)[2:]]), "b": torch.cat([read(1)[1:], read(2)[:2]]), "c": read(4)}
    rows = {"a": [0, 29, 30, 39], "b": [6, 7, 8], "c": [32]}
    for k in got:
        assert U.close(got[k], want[k][rows[k]], "float32"), (k, U.rel_err(got[k], want[k][rows[k]]))


# ----------------------------------------------------------------- kernels against plain functions
def _ctx(q_lens, kv_lens, rows=None, tokens=None):
    from llm_singularity_b200.engine.batch import ContextBuilder
    b = ContextBuilder("cuda", 4096, 64)
    ctx, _ = b.build(tokens or [[0] * n for n in q_lens], [kv - q for kv, q in zip(kv_lens, q_lens)],
                     rows or list(range(len(q_lens))), [[] for _ in q_lens])
    ctx._keep = b
    return ctx


def _pages(slots, max_kv, nkv, dk, dv, page, dtype, seed=0):
    from llm_singularity_b200.parts import KVCacheView
    per = -(-max_kv // page)
    n = slots * per + 3
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(seed))[:slots * per].view(slots, per)
    return KVCacheView(torch.zeros(n, nkv, page, dk, dtype=dtype, device="cuda"),
                       torch.zeros(n, nkv, page, dv, dtype=dtype, device="cuda"),
                       perm.to(torch.int32).cuda(), page, None, 0)


def _fill(cache, row, K, V):
    pos = torch.arange(K.shape[0])
    pages = cache.block_table[row].cpu()[pos // cache.page_size].long()
    cache.k_pages[pages, :, pos % cache.page_size, :] = K.to(cache.k_pages.dtype).cuda()
    cache.v_pages[pages, :, pos % cache.page_size, :] = V.to(cache.v_pages.dtype).cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, dk, dv, cap, page", [(4, 2, 32, 16, 7.0, 16), (6, 2, 96, 48, 0.0, 16), (3, 3, 10, 14, 2.5, 8),
                                                        (4, 1, 64, 64, 11.0, 16), (2, 2, 128, 128, 30.0, 32), (8, 2, 64, 64, 0.0, 16)])
@pytest.mark.parametrize("single_first", [False, True])
def test_capped_biased_attention_kernel_one_score_standing_out(dtype, nh, nkv, dk, dv, cap, page, single_first):
    """Three requests in one launch (a prompt portion, a single token, a long whole prompt).  All keys
    are alike but one per request, which every query scores high, up to the cap: the heads with a small
    slope then take its value from far back, the heads with a large slope prefer near keys.  The
    standing-out key is put far back, on a page border, first in the sequence and last."""
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(dk + dv)
    q_lens, kv_lens = ([1, 37, 170], [131, 90, 170]) if single_first else ([37, 1, 170], [90, 131, 170])
    slot_rows = [0, 2, 1] if single_first else [2, 0, 1]
    ctx = _ctx(q_lens, kv_lens, rows=slot_rows)
    scale = 1.0 / math.sqrt(dk)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / nh) for h in range(nh)], dtype=F64)
    for targets in ([3, 0, 15], [16, 64, 48], [0, 79, 0], [89, 89, 169]):
        cache = _pages(3, 176, nkv, dk, dv, page, dtype, seed=1)
        qs, outs = [], []
        for r, (ql, kv, tgt) in enumerate(zip(q_lens, kv_lens, targets)):
            Kd = 0.1 * torch.randn(kv, nkv, dk, generator=g)
            Kd[tgt, :, 0] = 6.0
            Vd = torch.randn(kv, nkv, dv, generator=g)
            q = 0.1 * torch.randn(ql, nh, dk, generator=g)
            q[:, :, 0] = 1.5 / scale
            Kd, Vd, q = (t.to(dtype).double() for t in (Kd, Vd, q))
            _fill(cache, slot_rows[r], Kd, Vd)
            pos_q, pos_k = torch.arange(kv - ql, kv), torch.arange(kv)
            seen = pos_k[None, :] <= pos_q[:, None]
            o = torch.zeros(ql, nh, dv, dtype=F64)
            for h in range(nh):
                s = (q[:, h] @ Kd[:, h // (nh // nkv)].T) * scale
                if cap:
                    s = cap * torch.tanh(s / cap)
                s = s - slopes[h] * (pos_q[:, None] - pos_k[None, :]).to(F64)
                o[:, h] = torch.softmax(s.masked_fill(~seen, float("-inf")), dim=-1) @ Vd[:, h // (nh // nkv)]
            outs.append(o)
            qs.append(q)
        T = sum(q_lens)
        q = torch.cat(qs).reshape(T, nh * dk).to(dtype).cuda()
        out = torch.zeros(T, nh * dv, dtype=dtype, device="cuda")
        K.attention_dv(q, nh, nkv, dk, dv, ctx, cache, scale, 0, 0, None, out, softcap=cap, linear_bias=True)
        want = torch.cat(outs).reshape(T, nh * dv)
        assert (out.double().cpu() - want).abs().max() <= tol * 4, (targets, (out.double().cpu() - want).abs().max())
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [52, 128, 1030])
def test_centred_norm_kernel(dtype, hidden):
    """The norm behind a sublayer, the sum and the norm in front of the next one as one kernel, rows with a
    large common offset (which a norm that does not take the mean off first would lose digits on)."""
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(hidden)
    T = 19
    x = (torch.randn(T, hidden, generator=g) + 30.0).cuda()
    y = (3.0 * torch.randn(T, hidden, generator=g) - 7.0).to(dtype).cuda()
    w1, b1, w2, b2 = (torch.randn(hidden, generator=g).cuda() for _ in range(4))
    eps = 1e-5
    xd, yd = x.double().cpu(), y.double().cpu()
    stream = xd + 0.5 * P.centred_norm(yd, w1.double().cpu(), b1.double().cpu(), eps)
    want = P.centred_norm(stream, w2.double().cpu(), b2.double().cpu(), eps)
    tol = 1e-4 if dtype == torch.float32 else 8e-2
    rows = torch.tensor([4, 0, 18, 4], dtype=torch.int32).cuda()
    picked = torch.empty(4, hidden, dtype=dtype, device="cuda")
    K.stream_centred_norm(x, y, w1, b1, eps, 0.5, rows, w2, b2, eps, picked)           # the stream stays as it is
    assert torch.equal(x.cpu(), xd.float())
    assert (picked.double().cpu() - want[rows.cpu().long()]).abs().max() < tol
    out = torch.empty(T, hidden, dtype=dtype, device="cuda")
    K.stream_centred_norm(x, y, w1, b1, eps, 0.5, None, w2, b2, eps, out)
    assert (x.double().cpu() - stream).abs().max() < 1e-4
    assert (out.double().cpu() - want).abs().max() < tol
    K.stream_centred_norm(x, y, None, None, 0.0, 2.0, None, None, None, 0.0, None)     # a plain sum
    assert (x.double().cpu() - (stream + 2.0 * yd)).abs().max() < 1e-4
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_pair_embedding_keeps_the_last_token_of_a_slot(dtype):
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(3)
    vocab, hidden, buckets, mp, mc = 50, 24, 17, 13, 5
    table = torch.randn(vocab, hidden, generator=g).to(dtype).cuda()
    pairs = torch.randn(buckets + 1, hidden, generator=g).to(dtype).cuda()
    last = torch.full((4,), 49, dtype=torch.int32, device="cuda")            # (what other requests left there)
    seqs = {0: torch.randint(0, vocab, (11,), generator=g).tolist(), 3: torch.randint(0, vocab, (7,), generator=g).tolist()}
    want = {s: P.embed({"embedding": {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}},
                       {"embed": table.double().cpu(), "bigram": pairs.double().cpu()}, t) for s, t in seqs.items()}
    got = {0: [], 3: []}
    for (a0, a1), (b0, b1) in (((0, 4), (0, 1)), ((4, 5), (1, 6)), ((5, 11), (6, 7))):
        parts = [(3, a0, min(a1, 7)), (0, b0, b1)]
        parts = [(s, lo, hi) for s, lo, hi in parts if hi > lo]
        ctx = _ctx([hi - lo for _, lo, hi in parts], [hi for _, lo, hi in parts], rows=[s for s, _, _ in parts],
                   tokens=[seqs[s][lo:hi] for s, lo, hi in parts])
        out = torch.empty(ctx.n_tokens, hidden, dtype=torch.float32, device="cuda")
        K.embedding_pair(table, pairs, ctx, last, buckets, mp, mc, out)
        at = 0
        for s, lo, hi in parts:
            got[s].append(out[at:at + hi - lo].double().cpu())
            at += hi - lo
    assert (torch.cat(got[0]) - want[0][:7]).abs().max() < 1e-6
    assert (torch.cat(got[3]) - want[3]).abs().max() < 1e-6
    assert last.cpu().tolist() == [seqs[0][6], 49, 49, seqs[3][6]]
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width, blocks, taps", [(64, 4, 4), (40, 5, 2), (96, 1, 1), (132, 3, 6)])
def test_recurrence_kernels_carry_state_and_inputs(dtype, width, blocks, taps, monkeypatch):
    """Convolution, gates and walk of two requests in portions of unequal length (one shorter than the
    convolution's taps, one walked in segments) against the plain recurrence on the whole sequences."""
    from llm_singularity_b200 import kernels as K
    monkeypatch.setattr(K, "RGLRU_SEGMENT", 8)
    monkeypatch.setattr(K, "RGLRU_SEGMENT_FROM", 24)
    g = torch.Generator().manual_seed(width + taps)
    bw, lens = width // blocks, {1: 61, 2: 9}
    W = {"y": torch.zeros(width, 1), "x": torch.zeros(width, 1), "o": torch.eye(width),
         "y.b": 0.3 * torch.randn(width, generator=g), "x.b": 0.3 * torch.randn(width, generator=g),
         "conv": 0.6 * torch.randn(width, taps, generator=g), "conv.b": 0.2 * torch.randn(width, generator=g),
         "ra": 2.0 * torch.randn(blocks, bw, bw, generator=g) / math.sqrt(bw), "ra.b": torch.randn(blocks, bw, generator=g),
         "ri": 2.0 * torch.randn(blocks, bw, bw, generator=g) / math.sqrt(bw), "ri.b": torch.randn(blocks, bw, generator=g),
         "lam": -2.0 + 1.5 * torch.randn(width, generator=g)}
    W = {n: t.to(torch.bfloat16).double() for n, t in W.items()}
    proj = {s: torch.randn(n, 2 * width, generator=g).float() for s, n in lens.items()}     # [y | x] before the biases
    want = {}
    for s, n in lens.items():
        # the plain block with the two projections taken out: h is one constant column, the maps add the rows
        y = P.gelu_tanh(proj[s][:, :width].double() + W["y.b"])
        u = P.short_conv(proj[s][:, width:].double() + W["x.b"], W["conv"], W["conv.b"])
        ub = u.view(n, blocks, bw)
        r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, W["ra"]) + W["ra.b"]).reshape(n, width)
        i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, W["ri"]) + W["ri.b"]).reshape(n, width)
        a = torch.exp(-8.0 * r * P.softplus(W["lam"]))
        S, rows = torch.zeros(width, dtype=F64), []
        for t in range(n):
            S = a[t] * S + torch.sqrt(1.0 - a[t] * a[t]) * i[t] * u[t]
            rows.append(S * y[t])
        want[s] = torch.stack(rows)
    state = torch.zeros(4, width, device="cuda")
    conv_state = torch.zeros(4, max(taps - 1, 1), width, device="cuda")
    state[0] = 5.0                                                             # (another request's)
    w_gates = torch.cat([W["ra"], W["ri"]], dim=1).to(dtype).cuda().contiguous()
    f = lambda n: W[n].float().reshape(-1).cuda().contiguous()
    got = {1: [], 2: []}
    for cuts in (((1, 0, 2), (2, 0, 1)), ((2, 1, 3), (1, 2, 40)), ((1, 40, 41), (2, 3, 9)), ((1, 41, 61),)):
        ctx = _ctx([hi - lo for _, lo, hi in cuts], [hi for _, _, hi in cuts], rows=[s for s, _, _ in cuts])
        pj = torch.cat([proj[s][lo:hi] for s, lo, hi in cuts]).cuda().contiguous()
        T = pj.shape[0]
        u = torch.empty(T, width, device="cuda")
        gates = torch.empty(T, 2 * width, device="cuda")
        if dtype == torch.bfloat16:          # u as two bfloat16 numbers against the maps repeated along k
            halves = torch.empty(T, 2 * width, dtype=dtype, device="cuda")
            K.rglru_conv(pj, width, f("x.b"), W["conv"].float().cuda().contiguous(), f("conv.b"), conv_state, ctx, u,
                         split=halves, blocks=blocks)
            K.batched_nt(halves.view(T, blocks, 2 * bw), torch.cat([w_gates, w_gates], dim=2).contiguous(),
                         gates.view(T, blocks, 2 * bw))
            exact = torch.empty_like(gates)
            K.batched_nt(u.view(T, blocks, bw), w_gates, exact.view(T, blocks, 2 * bw), exact=True)
            assert (gates - exact).abs().max() < 2e-4 * max(1.0, exact.abs().max().item())
        else:
            K.rglru_conv(pj, width, f("x.b"), W["conv"].float().cuda().contiguous(), f("conv.b"), conv_state, ctx, u)
            K.batched_nt(u.view(T, blocks, bw), w_gates, gates.view(T, blocks, 2 * bw), exact=True)
        K.rglru_gates(gates, f("ra.b"), f("ri.b"), f("lam"), 8.0, u, pj, 0, f("y.b"), blocks)
        out = torch.empty(T, width, dtype=dtype, device="cuda")
        K.rglru_walk(gates, pj, width, 0, f("x.b"), taps, state, conv_state, ctx, out, blocks)
        at = 0
        for s, lo, hi in cuts:
            got[s].append(out[at:at + hi - lo].double().cpu())
            at += hi - lo
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for s in lens:
        assert (torch.cat(got[s]) - want[s]).abs().max() < tol * max(1.0, want[s].abs().max().item()), s
    assert torch.equal(state[0].cpu(), torch.full((width,), 5.0))
    K.check_status()


@pytest.mark.parametrize("E, top", [(5, 2), (12, 3), (3, 1), (40, 4)])
def test_router_chooses_with_the_correction_and_weighs_without(E, top):
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(E)
    T = 64
    z = 2.0 * torch.randn(T, E, generator=g)
    corr = 0.3 * torch.randn(E, generator=g)
    s = torch.softmax(z.double(), dim=-1)
    idx = torch.topk(s + corr.double(), top, dim=-1).indices
    assert not torch.equal(idx.sort(-1).values, torch.topk(s, top, dim=-1).indices.sort(-1).values)   # the correction matters
    w = torch.gather(s, 1, idx)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * 1.7
    ids = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(T, top, dtype=torch.float32, device="cuda")
    K.moe_route(z.cuda(), top, "softmax", True, ids, wts, choice_bias=corr.cuda(), weight_scale=1.7, renorm_eps=1e-20)
    assert torch.equal(ids.cpu().long(), idx)
    assert (wts.double().cpu() - w).abs().max() < 1e-6
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [5, 300])
def test_capped_gated_product(dtype, T):
    """Gate and up values well beyond the limit on both sides, through the product's own epilogue (many rows,
    bfloat16) and through the activation kernel."""
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(T)
    H, F, limit = 64, 48, 0.75
    x = torch.randn(T, H, generator=g).to(dtype)
    wg, wu = (1.5 * torch.randn(F, H, generator=g) / 8.0).to(dtype), (1.5 * torch.randn(F, H, generator=g) / 8.0).to(dtype)
    gate, up = x.double() @ wg.double().T, x.double() @ wu.double().T
    assert (gate > limit).any() and (up > limit).any() and (up < -limit).any()
    gc = torch.clamp(gate, max=limit)
    want = gc * torch.sigmoid(1.702 * gc) * (torch.clamp(up, -limit, limit) + 1.0)
    w = torch.stack([wg, wu], dim=1).reshape(2 * F, H).contiguous().cuda()
    got = K.linear(x.cuda(), w, gated=True, activation="capped_glu", limit=limit)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert (got.double().cpu() - want).abs().max() < tol
    K.check_status()


# ------------------------------------------------------------------------ as a user runs it
@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_as_a_user_runs_it(tmp_path, dtype):
    """bin/trace_run as a process of its own, fed step by step: seven requests through four slots
    and a pool smaller than their sum (mixed portions and single tokens), then each request in
    portions of changing size; every position against the plain model."""
    import cuttings
    import numpy as np
    import replay_util
    cfg = U.CONFIGS["mix_a"]
    W, path = _setup(tmp_path, cfg, 23)
    seqs = {f"q{i}": U.tokens_for(cfg, n, 60 + i) for i, n in enumerate((5, 70, 33, 1, 100, 64, 21))}
    want = {rid: U.plain_logits(cfg, W, t) for rid, t in seqs.items()}
    for k, (steps, max_tokens) in enumerate((cuttings.mixed(seqs, seed=3), cuttings.portions(seqs))):
        out = str(tmp_path / f"out{k}")
        replay_util.replay_subprocess(path, dtype, steps, out, max_tokens)
        rows = replay_util.collect(steps, out, cfg["vocab"])
        assert len(rows) == sum(len(t) for t in seqs.values())
        for rid, t in seqs.items():
            got = torch.from_numpy(np.stack([rows[(rid, p)] for p in range(len(t))]))
            assert U.close(got, want[rid], dtype), (k, rid, U.rel_err(got, want[rid]))


def test_command_line_serves_the_design(tmp_path):
    """bin/llm-serve-llama picks the design by config.json and generates greedily what the plain
    model picks (where its choice is clear)."""
    cfg = U.CONFIGS["mix_b"]
    W, path = _setup(tmp_path, cfg, 29)
    prompts = [U.tokens_for(cfg, n, 70 + n) for n in (4, 19)]
    (tmp_path / "p.json").write_text(json.dumps(prompts))
    cmd = [sys.executable, os.path.join(ROOT, "bin", "llm-serve-llama"), "--model-dir", path, "--dtype", "fp32",
           "--prompt-ids", str(tmp_path / "p.json"), "--max-new-tokens", "6", "--ignore-eos",
           "--num-kv-blocks", "16", "--max-batch-size", "2"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    outs = [json.loads(line)["tokens"] for line in res.stdout.splitlines()]
    assert len(outs) == 2 and all(len(o) == 6 for o in outs)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            logits = U.plain_logits(cfg, W, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if top2[0] - top2[1] > 0.05:
                assert tok == int(logits.argmax())
            seq.append(tok)
