"""The Fikizen design in the engine against tests/plain_fikizen.py (float64, whole sequences, one
function per mechanism, no cache).  Every test makes its own small model (tests/fikizen_util.py).

Covered: each mixer alone, with and without feed-forward; whole prompts against token-by-token
stepping; portions of changing size down to two tokens; batches of unequal requests against each
alone; pages and state slots given back and used again, also pages that a window has passed; keys
far back, at page borders, among the first tokens and just inside and just outside a window, in
prompts and in decoding, with one score made to stand out; the sink alone; the memories' walk with
state carried over many steps and a write far back read much later; the convolution's carried
inputs over portions shorter than its taps; long decoding; other sizes; greedy generation through
the engine's entry point, the trace runner and the command line.
"""
import math

import pytest
import torch

import fikizen_util as U
import plain_fikizen as P

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
F64 = torch.float64


def _setup(tmp_path, cfg, seed, **kw):
    W = U.make_weights(cfg, seed, **kw)
    return W, U.write_model(str(tmp_path / f"m{seed}"), cfg, W)


# ----------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", DTYPES)
def test_each_mixer_alone(tmp_path, dtype):
    cases = [("attention", True, {}), ("delta", True, {}), ("parallel", True, {}),
             ("attention", False, dict(heads=4, kv=4, dim=32, vdim=32, window=9, rot=(32, 77.0))),
             ("attention", True, dict(heads=3, kv=1, dim=64, vdim=16, window=200, rot=(2, 10.0), cap=5.0)),
             ("delta", False, dict(heads=2, kv=2, dim=64, vdim=64, conv=1)),
             ("delta", True, dict(heads=8, kv=1, dim=8, vdim=40, conv=2, cap=20.0)),
             ("parallel", False, dict(heads=2, kv=1, dim=64, vdim=32, window=17, rot=(64, 100.0), rheads=1, rdim=64,
                                      left_scale=1.0, right_scale=2.0)),
             ("parallel", True, dict(heads=5, kv=5, dim=12, vdim=20, window=70, rot=(4, 1e6), rheads=7, rdim=10))]
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
    W, path = _setup(tmp_path, cfg, 7, rank=U.DECAY_RANKS[name])
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
    """The memories' long portions cut into segments of 16 and of 5 tokens (half as many for portions of
    up to eight segments) that are walked side by side:
    a whole prompt, a long portion after a short one, and two long portions of unequal length in one
    batch, against the plain model."""
    from llm_singularity_b200 import kernels as K
    from llm_singularity_b200.engine.batch import StepEntry
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 11, rank=U.DECAY_RANKS[name])
    toks, other = U.tokens_for(cfg, n, 4), U.tokens_for(cfg, 97, 5)
    want, want_other = U.plain_logits(cfg, W, toks), U.plain_logits(cfg, W, other)
    for seg in (16, 5):
        monkeypatch.setattr(K, "DELTA_SEGMENT", seg)
        r = U.make_runner(path, dtype, pages=24)                  # (a runner keeps the graphs of the shapes it has met)
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
    """Portions of 140 to 150 tokens in one step with another request's single token, the single token
    before the portion and after it (the attention layers with equal key and value sizes send such
    portions to another kernel than single tokens and short portions), against the plain model of
    each request alone."""
    from llm_singularity_b200.engine.batch import StepEntry
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 13, rank=U.DECAY_RANKS[name])
    x, y = U.tokens_for(cfg, 300, 6), U.tokens_for(cfg, 170, 7)
    want_x, want_y = U.plain_logits(cfg, W, x), U.plain_logits(cfg, W, y)
    r = U.make_runner(path, dtype, pages=40)
    assert r.open("x") and r.open("y")
    every = lambda n: list(range(n))
    a = r.step([StepEntry("y", y[:139], every(139))]).float().cpu()
    b = r.step([StepEntry("y", y[139:140], [0]), StepEntry("x", x[:150], every(150))]).float().cpu()
    c = r.step([StepEntry("x", x[150:290], every(140)), StepEntry("y", y[140:141], [0])]).float().cpu()
    d = r.step([StepEntry("y", y[141:], every(29)), StepEntry("x", x[290:], every(10))]).float().cpu()
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
    freed pages) against the plain model of each alone."""
    from llm_singularity_b200.engine.batch import StepEntry
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 9, rank=U.DECAY_RANKS[name])
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
def test_far_keys_page_borders_window_edges_and_first_tokens(tmp_path, dtype):
    """A strongly peaked softmax, windows of 50 and 130 against pages of 16: a key that is lost, one
    page or one place off, a first token left out or a window edge one token off changes the logits
    by far more than the tolerance."""
    for kind, kw, seed in (("attention", dict(window=50), 31), ("parallel", dict(window=130), 32),
                           ("attention", dict(window=1000), 33)):
        cfg = U.single(kind, mlp=False, **kw)
        W, path = _setup(tmp_path, cfg, seed, sharpen=8.0)
        n = 300
        toks = U.tokens_for(cfg, n, 5)
        want = U.plain_logits(cfg, W, toks)
        r = U.make_runner(path, dtype, pages=20)
        for cuts in ([n], [255, 1, 1, 15, 17, 11], [n - 64] + [1] * 64, [49, 2, 48, 1, 1, 49, 50, 100], [129, 2, 130, 39]):
            got = U.run_cuts(r, "f", toks, cuts)
            assert U.close(got, want, dtype), (kind, cuts[:4], U.rel_err(got, want))


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_a_window_has_passed_are_used_again(tmp_path, dtype):
    """300 tokens through a pool of 7 pages of 16 places: the window of 40 gives its pages back as it
    moves on, and the logits do not change."""
    cfg = U.single("attention", window=40)
    W, path = _setup(tmp_path, cfg, 35, sharpen=6.0)
    n = 300
    toks = U.tokens_for(cfg, n, 4)
    want = U.plain_logits(cfg, W, toks)
    r = U.make_runner(path, dtype, pages=7, max_len=512)
    for cuts in ([30] * 10, [40, 3, 1, 1, 19] + [1] * 236, [7, 33] * 7 + [20]):
        got = U.run_cuts(r, "w", toks, cuts)
        assert U.close(got, want, dtype), (cuts[:5], U.rel_err(got, want))
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tmp_path, dtype, name="mix_b"):
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 13, rank=U.DECAY_RANKS[name])
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
    W, path = _setup(tmp_path, cfg, 17, rank=U.DECAY_RANKS[name])
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


# ----------------------------------------------------------------- kernels against plain functions
def _ctx(q_lens, kv_lens, rows=None):
    from llm_singularity_b200.engine.batch import ContextBuilder
    b = ContextBuilder("cuda", 4096, 64)
    ctx, _ = b.build([[0] * n for n in q_lens], [kv - q for kv, q in zip(kv_lens, q_lens)],
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
@pytest.mark.parametrize("nh, nkv, dk, dv, window, page", [(4, 2, 32, 16, 24, 16), (6, 2, 96, 48, 40, 16), (3, 3, 10, 14, 5, 8),
                                                           (4, 1, 64, 128, 1000, 16), (2, 2, 128, 64, 33, 16),
                                                           (8, 2, 48, 80, 64, 32), (5, 5, 112, 16, 1, 8)])
def test_sink_attention_kernel_one_score_standing_out(dtype, nh, nkv, dk, dv, window, page):
    """Three requests in one launch (a prompt portion, a single token, a longer portion that is a
    whole prompt).  All keys are alike but one per request, which every query scores high: where it
    is visible the output is nearly its value, where it is not the output is the visible values'
    mean shrunk by the sink's share.  The standing-out key is put far back, on a page border, first
    in the sequence, just inside and just outside the last query's window, and last.  With and
    without the sink, and with a gate of one number per head."""
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(dk + dv)
    q_lens, kv_lens = [37, 1, 70], [90, 131, 70]
    ctx = _ctx(q_lens, kv_lens, rows=[2, 0, 1])
    scale = 1.0 / math.sqrt(dk)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    lows = [max(0, kv - window) for kv in kv_lens]                 # the last query's first visible key
    for targets in ([3, 0, 15], [max(lo - 1, 0) for lo in lows], lows, [16, 127, 48], [89, 130, 69]):
        cache = _pages(3, 144, nkv, dk, dv, page, dtype, seed=1)
        qs, outs = [], {True: [], False: []}
        for r, (ql, kv, tgt) in enumerate(zip(q_lens, kv_lens, targets)):
            Kd = 0.1 * torch.randn(kv, nkv, dk, generator=g)
            Kd[tgt, :, 0] = 6.0
            Vd = torch.randn(kv, nkv, dv, generator=g)
            q = 0.1 * torch.randn(ql, nh, dk, generator=g)
            q[:, :, 0] = 4.0 / scale
            Kd, Vd, q = (t.to(dtype).double() for t in (Kd, Vd, q))
            _fill(cache, [2, 0, 1][r], Kd, Vd)
            ok = P.in_window(torch.arange(kv), window)[kv - ql:]
            for sink in (True, False):
                o = torch.zeros(ql, nh, dv, dtype=F64)
                for h in range(nh):
                    s = ((q[:, h] @ Kd[:, h // (nh // nkv)].T) * scale).masked_fill(~ok, float("-inf"))
                    e = torch.exp(s)
                    o[:, h] = (e / (e.sum(-1, keepdim=True) + (1.0 if sink else 0.0))) @ Vd[:, h // (nh // nkv)]
                outs[sink].append(o)
            qs.append(q)
        T = sum(q_lens)
        q = torch.cat(qs).reshape(T, nh * dk).to(dtype).cuda()
        gate = torch.randn(T, nh + 6, generator=g).to(dtype).cuda()
        out = torch.empty(T, nh * dv, dtype=dtype, device="cuda")
        for sink in (True, False):
            want = torch.cat(outs[sink])
            out.zero_()
            K.attention_dv(q, nh, nkv, dk, dv, ctx, cache, scale, window, 0, None, out, sink=sink)
            assert (out.double().cpu() - want.reshape(T, nh * dv)).abs().max() <= tol * 4, (targets, sink)
        K.attention_dv(q, nh, nkv, dk, dv, ctx, cache, scale, window, 0, gate[:, 6:], out, sink=True, gate_per_head=True)
        gated = (torch.cat(outs[True]) * torch.sigmoid(gate[:, 6:].double().cpu())[:, :, None]).reshape(T, nh * dv)
        assert (out.double().cpu() - gated).abs().max() <= tol * 4, targets
    K.check_status()


@pytest.mark.parametrize("nh, nkv, hd, window, page", [(4, 2, 128, 40, 16), (6, 1, 64, 1000, 16), (2, 2, 128, 129, 32),
                                                       (8, 4, 64, 1, 8)])
@pytest.mark.parametrize("singles", [0, 2])
def test_sink_attention_of_steps_with_long_portions(nh, nkv, hd, window, page, singles, monkeypatch):
    """Equal key and value sizes, bfloat16: the route through the tensor-memory prompt kernel (sink and
    gate per head in its last step; single tokens that come first in the step go through the
    warp-level kernel in the same call) and the route through the warp-level kernel alone both match
    plain arithmetic.  Three portions of 131 to 200 rows, two of them continuing a longer sequence,
    with or without two single tokens before them; one key per request stands out, just inside or
    just outside the last query's window."""
    from llm_singularity_b200 import kernels as K
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(hd + window)
    q_lens, kv_lens, rows = [150, 200, 131], [150, 260, 400], [1, 2, 0]
    if singles:
        q_lens, kv_lens, rows = [1, 1] + q_lens, [77, 300] + kv_lens, [4, 3] + rows
    ctx = _ctx(q_lens, kv_lens, rows=rows)
    scale = 1.0 / math.sqrt(hd)
    lows = [max(0, kv - window) for kv in kv_lens]
    for targets in (lows, [max(lo - 1, 0) for lo in lows], [min(t, kv - 1) for t, kv in zip([40, 127, 16, 127, 300][-len(q_lens):], kv_lens)]):
        cache = _pages(5, 400, nkv, hd, hd, page, dtype, seed=2)
        qs, outs = [], {True: [], False: []}
        for r, (ql, kv, tgt) in enumerate(zip(q_lens, kv_lens, targets)):
            Kd = 0.1 * torch.randn(kv, nkv, hd, generator=g)
            Kd[tgt, :, 0] = 6.0
            Vd = torch.randn(kv, nkv, hd, generator=g)
            q = 0.1 * torch.randn(ql, nh, hd, generator=g)
            q[:, :, 0] = 4.0 / scale
            Kd, Vd, q = (t.to(dtype).double() for t in (Kd, Vd, q))
            _fill(cache, rows[r], Kd, Vd)
            pos = torch.arange(kv - ql, kv)[:, None]
            keys = torch.arange(kv)[None, :]
            ok = (keys <= pos) & (pos - keys < window)
            for sink in (True, False):
                o = torch.zeros(ql, nh, hd, dtype=F64)
                for h in range(nh):
                    sc = ((q[:, h] @ Kd[:, h // (nh // nkv)].T) * scale).masked_fill(~ok, float("-inf"))
                    e = torch.exp(sc)
                    o[:, h] = (e / (e.sum(-1, keepdim=True) + (1.0 if sink else 0.0))) @ Vd[:, h // (nh // nkv)]
                outs[sink].append(o)
            qs.append(q)
        T = sum(q_lens)
        q = torch.cat(qs).reshape(T, nh * hd).to(dtype).cuda()
        gate = torch.randn(T, nh + 6, generator=g).to(dtype).cuda()
        out = torch.empty(T, nh * hd, dtype=dtype, device="cuda")
        for tensor_memory in (True, False):
            monkeypatch.setattr(K, "USE_TCGEN05_ATTENTION", tensor_memory)
            for sink in (True, False):
                out.zero_()
                K.attention_dv(q, nh, nkv, hd, hd, ctx, cache, scale, window, 0, None, out, sink=sink)
                want = torch.cat(outs[sink]).reshape(T, nh * hd)
                assert (out.double().cpu() - want).abs().max() <= 8e-2, (targets, sink, tensor_memory)
            out.zero_()
            K.attention_dv(q, nh, nkv, hd, hd, ctx, cache, scale, window, 0, gate[:, 6:], out, sink=True, gate_per_head=True)
            gated = (torch.cat(outs[True]) * torch.sigmoid(gate[:, 6:].double().cpu())[:, :, None]).reshape(T, nh * hd)
            assert (out.double().cpu() - gated).abs().max() <= 8e-2, (targets, tensor_memory)
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sink_takes_everything_when_all_scores_are_low(dtype):
    """Scores of about -30 for every key: without the sink the output is the values' mean, with it
    the output vanishes; scores of about +30: the sink's share vanishes."""
    from llm_singularity_b200 import kernels as K
    nh, nkv, dk, dv, page = 4, 2, 32, 48, 16
    q_lens, kv_lens = [20, 1], [20, 45]
    ctx = _ctx(q_lens, kv_lens)
    cache = _pages(2, 48, nkv, dk, dv, page, dtype)
    g = torch.Generator().manual_seed(0)
    for r, kv in enumerate(kv_lens):
        Kd = torch.zeros(kv, nkv, dk)
        Kd[:, :, 0] = 1.0
        _fill(cache, r, Kd, 1.0 + torch.rand(kv, nkv, dv, generator=g))
    T = sum(q_lens)
    out = torch.empty(T, nh * dv, dtype=dtype, device="cuda")
    for level, lo, hi in ((-30.0, 0.0, 1e-9), (30.0, 0.99, 2.01)):
        q = torch.zeros(T, nh, dk)
        q[:, :, 0] = level
        K.attention_dv(q.reshape(T, nh * dk).to(dtype).cuda(), nh, nkv, dk, dv, ctx, cache, 1.0, 64, 0, None, out, sink=True)
        assert lo <= out.float().min().item() and out.float().max().item() <= hi, level
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_preparation_over_all_heads_and_unit_values(dtype):
    """Biases, the norm of q and of k over all their heads at once, rotation of the first dims with
    halves paired, value heads brought to unit rms, and the cache write, against plain arithmetic."""
    from llm_singularity_b200 import kernels as K
    from llm_singularity_b200.parts.rotary import rotary_inv_freq
    nh, nkv, dk, dv, rot, page, eps = 5, 2, 24, 10, 12, 8, 1e-4
    g = torch.Generator().manual_seed(3)
    q_lens, kv_lens = [9, 1, 4], [40, 33, 4]
    T, ld = sum(q_lens), nh * dk + nkv * dk + nkv * dv + 7
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    ctx = _ctx(q_lens, kv_lens, rows=[1, 2, 0])
    cache = _pages(3, 48, nkv, dk, dv, page, dtype, seed=2)
    proj = torch.randn(T, ld, generator=g).to(dtype).cuda()
    vec = {n: torch.randn(s, generator=g).cuda() for n, s in (("q_bias", nh * dk), ("k_bias", nkv * dk), ("v_bias", nkv * dv))}
    nrm = {n: (1 + 0.3 * torch.randn(s, generator=g)).cuda() for n, s in (("q_norm", nh * dk), ("k_norm", nkv * dk))}
    inv = rotary_inv_freq(rot, 900.0).float().cuda()
    q_out = torch.empty(T, nh * dk, dtype=dtype, device="cuda")
    K.attention_prep(proj, 3, 3 + nh * dk, 3 + (nh + nkv) * dk, nh, nkv, dk, dv, ctx, cache, q_out, norm_eps=eps,
                     inv_freq=inv, rotary_dim=rot, pairing="half", norm_all=True, v_unit=True, **vec, **nrm)
    pos = ctx.positions.cpu()
    x = proj.double().cpu()
    q = x[:, 3:3 + nh * dk] + vec["q_bias"].double().cpu()
    k = x[:, 3 + nh * dk:3 + (nh + nkv) * dk] + vec["k_bias"].double().cpu()
    v = x[:, 3 + (nh + nkv) * dk:3 + (nh + nkv) * dk + nkv * dv] + vec["v_bias"].double().cpu()
    q = (P.unit_rms(q, eps) * nrm["q_norm"].double().cpu()).view(T, nh, dk)
    k = (P.unit_rms(k, eps) * nrm["k_norm"].double().cpu()).view(T, nkv, dk)
    v = P.unit_rms(v.view(T, nkv, dv), eps)
    q, k = P.turn_halves(q, pos, rot, 900.0), P.turn_halves(k, pos, rot, 900.0)
    assert (q_out.double().cpu().view(T, nh, dk) - q).abs().max() <= tol * 8
    t0 = 0
    for r, (ql, kv) in enumerate(zip(q_lens, kv_lens)):
        p = torch.arange(kv - ql, kv)
        pages = cache.block_table[[1, 2, 0][r]].cpu()[p // page].long()
        got_k = cache.k_pages[pages, :, p % page, :].double().cpu()
        got_v = cache.v_pages[pages, :, p % page, :].double().cpu()
        assert (got_k - k[t0:t0 + ql]).abs().max() <= tol * 8
        assert (got_v - v[t0:t0 + ql]).abs().max() <= tol * 8
        t0 += ql
    K.check_status()


# ------------------------------------------------------------------ the memories' kernels
def _walk_scalar(S, q, k, v, fade, beta):
    """S [H, D, V] float64, walked over q, k [T, G, D], v [T, H, V], fade, beta [T, H]."""
    T, H = fade.shape
    G = q.shape[1]
    o = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        for h in range(H):
            g = h // (H // G)
            S[h] = fade[t, h] * S[h]
            S[h] = S[h] + torch.outer(k[t, g], beta[t, h] * (v[t, h] - S[h].T @ k[t, g]))
            o[t, h] = S[h].T @ q[t, g]
    return o


def _walk_channel(S, r, k, u, au, w, v):
    """S [H, D, V]; r, k, u, au, w [T, H, D]; v [T, H, V]."""
    T, H = r.shape[:2]
    o = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        for h in range(H):
            seen = u[t, h] @ S[h]
            S[h] = w[t, h][:, None] * S[h] - torch.outer(au[t, h], seen) + torch.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ r[t, h]
    return o


def _rand(*shape, g, scale=1.0):
    return (scale * torch.randn(*shape, generator=g)).float().double()


@pytest.mark.parametrize("H, G, D, V", [(3, 3, 16, 16), (4, 2, 32, 24), (2, 1, 64, 128), (5, 5, 6, 10), (6, 1, 48, 7),
                                        (1, 1, 128, 64), (2, 2, 200, 33), (8, 4, 96, 96)])
@pytest.mark.parametrize("segment", [None, 16, 7])
def test_delta_walk_with_state_carried_and_slots_used_again(H, G, D, V, segment, monkeypatch):
    """Both forms of the walk: four requests in changing portions (single tokens beside portions of
    hundreds), their slots in another order than the batch's, a slot given to a new request after it
    was zeroed, against a float64 walk of each request alone.  With short segments the long portions
    are walked in segments side by side (whole ones and a ragged last one, beside requests of one
    token in the same launch), the short steps in one walk each."""
    from llm_singularity_b200 import kernels as K
    if segment is not None:
        monkeypatch.setattr(K, "DELTA_SEGMENT", segment)
    g = torch.Generator().manual_seed(D + V)
    lens = {"a": 260, "b": 40, "c": 9, "d": 25}
    slot = {"a": 2, "b": 0, "c": 3, "d": 3}                       # d takes c's slot once c has ended
    plan = [[("a", 230), ("b", 3), ("c", 1)], [("b", 1), ("c", 8), ("a", 2)], [("d", 24), ("a", 1), ("b", 36)], [("a", 27), ("d", 1)]]
    for form in ("scalar", "channel"):
        heads_k = G if form == "scalar" else H
        data = {}
        for name, n in lens.items():
            k = _rand(n, heads_k, D, g=g)
            if form == "scalar":
                q = P.unit_length(_rand(n, G, D, g=g)) * D ** -0.5
                k = P.unit_length(k)
                fade = torch.sigmoid(_rand(n, H, g=g) + 3.0)
                beta = torch.sigmoid(_rand(n, H, g=g, scale=2.0))
                v = _rand(n, H, V, g=g)
                data[name] = dict(q=q, k=k, v=v, fade=fade, beta=beta)
            else:
                u = P.unit_length(k)
                au = torch.sigmoid(_rand(n, H, D, g=g, scale=2.0)) * u
                w = torch.exp(-0.6 * torch.sigmoid(_rand(n, H, D, g=g, scale=2.0)))
                data[name] = dict(r=_rand(n, H, D, g=g), k=k, u=u, au=au, w=w, v=_rand(n, H, V if form == "scalar" else D, g=g))
        Vf = V if form == "scalar" else D                         # the channel form's values have the keys' size
        want = {}
        for name, d in data.items():
            S = torch.zeros(H, D, Vf, dtype=F64)
            want[name] = _walk_scalar(S, d["q"], d["k"], d["v"], d["fade"], d["beta"]) if form == "scalar" \
                else _walk_channel(S, d["r"], d["k"], d["u"], d["au"], d["w"], d["v"])
        state = torch.randn(4, H, Vf, D, generator=g).cuda()        # what requests before left behind
        at, got, opened = {k: 0 for k in lens}, {k: [] for k in lens}, set()
        for step in plan:
            for name, _ in step:
                if name not in opened:
                    state[slot[name]].zero_()
                    opened.add(name)
            ctx = _ctx([n for _, n in step], [at[k] + n for k, n in step], rows=[slot[k] for k, _ in step])
            cut = lambda key: torch.cat([data[k][key][at[k]:at[k] + n] for k, n in step]).float().cuda().contiguous()
            T = sum(n for _, n in step)
            out = torch.empty(T, H * Vf, dtype=torch.float32, device="cuda")
            if form == "scalar":
                vecs = torch.cat([cut("q").reshape(T, G * D), cut("k").reshape(T, G * D)], dim=1).contiguous()
                scal = torch.cat([cut("fade"), cut("beta")], dim=1).contiguous()
                K.delta_scan("scalar", vecs, scal, cut("v").reshape(T, H * Vf), state, ctx, out, H, G, D, Vf)
            else:
                vecs = torch.stack([cut(n) for n in ("r", "k", "u", "au", "w")], dim=2).contiguous()      # [T, H, 5, D]
                K.delta_scan("channel", vecs, None, cut("v").reshape(T, H * Vf), state, ctx, out, H, H, D, Vf)
            o = 0
            for name, n in step:
                got[name].append(out[o:o + n].double().cpu().view(n, H, Vf))
                o += n
                at[name] += n
        assert at == lens
        for name in lens:
            scale = want[name].abs().max().item()
            assert (torch.cat(got[name]) - want[name]).abs().max() <= 2e-4 * scale, (form, name)
    K.check_status()


@pytest.mark.parametrize("where", [0, 5, 12])
def test_delta_walk_one_long_portion_beside_many_single_tokens(where, monkeypatch):
    """Thirteen requests in one launch, one of them with a portion of 101 tokens (first, in the middle
    or last in the batch) and the others with one to three tokens, every request from a state of its
    own: the long portion is walked in segments of 16, the short ones ride along, and each request
    matches a float64 walk of it alone.  Both forms."""
    from llm_singularity_b200 import kernels as K
    monkeypatch.setattr(K, "DELTA_SEGMENT", 16)
    H, G, D, V = 4, 2, 24, 20
    g = torch.Generator().manual_seed(where)
    q_lens = [1 + (i % 3) for i in range(13)]
    q_lens[where] = 101
    rows = [(5 * i + 3) % 13 for i in range(13)]                  # the slots in another order than the batch
    T = sum(q_lens)
    ctx = _ctx(q_lens, [n + 7 for n in q_lens], rows=rows)
    start = torch.randn(13, H, V, D, generator=g)                 # [slot, head, value, key]
    k = _rand(T, G, D, g=g)
    q = P.unit_length(_rand(T, G, D, g=g)) * D ** -0.5
    fade, beta = torch.sigmoid(_rand(T, H, g=g) + 3.0), torch.sigmoid(_rand(T, H, g=g, scale=2.0))
    v = _rand(T, H, V, g=g)
    kh = _rand(T, H, D, g=g)
    u = P.unit_length(kh)
    au = torch.sigmoid(_rand(T, H, D, g=g, scale=2.0)) * u
    w = torch.exp(-0.6 * torch.sigmoid(_rand(T, H, D, g=g, scale=2.0)))
    rr, vd = _rand(T, H, D, g=g), _rand(T, H, D, g=g)
    startd = torch.randn(13, H, D, D, generator=g)
    for form in ("scalar", "channel"):
        st0 = start if form == "scalar" else startd
        state = st0.clone().cuda()
        Vf = V if form == "scalar" else D
        out = torch.empty(T, H * Vf, dtype=torch.float32, device="cuda")
        f32 = lambda x: x.float().cuda().contiguous()
        if form == "scalar":
            vecs = torch.cat([f32(q).reshape(T, G * D), f32(P.unit_length(k)).reshape(T, G * D)], dim=1).contiguous()
            K.delta_scan("scalar", vecs, torch.cat([f32(fade), f32(beta)], dim=1).contiguous(), f32(v).reshape(T, H * Vf),
                         state, ctx, out, H, G, D, Vf)
        else:
            vecs = torch.stack([f32(x) for x in (rr, kh, u, au, w)], dim=2).contiguous()
            K.delta_scan("channel", vecs, None, f32(vd).reshape(T, H * Vf), state, ctx, out, H, H, D, Vf)
        t0 = 0
        for i, n in enumerate(q_lens):
            S = st0[rows[i]].double().transpose(1, 2).contiguous()        # [head, key, value]
            sl = slice(t0, t0 + n)
            want = _walk_scalar(S, q[sl], P.unit_length(k)[sl], v[sl], fade[sl], beta[sl]) if form == "scalar" \
                else _walk_channel(S, rr[sl], kh[sl], u[sl], au[sl], w[sl], vd[sl])
            got = out[sl].double().cpu().view(n, H, Vf)
            scale = max(want.abs().max().item(), 1.0)
            assert (got - want).abs().max() <= 2e-4 * scale, (form, i, n)
            assert (state[rows[i]].double().cpu().transpose(1, 2) - S).abs().max() <= 2e-4 * max(S.abs().max().item(), 1.0), (form, i)
            t0 += n
    K.check_status()


@pytest.mark.parametrize("segment", [None, 16])
def test_delta_walk_reads_a_write_from_far_back(segment, monkeypatch):
    """Scalar form, no fading: token 2 writes value x under key e0 with full strength, every later
    token writes under other keys, and the query at the very end, 400 tokens and many steps later,
    asks along e0: the answer is x exactly.  With a fade of 0.99 a token it is x * 0.99^(n-3).  With
    segments the write has to pass through a dozen segments' products."""
    from llm_singularity_b200 import kernels as K
    if segment is not None:
        monkeypatch.setattr(K, "DELTA_SEGMENT", segment)
    H, D, V, n = 2, 32, 16, 403
    g = torch.Generator().manual_seed(5)
    x = torch.randn(H, V, generator=g)
    for fade_value in (1.0, 0.99):
        k = torch.zeros(n, H, D)
        k[torch.arange(n), :, 1 + torch.arange(n) % (D - 1)] = 1.0
        k[2] = 0.0
        k[2, :, 0] = 1.0
        q = torch.zeros(n, H, D)
        q[:, :, 0] = 1.0
        v = torch.randn(n, H, V, generator=g)
        v[2] = x
        beta = torch.ones(n, H)
        fade = torch.full((n, H), fade_value)
        state = torch.randn(3, H, V, D, generator=g).cuda()
        state[1].zero_()
        at, last = 0, None
        for c in (1, 1, 1, 200, 1, 1, 2, 195, 1):
            ctx = _ctx([c], [at + c], rows=[1])
            out = torch.empty(c, H * V, dtype=torch.float32, device="cuda")
            sl = slice(at, at + c)
            vecs = torch.cat([q[sl].reshape(c, H * D), k[sl].reshape(c, H * D)], dim=1).contiguous().cuda()
            scal = torch.cat([fade[sl], beta[sl]], dim=1).contiguous().cuda()
            K.delta_scan("scalar", vecs, scal, v[sl].reshape(c, H * V).contiguous().cuda(), state, ctx, out, H, H, D, V)
            last = out[-1].cpu().view(H, V)
            at += c
        assert at == n
        assert (last - x * fade_value ** (n - 3)).abs().max() <= 1e-5
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("G, H, D, V, taps", [(2, 4, 16, 24, 3), (1, 2, 32, 32, 4), (3, 3, 10, 6, 5), (2, 2, 64, 32, 1), (1, 8, 8, 40, 2)])
def test_gated_memory_preparation_carries_the_convolutions_inputs(dtype, G, H, D, V, taps):
    """Two requests in portions shorter and longer than the taps (1, 2, 1, 7, ... tokens), slots in
    another order, one slot used again by a third request: convolution, silu, unit length, the
    write strength and the fade against plain arithmetic over each whole sequence."""
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(taps + D)
    GD, HV = G * D, H * V
    C, ld = 2 * GD + HV, 2 * GD + HV + HV + 5
    lens = {"a": 30, "b": 12, "c": 9}
    slot = {"a": 1, "b": 0, "c": 0}
    plan = [[("a", 1), ("b", 2)], [("a", 2), ("b", 1)], [("b", 7), ("a", 1)], [("a", 20), ("b", 2)], [("c", 2), ("a", 6)], [("c", 7)]]
    tap = [torch.randn(n, taps, generator=g) for n in (GD, GD, HV)]
    a_log, dt_bias = torch.randn(H, generator=g) - 1.0, torch.randn(H, generator=g)
    proj = {k: torch.randn(n, ld, generator=g).to(dtype) for k, n in lens.items()}
    raw = {k: 2 * torch.randn(n, 2 * H, generator=g) for k, n in lens.items()}
    want = {}
    for name, n in lens.items():
        x = proj[name].double()
        q = P.silu(P.short_conv(x[:, 3:3 + GD], tap[0].double())).view(n, G, D)
        k = P.silu(P.short_conv(x[:, 3 + GD:3 + 2 * GD], tap[1].double())).view(n, G, D)
        v = P.silu(P.short_conv(x[:, 3 + 2 * GD:3 + C], tap[2].double()))
        qk = torch.cat([(P.unit_length(q) * D ** -0.5).reshape(n, GD), P.unit_length(k).reshape(n, GD)], dim=1)
        r = raw[name].double()
        fade = torch.exp(-torch.exp(a_log.double()) * P.softplus(r[:, H:] + dt_bias.double()))
        want[name] = (qk, v, torch.cat([fade, torch.sigmoid(r[:, :H])], dim=1))
    conv_state = torch.randn(2, max(taps - 1, 1), C, generator=g).cuda() if taps > 1 else None
    dev_taps = tuple(t.cuda() for t in tap)
    at, got, opened = {k: 0 for k in lens}, {k: [] for k in lens}, set()
    for step in plan:
        for name, _ in step:
            if name not in opened:
                opened.add(name)
                if conv_state is not None:
                    conv_state[slot[name]].zero_()
        T = sum(n for _, n in step)
        ctx = _ctx([n for _, n in step], [at[k] + n for k, n in step], rows=[slot[k] for k, _ in step])
        rows = torch.cat([proj[k][at[k]:at[k] + n] for k, n in step]).cuda()
        rw = torch.cat([raw[k][at[k]:at[k] + n] for k, n in step]).cuda()
        qk, v, scal = (torch.empty(T, w, dtype=torch.float32, device="cuda") for w in (2 * GD, HV, 2 * H))
        K.gated_delta_prep(rows, 3, 3 + GD, 3 + 2 * GD, G, H, D, V, dev_taps, conv_state, rw, a_log.cuda(), dt_bias.cuda(), ctx,
                           qk, v, scal)
        o = 0
        for name, n in step:
            got[name].append(tuple(t[o:o + n].double().cpu() for t in (qk, v, scal)))
            o += n
            at[name] += n
    assert at == lens
    for name in lens:
        for i, what in enumerate(("q and k", "v", "fade and strength")):
            have = torch.cat([p[i] for p in got[name]])
            assert (have - want[name][i]).abs().max() <= 3e-5, (name, what)
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_channel_memory_preparation_and_read_out(dtype):
    from llm_singularity_b200 import kernels as K
    H, D, T, rate, eps = 3, 20, 11, math.exp(-0.5), 1e-5
    HD = H * D
    g = torch.Generator().manual_seed(2)
    proj = torch.randn(T, 4 * HD + 3, generator=g).to(dtype)
    decay_raw, remove_raw = 2 * torch.randn(T, HD, generator=g), 2 * torch.randn(T, HD + 4, generator=g)
    w0, ab = torch.randn(HD, generator=g), torch.randn(HD, generator=g)
    vecs = torch.empty(T, H, 5, D, dtype=torch.float32, device="cuda")
    v = torch.empty(T, HD, dtype=torch.float32, device="cuda")
    K.channel_delta_prep(proj.cuda(), 3, 3 + HD, 3 + 2 * HD, H, D, D, decay_raw.cuda(), w0.cuda(), remove_raw.cuda()[:, :HD],
                         ab.cuda(), rate, vecs, v)
    x = proj.double()
    r, k = x[:, 3:3 + HD].view(T, H, D), x[:, 3 + HD:3 + 2 * HD].view(T, H, D)
    u = P.unit_length(k)
    a = torch.sigmoid(remove_raw[:, :HD].double() + ab.double()).view(T, H, D)
    w = torch.exp(-rate * torch.sigmoid(decay_raw.double() + w0.double())).view(T, H, D)
    want = torch.stack([r, k, u, a * u, w], dim=2)
    assert (vecs.double().cpu() - want).abs().max() <= 3e-5
    assert (v.double().cpu() - x[:, 3 + 2 * HD:3 + 3 * HD]).abs().max() == 0
    # the read-out: unit rms per head, a weight over the row or one per head, sigmoid or silu of a gate
    o = torch.randn(T, HD, generator=g)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for weight, act in ((1 + 0.3 * torch.randn(HD, generator=g), "sigmoid"), (1 + 0.3 * torch.randn(D, generator=g), "silu")):
        y = torch.empty(T, HD, dtype=dtype, device="cuda")
        gate = proj.cuda()[:, 3 + 3 * HD:]
        K.delta_output(o.cuda(), weight.cuda(), H, eps, gate, act, y)
        z = gate.double().cpu()
        full = weight.double() if weight.numel() == HD else weight.double().repeat(H)
        ref = P.unit_rms(o.double().view(T, H, D), eps).reshape(T, HD) * full * (torch.sigmoid(z) if act == "sigmoid" else P.silu(z))
        assert (y.double().cpu() - ref).abs().max() <= tol * 4
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_activation_soft_cap_and_branch_sum(dtype):
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(4)
    tol = 3e-6 if dtype == torch.float32 else 2e-2
    z = (3 * torch.randn(37, 50, generator=g)).to(dtype)
    z[0, :4] = torch.tensor([0.0, -0.0, 1e-3, -1e-3]).to(dtype)
    p, q = torch.tensor(0.4, dtype=F64), torch.tensor(-0.7, dtype=F64)
    out = torch.empty_like(z, device="cuda")
    K.plain_activation(z.cuda(), out, "bent_square", float(P.softplus(p)), float(0.5 + P.softplus(q)))
    want = P.bent_square(z.double(), p, q)
    assert ((out.double().cpu() - want).abs() <= tol * (1 + want.abs())).all()
    x = (40 * torch.randn(9, 33, generator=g)).cuda()
    keep = x.clone()
    K.softcap(x, 12.5)
    assert (x.double().cpu() - 12.5 * torch.tanh(keep.double().cpu() / 12.5)).abs().max() <= 1e-5
    ys = [torch.randn(21, 90, generator=g).to(dtype).cuda() for _ in range(2)]
    out = torch.empty(21, 90, dtype=dtype, device="cuda")
    K.branch_sum(ys, (0.6, -1.5), out)
    assert (out.double().cpu() - (0.6 * ys[0].double().cpu() - 1.5 * ys[1].double().cpu())).abs().max() <= tol * 4
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
    W, path = _setup(tmp_path, cfg, 23, rank=U.DECAY_RANKS["mix_a"])
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
    import json
    import os
    import subprocess
    import sys
    cfg = U.CONFIGS["mix_b"]
    W, path = _setup(tmp_path, cfg, 29, rank=U.DECAY_RANKS["mix_b"])
    prompts = [U.tokens_for(cfg, n, 70 + n) for n in (4, 19)]
    (tmp_path / "p.json").write_text(json.dumps(prompts))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, os.path.join(root, "bin", "llm-serve-llama"), "--model-dir", path, "--dtype", "fp32",
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
