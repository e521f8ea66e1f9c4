"""The layered model family on the GPU against the plain fp32 restatement in oracle/gitozen_oracle.py.

Every test builds its own small configuration and random weights.  Logits are compared at EVERY position; the engine
computes this family in fp32 on bf16 weights, so the bound is rounding: 1e-4 of the largest logit.
"""
import numpy as np
import pytest
import torch

from oracle import gitozen_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-4


def latent(heads=3, dim=24, vdim=20, kv_rank=40, scale=0.21, **mlp):
    return dict(mixer="latent_attention", heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, scale=scale, **mlp)


def delta(heads=4, kv_heads=2, dim=16, vdim=24, conv=4, rank_a=8, rank_g=12, **mlp):
    return dict(mixer="channel_delta", heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, rank_a=rank_a,
                rank_g=rank_g, **mlp)


def moe(ff=40, experts=12, top=3, groups=4, keep=2):
    return dict(ff=ff, experts=experts, top=top, groups=groups, keep=keep)


def make(layers, width=96, vocab=160, softcap=12.0, eps=1e-5, seed=0, tweak=None):
    from fasttalk_llm_microservice_b200.layered import LayeredSpec, LayerSpec, init_weights
    spec = LayeredSpec(name="test", architecture="Gitozen", width=width, vocab=vocab, eps=eps, logit_softcap=softcap,
                       layers=tuple(LayerSpec(**l) for l in layers))
    w = init_weights(spec, seed=seed)
    if tweak:
        tweak(w)
    return spec, w


def engine(spec, w, **kw):
    from fasttalk_llm_microservice_b200 import build
    from fasttalk_llm_microservice_b200.engine import Engine, EngineLimits
    build.build()
    lim = EngineLimits(**{"max_batch": 4, "max_batched_tokens": 512, "max_context": 512, "num_pages": 16,
                          "max_sessions": 4, "debug_logit_rows": 512, **kw})
    return Engine(spec, w, lim, eos_ids=())


def oracle_logits(spec, w, tokens):
    with torch.no_grad():
        return O.forward(spec.config(), w, list(tokens)).numpy()


def rel(got, ref):
    return float(np.abs(got - ref).max() / np.abs(ref).max())


def tokens_of(spec, n, seed):
    return np.random.default_rng(seed).integers(0, spec.vocab, n).tolist()


def feed_cut(eng, sid, toks, cuts):
    """Feed `toks` to session `sid` in portions of the given sizes (the last size repeats); logits of every position."""
    out, pos, k = [], 0, 0
    while pos < len(toks):
        n = min(cuts[min(k, len(cuts) - 1)], len(toks) - pos)
        out.append(eng.feed([(sid, toks[pos:pos + n], list(range(n)))]))
        pos, k = pos + n, k + 1
    return np.concatenate(out)


MIXED = [delta(**moe()), latent(**moe(experts=6, top=3, groups=3, keep=2, ff=24)), delta(heads=2, kv_heads=2, dim=24, vdim=8, conv=2),
         latent(heads=5, dim=8, vdim=12, kv_rank=33, scale=0.4)]


@pytest.mark.parametrize("layers", [
    [latent()],                                        # the mixers alone, no feed-forward
    [delta()],
    [delta(heads=3, kv_heads=1, dim=40, vdim=72, conv=5, rank_a=3, rank_g=5)],
    [delta(heads=2, kv_heads=2, dim=8, vdim=8, conv=1)],
    [delta(heads=2, kv_heads=1, dim=32, vdim=40, conv=3), delta(heads=3, kv_heads=3, dim=64, vdim=16, conv=2)],   # whole runs of channels per lane
    [latent(**moe())],                                 # experts: groups that matter, then one group, then top = all
    [latent(**moe(experts=6, top=2, groups=1, keep=1))],
    [latent(**moe(experts=4, top=4, groups=2, keep=2, ff=17))],
    MIXED,
], ids=["latent", "delta", "delta-odd", "delta-conv1", "delta-full-runs", "moe-groups", "moe-flat", "moe-all", "mixed"])
def test_whole_prompt_matches_oracle(layers):
    spec, w = make(layers, seed=3)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 150, 1)
        got = eng.feed([("s", toks, list(range(len(toks))))])
        assert rel(got, oracle_logits(spec, w, toks)) < TOL
    finally:
        eng.close()


def test_other_sizes_and_no_softcap():
    spec, w = make([latent(heads=1, dim=48, vdim=56, kv_rank=72, scale=0.15, **moe(ff=88, experts=16, top=6, groups=8, keep=5)),
                    delta(heads=6, kv_heads=3, dim=20, vdim=16, conv=2, rank_a=10, rank_g=2)],
                   width=200, vocab=333, softcap=0.0, eps=1e-6, seed=9)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 90, 2)
        got = eng.feed([("s", toks, list(range(len(toks))))])
        assert rel(got, oracle_logits(spec, w, toks)) < TOL
    finally:
        eng.close()


def test_residual_after_every_layer():
    spec, w = make(MIXED, seed=4)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 70, 5)
        eng.debug_trail(True)
        eng.feed([("s", toks, [])])
        got = eng.read_trail(len(toks))
        trail = []
        with torch.no_grad():
            O.forward(spec.config(), w, toks, trail)
        for i, x in enumerate(trail):
            assert rel(got[i], x.numpy()) < TOL, f"layer {i}"
    finally:
        eng.close()


def test_router_groups_change_the_choice():
    """The test weights are such that the group limit matters: without it other experts would be chosen."""
    spec, w = make([latent(**moe())], seed=3)
    h = torch.randn(200, spec.width)
    r = dict(experts=12, top=3, groups={"count": 4, "keep": 2})
    limited, _ = O.route(h, w["l0.mlp.router"], r)
    free, _ = O.route(h, w["l0.mlp.router"], dict(r, groups={"count": 1, "keep": 1}))
    assert (limited.sort(-1).values != free.sort(-1).values).any()


@pytest.mark.parametrize("cuts", [[1], [2], [3, 2, 29, 1, 1, 17, 2], [64], [63, 1, 1, 64, 2], [65, 2]],
                         ids=["token-by-token", "pairs", "ragged", "pages", "page-edges", "over-a-page"])
def test_portions_and_decoding_match_the_whole_prompt(cuts):
    spec, w = make(MIXED, seed=5)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 200, 6)
        ref = oracle_logits(spec, w, toks)
        whole = eng.feed([("whole", toks, list(range(len(toks))))])
        eng.close_session("whole")
        got = feed_cut(eng, "cut", toks, cuts)
        assert rel(whole, ref) < TOL and rel(got, ref) < TOL
        assert rel(got, whole) < 2e-5          # the same arithmetic, apart from summation order in few-row launches
    finally:
        eng.close()


def sharpen(factor):
    def f(w):
        for k in list(w):
            if k.endswith("mix.q") and k.replace("mix.q", "mix.dkv") in w:
                w[k] = (w[k].float() * factor).to(torch.bfloat16)
    return f


def test_far_keys_and_page_borders_with_sharp_attention():
    """Queries scaled up: each position attends to a few keys, often hundreds of tokens back, so a key that is lost
    or misplaced (a page's last or first row, a stale page) changes the logits by far more than the bound."""
    layers = [latent(heads=2, dim=16, vdim=16, kv_rank=24, scale=0.25), latent(heads=4, dim=8, vdim=8, kv_rank=16, scale=0.35)]
    spec, w = make(layers, width=64, vocab=96, seed=7, tweak=sharpen(24.0))
    cfg = spec.config()
    toks = tokens_of(spec, 330, 8)
    with torch.no_grad():          # the test means something: the attention of the first layer is peaked and reaches back
        h = O.scalar_norm(w["embed"].float()[torch.tensor(toks)], w["l0.norm1"], spec.eps)
        m = cfg["layers"][0]["mixer"]
        q = (h @ w["l0.mix.q"].float().T).reshape(len(toks), m["heads"], m["dim"])
        c = O.rms_unit(h @ w["l0.mix.dkv"].float().T, spec.eps) * w["l0.mix.dkv.norm"].float()
        k = (c @ w["l0.mix.uk"].float().T).reshape(len(toks), m["heads"], m["dim"])
        s = torch.einsum("hd,jhd->hj", q[-1], k) * m["scale"]
        a = torch.softmax(s, -1)
        # (a token that occurs r times shares its weight among r equal keys: there are no positions in this attention)
        assert a.max() > 20.0 / len(toks) and float(a[:, :len(toks) - 100].sum(-1).min()) > 0.4
    eng = engine(spec, w)
    try:
        ref = oracle_logits(spec, w, toks)
        got = feed_cut(eng, "a", toks, [190, 1, 1, 62, 1, 1, 1, 5, 1])
        assert rel(got, ref) < TOL
    finally:
        eng.close()


def test_delta_rule_remembers_a_far_write():
    """One early token writes a large value; with decays near one it must still be read hundreds of tokens later."""
    def slow_decay(w):
        w["l0.mix.dt_bias"] = torch.full_like(w["l0.mix.dt_bias"], -9.0)
        w["l0.mix.a2"] = torch.zeros_like(w["l0.mix.a2"])
    spec, w = make([delta(heads=2, kv_heads=1, dim=16, vdim=16, conv=3)], width=64, vocab=96, seed=11, tweak=slow_decay)
    toks = tokens_of(spec, 260, 12)
    other = list(toks)
    other[3] = (toks[3] + 1) % spec.vocab
    ref, ref_other = oracle_logits(spec, w, toks), oracle_logits(spec, w, other)
    assert rel(ref[-1], ref_other[-1]) > 20 * TOL          # position 259 still depends on token 3
    eng = engine(spec, w)
    try:
        got = feed_cut(eng, "a", toks, [100, 1, 1, 2, 64, 1])
        assert rel(got, ref) < TOL
    finally:
        eng.close()


def test_unequal_requests_in_one_batch_match_each_alone():
    spec, w = make(MIXED, seed=13)
    eng = engine(spec, w)
    try:
        seqs = {n: tokens_of(spec, ln, 20 + i) for i, (n, ln) in enumerate([("a", 140), ("b", 33), ("c", 70), ("d", 9)])}
        ref = {n: oracle_logits(spec, w, t) for n, t in seqs.items()}
        alone = {}
        for n, t in seqs.items():
            alone[n] = eng.feed([(n + "-alone", t, list(range(len(t))))])
            eng.close_session(n + "-alone")
        # a schedule of mixed steps: portions of some beside single tokens of others, one request pausing for a step
        plan = [{"a": 64, "b": 1}, {"a": 2, "b": 1, "c": 29}, {"b": 16, "c": 1, "d": 3}, {"a": 1, "c": 1, "d": 1},
                {"a": 70, "b": 15, "c": 39, "d": 5}, {"a": 3}]
        at = {n: 0 for n in seqs}
        got = {n: [] for n in seqs}
        for step in plan:
            entries, names = [], []
            for n, cnt in step.items():
                cnt = min(cnt, len(seqs[n]) - at[n])
                if cnt:
                    entries.append((n, seqs[n][at[n]:at[n] + cnt], list(range(cnt))))
                    names.append((n, cnt))
            out = eng.feed(entries)
            o = 0
            for n, cnt in names:
                got[n].append(out[o:o + cnt])
                o += cnt
                at[n] += cnt
        for n in seqs:
            assert at[n] == len(seqs[n])
            g = np.concatenate(got[n])
            assert rel(g, ref[n]) < TOL, n
            assert rel(g, alone[n]) < 2e-5, n
    finally:
        eng.close()


def test_pages_and_state_slots_are_used_again():
    """A pool of 6 pages and 2 slots serves 6 sequences one after the other and two at a time: what an ended session
    left in its pages and its slot must not reach the next one."""
    spec, w = make(MIXED, seed=17)
    eng = engine(spec, w, max_batch=2, max_sessions=2, num_pages=6, max_context=384, max_batched_tokens=384,
                 debug_logit_rows=384)
    try:
        seqs = [tokens_of(spec, ln, 40 + i) for i, ln in enumerate([190, 100, 130, 64, 65, 180])]
        ref = [oracle_logits(spec, w, t) for t in seqs]
        for i in (0, 1):                                       # alone, the whole pool in turn
            assert rel(feed_cut(eng, f"s{i}", seqs[i], [50, 1, 1, 90]), ref[i]) < TOL
            eng.close_session(f"s{i}")
            assert eng.stats()["free_pages"] == 6
        for a, b in ((2, 3), (4, 5)):                          # two at a time, the shorter one ends first
            la, lb = len(seqs[a]), len(seqs[b])
            ga, gb, pa, pb = [], [], 0, 0
            while pa < la or pb < lb:
                entries = []
                na, nb = min(37, la - pa), min(1 if pb else 20, lb - pb)
                if na:
                    entries.append((f"s{a}", seqs[a][pa:pa + na], list(range(na))))
                if nb:
                    entries.append((f"s{b}", seqs[b][pb:pb + nb], list(range(nb))))
                out = eng.feed(entries)
                ga.append(out[:na]); gb.append(out[na:na + nb])
                pa, pb = pa + na, pb + nb
                if pa == la and na:
                    eng.close_session(f"s{a}")
                if pb == lb and nb:
                    eng.close_session(f"s{b}")
            assert rel(np.concatenate(ga), ref[a]) < TOL and rel(np.concatenate(gb), ref[b]) < TOL
        st = eng.stats()
        assert st["free_pages"] == 6 and st["live_sessions"] == 0
    finally:
        eng.close()


def test_first_tokens_and_long_decoding():
    spec, w = make(MIXED, seed=19)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 300, 21)
        ref = oracle_logits(spec, w, toks)
        got = feed_cut(eng, "a", toks, [1, 1, 1, 2, 1, 30, 1])      # a sequence that starts with single tokens, then 264 decoded
        assert rel(got[:8], ref[:8]) < TOL
        assert rel(got, ref) < TOL
    finally:
        eng.close()


def test_greedy_generation_through_the_scheduler():
    """Engine.generate: submit -> the scheduler's own chunked prefill and decode steps -> argmax sampling; three requests
    of unequal length run together, prompts longer than a step's token budget are cut by the scheduler itself."""
    spec, w = make(MIXED, seed=23)
    eng = engine(spec, w, max_batched_tokens=48, decode_prefill_cap=16)
    try:
        prompts = [tokens_of(spec, ln, 60 + i) for i, ln in enumerate([100, 7, 51])]
        n_new = 24
        got = eng.generate(prompts, n_new, temperature=0.0, ignore_eos=True)
        for p, g in zip(prompts, got):
            assert len(g) == n_new
            toks = list(p)
            for t in g:                     # teacher-forced on the engine's own tokens: each must be the oracle's argmax
                lg = oracle_logits(spec, w, toks)[-1]
                top2 = np.sort(lg)[-2:]
                assert t == int(lg.argmax()) or (top2[1] - lg[t]) < 1e-4 * np.abs(lg).max()
                toks.append(t)
        # the same conversation again, longer: the cached state and latents are continued, not rebuilt
        more = prompts[1] + got[1] + tokens_of(spec, 5, 99)
        again = eng.generate([more], 4, sessions=["gen-1"], temperature=0.0, ignore_eos=True)[0]
        assert eng.stats()["prefix_hit_tokens"] >= len(prompts[1]) + n_new - 1
        assert again == O.greedy(spec.config(), w, more, 4)
        # and one that diverges early: a recurrent state cannot be rewound, the whole prompt runs again
        other = [more[0], (more[1] + 1) % spec.vocab] + more[2:20]
        assert eng.generate([other], 3, sessions=["gen-1"], temperature=0.0, ignore_eos=True)[0] == O.greedy(spec.config(), w, other, 3)
    finally:
        eng.close()


def test_sampling_with_temperature_runs():
    spec, w = make([delta(**moe()), latent()], seed=29)
    eng = engine(spec, w)
    try:
        out = eng.generate([tokens_of(spec, 20, 1), tokens_of(spec, 5, 2)], 8, temperature=0.8, top_k=20, top_p=0.9,
                           seed=5, ignore_eos=True)
        assert all(len(o) == 8 and all(0 <= t < spec.vocab for t in o) for o in out)
    finally:
        eng.close()


def test_trace_runner_replays_a_schedule(tmp_path):
    """bin/trace_run on a saved checkpoint: two steps, one wanted place each, then a session ends."""
    import json
    import os
    import subprocess
    import sys
    from fasttalk_llm_microservice_b200.layered import save_checkpoint
    spec, w = make(MIXED, seed=31)
    save_checkpoint(spec, w, str(tmp_path / "model"))
    toks = tokens_of(spec, 40, 3)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[30:31], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[31:], "want": [8]}, {"id": "y", "tokens": toks[:5], "want": [4]}],
              "end": ["x", "y"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / ("out-" + dtype)
        r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path / "model"), "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        ref = oracle_logits(spec, w, toks)
        a = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, spec.vocab)
        c = np.fromfile(out / "2.f32", dtype="<f4").reshape(2, spec.vocab)
        assert not (out / "1.f32").exists()
        tol = TOL if dtype == "float32" else 3e-2
        assert rel(a, ref[[0, 29]]) < tol and rel(c[0], ref[39]) < tol and rel(c[1], ref[4]) < tol


@pytest.mark.parametrize("exact", [False, True], ids=["tensor-cores", "exact-fp32"])
def test_projections_on_tensor_cores_and_in_exact_fp32(exact):
    """Shapes that tile (width and heads * vdim multiples of 64, vocab of 128): with enough rows the input, output and head
    projections run on the tensor cores from bf16 hi + lo planes unless the engine was made exact, and so do the experts of
    the first layer (ff a multiple of 64) in the 100-token portion, one GEMM per expert; single tokens and short portions
    take the CUDA-core kernels either way, so the two forms must agree along one sequence."""
    layers = [latent(heads=4, dim=16, vdim=32, kv_rank=48, scale=0.25, **moe(ff=64, experts=6, top=2, groups=3, keep=1)),
              delta(heads=4, kv_heads=2, dim=16, vdim=16, conv=3, rank_a=8, rank_g=8, **moe(ff=24, experts=4, top=2, groups=2, keep=1))]
    spec, w = make(layers, width=128, vocab=256, seed=37)
    eng = engine(spec, w, exact_f32=exact)
    try:
        toks = tokens_of(spec, 180, 38)
        ref = oracle_logits(spec, w, toks)
        got = feed_cut(eng, "a", toks, [150, 1, 1, 12, 3, 10, 1])
        assert rel(got, ref) < (TOL if exact else 3e-4)
    finally:
        eng.close()


def test_served_through_the_handler(tmp_path, monkeypatch):
    """A layered checkpoint behind the serving path: FASTTALK_CHECKPOINT -> registry -> engine -> NativeHandler streams text."""
    from fasttalk_llm_microservice_b200.handler import NativeHandler
    from fasttalk_llm_microservice_b200.layered import save_checkpoint
    spec, w = make([delta(**moe()), latent()], width=64, vocab=600, seed=41)
    save_checkpoint(spec, w, str(tmp_path / "ckpt"))
    monkeypatch.setenv("FASTTALK_CHECKPOINT", str(tmp_path / "ckpt"))
    monkeypatch.setenv("FASTTALK_ALLOW_BYTE_TOKENIZER", "1")
    monkeypatch.setenv("FASTTALK_MAX_SESSIONS", "4")
    monkeypatch.setenv("FASTTALK_MAX_CONTEXT", "512")
    monkeypatch.setenv("FASTTALK_MAX_BATCHED_TOKENS", "256")
    from fasttalk_llm_microservice_b200.handler import build_runner
    runner = build_runner("gitozen-test")
    h = NativeHandler(model="gitozen-test", runner=runner)
    try:
        assert h.check_connection()
        chunks = list(h.generate_stream([{"role": "user", "content": "hello there"}], temperature=0.0, max_tokens=12,
                                        request_id="conv-1"))
        assert 1 <= len(chunks) <= 12
        st = h.runner.engine.stats()
        assert st["prefill_tokens"] > 0 and st["decode_tokens"] > 0
    finally:
        h.close()
        runner.shutdown()
        runner.engine.close()


@pytest.mark.parametrize("sharp", [1.0, 16.0], ids=["plain", "sharp"])
def test_latent_attention_on_tensor_cores(sharp):
    """Latent sizes that are multiples of 32 take the mma.sync kernel in the serving form (bf16 queries, latents and softmax
    weights, fp32 sums): 3 heads (one partly filled group of 16), 20 heads (two groups), prompts over several pages, single
    tokens with key shares.  bf16 operands bound the agreement with the fp32 restatement; the exact engine stays at 1e-4.
    With sharpened queries a lost or misplaced key would show far above either bound."""
    layers = [latent(heads=3, dim=16, vdim=24, kv_rank=64, scale=0.3),
              latent(heads=20, dim=8, vdim=8, kv_rank=32, scale=0.4, **moe(ff=24, experts=4, top=2, groups=2, keep=1))]
    spec, w = make(layers, width=64, vocab=96, seed=43, tweak=sharpen(sharp))
    toks = tokens_of(spec, 330, 44)
    ref = oracle_logits(spec, w, toks)
    for exact, tol in ((False, 2e-2), (True, TOL)):
        eng = engine(spec, w, exact_f32=exact)
        try:
            got = feed_cut(eng, "a", toks, [190, 1, 1, 62, 1, 1, 1, 5, 1])
            assert rel(got, ref) < tol, ("exact" if exact else "tensor cores")
        finally:
            eng.close()
