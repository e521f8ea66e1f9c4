"""The Gedelorn design on the GPU against the plain restatement in oracle/gedelorn_oracle.py.

Every test builds its own small configuration and random weights (none of them a published model's sizes).  Logits are
compared at EVERY position; the engine keeps this family in fp32 on bf16 weights, so the bound is rounding: 1e-4 of the
largest logit in the exact form, a few times that when projections run on the tensor cores from bf16 hi + lo planes.
"""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import gedelorn_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-4


# ------------------------------------------------------------------------------------------------ configurations
def memory(heads=3, dim=12, vdim=20, gate_cap=9.0):
    return {"type": "mlstm", "mixer": {"dim": dim, "gate_cap": gate_cap, "heads": heads, "vdim": vdim}}


def space(heads=6, vdim=8, state=12, groups=3, norm_groups=2, conv=4):
    return {"type": "mamba2", "mixer": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups,
                                        "state": state, "vdim": vdim}}


def window(heads=6, kv_heads=2, dim=16, size=17, rot=(8, 5000.0), softcap=30.0, scale=0.3):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": size}, "scale": scale, "vdim": dim}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if softcap:
        m["softcap"] = softcap
    return m


def decaying(heads=3, dim=20, vdim=12, decay=(0.7, 0.95, 0.999)):
    return {"decay": list(decay), "dim": dim, "heads": heads, "vdim": vdim}


def parallel(left=None, right=None, left_scale=0.6, right_scale=1.3):
    return {"type": "parallel", "mixer": {"left": left or window(), "left_scale": left_scale, "right": right or decaying(),
                                          "right_scale": right_scale}}


def dense(ff=72):
    return {"ff": ff, "kind": "dense"}


def moe(ff=24, experts=7, top=3, scale=1.7, shared=40):
    m = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}
    if scale is not None:
        m["router"]["scale"] = scale
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp=None):
    return {**mixer, "mlp": mlp}


def make(layers, width=80, vocab=150, eps=1e-5, seed=0, tweak=None):
    from fasttalk_llm_microservice_b200.layered import init_weights, spec_from_config
    cfg = {"architecture": "Gedelorn", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    spec = spec_from_config(cfg, name="test")
    assert spec_from_config(spec.config(), name="test") == spec
    w = init_weights(spec, seed=seed)
    if tweak:
        tweak(w)
    return spec, w


def engine(spec, w, **kw):
    from fasttalk_llm_microservice_b200 import build
    from fasttalk_llm_microservice_b200.engine import Engine, EngineLimits
    build.build()
    lim = EngineLimits(**{"max_batch": 4, "max_batched_tokens": 512, "max_context": 512, "num_pages": 16,
                          "max_sessions": 4, "debug_logit_rows": 512, "exact_f32": True, **kw})
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


MIXED = [layer(space(), dense()), layer(parallel(), moe()), layer(memory(), dense(ff=33)), layer(space(heads=4, vdim=12, state=8, groups=1, norm_groups=4, conv=2), moe(experts=4, top=2, scale=None, shared=0)),
         layer(parallel(window(heads=2, kv_heads=2, dim=24, size=70, rot=(24, 1e6), softcap=0), decaying(heads=1, dim=8, vdim=40, decay=(0.9,))))]


# ------------------------------------------------------------------------------------------------ every mechanism alone
@pytest.mark.parametrize("layers", [
    [layer(memory())],
    [layer(memory(heads=1, dim=40, vdim=8, gate_cap=4.0))],
    [layer(memory(heads=2, dim=72, vdim=33))],                           # more key channels than one run of lanes holds
    [layer(space())],
    [layer(space(heads=4, vdim=20, state=6, groups=1, norm_groups=1, conv=1))],
    [layer(space(heads=4, vdim=4, state=130, groups=4, norm_groups=4, conv=7))],
    [layer(parallel())],
    [layer(parallel(window(heads=4, kv_heads=4, dim=10, size=1, rot=(10, 100.0), softcap=0), decaying(heads=2, dim=4, vdim=70, decay=(1.0, 0.5))))],
    [layer(parallel(window(heads=3, kv_heads=1, dim=36, size=400, rot=None), left_scale=1.0, right_scale=0.25))],
    [layer(parallel(window(heads=2, kv_heads=1, dim=160, size=90, rot=(64, 1e4), scale=0.08), decaying(heads=1, dim=300, vdim=8, decay=(0.97,))))],
    [layer(parallel(window(heads=1, kv_heads=1, dim=264, size=50, rot=(8, 1e4), scale=0.06), decaying(heads=1, dim=8, vdim=8, decay=(0.9,))))],
    [layer(space(), dense())],
    [layer(memory(), moe())],
    [layer(memory(), moe(experts=3, top=3, shared=0))],                  # every expert chosen, no shared expert
    [layer(memory(), moe(experts=40, top=1, scale=None, shared=9))],     # more experts than lanes, one chosen
    MIXED,
], ids=["memory", "memory-1head", "memory-wide", "space", "space-1group-1tap", "space-big-state", "parallel", "parallel-window1",
        "parallel-norot", "parallel-wide-heads", "parallel-widest-head", "dense", "moe", "moe-all", "moe-top1", "mixed"])
def test_whole_prompt_matches_oracle(layers):
    spec, w = make(layers, seed=3)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 150, 1)
        got = eng.feed([("s", toks, list(range(len(toks))))])
        assert rel(got, oracle_logits(spec, w, toks)) < TOL
    finally:
        eng.close()


def test_other_sizes():
    layers = [layer(parallel(window(heads=10, kv_heads=5, dim=12, size=33, rot=(4, 77.0), softcap=5.0, scale=0.5),
                             decaying(heads=5, dim=6, vdim=14, decay=(0.1, 0.3, 0.5, 0.8, 0.99)), 1.5, 0.5), dense(ff=50)),
              layer(space(heads=9, vdim=6, state=10, groups=3, norm_groups=9, conv=5), moe(ff=10, experts=9, top=5, scale=0.5, shared=3)),
              layer(memory(heads=5, dim=6, vdim=14, gate_cap=20.0))]
    spec, w = make(layers, width=70, vocab=333, eps=1e-6, seed=9)
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
            O.forward(spec.config(), w, toks, trail=trail)
        for i, t in enumerate(trail):
            assert rel(got[i], t.numpy()) < TOL, i
    finally:
        eng.close()


# ------------------------------------------------------------------------------------------------ portions, decoding
@pytest.mark.parametrize("cuts", [[1], [2], [3, 2, 29, 1, 1, 17, 2], [64], [63, 1, 1, 64, 2], [65, 2]],
                         ids=["token-by-token", "twos", "ragged", "pages", "around-pages", "over-a-page"])
def test_portions_and_decoding_match_the_whole_prompt(cuts):
    spec, w = make(MIXED, seed=7)
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 200, 8)
        ref = oracle_logits(spec, w, toks)
        whole = eng.feed([("w", toks, list(range(len(toks))))])
        got = feed_cut(eng, "c", toks, cuts)
        assert rel(whole, ref) < TOL and rel(got, ref) < TOL
        assert rel(got, whole) < 2e-5
    finally:
        eng.close()


def sharpen(factor):
    """Queries of every window attention times `factor`: the softmax then rests on one or two keys, so a key that is
    wrongly seen or wrongly hidden (one off at a window's edge, a wrong page) moves the result by far more than rounding."""
    def tweak(w):
        for k in list(w):
            if k.endswith("left.q") or k.endswith("left.q.b"):
                w[k] = (w[k].float() * factor).to(torch.bfloat16)
    return tweak


@pytest.mark.parametrize("size", [2, 5, 63, 64, 65, 129, 1000])
def test_window_edges_with_sharp_attention(size):
    """Windows shorter than, equal to and longer than a page, and longer than the sequence; prompt portions and single
    decoded tokens both cross every edge."""
    layers = [layer(parallel(window(heads=4, kv_heads=2, dim=16, size=size, rot=(16, 10000.0), softcap=0, scale=0.25)))]
    spec, w = make(layers, width=64, seed=11, tweak=sharpen(12.0))
    eng = engine(spec, w)
    try:
        toks = tokens_of(spec, 260, 12)
        ref = oracle_logits(spec, w, toks)
        got = feed_cut(eng, "a", toks, [130, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 60, 1])
        assert rel(got, ref) < TOL
        # the test has teeth: a window one longer or one shorter gives another result
        cfg = spec.config()
        cfg["layers"][0]["mixer"]["left"]["mask"]["size"] = size + 1
        if size < 260:
            with torch.no_grad():
                assert rel(O.forward(cfg, w, toks).numpy(), ref) > 50 * TOL
    finally:
        eng.close()


def test_one_key_just_inside_and_just_outside_the_window():
    """One marked token in a run of equal tokens: the query scaled so that the marked key takes all the weight while it is
    visible.  The logits must change exactly when the marked token leaves the window, in a prompt and in decoding."""
    size = 37
    layers = [layer(parallel(window(heads=2, kv_heads=1, dim=8, size=size, rot=None, softcap=0, scale=1.0), left_scale=1.0, right_scale=0.0))]

    def tweak(w):
        # token 1 is the marked one: its key has a large component that every query of token 0 likes
        w["embed"][:] = 0
        w["embed"][0, 0], w["embed"][1, 1], w["embed"][0, 2], w["embed"][1, 3] = 1.0, 1.0, 0.5, -0.5
        for n in ("l0.mix.left.q", "l0.mix.left.k"):
            w[n][:] = 0
        w["l0.mix.left.q.b"][:] = 0
        w["l0.mix.left.k.b"][:] = 0
        w["l0.mix.left.q"][0, 0] = w["l0.mix.left.q"][8, 0] = 8.0      # token 0's queries point along key channel 0
        w["l0.mix.left.k"][0, 1] = 8.0                                    # only token 1's key has that channel
        w["l0.mix.left.k"][1, 0] = w["l0.mix.left.k"][2, 1] = 1.0         # values (= keys) that tell the two tokens apart
    spec, w = make(layers, width=32, vocab=40, seed=2, tweak=tweak)
    eng = engine(spec, w)
    try:
        mark = 70
        toks = [0] * 200
        toks[mark] = 1
        ref = oracle_logits(spec, w, toks)
        inside, outside = ref[mark + size - 1], ref[mark + size]
        assert np.abs(inside - outside).max() > 1e-2 * np.abs(ref).max()          # the oracle itself sees the edge
        for cuts in ([200], [mark + size - 1, 1, 1, 1], [mark + 3, 1], [64, 2, 2]):
            got = feed_cut(eng, "s", toks, cuts)
            eng.close_session("s")
            assert rel(got, ref) < TOL, cuts
    finally:
        eng.close()


def test_recurrent_branches_remember_a_far_write():
    """Slow decays (a decay of 0.9995 per step; forget gates pushed open; small step sizes): one marked token early in the
    sequence still shows 300 tokens later, across portions and decoded tokens."""
    def tweak(w):
        for k in list(w):
            if k.endswith("f.b"):
                w[k] = (w[k].float() + 8.0).to(torch.bfloat16)
            if k.endswith("dt_bias"):
                w[k] = (w[k].float() - 5.0).to(torch.bfloat16)
    layers = [layer(parallel(window(size=4), decaying(heads=2, dim=12, vdim=12, decay=(0.9995, 0.98)), 0.1, 1.5)), layer(memory()),
              layer(space())]
    spec, w = make(layers, seed=29, tweak=tweak)
    eng = engine(spec, w)
    try:
        toks = [3] * 340
        toks[5] = 77
        ref = oracle_logits(spec, w, toks)
        other = list(toks)
        other[5] = 78
        assert rel(oracle_logits(spec, w, other)[330:], ref[330:]) > 20 * TOL      # the write is still felt at the end
        got = feed_cut(eng, "a", toks, [40, 2, 100, 1, 1, 1, 150, 1])
        assert rel(got, ref) < TOL and rel(got[330:], ref[330:]) < TOL
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


# ------------------------------------------------------------------------------------------------ batches, pools
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
    left in its pages and its slot (states, running maxima, convolution tails) must not reach the next one."""
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


# ------------------------------------------------------------------------------------------------ tensor cores
TILING = [layer(space(heads=8, vdim=16, state=16, groups=2, norm_groups=2, conv=3), dense(ff=64)),
          layer(parallel(window(heads=4, kv_heads=2, dim=32, size=50, rot=(32, 1e4)), decaying(heads=4, dim=16, vdim=16, decay=(0.5, 0.8, 0.9, 0.99))),
                moe(ff=128, experts=4, top=2, scale=2.0, shared=64)),
          layer(memory(heads=2, dim=16, vdim=64), dense(ff=100))]


@pytest.mark.parametrize("exact", [False, True], ids=["tensor-cores", "exact-fp32"])
def test_projections_on_tensor_cores_and_in_exact_fp32(exact):
    """Shapes that tile (width, heads * vdim and the feed-forward sizes multiples of 64 or 128): with enough rows the input
    and output projections, the dense feed-forward, the shared expert and (from 256 (token, choice) pairs) the experts run
    on the tensor cores from bf16 hi + lo planes unless the engine was made exact; single tokens and short portions take the
    CUDA-core kernels either way, so the two forms must agree along one sequence.  The last layer's feed-forward (100) does
    not tile and stays on the CUDA cores."""
    spec, w = make(TILING, width=128, vocab=256, seed=37)
    eng = engine(spec, w, exact_f32=exact)
    try:
        toks = tokens_of(spec, 200, 38)
        ref = oracle_logits(spec, w, toks)
        got = feed_cut(eng, "a", toks, [150, 1, 1, 12, 3, 10, 1])
        assert rel(got, ref) < (TOL if exact else 4e-4)
    finally:
        eng.close()


# ------------------------------------------------------------------------------------------------ the serving path
def test_greedy_generation_through_the_scheduler():
    """Engine.generate: submit -> the scheduler's own chunked prefill and decode steps -> argmax sampling; three requests
    of unequal length run together, prompts longer than a step's token budget are cut by the scheduler itself."""
    spec, w = make(MIXED, seed=23)
    eng = engine(spec, w, max_batched_tokens=48, decode_prefill_cap=16)
    try:
        prompts = [tokens_of(spec, ln, 60 + i) for i, ln in enumerate([100, 7, 51])]
        n_new = 12
        got = eng.generate(prompts, n_new, temperature=0.0, ignore_eos=True)
        with torch.no_grad():
            for p, g in zip(prompts, got):
                assert g == O.greedy(spec.config(), w, p, n_new)
        # a conversation that continues keeps its state; one that diverges is rebuilt from its start
        eng.close()
        eng = engine(spec, w, max_batched_tokens=48, decode_prefill_cap=16)
        first = eng.generate([prompts[1]], 5, sessions=["gen-1"], temperature=0.0, ignore_eos=True)[0]
        more = prompts[1] + first + tokens_of(spec, 6, 99)
        with torch.no_grad():
            assert eng.generate([more], 4, sessions=["gen-1"], temperature=0.0, ignore_eos=True)[0] == O.greedy(spec.config(), w, more, 4)
            other = tokens_of(spec, 11, 98)
            assert eng.generate([other], 3, sessions=["gen-1"], temperature=0.0, ignore_eos=True)[0] == O.greedy(spec.config(), w, other, 3)
    finally:
        eng.close()


def test_sampling_with_temperature_runs():
    spec, w = make(MIXED, seed=25)
    eng = engine(spec, w)
    try:
        out = eng.generate([tokens_of(spec, 20, 1), tokens_of(spec, 5, 2)], 8, temperature=0.8, top_k=20, top_p=0.9,
                           ignore_eos=True)
        assert [len(o) for o in out] == [8, 8] and all(0 <= t < spec.vocab for o in out for t in o)
    finally:
        eng.close()


def test_trace_runner_replays_a_schedule(tmp_path):
    """bin/trace_run on a saved checkpoint: three steps, a session pausing and two ending, in both number formats."""
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
        tol = TOL if dtype == "float32" else 4e-4
        assert rel(a, ref[[0, 29]]) < tol and rel(c[0], ref[39]) < tol and rel(c[1], ref[4]) < tol


def test_served_through_the_handler(tmp_path, monkeypatch):
    """A Gedelorn checkpoint behind the serving path: FASTTALK_CHECKPOINT -> registry -> engine -> NativeHandler streams text."""
    from fasttalk_llm_microservice_b200.handler import NativeHandler, build_runner
    from fasttalk_llm_microservice_b200.layered import save_checkpoint
    spec, w = make([layer(space(), moe()), layer(parallel(), dense()), layer(memory())], width=64, vocab=600, seed=41)
    save_checkpoint(spec, w, str(tmp_path / "ckpt"))
    monkeypatch.setenv("FASTTALK_CHECKPOINT", str(tmp_path / "ckpt"))
    monkeypatch.setenv("FASTTALK_ALLOW_BYTE_TOKENIZER", "1")
    monkeypatch.setenv("FASTTALK_MAX_SESSIONS", "4")
    monkeypatch.setenv("FASTTALK_MAX_CONTEXT", "512")
    monkeypatch.setenv("FASTTALK_MAX_BATCHED_TOKENS", "256")
    runner = build_runner("gedelorn-test")
    h = NativeHandler(model="gedelorn-test", runner=runner)
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


# ------------------------------------------------------------------------------------------------ the rule alone
@pytest.mark.parametrize("lanes", [0, 4, 8, 16, 32])
@pytest.mark.parametrize("heads,qk_heads,dim,vd", [(3, 3, 20, 9), (4, 2, 64, 33), (2, 1, 128, 16), (1, 1, 7, 70)])
def test_decay_rule_kernel_alone(lanes, heads, qk_heads, dim, vd):
    """ft_decay_rule against the recurrence written out: three requests of unequal length in one launch, one of them
    continuing from a state that its slot already holds, every split of a column over lanes."""
    from fasttalk_llm_microservice_b200 import build, native
    build.build()
    lib = native.load()
    min_lanes = 4
    while min_lanes * 16 < dim and min_lanes < 32:      # runs of at most 16 channels per lane (32 beyond 512 channels)
        min_lanes *= 2
    if lanes and lanes < min_lanes:
        pytest.skip("fewer lanes than the channels need")
    g = torch.Generator().manual_seed(dim * 131 + vd)
    lens, pos0, slots = [37, 1, 90], [0, 5, 0], [2, 0, 1]
    T = sum(lens)
    q, k = torch.randn(T, qk_heads * dim, generator=g) * 0.3, torch.randn(T, qk_heads * dim, generator=g) * 0.3
    v = torch.randn(T, heads * vd, generator=g)
    ab = torch.stack([torch.rand(T, heads, generator=g) * 0.5 + 0.5, torch.rand(T, heads, generator=g) * 2.0], -1).contiguous()
    stride = heads * dim * vd + 4
    state = torch.randn(3 * stride, generator=g)
    ref_o = torch.zeros(T, heads * vd, dtype=torch.float64)
    ref_state = state.double().clone()
    start = [0, lens[0], lens[0] + lens[1], T]
    for r in range(3):
        for h in range(heads):
            S = ref_state[slots[r] * stride + h * dim * vd:][:dim * vd].reshape(dim, vd).clone()
            if pos0[r] == 0:
                S.zero_()
            gh = h // (heads // qk_heads)
            for t in range(start[r], start[r + 1]):
                S = ab[t, h, 0].double() * S + ab[t, h, 1].double() * torch.outer(k[t, gh * dim:(gh + 1) * dim].double(), v[t, h * vd:(h + 1) * vd].double())
                ref_o[t, h * vd:(h + 1) * vd] = S.T @ q[t, gh * dim:(gh + 1) * dim].double()
            ref_state[slots[r] * stride + h * dim * vd:][:dim * vd] = S.reshape(-1)
    dev = "cuda"
    dq, dk, dv, dab, dst = q.to(dev), k.to(dev), v.to(dev), ab.to(dev), state.to(dev)
    o = torch.zeros(T, heads * vd, device=dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    rs, rp, sl = i32(start), i32(pos0), i32(slots)
    rc = lib.ft_decay_rule(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dab.data_ptr(), o.data_ptr(), dst.data_ptr(), rs.data_ptr(),
                           rp.data_ptr(), sl.data_ptr(), 3, heads, qk_heads, dim, vd, stride, lanes, T, None)
    torch.cuda.synchronize()
    assert rc == 0, native.last_error()
    assert rel(o.cpu().double().numpy(), ref_o.numpy()) < 1e-5
    assert rel(dst.cpu().double().numpy(), ref_state.numpy()) < 1e-5
