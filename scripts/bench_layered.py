"""Prefill and decode throughput of the layered family (Gitozen) beside the closest Llama of equal size, random weights.

    python bench.py --design gitozen [--sizes s,m] [--steps K] [--warmup W]

For every size both models get the same width, depth, heads x head size, active feed-forward width (top x expert ff =
Llama's ffn) and vocabulary.  Each arm is driven through Engine.feed (ft_engine_feed: the engine's own batch builder and
forward pass, nothing sampled), timed with CUDA events on the engine's stream; a 512 MB write between timed steps
flushes L2.
  prefill  one fresh session, PREFILL tokens in one step
  decode   DECODE_SESSIONS sessions at context DECODE_CTX, one token each per step
One JSON line: per size and arm tok/s and ms per step; the Llama arm is the comparator, not a baseline of the reference.
"""
from __future__ import annotations

import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PREFILL = 2048
DECODE_SESSIONS = 16
DECODE_CTX = 1024

# name -> width, layers (mixer order), heads, head size, latent size, experts, top, expert ff, vocab
SIZES = {
    "s": dict(width=1024, order="ladl", heads=8, dim=128, kv_rank=128, experts=8, top=2, ff=512, vocab=16384),
    "m": dict(width=2048, order="ladl", heads=16, dim=128, kv_rank=256, experts=16, top=2, ff=1024, vocab=32768),
}


def gitozen_spec(name, c):
    from fasttalk_llm_microservice_b200.layered import LayeredSpec, LayerSpec
    moe = dict(ff=c["ff"], experts=c["experts"], top=c["top"], groups=4, keep=2)
    layers = []
    for k in c["order"]:
        if k == "l":
            layers.append(LayerSpec(mixer="latent_attention", heads=c["heads"], dim=c["dim"], vdim=c["dim"],
                                    kv_rank=c["kv_rank"], scale=c["dim"] ** -0.5, **moe))
        else:
            layers.append(LayerSpec(mixer="channel_delta", heads=c["heads"], kv_heads=c["heads"], dim=c["dim"], vdim=c["dim"],
                                    conv=4, rank_a=64, rank_g=64, **moe))
    return LayeredSpec(name=f"gitozen-{name}", architecture="Gitozen", width=c["width"], vocab=c["vocab"], eps=1e-6,
                       logit_softcap=30.0, layers=tuple(layers))


def llama_spec(name, c):
    from fasttalk_llm_microservice_b200.model_spec import ModelSpec
    return ModelSpec(name=f"llama-{name}", hidden=c["width"], ffn=c["top"] * c["ff"], layers=len(c["order"]),
                     n_q_heads=c["heads"], n_kv_heads=max(1, c["heads"] // 4), head_dim=c["dim"], vocab=c["vocab"],
                     tied_embeddings=False)


def measure(eng, vocab, steps, warmup):
    import numpy as np
    import torch
    rng = np.random.default_rng(0)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn):
        flush.zero_()
        torch.cuda.synchronize()
        eng.timer_start()
        fn()
        return eng.timer_stop_ms()

    out = {}
    ms = []
    for i in range(warmup + steps):
        toks = rng.integers(0, vocab, PREFILL).tolist()
        t = timed(lambda: eng.feed([("p", toks, [PREFILL - 1])]))
        eng.close_session("p")
        if i >= warmup:
            ms.append(t)
    out["prefill"] = {"tokens": PREFILL, "ms_per_step": sum(ms) / len(ms), "tok_s": PREFILL * len(ms) / (sum(ms) / 1e3)}
    names = [f"d{i}" for i in range(DECODE_SESSIONS)]
    for n in names:
        eng.feed([(n, rng.integers(0, vocab, DECODE_CTX).tolist(), [])])
    ms = []
    for i in range(warmup + steps):
        entries = [(n, [int(rng.integers(0, vocab))], [0]) for n in names]
        t = timed(lambda: eng.feed(entries))
        if i >= warmup:
            ms.append(t)
    for n in names:
        eng.close_session(n)
    out["decode"] = {"sessions": DECODE_SESSIONS, "context": DECODE_CTX, "ms_per_step": sum(ms) / len(ms),
                     "tok_s": DECODE_SESSIONS * len(ms) / (sum(ms) / 1e3)}
    return out


def run(args) -> None:
    import torch
    from fasttalk_llm_microservice_b200 import build
    from fasttalk_llm_microservice_b200.engine import Engine, EngineLimits
    from fasttalk_llm_microservice_b200.layered import init_weights as init_layered
    from fasttalk_llm_microservice_b200.weights import init_weights as init_llama
    build.build()
    torch.cuda.set_device(0)
    steps, warmup = max(1, min(args.steps, 20)), max(3, min(args.warmup, 5))
    lim = dict(max_batch=DECODE_SESSIONS, max_batched_tokens=PREFILL, max_context=PREFILL + 64, max_sessions=DECODE_SESSIONS + 1,
               num_pages=(DECODE_SESSIONS + 2) * (PREFILL // 64 + 1), debug_logit_rows=DECODE_SESSIONS)
    sizes = {}
    only = [s for s in (getattr(args, "sizes", "") or "s,m").split(",") if s]
    for name in only:
        c = SIZES[name]
        row = {"config": c}
        for arm in (getattr(args, "arms", "") or "gitozen,llama").split(","):
            if arm == "gitozen":
                spec = gitozen_spec(name, c)
                w = init_layered(spec, seed=0, device="cuda")
            else:
                spec = llama_spec(name, c)
                w = init_llama(spec, seed=0, device="cuda")
            eng = Engine(spec, w, EngineLimits(**lim), eos_ids=())
            row[arm] = measure(eng, c["vocab"], steps, warmup)
            row[arm]["kernel_launches"] = eng.stats()["kernel_launches"]
            eng.close()
            del eng, w
            torch.cuda.empty_cache()
        sizes[name] = row
    print(json.dumps({"metric": "prefill / decode tok/s, Gitozen beside the closest Llama of equal size", "design": "gitozen",
                      "dtype": "bf16 weights; Gitozen: fp32 activations, bf16 hi+lo planes on the tensor-core projections",
                      "data": "synthetic (random-init weights, random tokens)", "steps": steps, "warmup": warmup,
                      "l2": "512 MB write between timed steps", "sizes": sizes}), flush=True)
