"""CPU side of the layered model family: config <-> spec, checkpoint files, the packed layout, the family registry,
and properties of the plain restatement (oracle/gitozen_oracle.py) that the GPU tests lean on."""
import json
import os
import subprocess
import sys

import pytest
import torch

from fasttalk_llm_microservice_b200 import layered as LY
from fasttalk_llm_microservice_b200.registry import family_of, load_model
from oracle import gitozen_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def small_spec():
    layers = (LY.LayerSpec(mixer="channel_delta", heads=4, kv_heads=2, dim=8, vdim=12, conv=3, rank_a=5, rank_g=6,
                           ff=10, experts=6, top=2, groups=3, keep=2),
              LY.LayerSpec(mixer="latent_attention", heads=3, dim=8, vdim=4, kv_rank=10, scale=0.3))
    return LY.LayeredSpec(name="t", architecture="Gitozen", width=24, vocab=50, eps=1e-5, logit_softcap=8.0, layers=layers)


def test_config_roundtrip_and_shapes():
    spec = small_spec()
    cfg = spec.config()
    assert cfg["layers"][1]["mlp"] is None and cfg["layers"][0]["mlp"]["router"]["groups"] == {"count": 3, "keep": 2}
    shapes = LY.tensor_shapes(spec)
    again = LY.spec_from_config(json.loads(json.dumps(cfg)), shapes, name="t")
    assert again == spec
    assert shapes["l0.mix.a2"] == (32, 5) and shapes["l1.mix.uk"] == (24, 10) and shapes["l0.norm1"] == ()
    assert "l1.rg2" not in shapes and "l0.rg2.b" in shapes


def test_checkpoint_files_and_registry(tmp_path):
    spec = small_spec()
    w = LY.init_weights(spec, seed=1)
    LY.save_checkpoint(spec, w, str(tmp_path))
    with open(tmp_path / "config.json") as f:
        assert family_of(json.load(f)) == "layered"
    assert family_of({"model_type": "llama", "architectures": ["LlamaForCausalLM"]}) == "llama"
    with pytest.raises(ValueError):
        family_of({"model_type": "gpt2"})
    spec2, w2 = load_model(str(tmp_path), name="t")
    assert spec2 == spec and all(torch.equal(w[k], w2[k]) for k in w)
    bad = dict(w)
    bad["l0.mix.q"] = bad["l0.mix.q"][:-1]
    LY.save_checkpoint(spec, bad, str(tmp_path / "bad"))
    with pytest.raises(ValueError):
        LY.load_checkpoint(str(tmp_path / "bad"))


def test_packed_layout():
    spec = small_spec()
    w = LY.init_weights(spec, seed=2)
    model, keep = LY.pack(spec, w, "cpu")
    d0, d1 = model.layers[0], model.layers[1]
    assert model.n_layers == 2 and model.width == 24 and abs(model.logit_softcap - 8.0) < 1e-6
    # every part of the stacked input projection starts on a multiple of four rows and holds its tensor
    w_in0 = next(t for t in keep if isinstance(t, torch.Tensor) and t.data_ptr() == d0.w_in)
    for off in (d0.o_q, d0.o_beta, d0.o_a1, d0.o_g1, d0.o_rg1, d0.o_rg2, d0.o_router):
        assert off >= 0 and off % 4 == 0
    assert d0.o_k == d0.o_q + 16 and d0.o_v == d0.o_k + 16 and d0.o_dkv == -1
    assert torch.equal(w_in0[d0.o_k:d0.o_k + 16], w["l0.mix.k"]) and torch.equal(w_in0[d0.o_router:d0.o_router + 6], w["l0.mlp.router"])
    assert d1.ff_kind == LY.FF_NONE and d1.o_router == -1 and d1.o_rg2 == -1 and d1.o_gate >= 0
    gu = next(t for t in keep if isinstance(t, torch.Tensor) and t.data_ptr() == d0.w_gu)
    assert torch.equal(gu[3, 0::2], w["l0.mlp.e3.gate"]) and torch.equal(gu[3, 1::2], w["l0.mlp.e3.up"])
    uk = next(t for t in keep if isinstance(t, torch.Tensor) and t.data_ptr() == d1.w_uk_t)
    assert torch.equal(uk[2], w["l1.mix.uk"][16:24].T)


def test_oracle_is_causal_and_recurrent_state_is_what_carries_it():
    spec = small_spec()
    w = LY.init_weights(spec, seed=3)
    toks = torch.randint(0, spec.vocab, (30,)).tolist()
    with torch.no_grad():
        full = O.forward(spec.config(), w, toks)
        part = O.forward(spec.config(), w, toks[:17])
        assert torch.allclose(full[:17], part, atol=1e-5)
        changed = O.forward(spec.config(), w, [(toks[0] + 1) % spec.vocab] + toks[1:])
    assert (full[-1] - changed[-1]).abs().max() > 1e-4
    assert full.abs().max() <= spec.logit_softcap


def test_oracle_router_keeps_to_the_best_groups():
    h = torch.randn(64, 24)
    router = torch.randn(12, 24)
    idx, wt = O.route(h, router, {"experts": 12, "top": 3, "groups": {"count": 4, "keep": 2}})
    s = torch.softmax(h @ router.T, -1)
    best = s.reshape(64, 4, 3).amax(-1).topk(2, -1).indices
    for t in range(64):
        assert all(int(e) // 3 in best[t].tolist() for e in idx[t])
        assert torch.allclose(wt[t], s[t, idx[t]])
    assert (wt.sum(-1) < 1.0).all()          # the weights are the scores themselves, not renormalised


def test_trace_runner_is_an_executable_with_help():
    path = os.path.join(ROOT, "bin", "trace_run")
    assert os.access(path, os.X_OK)
    r = subprocess.run([sys.executable, path, "--help"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "--max-tokens" in r.stdout
