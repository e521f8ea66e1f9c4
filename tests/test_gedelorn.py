"""CPU side of the Gedelorn design: config <-> spec, checkpoint files, the family registry, the packed descriptors, and
properties of the plain restatement (oracle/gedelorn_oracle.py) that the GPU tests lean on."""
import json

import pytest
import torch

from fasttalk_llm_microservice_b200 import layered as LY
from fasttalk_llm_microservice_b200.registry import family_of, load_model
from oracle import gedelorn_oracle as O


def small_config():
    return {"architecture": "Gedelorn", "norm": {"eps": 1e-5}, "vocab": 50, "width": 24, "layers": [
        {"type": "mamba2", "mixer": {"conv": 3, "groups": 2, "heads": 4, "norm_groups": 4, "state": 6, "vdim": 5},
         "mlp": {"ff": 20, "kind": "dense"}},
        {"type": "parallel", "mixer": {
            "left": {"dim": 6, "heads": 4, "kv_heads": 2, "mask": {"size": 7}, "rot": {"base": 100.0, "dims": 4},
                     "scale": 0.4, "softcap": 20.0, "vdim": 6},
            "left_scale": 0.5, "right": {"decay": [0.9, 0.99], "dim": 5, "heads": 2, "vdim": 7}, "right_scale": 2.0},
         "mlp": {"expert": {"ff": 9}, "kind": "moe", "router": {"experts": 5, "scale": 1.5, "top": 2}, "shared": {"ff": 11}}},
        {"type": "mlstm", "mixer": {"dim": 4, "gate_cap": 10.0, "heads": 3, "vdim": 6}, "mlp": None}]}


def test_config_roundtrip_and_shapes():
    cfg = small_config()
    spec = LY.spec_from_config(cfg, name="t")
    assert spec.config() == cfg
    assert [l.form for l in spec.layers] == ["sandwich"] * 3
    assert [b.kind for l in spec.layers for b in l.branches] == ["state_space", "window_attention", "decay_attention", "matrix_memory"]
    shapes = LY.tensor_shapes(spec)
    assert shapes["l0.mix.in"] == (2 * 20 + 2 * 12 + 4, 24) and shapes["l0.mix.conv"] == (44, 3) and shapes["l0.norm2b"] == (24,)
    assert shapes["l1.mix.left.k.b"] == (12,) and shapes["l1.mix.right.g"] == (14, 24) and "l1.mix.left.v" not in shapes
    assert shapes["l1.mlp.e4.up"] == (9, 24) and "l1.mlp.e0.gate" not in shapes and shapes["l1.mlp.shared.down"] == (24, 11)
    assert shapes["l2.mix.f.b"] == (3,) and "l2.norm2" not in shapes and shapes["final.norm"] == (24,)
    with pytest.raises(ValueError):
        bad = small_config()
        bad["layers"][1]["mixer"]["right"]["decay"] = [0.5]
        LY.spec_from_config(bad)


def test_checkpoint_files_and_registry(tmp_path):
    spec = LY.spec_from_config(small_config(), name="t")
    w = LY.init_weights(spec, seed=1)
    LY.save_checkpoint(spec, w, str(tmp_path))
    with open(tmp_path / "config.json") as f:
        assert family_of(json.load(f)) == "layered"
    spec2, w2 = load_model(str(tmp_path), name="t")
    assert spec2 == spec and all(torch.equal(w[k], w2[k]) for k in w)
    bad = dict(w)
    del bad["l1.mix.left.q.b"]
    LY.save_checkpoint(spec, bad, str(tmp_path / "bad"))
    with pytest.raises(KeyError):
        LY.load_checkpoint(str(tmp_path / "bad"))


def test_packed_descriptors():
    spec = LY.spec_from_config(small_config(), name="t")
    w = LY.init_weights(spec, seed=2)
    model, keep = LY.pack(spec, w, "cpu")
    by_ptr = {t.data_ptr(): t for t in keep if isinstance(t, torch.Tensor)}
    assert model.n_layers == 3 and model.final_norm_w and torch.equal(by_ptr[model.final_norm_w], 1.0 + w["final.norm"].float())
    d0, d1, d2 = (model.layers[i] for i in range(3))
    assert all(d.form == LY.LAYER_SANDWICH and d.mixer == LY.MIXER_BRANCHES for d in (d0, d1, d2))
    assert torch.equal(by_ptr[d0.norm_post1], 1.0 + w["l0.norm1b"].float()) and not d2.norm_pre2
    s = d0.branch[0]                                   # z | x | B | C | dt of the state space, where the checkpoint has them
    assert (d0.n_branches, s.kind, s.kv_heads, s.dim, s.vdim) == (1, LY.BRANCH_STATE_SPACE, 2, 6, 5)
    assert (s.o_v - s.o_z, s.o_k - s.o_v, s.o_q - s.o_k, s.o_dt - s.o_q) == (20, 20, 12, 12)
    assert torch.equal(by_ptr[d0.w_in][s.o_z:s.o_z + 68], w["l0.mix.in"]) and d0.n_in % 128 == 0
    assert d0.ff_kind == LY.FF_DENSE and torch.equal(by_ptr[d0.w_gu][0::2], w["l0.mlp.gate"]) and torch.equal(by_ptr[d0.w_gu][1::2], w["l0.mlp.up"])
    a, r = d1.branch[0], d1.branch[1]
    assert (d1.n_branches, a.kind, r.kind) == (2, LY.BRANCH_WINDOW_ATTENTION, LY.BRANCH_DECAY_ATTENTION)
    assert (a.window, a.rot_dims, a.o_v) == (7, 4, -1) and abs(a.out_scale - 0.5) < 1e-7 and abs(r.out_scale - 2.0) < 1e-7
    freq = by_ptr[a.rot_freq]
    assert torch.allclose(freq, torch.tensor([1.0, 0.1])) and freq.dtype == torch.float32
    assert r.o_k == r.o_q + 10 and r.o_v == r.o_k + 10 and r.o_q % 4 == 0 and r.o_g % 4 == 0
    assert torch.equal(by_ptr[d1.w_in][r.o_v:r.o_v + 14], w["l1.mix.right.v"]) and torch.equal(by_ptr[d1.w_in][a.o_k:a.o_k + 12], w["l1.mix.left.k"])
    assert (d1.ff_kind, d1.ff_act, d1.route_kind, d1.route_norm, d1.experts, d1.top, d1.shared_ff) == (LY.FF_MOE, LY.ACT_RELU2, LY.ROUTE_SIGMOID, 1, 5, 2, 11)
    assert torch.equal(by_ptr[d1.w_gu][3], w["l1.mlp.e3.up"]) and torch.equal(by_ptr[d1.w_down][4], w["l1.mlp.e4.down"])
    m = d2.branch[0]
    assert m.kind == LY.BRANCH_MATRIX_MEMORY and d2.ff_kind == LY.FF_NONE and abs(m.gate_cap - 10.0) < 1e-6
    assert torch.equal(by_ptr[m.gate_bias], torch.cat([w["l2.mix.i.b"], w["l2.mix.f.b"]]).float())


def test_oracle_is_causal_and_the_window_hides_what_lies_before_it():
    cfg = small_config()
    spec = LY.spec_from_config(cfg, name="t")
    w = LY.init_weights(spec, seed=3)
    toks = torch.randint(0, spec.vocab, (30,)).tolist()
    with torch.no_grad():
        full = O.forward(cfg, w, toks)
        assert torch.allclose(full[:17], O.forward(cfg, w, toks[:17]), atol=1e-9)
        changed = O.forward(cfg, w, [(toks[0] + 1) % spec.vocab] + toks[1:])
        assert (full[-1] - changed[-1]).abs().max() > 1e-6          # the recurrent layers carry the first token to the end
        # the attention alone: a model of one parallel layer whose right branch is switched off
        only = {**cfg, "layers": [{**cfg["layers"][1], "mlp": None}]}
        only["layers"][0]["mixer"] = {**only["layers"][0]["mixer"], "right_scale": 0.0}
        w1 = LY.init_weights(LY.spec_from_config(only), seed=4)
        a = O.forward(only, w1, toks)
        b = O.forward(only, w1, [(toks[0] + 1) % spec.vocab] + toks[1:])
        assert (a[6] - b[6]).abs().max() > 1e-6 and (a[7:] - b[7:]).abs().max() == 0          # window 7: positions 0..6 see token 0


def test_oracle_router_weights():
    h = torch.randn(64, 24, dtype=torch.float64)
    router = torch.randn(12, 24, dtype=torch.float64)
    idx, wt = O.route(h, router, 4, 2.5)
    s = torch.sigmoid(h @ router.T)
    assert torch.equal(idx.sort(-1).values, s.topk(4, -1).indices.sort(-1).values)
    assert torch.allclose(wt.sum(-1), torch.full((64,), 2.5, dtype=torch.float64))
    assert torch.allclose(wt / wt.sum(-1, keepdim=True), s.gather(1, idx) / s.gather(1, idx).sum(-1, keepdim=True))


def test_oracle_state_space_convolution_and_memory_gates():
    u = torch.randn(9, 3, dtype=torch.float64)
    taps, bias = torch.randn(3, 4, dtype=torch.float64), torch.randn(3, dtype=torch.float64)
    y = O.causal_conv(u, taps, bias)
    assert torch.allclose(y[0], bias + taps[:, 3] * u[0])                          # zeros before the start
    assert torch.allclose(y[5], bias + sum(taps[:, 3 - j] * u[5 - j] for j in range(4)))
    z = torch.linspace(-40, 40, 9, dtype=torch.float64)
    assert torch.allclose(O.logsigmoid(z), torch.nn.functional.logsigmoid(z)) and torch.allclose(O.softplus(z), torch.nn.functional.softplus(z))
