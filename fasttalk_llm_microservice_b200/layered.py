"""Layered models: decoders that config.json describes layer by layer (ft_layer_desc in include/fasttalk_b200.h).

The first design of this family is Gitozen: parallel layers (mixer and feed-forward read one scalar-gain RMS norm and are
added through element-wise sigmoid gates), two token mixers — latent attention without positions, whose cache holds one
normed latent per token, and a gated delta rule with one decay per head and key channel, whose state lives in a
per-session slot — a mixture of experts with group-limited routing, and tanh-capped logits.

The reference names models by tag only and owns no model code (app/utils/config.py:86, docker-compose.vllm.yml:39); this
module is the model side of what its engine container would load: config.json -> LayeredSpec, model.safetensors -> the
tensors by their names in the file, pack() -> the device arrays and descriptors the native engine reads.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

MIXER_LATENT_ATTENTION, MIXER_CHANNEL_DELTA = 1, 2
FF_NONE, FF_MOE = 0, 1
MIXERS = {"latent_attention": MIXER_LATENT_ATTENTION, "channel_delta": MIXER_CHANNEL_DELTA}


@dataclass(frozen=True)
class LayerSpec:
    mixer: str                      # "latent_attention" | "channel_delta"
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0               # channel_delta
    conv: int = 0                   # channel_delta: taps
    rank_a: int = 0                 # channel_delta: inner size of the decay projection (from the tensor's shape)
    rank_g: int = 0                 # channel_delta: inner size of the gate projection
    kv_rank: int = 0                # latent_attention
    scale: float = 0.0              # latent_attention
    ff: int = 0                     # 0 = the layer has no feed-forward
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1


@dataclass(frozen=True)
class LayeredSpec:
    name: str
    architecture: str
    width: int
    vocab: int
    eps: float
    logit_softcap: float
    layers: Tuple[LayerSpec, ...] = field(default_factory=tuple)

    # the attributes the serving code reads from any model spec
    @property
    def hidden(self) -> int:
        return self.width

    def config(self) -> Dict:
        """The config.json of this spec."""
        out = []
        for l in self.layers:
            if l.mixer == "latent_attention":
                mixer = {"dim": l.dim, "heads": l.heads, "kv_rank": l.kv_rank, "scale": l.scale, "vdim": l.vdim}
            else:
                mixer = {"conv": l.conv, "dim": l.dim, "heads": l.heads, "kv_heads": l.kv_heads, "vdim": l.vdim}
            mlp = None
            if l.ff:
                mlp = {"expert": {"ff": l.ff}, "kind": "moe",
                       "router": {"experts": l.experts, "groups": {"count": l.groups, "keep": l.keep}, "top": l.top}}
            out.append({"mixer": mixer, "mlp": mlp, "type": l.mixer})
        return {"architecture": self.architecture, "layers": out, "logit_softcap": self.logit_softcap,
                "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}


def spec_from_config(cfg: Dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None, name: str = "checkpoint") -> LayeredSpec:
    """config.json (+ tensor shapes, for the sizes only a shape gives) -> LayeredSpec."""
    layers = []
    for i, l in enumerate(cfg["layers"]):
        kind, m = l["type"], l["mixer"]
        if kind not in MIXERS:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        kw = dict(mixer=kind, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]))
        if kind == "latent_attention":
            kw.update(kv_rank=int(m["kv_rank"]), scale=float(m["scale"]))
        else:
            kw.update(kv_heads=int(m.get("kv_heads", m["heads"])), conv=int(m["conv"]))
            if shapes is not None:
                kw.update(rank_a=int(shapes[f"l{i}.mix.a1"][0]), rank_g=int(shapes[f"l{i}.mix.g1"][0]))
            else:
                kw.update(rank_a=int(m.get("rank_a", 0)), rank_g=int(m.get("rank_g", 0)))
        mlp = l.get("mlp")
        if mlp:
            if mlp.get("kind", "moe") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            r = mlp["router"]
            g = r.get("groups") or {}
            kw.update(ff=int(mlp["expert"]["ff"]), experts=int(r["experts"]), top=int(r["top"]),
                      groups=int(g.get("count", 1)), keep=int(g.get("keep", g.get("count", 1))))
        layers.append(LayerSpec(**kw))
    cap = cfg.get("logit_softcap")
    return LayeredSpec(name=name, architecture=str(cfg.get("architecture", "Gitozen")), width=int(cfg["width"]),
                       vocab=int(cfg["vocab"]), eps=float(cfg["norm"]["eps"]), logit_softcap=float(cap) if cap else 0.0,
                       layers=tuple(layers))


def tensor_shapes(spec: LayeredSpec) -> Dict[str, Tuple[int, ...]]:
    """Names and shapes of a checkpoint of this spec."""
    W = spec.width
    out: Dict[str, Tuple[int, ...]] = {"embed": (spec.vocab, W)}
    for i, l in enumerate(spec.layers):
        p = f"l{i}."
        out[p + "norm1"] = ()
        if l.mixer == "latent_attention":
            out.update({p + "mix.q": (l.heads * l.dim, W), p + "mix.dkv": (l.kv_rank, W), p + "mix.dkv.norm": (l.kv_rank,),
                        p + "mix.uk": (l.heads * l.dim, l.kv_rank), p + "mix.uv": (l.heads * l.vdim, l.kv_rank),
                        p + "mix.g": (l.heads, W), p + "mix.o": (W, l.heads * l.vdim)})
        else:
            qk, hv = l.kv_heads * l.dim, l.heads * l.vdim
            out.update({p + "mix.q": (qk, W), p + "mix.q.conv": (qk, l.conv), p + "mix.k": (qk, W),
                        p + "mix.k.conv": (qk, l.conv), p + "mix.v": (hv, W), p + "mix.v.conv": (hv, l.conv),
                        p + "mix.b": (l.heads, W), p + "mix.A_log": (l.heads,), p + "mix.norm": (l.vdim,),
                        p + "mix.a1": (l.rank_a, W), p + "mix.a2": (l.heads * l.dim, l.rank_a),
                        p + "mix.dt_bias": (l.heads * l.dim,), p + "mix.g1": (l.rank_g, W),
                        p + "mix.g2": (hv, l.rank_g), p + "mix.o": (W, hv)})
        if l.ff:
            for e in range(l.experts):
                out.update({f"{p}mlp.e{e}.gate": (l.ff, W), f"{p}mlp.e{e}.up": (l.ff, W), f"{p}mlp.e{e}.down": (W, l.ff)})
            out[p + "mlp.router"] = (l.experts, W)
            out.update({p + "rg2": (W, W), p + "rg2.b": (W,)})
        out.update({p + "rg1": (W, W), p + "rg1.b": (W,)})
    out["final.norm"] = ()
    out["head"] = (spec.vocab, W)
    return out


def init_weights(spec: LayeredSpec, seed: int = 0, device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Deterministic random bf16 tensors under the checkpoint's names: projections ~ N(0, 1/fan_in), gains near 1, decay
    parameters in the range where the recurrence neither forgets at once nor never."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(spec).items():
        leaf = name.split(".")[-1]
        if name.endswith("norm1") or name == "final.norm" or name.endswith(".norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "A_log":
            t = torch.log(0.5 + 2.0 * torch.rand(shape, generator=g))
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=g) - 2.0
        elif leaf == "b" and name.split(".")[-2] in ("rg1", "rg2"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) * 0.5
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / (shape[-1] ** 0.5)
        w[name] = t.to(torch.bfloat16).to(device)
    return w


def read_safetensors_header(path: str) -> Dict:
    with open(path, "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        return json.loads(f.read(n))


def is_layered_config(cfg: Dict) -> bool:
    return isinstance(cfg.get("layers"), list) and "width" in cfg


def load_checkpoint(path: str, device: str = "cpu", name: Optional[str] = None) -> Tuple[LayeredSpec, Dict[str, torch.Tensor]]:
    """A folder with config.json and model.safetensors -> (spec, tensors by name)."""
    from safetensors.torch import load_file
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    st = os.path.join(path, "model.safetensors")
    shapes = {k: tuple(v["shape"]) for k, v in read_safetensors_header(st).items() if k != "__metadata__"}
    spec = spec_from_config(cfg, shapes, name or os.path.basename(os.path.normpath(path)))
    w = load_file(st, device=device)
    want = tensor_shapes(spec)
    for k, shape in want.items():
        if k not in w:
            raise KeyError(f"checkpoint has no tensor {k!r}")
        if tuple(w[k].shape) != tuple(shape):
            raise ValueError(f"{k}: shape {tuple(w[k].shape)} does not match config ({tuple(shape)})")
    return spec, w


def save_checkpoint(spec: LayeredSpec, w: Dict[str, torch.Tensor], path: str) -> None:
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(spec.config(), f, indent=1)
    save_file({k: v.detach().cpu().contiguous() for k, v in w.items()}, os.path.join(path, "model.safetensors"))


# ------------------------------------------------------------------ native side
class LayerDesc(C.Structure):
    """ft_layer_desc (include/fasttalk_b200.h)."""
    _fields_ = [
        ("mixer", C.c_int), ("heads", C.c_int), ("kv_heads", C.c_int), ("dim", C.c_int), ("vdim", C.c_int),
        ("kv_rank", C.c_int), ("scale", C.c_float), ("conv", C.c_int), ("rank_a", C.c_int), ("rank_g", C.c_int),
        ("ff_kind", C.c_int), ("experts", C.c_int), ("top", C.c_int), ("groups", C.c_int), ("keep", C.c_int),
        ("ff", C.c_int), ("n_in", C.c_int),
        ("o_q", C.c_int), ("o_k", C.c_int), ("o_v", C.c_int), ("o_dkv", C.c_int), ("o_gate", C.c_int),
        ("o_beta", C.c_int), ("o_a1", C.c_int), ("o_g1", C.c_int), ("o_rg1", C.c_int), ("o_rg2", C.c_int),
        ("o_router", C.c_int), ("norm_gain", C.c_float),
        ("w_in", C.c_void_p), ("w_o", C.c_void_p), ("rg_bias", C.c_void_p),
        ("w_uk_t", C.c_void_p), ("w_uv", C.c_void_p), ("dkv_norm", C.c_void_p),
        ("conv_w", C.c_void_p), ("w_a2", C.c_void_p), ("w_g2", C.c_void_p), ("dt_bias", C.c_void_p),
        ("a_log", C.c_void_p), ("out_norm", C.c_void_p),
        ("w_gu", C.c_void_p), ("w_down", C.c_void_p),
    ]


class LayeredModel(C.Structure):
    """ft_layered_model (include/fasttalk_b200.h)."""
    _fields_ = [
        ("width", C.c_int), ("vocab", C.c_int), ("n_layers", C.c_int),
        ("eps", C.c_float), ("logit_softcap", C.c_float), ("final_norm_gain", C.c_float),
        ("embed", C.c_void_p), ("head", C.c_void_p), ("layers", C.POINTER(LayerDesc)), ("exact_f32", C.c_int),
    ]


def _stack_inputs(parts: List[Tuple[str, torch.Tensor]], width: int, device) -> Tuple[torch.Tensor, Dict[str, int]]:
    """Projections that read the same input, one under the other; every part starts on a multiple of four rows (the
    kernels read its output columns four at a time) and the whole is a multiple of 128 rows (the tensor-core GEMM's
    tile); the gaps are zero rows."""
    offs, rows = {}, 0
    for name, t in parts:
        rows = (rows + 3) & ~3
        offs[name] = rows
        rows += t.shape[0]
    rows = (rows + 127) & ~127
    out = torch.zeros(rows, width, dtype=torch.bfloat16, device=device)
    for name, t in parts:
        out[offs[name]:offs[name] + t.shape[0]] = t
    return out, offs


def pack(spec: LayeredSpec, w: Dict[str, torch.Tensor], device, exact_f32: bool = False) -> Tuple[LayeredModel, list]:
    """Device arrays in the engine's layout + the descriptor structs.  Returns (model, keepalive): the engine borrows
    the pointers, so `keepalive` has to live as long as the engine."""
    keep: list = []
    bf = torch.bfloat16

    def dev(t: torch.Tensor, dtype=bf) -> torch.Tensor:
        t = t.to(device=device, dtype=dtype).contiguous()
        keep.append(t)
        return t

    descs = (LayerDesc * len(spec.layers))()
    W = spec.width
    for i, l in enumerate(spec.layers):
        p, d = f"l{i}.", descs[i]
        m = p + "mix."
        d.mixer, d.heads, d.dim, d.vdim = MIXERS[l.mixer], l.heads, l.dim, l.vdim
        d.norm_gain = float(w[p + "norm1"].float().item())
        for f_ in ("o_q", "o_k", "o_v", "o_dkv", "o_gate", "o_beta", "o_a1", "o_g1", "o_rg1", "o_rg2", "o_router"):
            setattr(d, f_, -1)
        if l.mixer == "latent_attention":
            parts = [("q", w[m + "q"]), ("dkv", w[m + "dkv"]), ("gate", w[m + "g"])]
        else:
            # q | k | v stay adjacent: the convolution kernel addresses them as one run of channels
            qkv = torch.cat([w[m + "q"], w[m + "k"], w[m + "v"]], 0)
            parts = [("q", qkv), ("beta", w[m + "b"]), ("a1", w[m + "a1"]), ("g1", w[m + "g1"])]
        parts.append(("rg1", w[p + "rg1"]))
        if l.ff:
            parts += [("rg2", w[p + "rg2"]), ("router", w[p + "mlp.router"])]
        w_in, offs = _stack_inputs([(n, t.to(device)) for n, t in parts], W, device)
        keep.append(w_in)
        d.w_in, d.n_in = w_in.data_ptr(), w_in.shape[0]
        for n, o in offs.items():
            setattr(d, "o_" + n, o)
        d.w_o = dev(w[m + "o"]).data_ptr()
        bias = [w[p + "rg1.b"].float(), w[p + "rg2.b"].float() if l.ff else torch.zeros(W)]
        d.rg_bias = dev(torch.cat([b.to("cpu") for b in bias]), torch.float32).data_ptr()
        if l.mixer == "latent_attention":
            d.kv_rank, d.scale = l.kv_rank, l.scale
            uk = w[m + "uk"].reshape(l.heads, l.dim, l.kv_rank).transpose(1, 2)      # [heads][kv_rank][dim]
            d.w_uk_t = dev(uk).data_ptr()
            d.w_uv = dev(w[m + "uv"]).data_ptr()
            d.dkv_norm = dev(w[m + "dkv.norm"], torch.float32).data_ptr()
        else:
            d.kv_heads, d.conv, d.rank_a, d.rank_g = l.kv_heads, l.conv, l.rank_a, l.rank_g
            d.o_k = d.o_q + l.kv_heads * l.dim
            d.o_v = d.o_k + l.kv_heads * l.dim
            conv = torch.cat([w[m + "q.conv"], w[m + "k.conv"], w[m + "v.conv"]], 0)
            d.conv_w = dev(conv, torch.float32).data_ptr()
            d.w_a2 = dev(w[m + "a2"]).data_ptr()
            d.w_g2 = dev(w[m + "g2"]).data_ptr()
            d.dt_bias = dev(w[m + "dt_bias"], torch.float32).data_ptr()
            d.a_log = dev(w[m + "A_log"], torch.float32).data_ptr()
            d.out_norm = dev(w[m + "norm"], torch.float32).data_ptr()
        if l.ff:
            d.ff_kind, d.experts, d.top, d.groups, d.keep, d.ff = FF_MOE, l.experts, l.top, l.groups, l.keep, l.ff
            gu = torch.empty(l.experts, 2 * l.ff, W, dtype=bf, device=device)
            dn = torch.empty(l.experts, W, l.ff, dtype=bf, device=device)
            for e in range(l.experts):
                gu[e, 0::2] = w[f"{p}mlp.e{e}.gate"].to(device)
                gu[e, 1::2] = w[f"{p}mlp.e{e}.up"].to(device)
                dn[e] = w[f"{p}mlp.e{e}.down"].to(device)
            keep += [gu, dn]
            d.w_gu, d.w_down = gu.data_ptr(), dn.data_ptr()
        else:
            d.ff_kind = FF_NONE
    model = LayeredModel()
    model.width, model.vocab, model.n_layers = W, spec.vocab, len(spec.layers)
    model.eps, model.logit_softcap = spec.eps, spec.logit_softcap
    model.final_norm_gain = float(w["final.norm"].float().item())
    model.embed = dev(w["embed"]).data_ptr()
    model.head = dev(w["head"]).data_ptr()
    model.layers = C.cast(descs, C.POINTER(LayerDesc))
    model.exact_f32 = int(exact_f32)
    keep.append(descs)
    return model, keep
