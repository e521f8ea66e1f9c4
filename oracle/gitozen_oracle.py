"""Plain fp32 restatement of the Gitozen decoder, one function per mechanism, token by token where the
mechanism is a recurrence.  It is slow on purpose: no cache, no batching, no shared code with the engine.

A model is described by a dict `cfg` (the keys of the model's config.json) and a dict `w` of tensors named
as in its safetensors file.  Everything is computed in float32 on the CPU.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float32


def _f(t: torch.Tensor) -> torch.Tensor:
    return t.to(F)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose gain is one number for all coordinates."""
    return rms_unit(x, eps) * _f(g).reshape(())


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K] with the last column acting on the current token; zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    out = torch.zeros(T, C, dtype=F)
    for t in range(T):
        for j in range(K):
            s = t - (K - 1 - j)
            if s >= 0:
                out[t] += _f(taps[:, j]) * x[s]
    return out


def channel_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """Gated delta rule with one decay per head and key channel.  h [T, width] -> [T, width]."""
    T = h.shape[0]
    H, KH, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ _f(w[p + "q"]).T, w[p + "q.conv"])).reshape(T, KH, D)
    k = silu(causal_conv(h @ _f(w[p + "k"]).T, w[p + "k.conv"])).reshape(T, KH, D)
    v = silu(causal_conv(h @ _f(w[p + "v"]).T, w[p + "v.conv"])).reshape(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ _f(w[p + "b"]).T)                                   # [T, H]
    a = (h @ _f(w[p + "a1"]).T) @ _f(w[p + "a2"]).T + _f(w[p + "dt_bias"])       # [T, H*D]
    decay = torch.exp(-torch.exp(_f(w[p + "A_log"]))[None, :, None] * torch.nn.functional.softplus(a).reshape(T, H, D))
    gate = torch.sigmoid((h @ _f(w[p + "g1"]).T) @ _f(w[p + "g2"]).T).reshape(T, H, V)
    S = torch.zeros(H, D, V, dtype=F)
    out = torch.zeros(T, H, V, dtype=F)
    rep = H // KH
    for t in range(T):
        for hh in range(H):
            kk, qq = k[t, hh // rep], q[t, hh // rep]
            S[hh] = decay[t, hh][:, None] * S[hh]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ kk)
            S[hh] = S[hh] + torch.outer(kk, u)
            out[t, hh] = S[hh].T @ qq
    out = rms_unit(out, eps) * _f(w[p + "norm"]) * gate
    return out.reshape(T, H * V) @ _f(w[p + "o"]).T


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """Causal softmax attention whose keys and values are expanded from one cached latent per token."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ _f(w[p + "q"]).T).reshape(T, H, D)
    c = rms_unit(h @ _f(w[p + "dkv"]).T, eps) * _f(w[p + "dkv.norm"])
    k = (c @ _f(w[p + "uk"]).T).reshape(T, H, D)
    v = (c @ _f(w[p + "uv"]).T).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        s = torch.einsum("hd,jhd->hj", q[t], k[: t + 1]) * float(m["scale"])
        a = torch.softmax(s, dim=-1)
        out[t] = torch.einsum("hj,jhv->hv", a, v[: t + 1])
    out = out * torch.sigmoid(h @ _f(w[p + "g"]).T)[:, :, None]
    return out.reshape(T, H * V) @ _f(w[p + "o"]).T


def route(h: torch.Tensor, router: torch.Tensor, r: Dict):
    """Scores over all experts; the `top` largest among the experts of the `keep` best groups."""
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.softmax(h @ _f(router).T, dim=-1)                                   # [T, E]
    per = E // groups["count"]
    gs = s.reshape(-1, groups["count"], per).amax(-1)
    best = torch.topk(gs, groups["keep"], dim=-1).indices
    allowed = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, best, True).repeat_interleave(per, dim=1)
    idx = torch.topk(torch.where(allowed, s, torch.full_like(s, -1.0)), top, dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def moe(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: Dict) -> torch.Tensor:
    idx, wt = route(h, w[p + "router"], mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t].tolist(), wt[t]):
            pe = f"{p}e{e}."
            y = silu(_f(w[pe + "gate"]) @ h[t]) * (_f(w[pe + "up"]) @ h[t])
            out[t] += s * (_f(w[pe + "down"]) @ y)
    return out


def layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, spec: Dict, eps: float) -> torch.Tensor:
    """One parallel layer: both sublayers read the same normed input and are gated element by element."""
    p = f"l{i}."
    h = scalar_norm(x, w[p + "norm1"], eps)
    mixer = {"channel_delta": channel_delta, "latent_attention": latent_attention}[spec["type"]]
    y = torch.sigmoid(h @ _f(w[p + "rg1"]).T + _f(w[p + "rg1.b"])) * mixer(h, w, p + "mix.", spec["mixer"], eps)
    if spec.get("mlp"):
        y = y + torch.sigmoid(h @ _f(w[p + "rg2"]).T + _f(w[p + "rg2.b"])) * moe(h, w, p + "mlp.", spec["mlp"])
    return x + y


def forward(cfg: Dict, w: Dict[str, torch.Tensor], tokens: List[int], trail: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of every position of one sequence; `trail` collects the residual after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = _f(w["embed"])[torch.tensor(tokens)]
    for i, spec in enumerate(cfg["layers"]):
        x = layer(x, w, i, spec, eps)
        if trail is not None:
            trail.append(x.clone())
    logits = scalar_norm(x, w["final.norm"], eps) @ _f(w["head"]).T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy(cfg: Dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(forward(cfg, w, toks)[-1].argmax())
        out.append(t)
        toks.append(t)
    return out
