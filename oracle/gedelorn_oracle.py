"""Plain restatement of the Gedelorn design: one function per mechanism, token by token where the design is a recurrence.

Slow on purpose and independent of the engine: it shares no code with the package, takes the config dictionary and the
tensors by their checkpoint names, and computes in one floating type (float64 by default) from the bf16 weight values.
The reference service names models by tag and has no model code (app/utils/config.py:86), so nothing here restates it.

Notation: x residual stream [T, W]; h a sublayer's normed input; S a matrix state [key dim, value dim] per head.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the gain minus one."""
    return rms_unit(x, eps) * (1.0 + w)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def logsigmoid(z: torch.Tensor) -> torch.Tensor:
    return -softplus(-z)


# ------------------------------------------------------------------------------------------------ mixers
def mlstm_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """Matrix memory with exponential gates and a running maximum that starts at 0."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, V)
    gi = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    gf = logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        n = torch.zeros(D, dtype=h.dtype)
        mx = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            m_new = torch.maximum(gf[t, a] + mx, gi[t, a])
            keep, put = torch.exp(gf[t, a] + mx - m_new), torch.exp(gi[t, a] - m_new)
            S = keep * S + put * torch.outer(k[t, a], v[t, a])
            n = keep * n + put * k[t, a]
            mx = m_new
            den = torch.maximum(torch.abs(n @ q[t, a]), torch.exp(-mx)) + 1e-6
            out[t, a] = (S.T @ q[t, a]) / den
    out = rms_unit(out, eps).reshape(T, H * V) * w[p + "norm"]
    return (out * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y[t, c] = bias[c] + sum_j taps[c, K-1-j] u[t-j, c], zeros before the start."""
    T, K = u.shape[0], taps.shape[1]
    y = bias.expand(T, -1).clone()
    for j in range(K):
        y[j:] += u[:T - j] * taps[:, K - 1 - j]
    return y


def mamba2_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """Selective state space with one decay per head and step."""
    T = h.shape[0]
    H, P, N, G, NG = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * P
    zxbcdt = h @ w[p + "in"].T
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    A = -torch.exp(w[p + "A_log"])
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(A[a] * dt[t, a]) * S + dt[t, a] * torch.outer(B[t, g], x[t, a])
            y[t, a] = S.T @ Cm[t, g] + w[p + "D"][a] * x[t, a]
    y = y.reshape(T, inner) * silu(z)
    y = rms_unit(y.reshape(T, NG, inner // NG), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def rotate_pairs(u: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotary positions on the first `dims` coordinates of the last axis, coordinate 2i paired with 2i+1."""
    i = torch.arange(dims // 2, dtype=u.dtype)
    ang = pos.to(u.dtype)[:, None] * base ** (-2.0 * i / dims)          # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = u.clone()
    a, b = u[..., 0:dims:2], u[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict) -> torch.Tensor:
    """Grouped-query softmax attention over a sliding window; the unrotated keys serve as values."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, D)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, D)
    v = k
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        q, k = rotate_pairs(q, pos, rot["dims"], rot["base"]), rotate_pairs(k, pos, rot["dims"], rot["base"])
    out = torch.zeros(T, H, D, dtype=h.dtype)
    cap, win = m.get("softcap"), m["mask"]["size"]
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        d = pos[:, None] - pos[None, :]
        s = s.masked_fill((d < 0) | (d >= win), float("-inf"))
        out[:, a] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * D) @ w[p + "o"].T


def lightning_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """Linear attention with one constant decay per head."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, D)
    k = silu(h @ w[p + "k"].T).reshape(T, H, D)
    v = silu(h @ w[p + "v"].T).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = m["decay"][a] * S + torch.outer(k[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    out = rms_unit(out.reshape(T, H * V), eps) * w[p + "norm"]
    return (out * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    left = window_attention(h, w, p + "left.", m["left"])
    right = lightning_attention(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ------------------------------------------------------------------------------------------------ feed-forward
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def squared_relu_expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (torch.relu(h @ up.T) ** 2) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, top: int, scale: float):
    """(indices [T, top], weights [T, top]): sigmoid scores, the largest `top`, normalised to sum to `scale`."""
    s = torch.sigmoid(h @ router.T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20) * scale


def moe_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict) -> torch.Tensor:
    r = m["router"]
    idx, wt = route(h, w[p + "router"], r["top"], float(r.get("scale", 1.0)))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * squared_relu_expert(h[t:t + 1], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])[0]
    if m.get("shared"):
        out = out + squared_relu_expert(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


# ------------------------------------------------------------------------------------------------ the model
MIXERS = {"mlstm": mlstm_mixer, "mamba2": mamba2_mixer, "parallel": parallel_mixer}


def forward(cfg: Dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            trail: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its start; `trail` collects the stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = offset_norm(x, w[p + "norm1"], eps)
        x = x + offset_norm(MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], eps), w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = offset_norm(x, w[p + "norm2"], eps)
            y = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp)
            x = x + offset_norm(y, w[p + "norm2b"], eps)
        if trail is not None:
            trail.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg: Dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    """n tokens of argmax decoding, each from a full forward pass over everything so far."""
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(forward(cfg, w, toks)[-1].argmax())
        out.append(t)
        toks.append(t)
    return out
