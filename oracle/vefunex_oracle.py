"""Vefunex restated on the CPU in float64, one function per mechanism, token loops where the design has a recurrence.

Test infrastructure only: nothing here is imported by the product, and nothing of the product is imported here. The functions take
plain tensors (a checkpoint's state dict under its own names) and the config.json dictionary.

Notation: T tokens of ONE sequence at positions 0..T-1, C the width, rows are tokens.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------------------ small pieces
def dyt(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    """Dynamic tanh: a norm without statistics, tanh(alpha x) w + b with a scalar alpha."""
    return torch.tanh(alpha.to(F64) * x) * w.to(F64) + b.to(F64)


def shift_conv(h: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal convolution over time per channel: y_t = sum_j w[:, j] h_(t - taps + 1 + j), zeros before the start. h [T, ch], w [ch, taps]."""
    T, taps = h.shape[0], w.shape[1]
    y = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j].to(F64) * h[s]
    if bias is not None:
        y = y + bias.to(F64)
    return y


def input_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """What a sublayer reads: h + conv(h)."""
    return h + shift_conv(h, w)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: the pair (2i, 2i + 1), i < dims / 2, turns by pos * base^(-2i / dims); the other dimensions pass."""
    out = x.clone()
    for i in range(dims // 2):
        a = pos.to(F64) * base ** (-2.0 * i / dims)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def query_temperature(pos: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """1 + coef ln(floor((p + 1) / every) + 1)."""
    return 1.0 + coef * torch.log(torch.floor((pos.to(F64) + 1.0) / every) + 1.0)


def causal_softmax_attention(q, k, v, scale: float, softcap: float = 0.0, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; head h reads key/value head h // (H / G); row i sees j <= i; the
    denominator of head h also holds exp(sink[h])."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), -math.inf)
        m = s.max(dim=1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].to(F64).expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(dim=1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h].to(F64) - m)
        out[:, h] = (e / den) @ v[:, g]
    return out


# ------------------------------------------------------------------------------------------------------------------ mixers
def attention_mixer(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ W[p + "q"].to(F64).T).view(T, H, d)
    k = (h @ W[p + "k"].to(F64).T).view(T, G, d)
    v = (h @ W[p + "v"].to(F64).T).view(T, G, dv)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(pos, qt["coef"], qt["every"])[:, None, None]
    v = unit_rms(v, eps)
    o = causal_softmax_attention(q, k, v, m["scale"])
    return o.reshape(T, H * dv) @ W[p + "o"].to(F64).T


def gated_sink_attention(h, W, p: str, m: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ W[p + "q"].to(F64).T).view(T, H, d)
    k = (h @ W[p + "k"].to(F64).T).view(T, G, d)
    v = (h @ W[p + "v"].to(F64).T).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q = rotate_pairs(q, pos, rot["dims"], rot["base"])
        k = rotate_pairs(k, pos, rot["dims"], rot["base"])
    o = causal_softmax_attention(q, k, v, m["scale"], m.get("softcap") or 0.0, W[p + "sink"])
    o = o.reshape(T, H * dv) * torch.sigmoid(h @ W[p + "g"].to(F64).T)
    return o @ W[p + "o"].to(F64).T


def selective_scan(h, W, p: str, m: dict) -> torch.Tensor:
    T = h.shape[0]
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ W[p + "in"].to(F64).T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(shift_conv(x, W[p + "conv"], W[p + "conv.b"]))
    proj = x @ W[p + "x"].to(F64).T
    dt, B, Cm = proj[:, :R], proj[:, R:R + N], proj[:, R + N:R + 2 * N]
    dt = softplus(dt @ W[p + "dt"].to(F64).T + W[p + "dt.b"].to(F64))          # [T, inner]
    A = -torch.exp(W[p + "A_log"].to(F64))                                    # [inner, N]
    S = torch.zeros(inner, N, dtype=F64)
    y = torch.zeros(T, inner, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ Cm[t] + W[p + "D"].to(F64) * x[t]
    return (y * silu(z)) @ W[p + "o"].to(F64).T


def parallel_mixer(h, W, p: str, m: dict) -> torch.Tensor:
    return m["left_scale"] * gated_sink_attention(h, W, p + "left.", m["left"]) + m["right_scale"] * selective_scan(h, W, p + "right.", m["right"])


def gla_mixer(h, W, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (h @ W[p + "q"].to(F64).T).view(T, H, d) * d ** -0.5
    k = (h @ W[p + "k"].to(F64).T).view(T, H, d)
    v = (h @ W[p + "v"].to(F64).T).view(T, H, dv)
    z = (h @ W[p + "a1"].to(F64).T) @ W[p + "a2"].to(F64).T + W[p + "a2.b"].to(F64)
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit_rms(o, eps) * W[p + "norm"].to(F64)
    o = o.reshape(T, H * dv) * silu(h @ W[p + "g"].to(F64).T)
    return o @ W[p + "o"].to(F64).T


# ------------------------------------------------------------------------------------------------------------ feed-forward
def moe(h, W, p: str, m: dict) -> torch.Tensor:
    """Sigmoid router, the `top` largest scores, the score scales the expert's INPUT."""
    E, top = m["router"]["experts"], m["router"]["top"]
    s = torch.sigmoid(h @ W[p + "router"].to(F64).T)
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(s[t, e]), e))[:top]
        for e in order:
            u = s[t, e] * h[t]
            a = silu(W[f"{p}e{e}.gate"].to(F64) @ u) * (W[f"{p}e{e}.up"].to(F64) @ u)
            out[t] += W[f"{p}e{e}.down"].to(F64) @ a
    return out


# ------------------------------------------------------------------------------------------------------------------- model
def mixer(h, W, i: int, layer: dict, eps: float) -> torch.Tensor:
    p, typ = f"l{i}.mix.", layer["type"]
    if typ == "attention":
        return attention_mixer(h, W, p, layer["mixer"], eps)
    if typ == "parallel":
        return parallel_mixer(h, W, p, layer["mixer"])
    if typ == "gla":
        return gla_mixer(h, W, p, layer["mixer"], eps)
    raise ValueError(typ)


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], collect: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one sequence. collect: receives the stream after every layer (after the depth average)."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = W["embed"].to(F64)[torch.tensor(tokens, dtype=torch.long)]
    streams = [x]
    for i, layer in enumerate(cfg["layers"]):
        n = f"l{i}."
        h = input_conv(dyt(x, W[n + "norm1"], W[n + "norm1.b"], W[n + "norm1.alpha"]), W[n + "canon1"])
        x = x + mult * mixer(h, W, i, layer, eps)
        if layer.get("mlp"):
            h = input_conv(dyt(x, W[n + "norm2"], W[n + "norm2.b"], W[n + "norm2.alpha"]), W[n + "canon2"])
            x = x + mult * moe(h, W, n + "mlp.", layer["mlp"])
        streams.append(x)
        x = sum(W[n + "dwa"][j].to(F64) * streams[j] for j in range(i + 2))
        if collect is not None:
            collect.append(x)
    x = dyt(x, W["final.norm"], W["final.norm.b"], W["final.norm.alpha"])
    z = x @ W["embed"].to(F64).T
    cap = cfg.get("logit_softcap") or 0.0
    return cap * torch.tanh(z / cap) if cap else z
