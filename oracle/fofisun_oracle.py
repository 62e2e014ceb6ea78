"""Plain, slow restatement of the Fofisun decoder: one function per mechanism, whole sequences only, explicit loops.

Test infrastructure: the product never imports this file. Everything runs on the CPU in float64; attention materialises the whole
score matrix and its visibility mask, convolutions loop over taps, the router loops over tokens. The product does the opposite
(packed steps, paged keys, convolution rings in state slots, fused kernels), so the two share neither code nor structure.

Notation. x is the residual stream [T, C], p_t the position of token t (from 0).
    x_0 = E[token] + s(p),   s(p)[2i] = sin(p * 10000^(-2i/C)),  s(p)[2i+1] = cos(p * 10000^(-2i/C))
    layer:  x <- x + Nb1(mixer(Na1(x)));  x <- x + Nb2(ff(Na2(x)))        N(y) = y / sqrt(mean(y^2) + eps) * (1 + g)
    layers [start, stop) are run `times` times in a row with the same tensors
Mixer: differential attention - two score maps per head over one set of values - with short causal convolutions behind the q, k, v
projections, per-head RMS norms of queries and keys, a sliding window that also keeps the first tokens of the sequence, and a sigmoid
output gate. Feed-forward: W_d gelu(W_u x), or a softmax-over-the-chosen mixture of clamped gated experts plus a gated shared expert.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


def unit_rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def norm_zero_centred(y, g, eps):
    return unit_rms(y, eps) * (1.0 + g)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def position_vectors(T: int, C: int, first: int = 0) -> torch.Tensor:
    """[T, C]: even entries sin, odd entries cos of position * 10000^(-2i / C), i = entry // 2."""
    out = torch.zeros(T, C, dtype=DT)
    for t in range(T):
        for c in range(C):
            ang = (first + t) * 10000.0 ** (-2.0 * (c // 2) / C)
            out[t, c] = math.sin(ang) if c % 2 == 0 else math.cos(ang)
    return out


def causal_conv(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, ch], w [ch, taps]; the last tap multiplies the current token, earlier taps the tokens before it, zeros before
    the sequence starts. No activation."""
    T, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1 - j)
            if s >= 0:
                y[t] += w[:, j] * x[s]
    return y


def visible(i: int, j: int, window: Optional[int], keep_first: int) -> bool:
    """Query position i sees key position j."""
    if j > i:
        return False
    return window is None or i - j < window or j < keep_first


def visibility(T: int, window: Optional[int], keep_first: int) -> torch.Tensor:
    """bool [T, T]: entry (i, j) says whether query position i sees key position j."""
    return torch.tensor([[visible(i, j, window, keep_first) for j in range(T)] for i in range(T)], dtype=torch.bool).view(T, T)


def softmax_attention(q, k, v, scale: float, see: torch.Tensor) -> torch.Tensor:
    """One score map of one head: q, k [T, d], v [T, dv], see bool [T, T] -> [T, dv]. The whole score matrix is materialised."""
    s = (q @ k.T) * scale
    s = s.masked_fill(~see, float("-inf"))
    return torch.softmax(s, dim=-1) @ v


def diff_lambda(lq1, lk1, lq2, lk2, diff: float) -> float:
    return math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + diff


def diff_attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """h [T, C] -> [T, C]. w: the mixer's tensors by their short names ('q', 'q.conv', 'q.norm', 'lq1', 'g', 'o', ...).
    m: heads, kv_heads, dim, vdim, scale, diff, window (None: all earlier keys), keep_first."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    if "q.conv" in w:
        q, k, v = causal_conv(q, w["q.conv"]), causal_conv(k, w["k.conv"]), causal_conv(v, w["v.conv"])
    q = unit_rms(q.view(T, H, 2, d), eps) * w["q.norm"]
    k = unit_rms(k.view(T, G, 2, d), eps) * w["k.norm"]
    v = v.view(T, G, dv)
    lam = diff_lambda(w["lq1"], w["lk1"], w["lq2"], w["lk2"], m["diff"])
    see = visibility(T, m["window"], m["keep_first"])
    heads = []
    for hd in range(H):
        g = hd // (H // G)
        a1 = softmax_attention(q[:, hd, 0], k[:, g, 0], v[:, g], m["scale"], see)
        a2 = softmax_attention(q[:, hd, 1], k[:, g, 1], v[:, g], m["scale"], see)
        heads.append(unit_rms(a1 - lam * a2, eps) * (1.0 - m["diff"]))
    o = torch.cat(heads, dim=-1) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def dense_ff(h, w):
    return gelu_erf(h @ w["up"].T) @ w["down"].T


def clamped_expert(h, gate, up, down, limit: float):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def moe_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], s: dict) -> torch.Tensor:
    """s: experts, top, limit, shared (None or {'limit': ...})."""
    T = h.shape[0]
    z = h @ w["router"].T + w["router.b"]
    out = torch.zeros_like(h)
    for t in range(T):
        order = sorted(range(s["experts"]), key=lambda e: (-float(z[t, e]), e))[: s["top"]]
        p = torch.softmax(torch.stack([z[t, e] for e in order]), dim=0)
        for pe, e in zip(p, order):
            out[t] += pe * clamped_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], s["limit"])[0]
    if s.get("shared"):
        sg = torch.sigmoid(h @ w["shared.sg"].view(-1, 1))
        out = out + sg * clamped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], s["shared"]["limit"])
    return out


def layer_runs(n_layers: int, loop: Optional[dict]) -> List[int]:
    """The layer index of every layer run, in order."""
    if not loop:
        return list(range(n_layers))
    a, b, n = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * n + list(range(b, n_layers))


def forward(sd: Dict[str, torch.Tensor], cfg: dict, tokens, collect: Optional[list] = None) -> torch.Tensor:
    """cfg: the config.json dictionary. Returns logits [T, vocab] in float64; collect receives x after every layer run."""
    sd = {k: v.to(DT) for k, v in sd.items()}
    eps = float(cfg["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T, C = tokens.numel(), int(cfg["width"])
    x = sd["embed"][tokens] + position_vectors(T, C)
    for li in layer_runs(len(cfg["layers"]), cfg.get("loop")):
        L = cfg["layers"][li]
        p = f"l{li}."
        mw = {k[len(p) + 4:]: v for k, v in sd.items() if k.startswith(p + "mix.")}
        mm = L["mixer"]
        mask = mm.get("mask") or {}
        m = {"heads": int(mm["heads"]), "kv_heads": int(mm.get("kv_heads", mm["heads"])), "dim": int(mm["dim"]), "vdim": int(mm["vdim"]),
             "scale": float(mm["scale"]), "diff": float(mm["diff"]), "window": int(mask["size"]) if mask.get("size") else None,
             "keep_first": int(mask.get("keep_first", 0))}
        x = x + norm_zero_centred(diff_attention_mixer(norm_zero_centred(x, sd[p + "norm1"], eps), mw, m, eps), sd[p + "norm1b"], eps)
        if L.get("mlp"):
            fw = {k[len(p) + 4:]: v for k, v in sd.items() if k.startswith(p + "mlp.")}
            hin = norm_zero_centred(x, sd[p + "norm2"], eps)
            if L["mlp"].get("kind", "dense") == "dense":
                y = dense_ff(hin, fw)
            else:
                r = L["mlp"]["router"]
                y = moe_ff(hin, fw, {"experts": int(r["experts"]), "top": int(r["top"]), "limit": float(L["mlp"]["expert"]["limit"]),
                                     "shared": L["mlp"].get("shared")})
            x = x + norm_zero_centred(y, sd[p + "norm2b"], eps)
        if collect is not None:
            collect.append(x.clone())
    return norm_zero_centred(x, sd["final.norm"], eps) @ sd["head"].T
