"""Fofisun: a decoder-only language model of differential-attention layers with dense or mixture-of-experts feed-forwards, sinusoidal
position vectors added to the embedding, and a block of layers that runs several times in a row with the same tensors.

    x_0 = E[token] + s(position)                              s(p)[2i] = sin(p f_i), s(p)[2i + 1] = cos(p f_i), f_i = 10000^(-2i / C)
    x <- x + Nb1(mixer(Na1(x)));  x <- x + Nb2(ff(Na2(x)))    N(y) = y / rms(y) * (1 + g) on both sides of every sublayer
The residual stream x is fp32 on the device. A layer RUN is one pass through a layer; the layers [loop_start, loop_stop) make
loop_times passes with the same tensors, and every run owns its pages of keys / values and its convolution ring.

Mixer (config.DiffAttentionSpec): one stacked projection q | k | v | gate; a short causal convolution over time on q, k, v (the last
taps - 1 projected rows of a sequence live in its state slot); RMS norm of queries and keys per head and score map; two softmax maps
per head over the same values inside a sliding window that also keeps the first tokens of the sequence; o = a1 - lambda a2, RMS norm
over the head, times 1 - diff, times sigmoid(gate); output projection. Feed-forward: W_d gelu(W_u x) (config.GeluMlpSpec) or routed
clamped gated experts plus a sigmoid-gated shared expert (config.ClampedMoeSpec).

Like the other sequence-step decoders (model/voduzen.py, model/tifisun.py) the model owns no cache and no loop: `step()` runs ONE
packed batch of rows - portions of prompts beside single decoded tokens, each row addressed by (slot, position) - against a
PagedStateCache that the caller (serving.StepScheduler) manages. `generate()` goes through that scheduler.

Kernels: embedding + position vector (rownorm32.cu), stacked projection (seq_linear), causal convolution over state slots
(state_mixers.cu), per-group query / key norm + cache append, windowed attention with kept first keys and two score maps, the
differential combine + head norm + gate (window_attention.cu), router with bias and softmax over the chosen, expert-sorted grouped
products, clamped gate * up, combine + post norm + residual + next pre-norm (router_moe.cu), post norm + residual + next pre-norm
(rownorm32.cu).

Compute dtype bfloat16: bf16 matrix operands with fp32 accumulation, bf16 keys / values; positions and angles, attention scores and
weights, norms, router, residual in fp32. Compute dtype float32: everything in fp32 on the FMA pipe.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .. import lib, seqlib
from ..config import ClampedMoeSpec, DiffAttentionSpec, FofisunConfig, GeluMlpSpec
from .paged_cache import PagedStateCache
from .seq_linear import dense_linear
from .seq_moe import SMALL_STEP_ROWS, expert_workspace, grouped_tensor_gemm_ok, run_sorted_experts  # noqa: F401
from .seq_model import GraphedDecodeMixin, SequenceStepLM


# ------------------------------------------------------------------------------------------------------------------- weights
@dataclass
class DiffAttnW:
    w_in: torch.Tensor             # [q | k | v | gate | zero rows, C]
    cols: Dict[str, slice]         # column ranges of the stacked projection's output
    conv: Optional[torch.Tensor]   # [q + k + v channels, taps]
    q_norm: torch.Tensor           # [dim]
    k_norm: torch.Tensor
    lam: float                     # exp(lq1 . lk1) - exp(lq2 . lk2) + diff
    o: torch.Tensor                # [C, H * vdim]


@dataclass
class GeluMlpW:
    up: torch.Tensor               # [ff, C]
    down: torch.Tensor             # [C, ff]


@dataclass
class ClampedMoeW:
    router_cat: torch.Tensor            # [experts (+ 1) rounded up to 8, C]: router rows, the shared expert's gate row, zero rows
    router_bias: torch.Tensor           # fp32 [experts]
    gate_up: torch.Tensor               # [E, 2 * ff, C]: per expert gate rows then up rows
    down: torch.Tensor                  # [E, C, ff]
    shared_gate_up: Optional[torch.Tensor]   # [2 * ffs, C]
    shared_down: Optional[torch.Tensor]      # [C, ffs]


@dataclass
class FofisunLayerW:
    norm1: torch.Tensor
    norm1b: torch.Tensor
    norm2: Optional[torch.Tensor]
    norm2b: Optional[torch.Tensor]
    mix: DiffAttnW
    mlp: object


@dataclass
class FofisunW:
    embed: torch.Tensor
    final_norm: torch.Tensor
    head: torch.Tensor
    layers: List[FofisunLayerW]
    pos_freq: torch.Tensor         # float64 [ceil(C / 2)]


def _stack(parts: Sequence[tuple], device, dtype):
    """[(name, matrix [n_i, C])] -> (stacked matrix with zero rows up to a multiple of 8, {name: column slice of its output})."""
    cols, rows, at = {}, [], 0
    for name, m in parts:
        cols[name] = slice(at, at + m.shape[0])
        at += m.shape[0]
        rows.append(m)
    if at % 8:   # the tensor-core GEMMs take N % 8 == 0; the extra outputs are never read
        rows.append(torch.zeros(8 - at % 8, rows[0].shape[1], device=device, dtype=dtype))
    return torch.cat(rows, dim=0).contiguous(), cols


def weights_from_state_dict(sd: Dict[str, torch.Tensor], cfg: FofisunConfig, device, dtype: torch.dtype) -> FofisunW:
    """Checkpoint names: 'embed', 'final.norm', 'head', per layer i 'l<i>.norm1|norm1b|norm2|norm2b', 'l<i>.mix.*', 'l<i>.mlp.*';
    linear weights [out, in]. Load-time re-layouts: the mixer's projections are stacked into one matrix, the three convolutions
    into one, gate and up of every expert likewise, the experts into one tensor, the shared expert's gate row goes behind the router
    rows; lambda is evaluated once (in double precision)."""
    def g(name, dt=dtype):
        if name not in sd:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        return sd[name].to(device=device, dtype=dt).contiguous()

    def need(t: torch.Tensor, shape, what: str):
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"{what} has shape {tuple(t.shape)}, the config says {tuple(shape)}")
        return t

    C, f64 = cfg.hidden_size, torch.float64
    layers = []
    for i, spec in enumerate(cfg.layers):
        m, p = spec.mixer, f"l{i}.mix."
        nq, nk, nv = m.heads * 2 * m.dim, m.kv_heads * 2 * m.dim, m.kv_heads * m.vdim
        w_in, cols = _stack([("q", need(g(p + "q"), (nq, C), p + "q")), ("k", need(g(p + "k"), (nk, C), p + "k")),
                             ("v", need(g(p + "v"), (nv, C), p + "v")), ("g", need(g(p + "g"), (m.heads * m.vdim, C), p + "g"))], device, dtype)
        conv = None
        if m.conv >= 1:
            conv = torch.cat([need(g(p + "q.conv"), (nq, m.conv), p + "q.conv"), need(g(p + "k.conv"), (nk, m.conv), p + "k.conv"),
                              need(g(p + "v.conv"), (nv, m.conv), p + "v.conv")], dim=0).contiguous()
        lam = math.exp(float((sd[p + "lq1"].to(f64) * sd[p + "lk1"].to(f64)).sum())) - \
            math.exp(float((sd[p + "lq2"].to(f64) * sd[p + "lk2"].to(f64)).sum())) + m.diff
        mix = DiffAttnW(w_in=w_in, cols=cols, conv=conv, q_norm=need(g(p + "q.norm"), (m.dim,), p + "q.norm"),
                        k_norm=need(g(p + "k.norm"), (m.dim,), p + "k.norm"), lam=lam,
                        o=need(g(p + "o"), (C, m.heads * m.vdim), p + "o"))
        mlp, q = None, f"l{i}.mlp."
        if isinstance(spec.mlp, GeluMlpSpec):
            mlp = GeluMlpW(up=need(g(q + "up"), (spec.mlp.ff, C), q + "up"), down=need(g(q + "down"), (C, spec.mlp.ff), q + "down"))
        elif isinstance(spec.mlp, ClampedMoeSpec):
            s = spec.mlp
            rows = [need(g(q + "router"), (s.experts, C), q + "router")]
            if s.shared_ff:
                rows.append(g(q + "shared.sg").view(1, -1))
            n_rows = sum(x.shape[0] for x in rows)
            if n_rows % 8:
                rows.append(torch.zeros(8 - n_rows % 8, C, device=device, dtype=dtype))
            mlp = ClampedMoeW(
                router_cat=torch.cat(rows, dim=0).contiguous(), router_bias=need(g(q + "router.b", torch.float32), (s.experts,), q + "router.b"),
                gate_up=torch.stack([torch.cat([need(g(f"{q}e{e}.gate"), (s.expert_ff, C), f"{q}e{e}.gate"), g(f"{q}e{e}.up")], dim=0)
                                     for e in range(s.experts)]).contiguous(),
                down=torch.stack([need(g(f"{q}e{e}.down"), (C, s.expert_ff), f"{q}e{e}.down") for e in range(s.experts)]).contiguous(),
                shared_gate_up=torch.cat([g(q + "shared.gate"), g(q + "shared.up")], dim=0).contiguous() if s.shared_ff else None,
                shared_down=need(g(q + "shared.down"), (C, s.shared_ff), q + "shared.down") if s.shared_ff else None)
        layers.append(FofisunLayerW(norm1=g(f"l{i}.norm1"), norm1b=g(f"l{i}.norm1b"), norm2=g(f"l{i}.norm2") if mlp else None,
                                    norm2b=g(f"l{i}.norm2b") if mlp else None, mix=mix, mlp=mlp))
    return FofisunW(embed=need(g("embed"), (cfg.vocab_size, C), "embed"), final_norm=g("final.norm"), head=g("head"), layers=layers,
                    pos_freq=seqlib.sinusoid_frequencies(C, FofisunConfig.POSITION_BASE, device))


def random_state_dict(cfg: FofisunConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bf16 weights under the checkpoint names (benchmarks, tests)."""
    gen = torch.Generator().manual_seed(seed)

    def rn(*shape, s=1.0, mean=0.0):
        return (torch.randn(*shape, generator=gen) * s + mean).to(torch.bfloat16)

    C, sd = cfg.hidden_size, {}
    sd["embed"] = rn(cfg.vocab_size, C, s=1.0)
    sd["final.norm"] = rn(C, s=0.2)
    sd["head"] = rn(cfg.vocab_size, C, s=C ** -0.5)
    for i, spec in enumerate(cfg.layers):
        m, p = spec.mixer, f"l{i}.mix."
        for n in ("norm1", "norm1b"):
            sd[f"l{i}.{n}"] = rn(C, s=0.2)
        for name, n in (("q", m.heads * 2 * m.dim), ("k", m.kv_heads * 2 * m.dim), ("v", m.kv_heads * m.vdim)):
            sd[p + name] = rn(n, C, s=C ** -0.5)
            if m.conv >= 1:
                sd[p + name + ".conv"] = rn(n, m.conv, s=0.5)
        sd[p + "q.norm"], sd[p + "k.norm"] = rn(m.dim, s=0.3, mean=1.2), rn(m.dim, s=0.3, mean=1.2)
        for n in ("lq1", "lk1", "lq2", "lk2"):
            sd[p + n] = rn(m.dim, s=0.6 * m.dim ** -0.5)
        sd[p + "g"] = rn(m.heads * m.vdim, C, s=C ** -0.5)
        sd[p + "o"] = rn(C, m.heads * m.vdim, s=(m.heads * m.vdim) ** -0.5)
        q = f"l{i}.mlp."
        if spec.mlp is not None:
            for n in ("norm2", "norm2b"):
                sd[f"l{i}.{n}"] = rn(C, s=0.2)
        if isinstance(spec.mlp, GeluMlpSpec):
            sd[q + "up"], sd[q + "down"] = rn(spec.mlp.ff, C, s=C ** -0.5), rn(C, spec.mlp.ff, s=spec.mlp.ff ** -0.5)
        elif isinstance(spec.mlp, ClampedMoeSpec):
            s = spec.mlp
            sd[q + "router"], sd[q + "router.b"] = rn(s.experts, C, s=2.0 * C ** -0.5), rn(s.experts, s=0.5)
            for e in range(s.experts):
                sd[f"{q}e{e}.gate"], sd[f"{q}e{e}.up"] = rn(s.expert_ff, C, s=1.5 * C ** -0.5), rn(s.expert_ff, C, s=1.5 * C ** -0.5)
                sd[f"{q}e{e}.down"] = rn(C, s.expert_ff, s=s.expert_ff ** -0.5)
            if s.shared_ff:
                sd[q + "shared.gate"], sd[q + "shared.up"] = rn(s.shared_ff, C, s=1.5 * C ** -0.5), rn(s.shared_ff, C, s=1.5 * C ** -0.5)
                sd[q + "shared.down"], sd[q + "shared.sg"] = rn(C, s.shared_ff, s=s.shared_ff ** -0.5), rn(1, C, s=C ** -0.5)
    return sd


# ------------------------------------------------------------------------------------------------------------------- decoder
class FofisunDecoder(GraphedDecodeMixin):
    def __init__(self, cfg: FofisunConfig, w: FofisunW, dtype: torch.dtype):
        self.cfg, self.w, self.dtype = cfg, w, dtype
        self.device = w.embed.device
        self.C = cfg.hidden_size
        self.eps = cfg.norm_eps
        self.runs = cfg.layer_runs()    # layer index of every layer run; cache pools and states are per run
        self.tensor_gemm = dtype == torch.bfloat16
        self.tensor_attention = True    # False: the plain attention kernel for every shape (A/B, tests)
        self.fused_maps = True          # False: prompt portions run one CTA per score map and the combine kernel behind it (A/B, tests)
        self.fused_conv_store = True    # False: convolution, query / key norm + cache append as separate launches (A/B, tests)
        self._moe_ws = {}
        self._init_graphs()

    # ---- cache
    def cache_widths(self) -> List[int]:
        """Cached numbers per token and layer run: both maps' keys and the values of every key/value head."""
        return [self.cfg.layers[li].mixer.kv_heads * (2 * self.cfg.layers[li].mixer.dim + self.cfg.layers[li].mixer.vdim) for li in self.runs]

    def state_shapes(self) -> List[dict]:
        """Per run: the ring of the last taps - 1 projected q | k | v rows (nothing for convolutions of one tap or none)."""
        out = []
        for li in self.runs:
            m = self.cfg.layers[li].mixer
            out.append({"conv": (m.conv - 1, (m.heads + m.kv_heads) * 2 * m.dim + m.kv_heads * m.vdim)} if m.conv > 1 else {})
        return out

    def new_cache(self, n_pages: int, n_slots: int, max_pages_per_slot: int = 0) -> PagedStateCache:
        return PagedStateCache(self.cache_widths(), self.state_shapes(), n_pages, n_slots, self.cfg.kv_page_size, self.dtype,
                               self.device, max_pages_per_slot)

    def _linear(self, x, w, out_dtype, act: int = seqlib.ACT_NONE):
        return dense_linear(x, w, out_dtype, tensor_gemm=self.tensor_gemm, act=act)

    # ---- mixer: compute-dtype rows [T, C] -> fp32 [T, C]
    def _mixer(self, run: int, xb, pos, slot, cache: PagedStateCache, single_rows: bool, plans: Optional[dict]):
        li = self.runs[run]
        m: DiffAttentionSpec = self.cfg.layers[li].mixer
        mw: DiffAttnW = self.w.layers[li].mix
        T, f32, dev = xb.shape[0], torch.float32, xb.device
        H, G, d, dv = m.heads, m.kv_heads, m.dim, m.vdim
        nq, nk, nv = H * 2 * d, G * 2 * d, G * dv
        z = self._linear(xb, mw.w_in, f32)                                    # [T, q | k | v | gate]
        pool = cache.pools[run]
        q = torch.empty(T, nq, device=dev, dtype=self.dtype)
        if mw.conv is not None and self.fused_conv_store:
            seqlib.conv_qk_norm_kv_store(z, mw.conv, pos, slot, cache.states[run].get("conv"), nq, nk, d, mw.q_norm, mw.k_norm, self.eps,
                                         cache.block_table, cache.page_size, pool, q, single_rows=single_rows)
        else:
            y = z
            if mw.conv is not None:
                y = torch.empty(T, nq + nk + nv, device=dev, dtype=f32)
                seqlib.causal_conv(z[:, :nq + nk + nv], mw.conv, pos, slot, cache.states[run].get("conv"), y, single_rows=single_rows)
            seqlib.qk_norm_kv_store(y[:, :nq], mw.q_norm, y[:, nq:nq + nk], mw.k_norm, y[:, nq + nk:nq + nk + nv], self.eps, pos, slot,
                                    cache.block_table, cache.page_size, pool, q, group=d)
        window = m.window if m.window is not None else seqlib.WINDOW_ALL
        on = torch.empty(T, H * dv, device=dev, dtype=self.dtype)
        gate = z[:, mw.cols["g"]]
        tensor = plans is not None and self.tensor_attention and seqlib.window_attn_mma_ok(H, G, d, dv, self.dtype)
        items = None
        if tensor and plans["portions"] is not None:
            rep = H // G
            items = plans.get(rep)
            if items is None:
                items = plans[rep] = seqlib.window_attn_items(plans["portions"], rep, dev)
        if items is not None and self.fused_maps and seqlib.diff_attn_pair_ok(H, G, d, dv, self.dtype):
            # prompt portions: both maps, the combine, the head norm and the gate in one kernel
            seqlib.diff_attn_pair(q, H, G, d, dv, pool, cache.block_table, cache.page_size, items, window, m.keep_first, m.scale, mw.lam,
                                  1.0 - m.diff, self.eps, gate, seqlib.GATE_SIGMOID, on)
            return self._linear(on, mw.o, f32)
        att = torch.empty(T, H * 2 * dv, device=dev, dtype=f32)
        if tensor:       # items None: one row per request, the kernel reads positions and slots itself
            seqlib.window_attn_mma(q, H, G, d, dv, pool, cache.block_table, cache.page_size, items, pos, slot, window, m.scale, 0.0, None,
                                   att, maps=2, keep_first=m.keep_first)
        else:
            seqlib.window_attn(q, H, G, d, dv, pool, cache.block_table, cache.page_size, pos, slot, window, m.scale, 0.0, None, att,
                               maps=2, keep_first=m.keep_first)
        seqlib.diff_heads_gate(att, H, dv, mw.lam, 1.0 - m.diff, self.eps, gate, seqlib.GATE_SIGMOID, on)
        return self._linear(on, mw.o, f32)

    # ---- feed-forwards: update h32 (and write the next sublayer's normed input to xb_out) in place
    def _dense(self, lw: FofisunLayerW, xb, h32, w_next, xb_out):
        act = self._linear(xb, lw.mlp.up, self.dtype, act=seqlib.ACT_GELU_ERF)
        y = self._linear(act, lw.mlp.down, torch.float32)
        seqlib.post_norm_residual(y, lw.norm2b, self.eps, 1.0, h32, w_next, xb_out)

    def _grouped_tensor_gemm(self, s: ClampedMoeSpec) -> bool:
        return grouped_tensor_gemm_ok(self.tensor_gemm, s.expert_ff, self.C)

    def _moe_workspace(self, T: int, s: ClampedMoeSpec, tile: int):
        return expert_workspace(self._moe_ws, T, s.experts, s.top, s.expert_ff, tile, self.C, self.dtype, self.device)

    def _moe(self, li: int, xb, h32, w_next, xb_out):
        s: ClampedMoeSpec = self.cfg.layers[li].mlp
        lw = self.w.layers[li]
        mw: ClampedMoeW = lw.mlp
        T, cfg = xb.shape[0], FofisunConfig
        grouped = self._grouped_tensor_gemm(s)
        tile = 128 if grouped else seqlib.LINEAR_TILE
        ws = self._moe_workspace(T, s, tile)
        has_gate = s.shared_ff is not None
        z32 = self._linear(xb, mw.router_cat, torch.float32)
        seqlib.router_topk(z32, s.experts, s.experts, s.top, None, has_gate, ws.ids, ws.w, ws.gate, ws.counts, bias=mw.router_bias, renorm=True)
        run_sorted_experts(ws, xb, s.experts, s.top, s.expert_ff, tile, mw.gate_up, mw.down, seqlib.ACT_CLAMP_SWISH, grouped=grouped,
                           limit=s.limit, slope=cfg.SWISH_SLOPE, shift=cfg.UP_SHIFT)
        ysh = None
        if has_gate:
            gu = self._linear(xb, mw.shared_gate_up, self.dtype)
            sact = seqlib.glu_mul(gu, s.shared_ff, seqlib.ACT_CLAMP_SWISH, torch.empty(T, s.shared_ff, device=xb.device, dtype=self.dtype),
                                  limit=s.shared_limit, slope=cfg.SWISH_SLOPE, shift=cfg.UP_SHIFT)
            ysh = self._linear(sact, mw.shared_down, torch.float32)
        seqlib.moe_combine_norm(ws.ys, ws.slot_of, ws.w, s.top, ws.gate if has_gate else None, ysh, lw.norm2b, self.eps, h32, xb_out,
                                w_next=w_next)

    # ---- the step
    @torch.no_grad()
    def step(self, tokens: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, cache: PagedStateCache,
             want_rows: Optional[torch.Tensor] = None, collect: Optional[list] = None,
             portions: Optional[Sequence] = None, one_row_each: bool = False) -> Optional[torch.Tensor]:
        """tokens / pos / slot: int32 [T] on the device - row t is token tokens[t] at position pos[t] of the request in slot slot[t];
        rows of one request are consecutive and ascending in position, and a request's rows continue where its previous step
        ended. Appends every row to the cache, advances the convolution rings and returns fp32 logits [len(want_rows), vocab] (None
        when no row is asked for). collect: receives the residual stream after every layer run. portions: the same batch as the
        host knows it, [(first_row, n_rows, slot, first_pos)] per request - the tensor-core attention kernel's work list is built
        from it; without it the plain kernel runs. one_row_each: every row is a request of its own (decode)."""
        T, dev, f32 = tokens.numel(), self.device, torch.float32
        single = one_row_each or (portions is not None and len(portions) == T)
        plans = {"portions": None} if one_row_each else ({"portions": list(portions)} if portions is not None else None)
        layers, runs = self.w.layers, self.runs
        h32 = torch.empty(T, self.C, device=dev, dtype=f32)
        xb = torch.empty(T, self.C, device=dev, dtype=self.dtype)
        seqlib.embed_sinusoid(tokens, pos, self.w.embed, 1.0, self.w.pos_freq, h32)
        if runs:
            seqlib.rms_rows(h32, layers[runs[0]].norm1, self.eps, xb, one_plus=True)
        for r, li in enumerate(runs):
            lw = layers[li]
            last = r + 1 == len(runs)
            nxt = None if last else layers[runs[r + 1]].norm1
            after_mixer = lw.norm2 if lw.mlp is not None else nxt
            y = self._mixer(r, xb, pos, slot, cache, single, plans)
            seqlib.post_norm_residual(y, lw.norm1b, self.eps, 1.0, h32, after_mixer, xb if (lw.mlp is not None or not last) else None)
            if isinstance(lw.mlp, GeluMlpW):
                self._dense(lw, xb, h32, nxt, None if last else xb)
            elif isinstance(lw.mlp, ClampedMoeW):
                self._moe(li, xb, h32, nxt, None if last else xb)
            if collect is not None:
                collect.append(h32.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        hw = h32.index_select(0, want_rows)
        xf = seqlib.rms_rows(hw, self.w.final_norm, self.eps, torch.empty(hw.shape[0], self.C, device=dev, dtype=self.dtype), one_plus=True)
        return self._linear(xf, self.w.head, f32)


# ------------------------------------------------------------------------------------------------------------------- model
class FofisunForCausalLM(SequenceStepLM):
    """Entry point: from_pretrained / from_state_dict, step() for serving loops, generate() for greedy generation."""
    config_class = FofisunConfig
    decoder_class = FofisunDecoder
    weights_from_state_dict = staticmethod(weights_from_state_dict)
