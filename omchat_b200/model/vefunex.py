"""Vefunex: a decoder-only language model that mixes three kinds of layers - causal softmax attention (query temperature, unit-RMS
values), attention beside a selective scan ('parallel': rotated, soft-capped attention with a sink and an output gate, plus a
state-space branch), and gated linear attention - with sigmoid-routed experts whose weights scale the experts' input.

Around the mixers: a tanh norm without statistics (tanh(alpha x) w + b), a short causal convolution on every sublayer's input
(h + conv(h); its last taps - 1 inputs are state), a residual factor m,
    x <- x + m * mixer(conv1(norm1(x)));   x <- x + m * ff(conv2(norm2(x)))
and a learned average over depth: what leaves layer i is sum_j dwa_i[j] X_j over the embedding output X_0 and the results X_1 .. X_(i+1)
of the layers so far. The output is the tanh norm, the embedding matrix as the head, and a soft cap on the logits.

Like the other sequence-step decoders the model owns no cache and no loop: `step()` runs ONE packed batch of rows - portions of prompts
beside single decoded tokens, each row addressed by (slot, position) - against a PagedStateCache that the caller
(serving.StepScheduler) manages: pages of keys and values for the attentions, per-slot fp32 states for the recurrences and the rings
of the convolutions. `generate()` goes through that scheduler; decode-only steps replay from a CUDA graph (seq_model.py).

Kernels: omc_dyt_conv (stream update + tanh norm + input convolution), omc_pos_qkv_store (rotation, query temperature, unit values,
cache append), omc_window_attn / omc_window_attn_mma with sink and gate, omc_causal_conv (bias + silu), omc_selective_scan,
omc_linear_state_scan with sigmoid-power decays, omc_gated_rms_rows, omc_router_topk (sigmoid scores), the expert-sorted products of
seq_moe.py, omc_moe_combine_depth (combine + residual + depth average), omc_dyt_rows, omc_tanh_cap_rows.

Compute dtype bfloat16: bf16 matrix operands with fp32 accumulation, bf16 keys / values; positions and angles, scores and softmax,
norms, router, residual stream, recurrent states and what enters them besides projections and convolutions in fp32. Compute dtype
float32: everything in fp32 on the FMA pipe.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .. import seqlib
from ..config import AttentionScanMixerSpec, GatedLinearAttentionSpec, SigmoidMoeSpec, SoftmaxAttentionSpec, VefunexConfig
from .paged_cache import PagedStateCache
from .seq_linear import dense_linear
from .seq_model import GraphedDecodeMixin, SequenceStepLM, portion_starts
from .seq_moe import expert_workspace, grouped_tensor_gemm_ok, run_sorted_experts


# ------------------------------------------------------------------------------------------------------------------- weights
@dataclass
class TanhNormW:
    alpha: torch.Tensor            # fp32 [1]
    w: torch.Tensor                # [C]
    b: torch.Tensor                # [C]


@dataclass
class AttentionW:
    w_in: torch.Tensor             # [q | k | v (| gate) (| the other branch's projection) | zero rows, C]
    cols: Dict[str, slice]
    o: torch.Tensor                # [C, H * vdim]
    freq: Optional[torch.Tensor]   # fp32 [rot.dims / 2]
    sink: Optional[torch.Tensor]   # fp32 [H]


@dataclass
class ScanW:
    conv: torch.Tensor             # [inner, taps]
    conv_b: torch.Tensor           # [inner]
    x_dt: torch.Tensor             # [dt_rank (+ zero rows), inner]: the rows of W_x that feed the step sizes
    x_bc: torch.Tensor             # [2 * state (+ zero rows), inner]: the rows that give B and C
    dt: torch.Tensor               # [inner, dt_rank]
    dt_b: torch.Tensor             # fp32 [inner]
    A_log: torch.Tensor            # fp32 [inner, state]
    D: torch.Tensor                # fp32 [inner]
    o: torch.Tensor                # [C, inner]


@dataclass
class ParallelW:
    left: AttentionW               # its w_in also holds the scan's input projection (columns 'rin')
    right: ScanW


@dataclass
class GlaW:
    w_in: torch.Tensor             # [q | k | v | gate | zero rows, C]
    cols: Dict[str, slice]
    a1: torch.Tensor               # [rank (+ zero rows), C]: the decay's first factor, a product of its own (its output feeds a product)
    a2: torch.Tensor               # [H * dim, rank]
    a2_b: torch.Tensor             # fp32 [H * dim]
    norm: torch.Tensor             # [vdim]
    o: torch.Tensor


@dataclass
class SigmoidMoeW:
    router: torch.Tensor           # [experts rounded up to 8, C]
    gate_up: torch.Tensor          # [E, 2 * ff, C]
    down: torch.Tensor             # [E, C, ff]


@dataclass
class VefunexLayerW:
    norm1: TanhNormW
    canon1: torch.Tensor           # [C, taps]
    norm2: Optional[TanhNormW]
    canon2: Optional[torch.Tensor]
    mix: object
    mlp: Optional[SigmoidMoeW]
    dwa: torch.Tensor              # [i + 2]


@dataclass
class VefunexW:
    embed: torch.Tensor
    final_norm: TanhNormW
    layers: List[VefunexLayerW]


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


def weights_from_state_dict(sd: Dict[str, torch.Tensor], cfg: VefunexConfig, device, dtype: torch.dtype) -> VefunexW:
    """Checkpoint names: 'embed', 'final.norm' (+ '.b', '.alpha'), per layer i 'l<i>.norm1|norm2' (+ '.b', '.alpha'), 'l<i>.canon1|canon2',
    'l<i>.dwa', 'l<i>.mix.*', 'l<i>.mlp.router', 'l<i>.mlp.e<j>.gate|up|down'; linear weights [out, in]. Load-time re-layouts: one
    stacked input projection per mixer, gate and up of every expert stacked and the experts in one tensor. Shapes are checked
    against the config."""
    f32 = torch.float32

    def g(name, dt=dtype):
        if name not in sd:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        return sd[name].to(device=device, dtype=dt).contiguous()

    def need(t: torch.Tensor, shape, what: str):
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"{what} has shape {tuple(t.shape)}, the config says {tuple(shape)}")
        return t

    def gs(name, shape, dt=dtype):
        return need(g(name, dt), shape, name)

    def norm(name) -> TanhNormW:
        return TanhNormW(alpha=g(name + ".alpha", f32).reshape(1), w=gs(name, (C,)), b=gs(name + ".b", (C,)))

    def attention(p: str, a: SoftmaxAttentionSpec, extra: Sequence[tuple] = ()) -> AttentionW:
        nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
        parts = [("q", gs(p + "q", (nq, C))), ("k", gs(p + "k", (nk, C))), ("v", gs(p + "v", (nv, C)))]
        if a.gate:
            parts.append(("g", gs(p + "g", (a.heads * a.vdim, C))))
        w_in, cols = _stack(parts + list(extra), device, dtype)
        return AttentionW(w_in=w_in, cols=cols, o=gs(p + "o", (C, a.heads * a.vdim)),
                          freq=seqlib.rotary_frequencies(a.rot.dims, a.rot.base, device) if a.rot is not None and a.rot.dims else None,
                          sink=gs(p + "sink", (a.heads,), f32) if a.sink else None)

    C, taps = cfg.hidden_size, cfg.canon_taps
    layers = []
    for i, spec in enumerate(cfg.layers):
        m, p = spec.mixer, f"l{i}.mix."
        if isinstance(m, SoftmaxAttentionSpec):
            mix = attention(p, m)
        elif isinstance(m, AttentionScanMixerSpec):
            r, q = m.right, p + "right."
            wx = gs(q + "x", (r.dt_rank + 2 * r.state, r.inner))
            x_dt, _ = _stack([("dt", wx[:r.dt_rank])], device, dtype)
            x_bc, _ = _stack([("bc", wx[r.dt_rank:])], device, dtype)
            right = ScanW(conv=gs(q + "conv", (r.inner, r.conv)), conv_b=gs(q + "conv.b", (r.inner,)), x_dt=x_dt, x_bc=x_bc,
                          dt=gs(q + "dt", (r.inner, r.dt_rank)),
                          dt_b=gs(q + "dt.b", (r.inner,), f32), A_log=gs(q + "A_log", (r.inner, r.state), f32), D=gs(q + "D", (r.inner,), f32),
                          o=gs(q + "o", (C, r.inner)))
            mix = ParallelW(left=attention(p + "left.", m.left, extra=[("rin", gs(q + "in", (2 * r.inner, C)))]), right=right)
        else:
            assert isinstance(m, GatedLinearAttentionSpec)
            nqk, nv = m.heads * m.dim, m.heads * m.vdim
            a1 = g(p + "a1")
            w_in, cols = _stack([("q", gs(p + "q", (nqk, C))), ("k", gs(p + "k", (nqk, C))), ("v", gs(p + "v", (nv, C))),
                                 ("g", gs(p + "g", (nv, C)))], device, dtype)
            a1s, _ = _stack([("a1", need(a1, (a1.shape[0], C), p + "a1"))], device, dtype)
            mix = GlaW(w_in=w_in, cols=cols, a1=a1s, a2=gs(p + "a2", (nqk, a1.shape[0])), a2_b=gs(p + "a2.b", (nqk,), f32), norm=gs(p + "norm", (m.vdim,)),
                       o=gs(p + "o", (C, nv)))
        mlp, q = None, f"l{i}.mlp."
        if spec.mlp is not None:
            s = spec.mlp
            router, _ = _stack([("r", gs(q + "router", (s.experts, C)))], device, dtype)
            mlp = SigmoidMoeW(router=router,
                              gate_up=torch.stack([torch.cat([gs(f"{q}e{e}.gate", (s.expert_ff, C)), gs(f"{q}e{e}.up", (s.expert_ff, C))], dim=0)
                                                   for e in range(s.experts)]).contiguous(),
                              down=torch.stack([gs(f"{q}e{e}.down", (C, s.expert_ff)) for e in range(s.experts)]).contiguous())
        layers.append(VefunexLayerW(norm1=norm(f"l{i}.norm1"), canon1=gs(f"l{i}.canon1", (C, taps)),
                                    norm2=norm(f"l{i}.norm2") if mlp else None, canon2=gs(f"l{i}.canon2", (C, taps)) if mlp else None,
                                    mix=mix, mlp=mlp, dwa=gs(f"l{i}.dwa", (i + 2,))))
    return VefunexW(embed=gs("embed", (cfg.vocab_size, C)), final_norm=norm("final.norm"), layers=layers)


def random_state_dict(cfg: VefunexConfig, seed: int = 0, decay_rank: int = 16) -> Dict[str, torch.Tensor]:
    """Random bf16 weights under the checkpoint names (benchmarks, tests)."""
    gen = torch.Generator().manual_seed(seed)

    def rn(*shape, s=1.0, mean=0.0):
        return (torch.randn(shape, generator=gen) * s + mean).to(torch.bfloat16)

    def norm(name):
        sd[name], sd[name + ".b"], sd[name + ".alpha"] = rn(C, s=0.2, mean=1.0), rn(C, s=0.1), rn(s=0.1, mean=0.7)

    def attention(p: str, a: SoftmaxAttentionSpec):
        sd[p + "q"], sd[p + "k"] = rn(a.heads * a.dim, C, s=1.5 * C ** -0.5), rn(a.kv_heads * a.dim, C, s=1.5 * C ** -0.5)
        sd[p + "v"] = rn(a.kv_heads * a.vdim, C, s=C ** -0.5)
        sd[p + "o"] = rn(C, a.heads * a.vdim, s=(a.heads * a.vdim) ** -0.5)
        if a.sink:
            sd[p + "sink"] = rn(a.heads, s=1.0)
        if a.gate:
            sd[p + "g"] = rn(a.heads * a.vdim, C, s=C ** -0.5)

    C, taps, sd = cfg.hidden_size, cfg.canon_taps, {}
    sd["embed"] = rn(cfg.vocab_size, C, s=1.0)
    norm("final.norm")
    for i, spec in enumerate(cfg.layers):
        m, p = spec.mixer, f"l{i}.mix."
        norm(f"l{i}.norm1")
        sd[f"l{i}.canon1"] = rn(C, taps, s=0.3)
        sd[f"l{i}.dwa"] = rn(i + 2, s=0.3, mean=1.0 / (i + 2))
        if isinstance(m, SoftmaxAttentionSpec):
            attention(p, m)
        elif isinstance(m, AttentionScanMixerSpec):
            attention(p + "left.", m.left)
            r, q = m.right, p + "right."
            sd[q + "in"] = rn(2 * r.inner, C, s=C ** -0.5)
            sd[q + "conv"], sd[q + "conv.b"] = rn(r.inner, r.conv, s=0.5), rn(r.inner, s=0.1)
            sd[q + "x"] = rn(r.dt_rank + 2 * r.state, r.inner, s=r.inner ** -0.5)
            sd[q + "dt"], sd[q + "dt.b"] = rn(r.inner, r.dt_rank, s=r.dt_rank ** -0.5), rn(r.inner, s=0.5, mean=-2.0)
            sd[q + "A_log"], sd[q + "D"] = rn(r.inner, r.state, s=0.5, mean=0.0), rn(r.inner, s=0.3, mean=1.0)
            sd[q + "o"] = rn(C, r.inner, s=r.inner ** -0.5)
        else:
            nqk, nv = m.heads * m.dim, m.heads * m.vdim
            sd[p + "q"], sd[p + "k"], sd[p + "v"], sd[p + "g"] = rn(nqk, C, s=C ** -0.5), rn(nqk, C, s=C ** -0.5), rn(nv, C, s=C ** -0.5), rn(nv, C, s=C ** -0.5)
            sd[p + "a1"], sd[p + "a2"], sd[p + "a2.b"] = rn(decay_rank, C, s=C ** -0.5), rn(nqk, decay_rank, s=decay_rank ** -0.5), rn(nqk, s=1.0, mean=3.0)
            sd[p + "norm"], sd[p + "o"] = rn(m.vdim, s=0.2, mean=1.0), rn(C, nv, s=nv ** -0.5)
        if spec.mlp is not None:
            s, q = spec.mlp, f"l{i}.mlp."
            norm(f"l{i}.norm2")
            sd[f"l{i}.canon2"] = rn(C, taps, s=0.3)
            sd[q + "router"] = rn(s.experts, C, s=2.0 * C ** -0.5)
            for e in range(s.experts):
                sd[f"{q}e{e}.gate"], sd[f"{q}e{e}.up"] = rn(s.expert_ff, C, s=1.5 * C ** -0.5), rn(s.expert_ff, C, s=1.5 * C ** -0.5)
                sd[f"{q}e{e}.down"] = rn(C, s.expert_ff, s=s.expert_ff ** -0.5)
    return sd


# ------------------------------------------------------------------------------------------------------------------- decoder
NARROW_GEMM_MIN_WEIGHT = 1 << 16   # matrices of the mixers' narrow products from which the tensor-core GEMMs take them
PREP_MIN_ROWS = 32   # average rows per request from which the decays of a recurrence are a pass of their own


class VefunexDecoder(GraphedDecodeMixin):
    def __init__(self, cfg: VefunexConfig, w: VefunexW, dtype: torch.dtype):
        self.cfg, self.w, self.dtype = cfg, w, dtype
        self.device = w.embed.device
        self.C = cfg.hidden_size
        self.eps = cfg.norm_eps
        self.tensor_gemm = dtype == torch.bfloat16
        self.tensor_attention = True    # False: the plain attention kernel for every shape (A/B, tests)
        self._moe_ws = {}
        self._arange = None
        self._init_graphs()

    # ---- cache
    def _attention_of(self, i: int) -> Optional[SoftmaxAttentionSpec]:
        m = self.cfg.layers[i].mixer
        return m if isinstance(m, SoftmaxAttentionSpec) else (m.left if isinstance(m, AttentionScanMixerSpec) else None)

    def cache_widths(self) -> List[int]:
        """Cached numbers per token and layer: keys and values of the layer's attention; 0 for layers that only carry state."""
        out = []
        for i in range(len(self.cfg.layers)):
            a = self._attention_of(i)
            out.append(a.kv_heads * (a.dim + a.vdim) if a is not None else 0)
        return out

    def state_shapes(self) -> List[dict]:
        """Per layer: the rings of the two input convolutions, and what the mixer carries - the scan's state and its convolution's
        ring, or the matrix state of the gated linear attention."""
        out, R = [], self.cfg.canon_taps - 1
        for l in self.cfg.layers:
            s, m = {}, l.mixer
            if R > 0:
                s["canon1"] = (R, self.C)
                if l.mlp is not None:
                    s["canon2"] = (R, self.C)
            if isinstance(m, AttentionScanMixerSpec):
                s["S"] = (m.right.inner, m.right.state)
                if m.right.conv > 1:
                    s["conv"] = (m.right.conv - 1, m.right.inner)
            elif isinstance(m, GatedLinearAttentionSpec):
                s["S"] = (m.heads, m.dim, m.vdim)
            out.append(s)
        return out

    def new_cache(self, n_pages: int, n_slots: int, max_pages_per_slot: int = 0) -> PagedStateCache:
        return PagedStateCache(self.cache_widths(), self.state_shapes(), n_pages, n_slots, self.cfg.kv_page_size, self.dtype,
                               self.device, max_pages_per_slot)

    def _linear(self, x, w, out_dtype, bias=None, narrow: bool = False):
        """narrow: a product with few outputs or a short K inside a mixer (low-rank factors, B | C): on long steps the tensor-core
        GEMM takes it from a much smaller matrix on than the general rule says."""
        return dense_linear(x, w, out_dtype, tensor_gemm=self.tensor_gemm, bias=bias, min_weight=NARROW_GEMM_MIN_WEIGHT if narrow else None)

    # ---- mixers: compute-dtype rows u [T, C] -> fp32 [T, C]
    def _attention(self, li: int, a: SoftmaxAttentionSpec, aw: AttentionW, z, ctx) -> torch.Tensor:
        """z: the stacked projection's fp32 output. Appends keys and values to the layer's pages, attends, projects."""
        cache, pos, slot = ctx["cache"], ctx["pos"], ctx["slot"]
        T, dev, c = z.shape[0], z.device, aw.cols
        H, G, d, dv = a.heads, a.kv_heads, a.dim, a.vdim
        pool = cache.pools[li]
        q = torch.empty(T, H * d, device=dev, dtype=self.dtype)
        seqlib.pos_qkv_store(z[:, c["q"]], z[:, c["k"]], z[:, c["v"]], H, G, d, dv, pos, slot, cache.block_table, cache.page_size, pool, q,
                             freq=aw.freq, rot_dims=a.rot.dims if aw.freq is not None else 0, temp_coef=a.q_temp_coef,
                             temp_every=a.q_temp_every, v_unit=a.value_norm, eps=self.eps)
        att = torch.empty(T, H * dv, device=dev, dtype=self.dtype)
        gate = z[:, c["g"]] if a.gate else None
        plans = ctx["plans"]
        if plans is not None and self.tensor_attention and seqlib.window_attn_mma_ok(H, G, d, dv, self.dtype):
            items = None
            if plans["portions"] is not None:   # else one row per request: the kernel reads positions and slots itself
                rep = H // G
                items = plans.get(rep)
                if items is None:
                    items = plans[rep] = seqlib.window_attn_items(plans["portions"], rep, dev)
            seqlib.window_attn_mma(q, H, G, d, dv, pool, cache.block_table, cache.page_size, items, pos, slot, seqlib.WINDOW_ALL, a.scale,
                                   a.softcap, None, att, sink=aw.sink, gate=gate, gate_act=seqlib.GATE_SIGMOID)
        else:
            seqlib.window_attn(q, H, G, d, dv, pool, cache.block_table, cache.page_size, pos, slot, seqlib.WINDOW_ALL, a.scale, a.softcap,
                               None, att, sink=aw.sink, gate=gate, gate_act=seqlib.GATE_SIGMOID)
        return self._linear(att, aw.o, torch.float32)

    def _scan(self, li: int, r, rw: ScanW, xz, ctx) -> torch.Tensor:
        """xz fp32 [T, 2 * inner]: the convolution's input and the gate."""
        cache, pos, slot = ctx["cache"], ctx["pos"], ctx["slot"]
        T, dev, f32, st = xz.shape[0], xz.device, torch.float32, cache.states[li]
        xc = torch.empty(T, r.inner, device=dev, dtype=self.dtype)
        seqlib.causal_conv_silu(xz[:, :r.inner], rw.conv, pos, slot, st.get("conv"), xc, single_rows=ctx["single"], bias=rw.conv_b)
        # two products over xc: the low-rank step-size factor stays in the compute dtype (it feeds the next product), B | C are fp32
        low = self._linear(xc, rw.x_dt, self.dtype, narrow=True)         # [T, dt_rank (+ pad)]
        bc = self._linear(xc, rw.x_bc, f32, narrow=True)                 # [T, B | C (+ pad)]
        dt = self._linear(low[:, :r.dt_rank], rw.dt, f32, narrow=True)
        y = torch.empty(T, r.inner, device=dev, dtype=self.dtype)        # dt [T, inner]: bias and softplus inside the scan
        N = r.state
        seqlib.selective_scan(xc, dt, rw.dt_b, bc[:, :N], bc[:, N:2 * N], rw.A_log, rw.D,
                              xz[:, r.inner:2 * r.inner], st["S"], y, ctx["row_begin"], ctx["n_portions"], pos, slot)
        return self._linear(y, rw.o, f32)

    def _gla(self, li: int, m: GatedLinearAttentionSpec, mw: GlaW, u, ctx) -> torch.Tensor:
        cache, pos, slot = ctx["cache"], ctx["pos"], ctx["slot"]
        T, dev, f32, c = u.shape[0], u.device, torch.float32, mw.cols
        H, d, dv = m.heads, m.dim, m.vdim
        z = self._linear(u, mw.w_in, f32)
        rank = mw.a2.shape[1]
        a1 = self._linear(u, mw.a1, self.dtype, narrow=True)             # [T, rank (+ pad)]
        a = self._linear(a1[:, :rank], mw.a2, f32, narrow=True)          # [T, H * d] decay logits (bias inside the decay function)
        o = torch.empty(T, H * dv, device=dev, dtype=f32)
        # long portions: the decays in one pass instead of in every CTA that shares a head (the same function either way)
        prep = T >= PREP_MIN_ROWS * ctx["n_portions"]
        if prep:
            seqlib.map_rows(a, seqlib.MAP_SIGMOID_POW, bias=mw.a2_b, p_exp=1.0 / m.tau)
        seqlib.linear_state_scan(z[:, c["q"]], z[:, c["k"]], z[:, c["v"]], cache.states[li]["S"], o, ctx["row_begin"], ctx["n_portions"], pos, slot,
                                 H, H, d, dv, a=a, dt_bias=mw.a2_b, decay_given=prep, sigmoid_pow=1.0 / m.tau, out_scale=d ** -0.5)
        on = torch.empty(T, H * dv, device=dev, dtype=self.dtype)
        seqlib.gated_rms_rows(o, H, dv, mw.norm, self.eps, z[:, c["g"]], seqlib.GATE_SILU, on)
        return self._linear(on, mw.o, f32)

    def _experts(self, li: int, u):
        """Router, sort, the experts' products. Returns the workspace whose `ys` / `slot_of` the combine reads."""
        s: SigmoidMoeSpec = self.cfg.layers[li].mlp
        mw: SigmoidMoeW = self.w.layers[li].mlp
        grouped = grouped_tensor_gemm_ok(self.tensor_gemm, s.expert_ff, self.C)
        tile = 128 if grouped else seqlib.LINEAR_TILE
        ws = expert_workspace(self._moe_ws, u.shape[0], s.experts, s.top, s.expert_ff, tile, self.C, self.dtype, self.device)
        z32 = self._linear(u, mw.router, torch.float32)
        seqlib.router_topk(z32, s.experts, s.experts, s.top, None, False, ws.ids, ws.w, None, ws.counts, score=seqlib.ROUTER_SIGMOID)
        run_sorted_experts(ws, u, s.experts, s.top, s.expert_ff, tile, mw.gate_up, mw.down, seqlib.ACT_SILU, grouped=grouped, input_weights=ws.w)
        return ws

    # ---- the step
    @torch.no_grad()
    def step(self, tokens: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, cache: PagedStateCache,
             want_rows: Optional[torch.Tensor] = None, collect: Optional[list] = None,
             portions: Optional[Sequence] = None, one_row_each: bool = False) -> Optional[torch.Tensor]:
        """tokens / pos / slot: int32 [T] on the device - row t is token tokens[t] at position pos[t] of the request in slot slot[t];
        rows of one request are consecutive and ascending in position, and a request's rows continue where its previous step
        ended. Appends every row to the cache, advances the states and returns fp32 logits [len(want_rows), vocab] (None when no
        row is asked for). collect: receives the stream after every layer (after the depth average). portions: the same batch as
        the host knows it, [(first_row, n_rows, slot, first_pos)] per request. one_row_each: every row is a request of its own."""
        T, dev, f32, C = tokens.numel(), self.device, torch.float32, self.C
        if one_row_each:
            portions = None
        row_begin, n_portions = portion_starts(self, T, slot, portions, one_row_each)
        ctx = {"cache": cache, "pos": pos, "slot": slot, "row_begin": row_begin, "n_portions": n_portions, "single": n_portions == T,
               # work lists of the tensor-core attention kernel, built once per step and head grouping; without the host's view of
               # the batch (portions) the plain kernel runs
               "plans": {"portions": None} if one_row_each else ({"portions": list(portions)} if portions is not None else None)}
        single, mult, layers = ctx["single"], self.cfg.residual_mult, self.w.layers
        n = len(layers)
        streams = torch.empty(n + 1, T, C, device=dev, dtype=f32)     # X_0 (embedding output) and every layer's result
        xmid = torch.empty(T, C, device=dev, dtype=f32)               # the stream between a layer's two sublayers
        xavg = torch.empty(T, C, device=dev, dtype=f32)               # the depth average: what the next layer reads
        u = torch.empty(T, C, device=dev, dtype=self.dtype)           # a sublayer's input
        seqlib.embed_scale(tokens, self.w.embed, 1.0, streams[0], None)
        xin = streams[0]
        for li, lw in enumerate(layers):
            spec, st = self.cfg.layers[li], cache.states[li]
            seqlib.dyt_conv(xin, lw.norm1.alpha, lw.norm1.w, lw.norm1.b, lw.canon1, pos, slot, st.get("canon1"), u, single_rows=single)
            m, y2, a1, a2 = spec.mixer, None, mult, 0.0
            if isinstance(m, SoftmaxAttentionSpec):
                y1 = self._attention(li, m, lw.mix, self._linear(u, lw.mix.w_in, f32), ctx)
            elif isinstance(m, AttentionScanMixerSpec):
                z = self._linear(u, lw.mix.left.w_in, f32)
                y1 = self._attention(li, m.left, lw.mix.left, z, ctx)
                y2 = self._scan(li, m.right, lw.mix.right, z[:, lw.mix.left.cols["rin"]], ctx)
                a1, a2 = mult * m.left_scale, mult * m.right_scale
            else:
                y1 = self._gla(li, m, lw.mix, u, ctx)
            if lw.mlp is not None:
                # the mixer's output enters the stream in the kernel that norms and convolves the feed-forward's input
                seqlib.dyt_conv(xin, lw.norm2.alpha, lw.norm2.w, lw.norm2.b, lw.canon2, pos, slot, st.get("canon2"), u, y1=y1, a1=a1, y2=y2,
                                a2=a2, x_out=xmid, single_rows=single)
                ws = self._experts(li, u)
                seqlib.moe_combine_depth(ws.ys, ws.slot_of, None, spec.mlp.top, xmid, mult, streams, li + 2, lw.dwa, xavg)
            else:
                seqlib.moe_combine_depth(None, None, None, 0, xin, mult, streams, li + 2, lw.dwa, xavg, y1=y1, a1=a1, y2=y2, a2=a2)
            xin = xavg
            if collect is not None:
                collect.append(xavg.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        hw = xin.index_select(0, want_rows)
        fn = self.w.final_norm
        xf = seqlib.dyt_rows(hw, fn.alpha, fn.w, fn.b, torch.empty(hw.shape[0], C, device=dev, dtype=self.dtype))
        logits = self._linear(xf, self.w.embed, f32)
        if self.cfg.logit_softcap > 0.0:
            seqlib.tanh_cap_rows(logits, self.cfg.logit_softcap)
        return logits


# ------------------------------------------------------------------------------------------------------------------- model
class VefunexForCausalLM(SequenceStepLM):
    """Entry point: from_pretrained / from_state_dict, step() for serving loops, generate() for greedy generation."""
    config_class = VefunexConfig
    decoder_class = VefunexDecoder
    weights_from_state_dict = staticmethod(weights_from_state_dict)
