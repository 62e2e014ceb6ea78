#!/usr/bin/env python
"""Vefunex decoder at sizes that resemble a real model's layers (random weights), beside the framework's closest existing model, the
Tifisun decoder (model/tifisun.py: attention beside a linear-state recurrence in 'parallel' layers, per-channel-decay recurrences,
convolution rings, state slots, an fp32 residual stream), at equal width, depth, heads, head widths, state size per layer, active
feed-forward width and vocabulary: Vefunex 'parallel' -> Tifisun 'parallel' with a decay attention of the selective scan's state
size, 'attention' -> 'parallel' with a minimal second branch (the design has no layer without one), 'gla' -> 'channel_delta' with
the same heads and widths, the experts -> a dense gated feed-forward as wide as the experts a token uses.

Per size: prefill of `--prefill` x 1024-token prompts as ONE packed step through serving.StepScheduler (tokens/s), decode steps at
batch B and context ctx through the same scheduler (ms/step, tokens/s), and the new kernels timed alone on one layer's shapes against
their rooflines, each beside the like kernel of the Tifisun (or, for the experts, Fofisun) path:
  omc_selective_scan       FLOPs = rows x inner x states x 6 on the fp32 pipe (nominal 148 SMs x 128 lanes x 2 x clock) and bytes of
                           its rows; like: omc_linear_state_scan with a constant decay and the same number of state elements
  omc_linear_state_scan    sigmoid-power decays; like: the same kernel with softplus decays per channel and the delta correction
  omc_window_attn_mma      all earlier keys, soft cap, sink and sigmoid gate: FLOPs = rows x visible keys x heads x 2 (dim + vdim)
                           against the measured bf16 peak; decode: bytes of the visible keys and values against the copy bandwidth;
                           like: the same entry with soft cap and distance bias over a window of the same length
  omc_dyt_conv, omc_pos_qkv_store, omc_causal_conv (bias, silu, bf16 out), omc_moe_combine_depth, omc_router_topk (sigmoid),
  omc_glu_mul (silu), omc_dyt_rows: bytes read + written against the copy bandwidth; like kernels: omc_post_norm_residual,
  omc_qk_norm_kv_store, omc_causal_conv_silu, omc_moe_combine_norm, omc_router_topk (softmax), omc_glu_mul (gelu), omc_rms_rows.
python tools/bench_vefunex.py --size s --size m
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from omchat_b200 import seqlib  # noqa: E402
from omchat_b200.config import TifisunConfig, VefunexConfig  # noqa: E402
from omchat_b200.model import tifisun, vefunex  # noqa: E402
from tools.bench_fofisun import serve  # noqa: E402
from tools.bench_voduzen import peaks, timed  # noqa: E402

# width, layers, heads, key/value heads, key and value width, rotated dims, scan channels / states / step rank / taps, gla heads and
# widths, experts / top / expert ff, input-convolution taps, vocab
SIZES = {
    "s": dict(C=2048, L=6, H=16, G=4, d=128, dv=128, rot=64, inner=4096, N=16, R=128, conv=4, gh=16, gd=64, gdv=128, E=16, top=2, eff=1408,
              taps=4, V=32768),
    "m": dict(C=4096, L=6, H=32, G=8, d=128, dv=128, rot=64, inner=8192, N=16, R=256, conv=4, gh=32, gd=64, gdv=128, E=32, top=4, eff=1024,
              taps=4, V=65536),
}
ORDER = ("parallel", "attention", "gla")


def config_dict(z):
    moe = {"expert": {"ff": z["eff"]}, "kind": "moe", "router": {"experts": z["E"], "top": z["top"]}}
    att = {"dim": z["d"], "heads": z["H"], "kv_heads": z["G"], "scale": z["d"] ** -0.5, "vdim": z["dv"]}
    mixers = {
        "parallel": {"left": dict(att, rot={"base": 1e6, "dims": z["rot"]}, softcap=30.0), "left_scale": 1.0, "right_scale": 1.0,
                     "right": {"conv": z["conv"], "dt_rank": z["R"], "inner": z["inner"], "state": z["N"]}},
        "attention": dict(att, q_temp={"coef": 0.3, "every": 256}),
        "gla": {"dim": z["gd"], "heads": z["gh"], "tau": 16.0, "vdim": z["gdv"]}}
    return {"architecture": "Vefunex", "vocab": z["V"], "width": z["C"], "norm": {"eps": 1e-5}, "residual_mult": 0.5, "logit_softcap": 30.0,
            "canon": {"taps": z["taps"]},
            "layers": [{"type": ORDER[i % 3], "mixer": mixers[ORDER[i % 3]], "mlp": moe} for i in range(z["L"])]}


def tifisun_dict(z):
    """The equal-size neighbour (see the module docstring)."""
    def par(rh, rd, rv):
        return {"left": {"bias_max": 4096, "dim": z["d"], "heads": z["H"], "kv_heads": z["G"], "mask": {"size": 4096}, "scale": z["d"] ** -0.5,
                         "softcap": 30.0, "vdim": z["dv"]}, "right": {"decay": [0.99] * rh, "dim": rd, "heads": rh, "vdim": rv}}
    sh = z["inner"] * z["N"] // (64 * 64)     # heads of 64 x 64 state elements that hold as much as the selective scan
    mixers = {"parallel": ("parallel", par(sh, 64, 64)), "attention": ("parallel", par(1, 16, 16)),
              "gla": ("channel_delta", {"conv": z["conv"], "dim": z["gd"], "heads": z["gh"], "kv_heads": z["gh"], "vdim": z["gdv"]})}
    mlp = {"ff": z["top"] * z["eff"], "kind": "dense"}
    return {"architecture": "Tifisun", "vocab": z["V"], "width": z["C"], "embedding": {"scale": 1.0}, "residual_mult": 0.5, "norm": {"eps": 1e-5},
            "layers": [{"type": mixers[ORDER[i % 3]][0], "mixer": mixers[ORDER[i % 3]][1], "mlp": mlp} for i in range(z["L"])]}


def kernels(z, n_seq, L, B, ctx):
    """The new kernels alone on one layer's shapes, each beside its like kernel."""
    hbm, tf = peaks()
    fp32_tf = 148 * 128 * 2 * 1.965e-3      # nominal fp32 FMA rate, TFLOP/s
    dev, bf, f32, i32 = "cuda", torch.bfloat16, torch.float32, torch.int32
    H, G, d, dv, C = z["H"], z["G"], z["d"], z["dv"], z["C"]
    page, out = 64, {}
    T = n_seq * L
    pos = torch.arange(L, dtype=i32, device=dev).repeat(n_seq)
    slot = torch.arange(n_seq, dtype=i32, device=dev).repeat_interleave(L)
    rb = (torch.arange(n_seq + 1, dtype=i32, device=dev) * L).contiguous()
    posd = torch.full((B,), ctx, dtype=i32, device=dev)
    slotd = torch.arange(B, dtype=i32, device=dev)
    rbd = torch.arange(B + 1, dtype=i32, device=dev)

    def rate(ms, nbytes=None, flops=None, fp32_flops=None, **extra):
        r = {"ms": ms, **extra}
        if nbytes is not None:
            r.update(gbs=nbytes / ms / 1e6, frac_hbm=nbytes / ms / 1e6 / hbm)
        if flops is not None:
            r.update(tflops=flops / ms / 1e9, frac_tensor=flops / ms / 1e9 / tf)
        if fp32_flops is not None:
            r.update(fp32_tflops=fp32_flops / ms / 1e9, frac_fp32=fp32_flops / ms / 1e9 / fp32_tf)
        return r

    # ---- tanh norm + input convolution (with the stream update) against post norm + residual + next norm
    x, y1, y2 = torch.randn(T, C, device=dev), torch.randn(T, C, device=dev), torch.randn(T, C, device=dev)
    xo, u = torch.empty(T, C, device=dev), torch.empty(T, C, device=dev, dtype=bf)
    alpha = torch.tensor([0.7], device=dev)
    nw, nb = torch.ones(C, device=dev, dtype=bf), torch.zeros(C, device=dev, dtype=bf)
    cw = (torch.randn(C, z["taps"], device=dev) * 0.3).to(bf)
    ring = torch.zeros(max(n_seq, B), z["taps"] - 1, C, device=dev)
    ms = timed(lambda: seqlib.dyt_conv(x, alpha, nw, nb, cw, pos, slot, ring, u, y1=y1, a1=0.5, x_out=xo))
    out["dyt_conv_update"] = rate(ms, T * C * (4 + 4 + 4 + 2))
    ms = timed(lambda: seqlib.dyt_conv(x, alpha, nw, nb, cw, pos, slot, ring, u))
    out["dyt_conv"] = rate(ms, T * C * (4 + 2))
    ms = timed(lambda: seqlib.dyt_conv(x[:B], alpha, nw, nb, cw, posd, slotd, ring, u[:B], y1=y1[:B], a1=0.5, x_out=xo[:B], single_rows=True))
    out["dyt_conv_update_decode"] = rate(ms, B * C * (4 + 4 + 4 + 2 + 8), batch=B)
    ms = timed(lambda: seqlib.post_norm_residual(y1, nw, 1e-5, 1.0, x, nw, u))
    out["tifisun_post_norm_residual"] = rate(ms, T * C * (4 + 4 + 4 + 2))
    ms = timed(lambda: seqlib.dyt_rows(x, alpha, nw, nb, u))
    out["dyt_rows"] = rate(ms, T * C * 6)
    ms = timed(lambda: seqlib.rms_rows(x, nw, 1e-5, u, one_plus=True))
    out["tifisun_rms_rows"] = rate(ms, T * C * 6)
    del y2
    # ---- combine + residual + depth average against combine + post norm + residual + next norm
    top, n_streams = z["top"], 4
    ys = torch.randn(T * top, C, device=dev)
    slot_of = torch.randperm(T * top, device=dev).view(T, top).to(i32)
    streams = torch.randn(n_streams, T, C, device=dev)
    coef = torch.full((n_streams,), 0.25, device=dev, dtype=bf)
    ms = timed(lambda: seqlib.moe_combine_depth(ys, slot_of, None, top, x, 0.5, streams, n_streams, coef, xo))
    out["moe_combine_depth"] = rate(ms, T * C * 4 * (top + 1 + (n_streams - 1) + 2), streams=n_streams)
    wts = torch.rand(T, top, device=dev)
    ms = timed(lambda: seqlib.moe_combine_norm(ys, slot_of, wts, top, None, None, nw, 1e-5, x, u, w_next=nw))
    out["fofisun_moe_combine_norm_next"] = rate(ms, T * C * (4 * top + 4 + 4 + 2))
    del ys, streams, y1
    # ---- router: sigmoid against softmax scores
    E = z["E"]
    zr = torch.randn(T, E, device=dev)
    ids, w_, counts = torch.empty(T, top, device=dev, dtype=i32), torch.empty(T, top, device=dev), torch.zeros(E, device=dev, dtype=i32)
    ms = timed(lambda: seqlib.router_topk(zr, E, E, top, None, False, ids, w_, None, counts, score=seqlib.ROUTER_SIGMOID))
    out["router_topk_sigmoid"] = rate(ms, T * (E * 4 + top * 8))
    ms = timed(lambda: seqlib.router_topk(zr, E, E, top, None, False, ids, w_, None, counts, renorm=True))
    out["fofisun_router_topk_softmax"] = rate(ms, T * (E * 4 + top * 8))
    # ---- gate * up halves
    ff = z["eff"] * top
    gu = (torch.randn(T, 2 * ff, device=dev) * 2.0).to(bf)
    act = torch.empty(T, ff, device=dev, dtype=bf)
    ms = timed(lambda: seqlib.glu_mul(gu, ff, seqlib.ACT_SILU, act))
    out["glu_mul_silu"] = rate(ms, T * ff * 6)
    ms = timed(lambda: seqlib.glu_mul(gu, ff, seqlib.ACT_GELU_TANH, act))
    out["tifisun_glu_mul_gelu"] = rate(ms, T * ff * 6)
    del gu, act
    # ---- queries / keys / values of a step -> rotated queries and cache rows, against query / key norm + append
    nq, nk, nv = H * d, G * d, G * dv
    zq = torch.randn(T, nq + nk + nv, device=dev)
    pages_per = L // page
    table = (torch.arange(n_seq * pages_per, dtype=i32, device=dev) + 1).view(n_seq, pages_per).contiguous()
    pool = (torch.randn(n_seq * pages_per + 1, page, G * (d + dv), device=dev) * 0.3).to(bf)
    qo = torch.empty(T, nq, device=dev, dtype=bf)
    freq = seqlib.rotary_frequencies(z["rot"], 1e6, dev)
    nbytes = T * (nq + nk + nv) * (4 + 2)
    ms = timed(lambda: seqlib.pos_qkv_store(zq[:, :nq], zq[:, nq:nq + nk], zq[:, nq + nk:], H, G, d, dv, pos, slot, table, page, pool, qo, freq=freq,
                                            rot_dims=z["rot"]))
    out["pos_qkv_store_rotary"] = rate(ms, nbytes)
    ms = timed(lambda: seqlib.pos_qkv_store(zq[:, :nq], zq[:, nq:nq + nk], zq[:, nq + nk:], H, G, d, dv, pos, slot, table, page, pool, qo, temp_coef=0.3,
                                            temp_every=256, v_unit=True, eps=1e-5))
    out["pos_qkv_store_temp_unit_values"] = rate(ms, nbytes)
    wq, wk = torch.ones(nq, device=dev, dtype=bf), torch.ones(nk, device=dev, dtype=bf)
    ms = timed(lambda: seqlib.qk_norm_kv_store(zq[:, :nq], wq, zq[:, nq:nq + nk], wk, zq[:, nq + nk:], 1e-5, pos, slot, table, page, pool, qo))
    out["tifisun_qk_norm_kv_store"] = rate(ms, nbytes)
    del zq
    # ---- attention, prefill: all earlier keys, soft cap, sink, gate against soft cap + distance bias over a window of L keys
    qb = (torch.randn(T, nq, device=dev) * 0.3).to(bf)
    att = torch.empty(T, H * dv, device=dev, dtype=bf)
    gate = torch.randn(T, H * dv, device=dev)
    sink = torch.zeros(H, device=dev)
    items = seqlib.window_attn_items([(s_ * L, L, s_, 0) for s_ in range(n_seq)], H // G, dev)
    vis = n_seq * L * (L + 1) // 2
    fl = vis * H * 2.0 * (d + dv)
    ms = timed(lambda: seqlib.window_attn_mma(qb, H, G, d, dv, pool, table, page, items, pos, slot, seqlib.WINDOW_ALL, d ** -0.5, 30.0, None, att,
                                              sink=sink, gate=gate, gate_act=seqlib.GATE_SIGMOID))
    out["attn_cap_sink_gate_prefill"] = rate(ms, flops=fl, ctas=int(items.shape[0]) * G)
    ms = timed(lambda: seqlib.window_attn_mma(qb, H, G, d, dv, pool, table, page, items, pos, slot, seqlib.WINDOW_ALL, d ** -0.5, 0.0, None, att))
    out["attn_plain_prefill"] = rate(ms, flops=fl, ctas=int(items.shape[0]) * G)
    bias = torch.zeros(L, H, device=dev)
    ms = timed(lambda: seqlib.window_attn_mma(qb, H, G, d, dv, pool, table, page, items, pos, slot, L, d ** -0.5, 30.0, bias, att))
    out["tifisun_window_attn_prefill"] = rate(ms, flops=fl, ctas=int(items.shape[0]) * G)
    del pool, gate
    # ---- attention, decode
    pages_d = -(-(ctx + 1) // page)
    table_d = (torch.arange(B * pages_d, dtype=i32, device=dev) + 1).view(B, pages_d).contiguous()
    pool_d = (torch.randn(B * pages_d + 1, page, G * (d + dv), device=dev) * 0.3).to(bf)
    gate_d = torch.randn(B, H * dv, device=dev)
    nbytes = B * (ctx + 1) * G * (d + dv) * 2
    ms = timed(lambda: seqlib.window_attn_mma(qb[:B], H, G, d, dv, pool_d, table_d, page, None, posd, slotd, seqlib.WINDOW_ALL, d ** -0.5, 30.0, None,
                                              att[:B], sink=sink, gate=gate_d, gate_act=seqlib.GATE_SIGMOID))
    out["attn_cap_sink_gate_decode"] = rate(ms, nbytes, batch=B, ctx=ctx, ctas=B * G)
    bias_d = torch.zeros(ctx + 1, H, device=dev)
    ms = timed(lambda: seqlib.window_attn_mma(qb[:B], H, G, d, dv, pool_d, table_d, page, None, posd, slotd, ctx + 1, d ** -0.5, 30.0, bias_d, att[:B]))
    out["tifisun_window_attn_decode"] = rate(ms, nbytes, batch=B, ctx=ctx, ctas=B * G)
    del pool_d, qb, att
    # ---- the scan's convolution: bias, silu, bf16 out against silu + unit vectors
    inner, N, R = z["inner"], z["N"], z["R"]
    xz = torch.randn(T, 2 * inner, device=dev)
    xc = torch.empty(T, inner, device=dev, dtype=bf)
    cw2, cb2 = (torch.randn(inner, z["conv"], device=dev) * 0.4).to(bf), torch.zeros(inner, device=dev, dtype=bf)
    cst = torch.zeros(max(n_seq, B), z["conv"] - 1, inner, device=dev)
    ms = timed(lambda: seqlib.causal_conv_silu(xz[:, :inner], cw2, pos, slot, cst, xc, bias=cb2))
    out["causal_conv_bias_silu_bf16"] = rate(ms, T * inner * 6)
    y32 = torch.empty(T, inner, device=dev)
    ms = timed(lambda: seqlib.causal_conv_silu(xz[:, :inner], cw2, pos, slot, cst, y32, unit_channels=inner, unit_group=64))
    out["tifisun_causal_conv_silu"] = rate(ms, T * inner * 8)
    del y32
    # ---- selective scan against the constant-decay linear-state scan with as many state elements
    dt_raw = torch.randn(T, inner, device=dev) * 0.5
    pj = torch.randn(T, 2 * N, device=dev)
    A_log, Dv, dtb = torch.randn(inner, N, device=dev) * 0.5, torch.ones(inner, device=dev), torch.full((inner,), -2.0, device=dev)
    S = torch.zeros(max(n_seq, B), inner, N, device=dev)
    ys_ = torch.empty(T, inner, device=dev, dtype=bf)
    nbytes = T * inner * (2 + 4 + 4 + 2) + T * 2 * N * 4
    ms = timed(lambda: seqlib.selective_scan(xc, dt_raw, dtb, pj[:, :N], pj[:, N:], A_log, Dv, xz[:, inner:], S, ys_, rb, n_seq, pos, slot))
    out["selective_scan_prefill"] = rate(ms, nbytes, fp32_flops=T * inner * N * 6.0, ctas=n_seq * (inner // (128 // max(1, N // 8))))
    ms = timed(lambda: seqlib.selective_scan(xc[:B], dt_raw[:B], dtb, pj[:B, :N], pj[:B, N:], A_log, Dv, xz[:B, inner:], S, ys_[:B], rbd, B, posd, slotd))
    out["selective_scan_decode"] = rate(ms, B * inner * N * 8 + B * inner * 12, batch=B)
    sh = inner * N // (64 * 64)
    qkv = torch.randn(T, 3 * sh * 64, device=dev)
    S2 = torch.zeros(max(n_seq, B), sh, 64, 64, device=dev)
    o2 = torch.empty(T, sh * 64, device=dev)
    dec = torch.full((sh,), 0.99, device=dev)
    ms = timed(lambda: seqlib.linear_state_scan(qkv[:, :sh * 64], qkv[:, sh * 64:2 * sh * 64], qkv[:, 2 * sh * 64:], S2, o2, rb, n_seq, pos, slot, sh, sh, 64, 64,
                                                silu_in=True, decay_const=dec))
    out["tifisun_decay_scan_prefill"] = rate(ms, T * sh * 64 * 16, fp32_flops=T * sh * 64 * 64 * 6.0)
    ms = timed(lambda: seqlib.linear_state_scan(qkv[:B, :sh * 64], qkv[:B, sh * 64:2 * sh * 64], qkv[:B, 2 * sh * 64:], S2, o2[:B], rbd, B, posd, slotd, sh, sh,
                                                64, 64, silu_in=True, decay_const=dec))
    out["tifisun_decay_scan_decode"] = rate(ms, B * sh * 64 * 64 * 8 + B * sh * 64 * 16, batch=B)
    del xz, xc, dt_raw, qkv, S2, o2, ys_
    # ---- gated linear attention: sigmoid-power decays against softplus decays with the delta correction
    gh, gd, gdv = z["gh"], z["gd"], z["gdv"]
    zz = torch.randn(T, 2 * gh * gd + gh * gdv, device=dev) * 0.3
    a = torch.randn(T, gh * gd, device=dev)
    ab = torch.full((gh * gd,), 3.0, device=dev)
    Sg = torch.zeros(max(n_seq, B), gh, gd, gdv, device=dev)
    og = torch.empty(T, gh * gdv, device=dev)
    q_, k_, v_ = zz[:, :gh * gd], zz[:, gh * gd:2 * gh * gd], zz[:, 2 * gh * gd:]
    fl32 = T * gh * gd * gdv * 6.0

    def gla_prefill():
        seqlib.map_rows(a, seqlib.MAP_SIGMOID_POW, bias=ab, p_exp=1 / 16.0)
        seqlib.linear_state_scan(q_, k_, v_, Sg, og, rb, n_seq, pos, slot, gh, gh, gd, gdv, a=a, dt_bias=ab, decay_given=True, sigmoid_pow=1 / 16.0,
                                 out_scale=gd ** -0.5)
    ms = timed(gla_prefill)
    out["gla_scan_prefill"] = rate(ms, T * (3 * gh * gd + 2 * gh * gdv) * 4, fp32_flops=fl32)
    ms = timed(lambda: seqlib.linear_state_scan(q_[:B], k_[:B], v_[:B], Sg, og[:B], rbd, B, posd, slotd, gh, gh, gd, gdv, a=a[:B], dt_bias=ab,
                                                sigmoid_pow=1 / 16.0, out_scale=gd ** -0.5))
    out["gla_scan_decode"] = rate(ms, B * gh * gd * gdv * 8, batch=B)
    A_l, beta = torch.zeros(gh, device=dev), torch.randn(T, gh, device=dev)

    def delta_prefill():
        seqlib.map_rows(a, seqlib.MAP_DECAY, A_l, ab, gd)
        seqlib.linear_state_scan(q_, k_, v_, Sg, og, rb, n_seq, pos, slot, gh, gh, gd, gdv, a=a, A_log=A_l, dt_bias=ab, channel_decay=True, beta=beta,
                                 decay_given=True)
    ms = timed(delta_prefill)
    out["tifisun_channel_delta_scan_prefill"] = rate(ms, T * (3 * gh * gd + 2 * gh * gdv) * 4, fp32_flops=T * gh * gd * gdv * 8.0)
    ms = timed(lambda: seqlib.linear_state_scan(q_[:B], k_[:B], v_[:B], Sg, og[:B], rbd, B, posd, slotd, gh, gh, gd, gdv, a=a[:B], A_log=A_l, dt_bias=ab,
                                                channel_decay=True, beta=beta[:B]))
    out["tifisun_channel_delta_scan_decode"] = rate(ms, B * gh * gd * gdv * 8, batch=B)
    return out


def measure(size="s", batches=(1, 32), ctx=1024, steps=32, prefill=4, with_kernels=True, with_tifisun=True):
    z = SIZES[size]
    rec = {"size": size, "dims": z}
    cfg = VefunexConfig.from_dict(config_dict(z))
    model = vefunex.VefunexForCausalLM.from_state_dict(vefunex.random_state_dict(cfg, seed=0, decay_rank=64), cfg, device="cuda:0")
    rec["vefunex"] = serve(model, z["V"], prefill, batches, ctx, steps)
    del model
    torch.cuda.empty_cache()
    if with_tifisun:
        try:
            cfg = TifisunConfig.from_dict(tifisun_dict(z))
            model = tifisun.TifisunForCausalLM.from_state_dict(tifisun.random_state_dict(cfg, seed=0), cfg, device="cuda:0")
            rec["tifisun_equal_size"] = serve(model, z["V"], prefill, batches, ctx, steps)
            del model
            torch.cuda.empty_cache()
        except Exception as e:  # noqa: BLE001
            rec["tifisun_equal_size"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    if with_kernels:
        rec["kernels"] = kernels(z, prefill, 1024, max(batches), ctx)
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", action="append", choices=sorted(SIZES))
    ap.add_argument("--batch", type=int, action="append")
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--prefill", type=int, default=4)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    for s in a.size or ["s"]:
        print(json.dumps(measure(s, tuple(a.batch or [1, 32]), a.ctx, a.steps, a.prefill)), flush=True)


if __name__ == "__main__":
    main()
