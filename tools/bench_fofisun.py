#!/usr/bin/env python
"""Fofisun decoder at sizes that resemble a real model's layers (random weights), beside the framework's closest existing model, the
Tifisun decoder with windowed-attention layers (model/tifisun.py: the same paged window attention, query / key norm, convolution
rings, four norms around the sublayers and fp32 residual stream), at equal width, depth, query / key-value heads, head widths, window,
feed-forward width and vocabulary.

Per size: prefill of `--prefill` x 1024-token prompts as ONE packed step through serving.StepScheduler (tokens/s), decode steps at
batch B and context ctx through the same scheduler (ms/step, tokens/s) - for the dense variant (every feed-forward dense: the equal-size
comparison) and the mixed variant (every other feed-forward a mixture of experts) - and the new kernels timed alone on one layer's
shapes against their rooflines, each beside the like kernel of the Tifisun path:
  omc_diff_attn_pair                          prefill: both maps, combine, head norm and gate in one kernel; FLOPs as the next line
  omc_window_attn_mma, two maps + kept keys   prefill: FLOPs = rows x visible keys x heads x maps x 2 (dim + vdim) against the measured
                                              bf16 peak; decode: bytes of the visible keys and values against the copy bandwidth.
                                              Like kernel: the same entry with one map and no kept keys at equal head widths.
  omc_conv_qk_norm_kv_store (the two below in one launch), omc_linear with a few outputs (the router),
  omc_causal_conv (linear), omc_qk_norm_kv_store (per group), omc_diff_heads_gate, omc_glu_mul (clamped), omc_embed_sinusoid,
  omc_moe_combine_norm (with the next norm): bytes read + written against the copy bandwidth; like kernels: omc_causal_conv_silu,
  omc_qk_norm_kv_store (whole projection), omc_gated_rms_rows, omc_glu_mul (gelu), omc_embed_scale, omc_post_norm_residual.
python tools/bench_fofisun.py --size s --size m
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from omchat_b200 import lib, seqlib  # noqa: E402
from omchat_b200.config import FofisunConfig, TifisunConfig  # noqa: E402
from omchat_b200.model import fofisun, tifisun  # noqa: E402
from omchat_b200.serving import StepScheduler  # noqa: E402
from tools.bench_voduzen import peaks, timed  # noqa: E402

# width, layers, heads, key/value heads, key width per map, value width, taps, window, kept first keys, ff, experts / top / expert ff / shared ff, vocab
SIZES = {
    "s": dict(C=2048, L=6, H=16, G=4, d=64, dv=128, conv=4, window=512, keep=64, ff=5632, E=16, top=2, eff=1408, sff=1408, V=32768),
    "m": dict(C=4096, L=6, H=32, G=8, d=64, dv=128, conv=4, window=512, keep=64, ff=8192, E=32, top=4, eff=1024, sff=2048, V=65536),
}


def config_dict(z, mixed: bool):
    mix = {"conv": z["conv"], "diff": 0.3, "dim": z["d"], "heads": z["H"], "kv_heads": z["G"],
           "mask": {"keep_first": z["keep"], "size": z["window"]}, "scale": z["d"] ** -0.5, "vdim": z["dv"]}
    dense = {"ff": z["ff"], "kind": "dense"}
    moe = {"expert": {"ff": z["eff"], "limit": 7.0}, "kind": "moe", "router": {"experts": z["E"], "top": z["top"]},
           "shared": {"ff": z["sff"], "limit": 7.0}}
    return {"architecture": "Fofisun", "vocab": z["V"], "width": z["C"], "norm": {"eps": 1e-5},
            "layers": [{"type": "attention", "mixer": mix, "mlp": moe if (mixed and i % 2) else dense} for i in range(z["L"])]}


def tifisun_dict(z):
    """Equal size: windowed attention with the two maps' key width as one head's key width (the same cache bytes per token and the
    same attention FLOPs), a one-head decay attention of minimal width beside it (the design has no layer without one)."""
    par = {"left": {"bias_max": z["window"], "dim": 2 * z["d"], "heads": z["H"], "kv_heads": z["G"], "mask": {"size": z["window"]},
                    "scale": (2 * z["d"]) ** -0.5, "softcap": 50.0, "vdim": z["dv"]},
           "right": {"decay": [0.99], "dim": 16, "heads": 1, "vdim": 16}}
    return {"architecture": "Tifisun", "vocab": z["V"], "width": z["C"], "embedding": {"scale": 1.0}, "residual_mult": 1.0, "norm": {"eps": 1e-5},
            "layers": [{"type": "parallel", "mixer": par, "mlp": {"ff": z["ff"], "kind": "dense"}} for _ in range(z["L"])]}


def kernels(z, n_seq, L, B, ctx):
    """The new kernels alone on one layer's shapes, each beside the like kernel of the Tifisun path."""
    hbm, tf = peaks()
    dev, bf, f32, i32 = "cuda", torch.bfloat16, torch.float32, torch.int32
    H, G, d, dv, C, W, keep = z["H"], z["G"], z["d"], z["dv"], z["C"], z["window"], z["keep"]
    page, out = 64, {}
    T = n_seq * L
    pos = torch.arange(L, dtype=i32, device=dev).repeat(n_seq)
    slot = torch.arange(n_seq, dtype=i32, device=dev).repeat_interleave(L)

    def rate(ms, nbytes=None, flops=None, **extra):
        r = {"ms": ms, **extra}
        if nbytes is not None:
            r.update(gbs=nbytes / ms / 1e6, frac_hbm=nbytes / ms / 1e6 / hbm)
        if flops is not None:
            r.update(tflops=flops / ms / 1e9, frac_tensor=flops / ms / 1e9 / tf)
        return r

    # ---- attention, prefill: two maps with kept keys against one map of twice the key width
    pages_per = L // page
    table = (torch.arange(n_seq * pages_per, dtype=i32, device=dev) + 1).view(n_seq, pages_per).contiguous()
    pool = (torch.randn(n_seq * pages_per + 1, page, G * (2 * d + dv), device=dev) * 0.3).to(bf)
    qb = (torch.randn(T, H * 2 * d, device=dev) * 0.3).to(bf)
    att2 = torch.empty(T, H * 2 * dv, device=dev, dtype=f32)
    att1 = torch.empty(T, H * dv, device=dev, dtype=bf)
    items = seqlib.window_attn_items([(s_ * L, L, s_, 0) for s_ in range(n_seq)], H // G, dev)
    vis = n_seq * sum(min(p + 1, W) + max(0, min(keep, p + 1 - W)) for p in range(L))
    ms = timed(lambda: seqlib.window_attn_mma(qb, H, G, d, dv, pool, table, page, items, pos, slot, W, d ** -0.5, 0.0, None, att2, maps=2, keep_first=keep))
    out["diff_window_attn_prefill"] = rate(ms, flops=vis * H * 2 * 2.0 * (d + dv), ctas=int(items.shape[0]) * G * 2)
    gate_a = torch.randn(T, H * dv, device=dev)
    on_a = torch.empty(T, H * dv, device=dev, dtype=bf)
    ms = timed(lambda: seqlib.diff_attn_pair(qb, H, G, d, dv, pool, table, page, items, W, keep, d ** -0.5, 0.4, 0.7, 1e-5, gate_a, seqlib.GATE_SIGMOID, on_a))
    out["diff_attn_pair_prefill"] = rate(ms, flops=vis * H * 2 * 2.0 * (d + dv), ctas=int(items.shape[0]) * G)
    del gate_a, on_a
    vis1 = n_seq * sum(min(p + 1, W) for p in range(L))
    ms = timed(lambda: seqlib.window_attn_mma(qb, H, G, 2 * d, dv, pool, table, page, items, pos, slot, W, d ** -0.5, 0.0, None, att1))
    out["tifisun_window_attn_prefill"] = rate(ms, flops=vis1 * H * 2.0 * (2 * d + dv), ctas=int(items.shape[0]) * G)
    # ---- attention, decode
    posd = torch.full((B,), ctx, dtype=i32, device=dev)
    slotd = torch.arange(B, dtype=i32, device=dev)
    pages_d = -(-(ctx + 1) // page)
    table_d = (torch.arange(B * pages_d, dtype=i32, device=dev) + 1).view(B, pages_d).contiguous()
    pool_d = (torch.randn(B * pages_d + 1, page, G * (2 * d + dv), device=dev) * 0.3).to(bf)
    seen = min(ctx + 1, W) + max(0, min(keep, ctx + 1 - W))
    nbytes = B * seen * G * (2 * d + dv) * 2
    ms = timed(lambda: seqlib.window_attn_mma(qb[:B], H, G, d, dv, pool_d, table_d, page, None, posd, slotd, W, d ** -0.5, 0.0, None, att2[:B], maps=2,
                                              keep_first=keep))
    out["diff_window_attn_decode"] = rate(ms, nbytes, batch=B, ctx=ctx, ctas=B * G * 2)
    ms = timed(lambda: seqlib.window_attn(qb[:B], H, G, d, dv, pool_d, table_d, page, posd, slotd, W, d ** -0.5, 0.0, None, att2[:B], maps=2, keep_first=keep))
    out["diff_window_attn_plain_decode"] = rate(ms, nbytes, batch=B, ctx=ctx)
    ms = timed(lambda: seqlib.window_attn_mma(qb[:B], H, G, 2 * d, dv, pool_d, table_d, page, None, posd, slotd, W, d ** -0.5, 0.0, None, att1[:B]))
    out["tifisun_window_attn_decode"] = rate(ms, B * min(ctx + 1, W) * G * (2 * d + dv) * 2, batch=B, ctx=ctx, ctas=B * G)
    del pool_d
    # ---- convolution: linear against silu + unit vectors
    ch = (H + G) * 2 * d + G * dv
    xz, yz = torch.randn(T, ch + H * dv, device=dev), torch.empty(T, ch, device=dev)
    cw = torch.randn(ch, z["conv"], device=dev).to(bf)
    cst = torch.zeros(n_seq, z["conv"] - 1, ch, device=dev)
    ms = timed(lambda: seqlib.causal_conv(xz[:, :ch], cw, pos, slot, cst, yz))
    out["causal_conv_linear"] = rate(ms, T * ch * 8)
    ms = timed(lambda: seqlib.causal_conv_silu(xz[:, :ch], cw, pos, slot, cst, yz, unit_channels=(H + G) * 2 * d, unit_group=d))
    out["tifisun_causal_conv_silu"] = rate(ms, T * ch * 8)
    # ---- query / key norm + cache append: per head and map against one norm over the projection
    nq, nk, nv = H * 2 * d, G * 2 * d, G * dv
    qo = torch.empty(T, nq, device=dev, dtype=bf)
    wd = torch.ones(d, device=dev, dtype=bf)
    wq, wk = torch.ones(nq, device=dev, dtype=bf), torch.ones(nk, device=dev, dtype=bf)
    nbytes = T * (nq + nk + nv) * (4 + 2)
    ms = timed(lambda: seqlib.qk_norm_kv_store(yz[:, :nq], wd, yz[:, nq:nq + nk], wd, yz[:, nq + nk:], 1e-5, pos, slot, table, page, pool, qo, group=d))
    out["qk_group_norm_kv_store"] = rate(ms, nbytes)
    ms = timed(lambda: seqlib.qk_norm_kv_store(yz[:, :nq], wq, yz[:, nq:nq + nk], wk, yz[:, nq + nk:], 1e-5, pos, slot, table, page, pool, qo))
    out["tifisun_qk_norm_kv_store"] = rate(ms, nbytes)
    ms_sep = out["causal_conv_linear"]["ms"] + out["qk_group_norm_kv_store"]["ms"]
    ms = timed(lambda: seqlib.conv_qk_norm_kv_store(xz, cw, pos, slot, cst, nq, nk, d, wd, wd, 1e-5, table, page, pool, qo))
    out["conv_qk_norm_kv_store_fused"] = rate(ms, T * ch * (4 + 2), ms_separate=ms_sep)
    out["tifisun_conv_then_qk_norm"] = rate(out["tifisun_causal_conv_silu"]["ms"] + out["tifisun_qk_norm_kv_store"]["ms"], T * ch * (4 + 2))
    # ---- the router's product: a few outputs over the width (rows of the step x router rows + the shared expert's gate row)
    nr = -(-(z["E"] + 1) // 8) * 8
    xr, wr, zr = (torch.randn(T, C, device=dev) * 0.5).to(bf), (torch.randn(nr, C, device=dev) * C ** -0.5).to(bf), torch.empty(T, nr, device=dev)
    ms = timed(lambda: seqlib.linear(xr, wr, zr))
    out["router_linear_prefill"] = rate(ms, T * C * 2 + T * nr * 4 + nr * C * 2)
    ms = timed(lambda: seqlib.linear(xr[:B], wr, zr[:B]))
    out["router_linear_decode"] = rate(ms, B * C * 2 + B * nr * 4 + nr * C * 2, batch=B)
    del xr, zr
    # ---- differential combine + head norm + gate against the gated RMS norm
    on = torch.empty(T, H * dv, device=dev, dtype=bf)
    gate = xz[:, ch:]
    ms = timed(lambda: seqlib.diff_heads_gate(att2, H, dv, 0.4, 0.7, 1e-5, gate, seqlib.GATE_SIGMOID, on))
    out["diff_heads_gate"] = rate(ms, T * H * dv * (8 + 4 + 2))
    o1 = torch.randn(T, H * dv, device=dev)
    nw = torch.ones(dv, device=dev, dtype=bf)
    ms = timed(lambda: seqlib.gated_rms_rows(o1, H, dv, nw, 1e-5, gate, seqlib.GATE_SIGMOID, on))
    out["tifisun_gated_rms_rows"] = rate(ms, T * H * dv * (4 + 4 + 2))
    del att2, o1
    # ---- gate * up halves
    ff = z["ff"]
    gu = (torch.randn(T, 2 * ff, device=dev) * 2.0).to(bf)
    act = torch.empty(T, ff, device=dev, dtype=bf)
    ms = timed(lambda: seqlib.glu_mul(gu, ff, seqlib.ACT_CLAMP_SWISH, act, limit=7.0, slope=1.702, shift=1.0))
    out["glu_mul_clamped"] = rate(ms, T * ff * 6)
    ms = timed(lambda: seqlib.glu_mul(gu, ff, seqlib.ACT_GELU_TANH, act))
    out["tifisun_glu_mul_gelu"] = rate(ms, T * ff * 6)
    del gu, act
    # ---- embedding
    table_e = torch.randn(z["V"], C, device=dev).to(bf)
    ids = torch.randint(0, z["V"], (T,), device=dev, dtype=i32)
    h = torch.empty(T, C, device=dev)
    freq = seqlib.sinusoid_frequencies(C, 10000.0, dev)
    ms = timed(lambda: seqlib.embed_sinusoid(ids, pos, table_e, 1.0, freq, h))
    out["embed_sinusoid"] = rate(ms, T * C * 6)
    ms = timed(lambda: seqlib.embed_scale(ids, table_e, 1.0, h, None))
    out["tifisun_embed_scale"] = rate(ms, T * C * 6)
    # ---- combine + post norm + residual + next norm against post norm + residual + next norm
    top = z["top"]
    ys, ysh = torch.randn(T * top, C, device=dev), torch.randn(T, C, device=dev)
    slot_of = torch.randperm(T * top, device=dev).view(T, top).to(i32)
    wts, gt = torch.rand(T, top, device=dev), torch.rand(T, device=dev)
    w = torch.zeros(C, device=dev, dtype=bf)
    xb = torch.empty(T, C, device=dev, dtype=bf)
    ms = timed(lambda: seqlib.moe_combine_norm(ys, slot_of, wts, top, gt, ysh, w, 1e-5, h, xb, w_next=w))
    out["moe_combine_norm_next"] = rate(ms, T * C * (4 * top + 4 + 4 + 4 + 2))
    ms = timed(lambda: seqlib.post_norm_residual(ysh, w, 1e-5, 1.0, h, w, xb))
    out["tifisun_post_norm_residual"] = rate(ms, T * C * (4 + 4 + 4 + 2))
    return out


def serve(model, V, prefill, batches, ctx, steps):
    """Prefill of `prefill` x 1024 tokens as one step and decode steps at every batch size, through the scheduler."""
    L = 1024
    g = torch.Generator().manual_seed(0)
    rec = {}

    def prefill_once():
        sched = StepScheduler(model, max_tokens=prefill * L, slots=prefill)
        entries = [(f"p{i}", torch.randint(0, V, (L,), generator=g).tolist(), [L - 1]) for i in range(prefill)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        sched.run_step(entries)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)
    for _ in range(2):
        prefill_once()
    n0 = lib.launch_count()
    ms = sorted(prefill_once() for _ in range(3))[1]
    T = prefill * L
    rec["prefill"] = {"tokens": T, "ms": ms, "tokens_per_sec": T / ms * 1e3, "launches": (lib.launch_count() - n0) // 3}
    rec["decode"] = []
    for B in batches:
        sched = StepScheduler(model, max_tokens=B * (ctx + steps + 80), slots=B)
        for lo in range(0, B, 8):     # contexts are filled by prefill steps of 8 prompts
            sched.run_step([(f"d{i}", torch.randint(0, V, (ctx,), generator=g).tolist(), []) for i in range(lo, min(B, lo + 8))])
        toks = torch.randint(0, V, (B,), generator=g).tolist()
        for _ in range(3):
            sched.run_step([(f"d{i}", [toks[i]], [0]) for i in range(B)])
        torch.cuda.synchronize()
        n0 = lib.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            lg = sched.run_step([(f"d{i}", [toks[i]], [0]) for i in range(B)])
            toks = lib.argmax(lg).tolist()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        rec["decode"].append({"batch": B, "ctx": ctx, "ms_per_step": ms, "tokens_per_sec": B / ms * 1e3,
                              "launches_per_step": (lib.launch_count() - n0) // steps})
        del sched
    return rec


def measure(size="s", batches=(1, 32), ctx=1024, steps=32, prefill=4, with_kernels=True, with_tifisun=True):
    z = SIZES[size]
    rec = {"size": size, "dims": z}
    for name, mixed in (("fofisun_dense", False), ("fofisun_mixed", True)):
        cfg = FofisunConfig.from_dict(config_dict(z, mixed))
        model = fofisun.FofisunForCausalLM.from_state_dict(fofisun.random_state_dict(cfg, seed=0), cfg, device="cuda:0")
        rec[name] = serve(model, z["V"], prefill, batches, ctx, steps)
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
