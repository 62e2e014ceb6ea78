"""Fofisun on the GPU against the plain restatement in oracle/fofisun_oracle.py (float64, whole sequences, explicit loops).

Small configurations of their own, random weights, and engineered inputs where random ones would hide a fault: one key whose score
stands out among hundreds, placed just inside / just outside the window and among / just behind the kept first keys, at page
borders, for prompt portions and for single decoded rows; states and pages poisoned with NaN before they are used again.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():  # collected on the CPU box too
    pytest.skip("needs a CUDA device", allow_module_level=True)

from omchat_b200 import seqlib  # noqa: E402
from omchat_b200.config import FofisunConfig  # noqa: E402
from omchat_b200.model.fofisun import FofisunForCausalLM, random_state_dict  # noqa: E402
from omchat_b200.serving import StepScheduler  # noqa: E402
from oracle import fofisun_oracle as O  # noqa: E402

DEV = "cuda:0"
F64 = torch.float64


def attention(heads, kv_heads, dim, vdim, window, keep, conv, mlp, diff=0.4, scale=None):
    return {"type": "attention", "mixer": {"conv": conv, "diff": diff, "dim": dim, "heads": heads, "kv_heads": kv_heads,
                                           "mask": {"keep_first": keep, "size": window}, "scale": scale if scale is not None else dim ** -0.5,
                                           "vdim": vdim}, "mlp": mlp}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def moe(experts, top, ff, limit, shared_ff=None, shared_limit=None):
    return {"expert": {"ff": ff, "limit": limit}, "kind": "moe", "router": {"experts": experts, "top": top},
            "shared": {"ff": shared_ff, "limit": shared_limit} if shared_ff else None}


def config_a(page=16):
    """Grouped heads, widths that are no multiples of 32, every kind of feed-forward and a layer without one, a looped block whose
    runs keep caches of their own, a window shorter than a page next to one longer than several."""
    return {"architecture": "Fofisun", "vocab": 131, "width": 72, "norm": {"eps": 1e-5}, "kv_page_size": page,
            "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
                attention(6, 2, 12, 20, 11, 3, 4, dense(100)),
                attention(4, 4, 24, 8, 37, 5, 2, moe(5, 2, 28, 0.8, 36, 1.3)),
                attention(3, 1, 20, 24, 9, 0, 3, None),
                attention(6, 2, 12, 20, 11, 3, 4, moe(7, 3, 20, 2.5))]}


def config_b(page=32):
    """Ones and equal values: one head, one expert out of one, every expert chosen, a window of one key, no kept keys, a convolution
    of one tap and none at all, value width = key width, no loop entry, an odd width."""
    return {"architecture": "Fofisun", "vocab": 67, "width": 45, "norm": {"eps": 1e-6}, "kv_page_size": page, "layers": [
        attention(1, 1, 16, 16, 1, 0, 1, moe(1, 1, 24, 1.0)),
        attention(1, 1, 8, 8, 200, 40, 0, moe(4, 4, 12, 0.5, 8, 0.25), diff=0.0),
        attention(2, 2, 16, 16, 4, 9, 2, dense(30), diff=0.9)]}


def config_c(page=16):
    """Attention shapes the tensor-core kernel takes (bf16): grouped heads, a window over several key tiles with kept keys that lie
    tiles behind it, a run of the same layer twice."""
    return {"architecture": "Fofisun", "vocab": 110, "width": 64, "norm": {"eps": 1e-5}, "kv_page_size": page,
            "loop": {"start": 0, "stop": 1, "times": 2}, "layers": [
                attention(4, 2, 32, 16, 75, 70, 3, dense(96)),
                attention(8, 1, 16, 64, 9, 2, 2, moe(6, 2, 32, 1.5, 32, 1.0))]}


def config_d(page=64):
    """Matrices large enough for the tensor-core GEMMs (erf-gelu epilogue, skinny decode GEMM, grouped expert GEMM over 128-row
    tiles) and head shapes of the tensor-core attention."""
    return {"architecture": "Fofisun", "vocab": 520, "width": 384, "norm": {"eps": 1e-6}, "kv_page_size": page,
            "loop": {"start": 1, "stop": 2, "times": 2}, "layers": [
                attention(4, 2, 32, 48, 50, 4, 3, dense(3328)),
                attention(6, 2, 64, 64, 120, 10, 4, moe(4, 2, 768, 3.0, 512, 2.0))]}


def build(cfg_dict, dtype, seed=0, edit=None):
    cfg = FofisunConfig.from_dict(cfg_dict)
    sd = random_state_dict(cfg, seed=seed)
    if edit:
        edit(sd)
    return FofisunForCausalLM.from_state_dict(sd, cfg, device=DEV, dtype=dtype), sd


def row_errors(got, want):
    """Per row: RMS difference of mean-free logits relative to the RMS of the reference row."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)


def rel_err(got, want):
    return float(row_errors(got, want).max())


def close(got, want, dtype):
    """fp32: every row within 2e-4. bf16: nine rows in ten within 6e-2 and none beyond 0.3 - with random weights a bf16 rounding
    now and then moves a token to another expert, which shows in that row and the few behind it, not in all of them."""
    e = row_errors(got, want)
    if dtype == torch.float32:
        return float(e.max()) < 2e-4
    return float(e.max()) < 0.3 and float(torch.quantile(e, 0.9)) < 6e-2


def tokens_for(cfg_dict, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg_dict["vocab"], (n,), generator=g).tolist()


TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


def run_schedule(model, steps, max_tokens, slots=4):
    """steps: [[(key, tokens, want)], end-keys]. Returns {key: [logit rows in the order they came]}."""
    sched = StepScheduler(model, max_tokens=max_tokens, slots=slots)
    out = {}
    for entries, end in steps:
        lg = sched.run_step(entries, end)
        at = 0
        for key, _, want in entries:
            for _ in want:
                out.setdefault(key, []).append(lg[at].float().cpu().clone())
                at += 1
    return out, sched


def _dev(t, dt=torch.float32):
    return t.to(device=DEV, dtype=dt).contiguous()


def _i32(x):
    return torch.tensor(x, device=DEV, dtype=torch.int32)


# ------------------------------------------------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("C", [72, 45, 2, 256])
def test_embedding_with_position_vectors(C):
    g = torch.Generator().manual_seed(C)
    table = torch.randn(19, C, generator=g).to(torch.bfloat16)
    ids = [3, 18, 0, 7, 7, 25, -1]                                 # the last two lie outside the table: position vector only
    pos = [0, 1, 2, 511, 4097, 5, 100000]
    h = torch.full((len(ids), C + 3), float("nan"), device=DEV)     # rows of a wider buffer
    seqlib.embed_sinusoid(_i32(ids), _i32(pos), table.to(DEV), 1.0, seqlib.sinusoid_frequencies(C, 10000.0, DEV), h[:, :C])
    for r, (i, p) in enumerate(zip(ids, pos)):
        want = O.position_vectors(1, C, first=p)[0] + (table[i].double() if 0 <= i < 19 else 0.0)
        assert torch.allclose(h[r, :C].double().cpu(), want, atol=3e-7 * (1 + want.abs().max())), (r, (h[r, :C].double().cpu() - want).abs().max())
    assert torch.isnan(h[:, C:]).all()


@pytest.mark.parametrize("taps,ch", [(3, 48), (2, 40), (1, 24), (7, 36)])
def test_linear_convolution_alone_and_in_portions(taps, ch):
    g = torch.Generator().manual_seed(taps)
    T = 23
    x = torch.randn(2, T, ch, generator=g, dtype=F64)
    w = torch.randn(ch, taps, generator=g, dtype=F64)
    want = [O.causal_conv(x[b], w) for b in range(2)]
    state = torch.full((3, max(taps - 1, 1), ch), float("nan"), device=DEV) if taps > 1 else None   # stale contents must never be read
    got = [torch.zeros(T, ch, dtype=F64), torch.zeros(T, ch, dtype=F64)]
    # request 0 in slot 2 in portions of 2, 1, 9, 11 tokens; request 1 in slot 0 as 20 + 3; the steps interleave them
    plan = [[(2, 0, 0, 2), (0, 1, 0, 20)], [(2, 0, 2, 1)], [(0, 1, 20, 3), (2, 0, 3, 9)], [(2, 0, 12, 11)]]
    for step in plan:
        pos = _i32([p for _, _, p0, n in step for p in range(p0, p0 + n)])
        slot = _i32([s for s, _, _, n in step for _ in range(n)])
        xin = torch.cat([x[b, p0:p0 + n] for _, b, p0, n in step])
        xin = torch.cat([_dev(xin), torch.zeros(xin.shape[0], 5, device=DEV)], dim=1)          # a column slice of a wider buffer
        y = torch.empty(xin.shape[0], ch, device=DEV)
        seqlib.causal_conv(xin[:, :ch], _dev(w), pos, slot, state, y, single_rows=all(n == 1 for _, _, _, n in step))
        at = 0
        for _, b, p0, n in step:
            got[b][p0:p0 + n] = y[at:at + n].double().cpu()
            at += n
    for b in range(2):
        assert torch.allclose(got[b], want[b], atol=2e-5, rtol=1e-5), (got[b] - want[b]).abs().max()


class Pages:
    """A hand-made paged pool for kernel tests: slots with shuffled, non-contiguous pages."""

    def __init__(self, width, n_slots, tokens_per_slot, page, dtype, seed=0):
        per = -(-tokens_per_slot // page)
        order = torch.randperm(n_slots * per, generator=torch.Generator().manual_seed(seed)) + 1
        self.page = page
        self.table = order.view(n_slots, per).to(torch.int32).to(DEV)
        self.pool = torch.full((n_slots * per + 1, page, width), float("nan"), device=DEV, dtype=dtype)

    def fill(self, slot, rows):
        """rows [L, width]: the cache rows of positions 0 .. L - 1 of `slot`."""
        j = torch.arange(rows.shape[0], device=DEV)
        self.pool[self.table[slot].long()[j // self.page], j % self.page] = rows.to(self.pool.dtype).to(DEV)


@pytest.mark.parametrize("H,G,d,dv,page", [(6, 2, 12, 20, 16), (1, 1, 16, 16, 8), (4, 4, 24, 8, 32)])
def test_group_norm_of_queries_and_keys_and_cache_append(H, G, d, dv, page):
    g = torch.Generator().manual_seed(H * d)
    T, eps = 13, 1e-5
    nq, nk, nv = H * 2 * d, G * 2 * d, G * dv
    y = torch.randn(T, nq + nk + nv, generator=g, dtype=F64) * 3.0
    wq, wk = torch.randn(d, generator=g, dtype=F64), torch.randn(d, generator=g, dtype=F64)
    pg = Pages(nk + nv, 2, 40, page, torch.float32)
    pos, slot = _i32([page - 2 + i for i in range(T)]), _i32([1] * T)        # crosses a page border
    q_out = torch.empty(T, nq, device=DEV)
    yd = _dev(y)
    seqlib.qk_norm_kv_store(yd[:, :nq], _dev(wq), yd[:, nq:nq + nk], _dev(wk), yd[:, nq + nk:], eps, pos, slot, pg.table, page, pg.pool, q_out,
                            group=d)
    want_q = (O.unit_rms(y[:, :nq].view(T, H * 2, d), eps) * wq).reshape(T, nq)
    want_k = (O.unit_rms(y[:, nq:nq + nk].view(T, G * 2, d), eps) * wk).reshape(T, nk)
    assert torch.allclose(q_out.double().cpu(), want_q, atol=1e-5, rtol=1e-5)
    for i in range(T):
        p = page - 2 + i
        row = pg.pool[int(pg.table[1, p // page]), p % page].double().cpu()
        assert torch.allclose(row[:nk], want_k[i], atol=1e-5, rtol=1e-5) and torch.allclose(row[nk:], y[i, nq + nk:], atol=1e-6)


@pytest.mark.parametrize("H,G,d,dv,taps,page,dtype", [(6, 2, 12, 20, 4, 16, torch.float32), (1, 1, 16, 16, 1, 8, torch.float32),
                                                     (4, 4, 24, 8, 2, 32, torch.bfloat16), (16, 4, 64, 128, 3, 16, torch.bfloat16)])
def test_convolution_norm_and_append_in_one_launch(H, G, d, dv, taps, page, dtype):
    """The fused kernel against convolution -> group norm -> append of the plain model, fed in portions (2 and 300 rows: one row and
    eight rows per CTA), then single rows; the ring carries the last inputs across the steps."""
    g = torch.Generator().manual_seed(H + taps)
    T, eps = 330, 1e-5
    nq, nk, nv = H * 2 * d, G * 2 * d, G * dv
    ch = nq + nk + nv
    x = torch.randn(T, ch + 7, generator=g, dtype=F64)              # columns behind the channels belong to somebody else
    w = torch.randn(ch, taps, generator=g, dtype=F64)
    wq, wk = torch.randn(d, generator=g, dtype=F64), torch.randn(d, generator=g, dtype=F64)
    xr, wr = x.to(torch.float32).double(), w.to(dtype).double()     # the values the kernel sees
    y = O.causal_conv(xr[:, :ch], wr)
    want_q = (O.unit_rms(y[:, :nq].view(T, H * 2, d), eps) * wq.to(dtype).double()).reshape(T, nq)
    want_k = (O.unit_rms(y[:, nq:nq + nk].view(T, G * 2, d), eps) * wk.to(dtype).double()).reshape(T, nk)
    pg = Pages(nk + nv, 2, T, page, dtype)
    state = torch.full((2, max(taps - 1, 1), ch), float("nan"), device=DEV) if taps > 1 else None
    q_out = torch.empty(T, nq, device=DEV, dtype=dtype)
    xd = _dev(x)
    at = 0
    for n in [2, 300] + [1] * 28:
        pos, slot = _i32(list(range(at, at + n))), _i32([1] * n)
        seqlib.conv_qk_norm_kv_store(xd[at:at + n], _dev(w, dtype), pos, slot, state, nq, nk, d, _dev(wq, dtype), _dev(wk, dtype), eps, pg.table,
                                     page, pg.pool, q_out[at:at + n], single_rows=n == 1)
        at += n
    assert at == T
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    assert torch.allclose(q_out.double().cpu(), want_q, atol=tol, rtol=tol)
    j = torch.arange(T, device=DEV)
    rows = pg.pool[pg.table[1].long()[j // page], j % page].double().cpu()
    assert torch.allclose(rows[:, :nk], want_k, atol=tol, rtol=tol) and torch.allclose(rows[:, nk:], y[:, nq + nk:], atol=tol, rtol=tol)


@pytest.mark.parametrize("M,N,K,batch", [(1, 11, 200, 1), (37, 24, 2048, 1), (9, 64, 256, 3), (300, 1, 45, 1)])
def test_linear_layer_with_few_outputs(M, N, K, batch):
    """Routers and gates: a handful of outputs over a long K, rows of strided buffers, a batch of column slices."""
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, batch * K + 3, generator=g, dtype=F64)
    w = torch.randn(batch, N, K, generator=g, dtype=F64) * K ** -0.5
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        xd, wd = _dev(x, dt), _dev(w, dt)
        out = torch.full((M, batch * N + 1), float("nan"), device=DEV)
        seqlib.linear(xd, wd, out, M=M, N=N, K=K, ldx=xd.stride(0), sx=K, ldw=K, sw=N * K, ldy=out.stride(0), sy=N, batch=batch, alpha=0.5)
        for b in range(batch):
            want = 0.5 * xd[:, b * K:(b + 1) * K].double().cpu() @ wd[b].double().cpu().T
            assert torch.allclose(out[:, b * N:(b + 1) * N].double().cpu(), want, atol=tol, rtol=tol)
        assert torch.isnan(out[:, batch * N:]).all()
        if batch == 1:      # a row's result does not depend on the rows beside it
            one = torch.empty(1, N, device=DEV)
            seqlib.linear(xd[M - 1:M], wd[0], one, K=K, alpha=0.5)
            assert torch.equal(one[0], out[M - 1, :N])


def plain_two_map_attention(q, k, v, H, G, d, dv, scale, window, keep, first_pos=0):
    """q [n, H, 2, d] for positions first_pos.., k [L, G, 2, d], v [L, G, dv] -> [n, H, 2, dv] with the oracle's mask, in float64."""
    n, L = q.shape[0], k.shape[0]
    out = torch.zeros(n, H, 2, dv, dtype=F64)
    see = torch.tensor([[O.visible(first_pos + i, j, window, keep) for j in range(L)] for i in range(n)], dtype=torch.bool).view(n, L)
    for h in range(H):
        gi = h // (H // G)
        for mp in range(2):
            s = (q[:, h, mp] @ k[:, gi, mp].T * scale).masked_fill(~see, float("-inf"))
            out[:, h, mp] = torch.softmax(s, dim=-1) @ v[:, gi]
    return out


ATT_SHAPES = [(6, 2, 12, 20, 16, torch.float32), (4, 2, 32, 16, 16, torch.bfloat16), (8, 1, 16, 64, 32, torch.bfloat16),
              (1, 1, 16, 16, 8, torch.float32), (2, 2, 48, 128, 16, torch.bfloat16)]


@pytest.mark.parametrize("H,G,d,dv,page,dtype", ATT_SHAPES)
@pytest.mark.parametrize("window,keep", [(23, 5), (70, 0), (1, 3), (9, 80), (None, 0)])
def test_two_map_attention_with_window_and_kept_keys(H, G, d, dv, page, dtype, window, keep):
    """Random queries, keys and values in a shuffled paged pool; a prompt portion that starts deep in the sequence and single decode
    rows, through the plain kernel and (bf16, eligible shapes) the tensor-core kernel."""
    g = torch.Generator().manual_seed(H + d + (window or 0))
    L, scale = 150, 1.3 * d ** -0.5
    k = torch.randn(L, G, 2, d, generator=g).to(dtype)
    v = torch.randn(L, G, dv, generator=g).to(dtype)
    q = torch.randn(L, H, 2, d, generator=g).to(dtype)
    pg = Pages(G * (2 * d + dv), 3, L, page, dtype, seed=1)
    pg.fill(2, torch.cat([k.reshape(L, -1), v.reshape(L, -1)], dim=1))
    win = window if window is not None else seqlib.WINDOW_ALL
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    cases = [("portion", 61, 150), ("first rows", 0, 40), ("decode", 149, 150), ("decode", 80, 81), ("decode", 0, 1)]
    for name, lo, hi in cases:
        n = hi - lo
        want = plain_two_map_attention(q[lo:hi].double(), k[:hi].double(), v[:hi].double(), H, G, d, dv, scale, window, keep, first_pos=lo)
        qd = q[lo:hi].reshape(n, -1).to(DEV)
        pos, slot = _i32(list(range(lo, hi))), _i32([2] * n)
        out = torch.empty(n, H * 2 * dv, device=DEV)
        seqlib.window_attn(qd, H, G, d, dv, pg.pool, pg.table, page, pos, slot, win, scale, 0.0, None, out, maps=2, keep_first=keep)
        assert torch.allclose(out.double().cpu().view(n, H, 2, dv), want, atol=tol, rtol=tol), (name, "plain")
        if seqlib.window_attn_mma_ok(H, G, d, dv, dtype):
            items = None if name == "decode" else seqlib.window_attn_items([(0, n, 2, lo)], H // G, DEV)
            out2 = torch.empty(n, H * 2 * dv, device=DEV)
            seqlib.window_attn_mma(qd, H, G, d, dv, pg.pool, pg.table, page, items, pos, slot, win, scale, 0.0, None, out2, maps=2, keep_first=keep)
            assert torch.allclose(out2.double().cpu().view(n, H, 2, dv), want, atol=tol, rtol=tol), (name, "tensor cores")
            if items is not None and seqlib.diff_attn_pair_ok(H, G, d, dv, dtype):     # both maps and the combine in one kernel
                lam, mult, eps = 0.45, 0.7, 1e-5
                gate = torch.randn(n, H * dv + 2, generator=g, dtype=F64)
                want_o = (O.unit_rms(want[:, :, 0] - lam * want[:, :, 1], eps) * mult).reshape(n, H * dv) * torch.sigmoid(gate[:, :H * dv])
                out3 = torch.empty(n, H * dv, device=DEV)
                seqlib.diff_attn_pair(qd, H, G, d, dv, pg.pool, pg.table, page, items, win, keep, scale, lam, mult, eps, _dev(gate)[:, :H * dv],
                                      seqlib.GATE_SIGMOID, out3)
                # the head norm divides by the size of a DIFFERENCE of two bf16-rounded maps: compare relative to the head's scale
                err = (out3.double().cpu() - want_o).view(n, H, dv).abs().amax(-1) / want_o.view(n, H, dv).abs().amax(-1).clamp_min(1e-3)
                assert float(err.max()) < 0.1 and float(err.median()) < 2e-2, (name, "paired maps", float(err.max()), float(err.median()))


@pytest.mark.parametrize("dtype,mma", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("window,keep,page", [(40, 6, 16), (64, 64, 64), (17, 1, 8)])
def test_one_key_that_stands_out_at_every_edge(dtype, mma, window, keep, page):
    """All keys but one score alike; the marked key's score is far above them and its value is a vector of its own. A row sees the
    mark iff the mark is a kept first key or lies inside the row's window - checked one position before and at every edge, for the
    rows of a prompt portion and for single decode rows, with the mark among hundreds of keys and at page borders."""
    H, G, d, dv, L = 4, 2, 16, 32, 400
    scale = 1.0
    for mark in (0, keep - 1, keep, keep + 1, page - 1, page, 2 * page + 3, 200):
        if mark < 0:
            continue
        k = torch.zeros(L, G, 2, d)
        k[..., 0] = 0.05
        k[mark, :, :, 0] = 12.0                                   # score 12 against 0.05 for everybody else
        v = torch.zeros(L, G, dv)
        v[..., 0] = 1.0
        v[mark] = 0.0
        v[mark, :, 1] = 1.0                                       # the mark's value points along another axis
        q = torch.zeros(L, H, 2, d)
        q[..., 0] = 1.0
        pg = Pages(G * (2 * d + dv), 2, L, page, dtype, seed=mark)
        pg.fill(1, torch.cat([k.reshape(L, -1), v.reshape(L, -1)], dim=1))
        rows = sorted({p for p in (mark, mark + 1, mark + window - 2, mark + window - 1, mark + window, mark + window + 1, mark + 250, L - 1)
                       if mark <= p < L})
        for mode in ("portion", "decode"):
            if mode == "portion":       # one portion that spans all the probed rows
                lo, hi = rows[0], rows[-1] + 1
                pos, slot, sel = _i32(list(range(lo, hi))), _i32([1] * (hi - lo)), [p - lo for p in rows]
                items = seqlib.window_attn_items([(0, hi - lo, 1, lo)], H // G, DEV)
            else:
                pos, slot, sel, items = _i32(rows), _i32([1] * len(rows)), list(range(len(rows))), None
            n = pos.numel()
            qd = q[:n].reshape(n, -1).to(dtype).to(DEV)
            out = torch.empty(n, H * 2 * dv, device=DEV)
            if mma:
                seqlib.window_attn_mma(qd, H, G, d, dv, pg.pool, pg.table, page, items, pos, slot, window, scale, 0.0, None, out, maps=2,
                                       keep_first=keep)
            else:
                seqlib.window_attn(qd, H, G, d, dv, pg.pool, pg.table, page, pos, slot, window, scale, 0.0, None, out, maps=2, keep_first=keep)
            o = out.view(n, H, 2, dv)
            paired = None
            if mma and items is not None and seqlib.diff_attn_pair_ok(H, G, d, dv, dtype):
                # the one-kernel path with lambda = 0: the first map alone, divided by its RMS over the head (1 / sqrt(dv) for a unit vector)
                paired = torch.empty(n, H * dv, device=DEV)
                seqlib.diff_attn_pair(qd, H, G, d, dv, pg.pool, pg.table, page, items, window, keep, scale, 0.0, dv ** -0.5, 0.0, None, 0, paired)
                paired = paired.view(n, H, dv)
            for p, r in zip(rows, sel):
                seen = mark < keep or p - mark < window
                share = o[r, :, :, 1]                             # weight of the mark's value in every head and map
                if seen:
                    assert (share > 0.99).all(), (mark, p, mode, "the mark must dominate")
                    assert paired is None or (paired[r, :, 1] > 0.99).all(), (mark, p, mode, "paired maps: the mark must dominate")
                else:
                    assert (share == 0).all(), (mark, p, mode, "the mark must be invisible")
                    assert paired is None or (paired[r, :, 1] == 0).all(), (mark, p, mode, "paired maps: the mark must be invisible")


@pytest.mark.parametrize("H,dv,lam,mult", [(6, 20, 0.37, 0.6), (1, 16, -1.2, 1.0), (3, 130, 0.0, 0.1)])
def test_differential_combine_head_norm_and_gate(H, dv, lam, mult):
    g = torch.Generator().manual_seed(H * dv)
    T, eps = 9, 1e-5
    a = torch.randn(T, H, 2, dv, generator=g, dtype=F64)
    gate = torch.randn(T, H * dv + 4, generator=g, dtype=F64) * 2.0
    want = (O.unit_rms(a[:, :, 0] - lam * a[:, :, 1], eps) * mult).reshape(T, H * dv) * torch.sigmoid(gate[:, :H * dv])
    for dt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 1e-2)):
        out = torch.empty(T, H * dv, device=DEV, dtype=dt)
        seqlib.diff_heads_gate(_dev(a.reshape(T, -1)), H, dv, lam, mult, eps, _dev(gate)[:, :H * dv], seqlib.GATE_SIGMOID, out)
        assert torch.allclose(out.double().cpu(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("E,top", [(10, 3), (5, 5), (1, 1), (40, 7)])
def test_router_with_bias_and_softmax_over_the_chosen(E, top):
    g = torch.Generator().manual_seed(E)
    T = 21
    z = torch.randn(T, E + 3, generator=g, dtype=F64) * 2.0        # one gate column and two unused ones behind the logits
    bias = torch.randn(E, generator=g, dtype=F64)
    zd = _dev(z)
    ids = torch.empty(T, top, device=DEV, dtype=torch.int32)
    w = torch.empty(T, top, device=DEV)
    gate = torch.empty(T, device=DEV)
    counts = torch.zeros(E, device=DEV, dtype=torch.int32)
    seqlib.router_topk(zd, E, E, top, None, True, ids, w, gate, counts, bias=_dev(bias), renorm=True)
    zb = z[:, :E].float().double() + bias.float().double()
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(zb[t, e]), e))[:top]
        assert ids[t].tolist() == order
        assert torch.allclose(w[t].double().cpu(), torch.softmax(zb[t, order], 0), atol=1e-6)
    assert torch.allclose(gate.double().cpu(), torch.sigmoid(z[:, E].float().double()), atol=1e-6)
    assert counts.sum().item() == T * top


@pytest.mark.parametrize("n,limit", [(28, 0.8), (64, 7.0), (5, 0.05)])
def test_clamped_gate_times_shifted_up(n, limit):
    g = torch.Generator().manual_seed(n)
    z = torch.randn(11, 2 * n, generator=g, dtype=F64) * 3.0
    gg = z[:, :n].clamp(max=limit)
    uu = z[:, n:].clamp(min=-limit, max=limit)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1.0)
    out = torch.empty(11, n, device=DEV)
    seqlib.glu_mul(_dev(z), n, seqlib.ACT_CLAMP_SWISH, out, limit=limit, slope=1.702, shift=1.0)
    assert torch.allclose(out.double().cpu(), want, atol=1e-5, rtol=1e-5)


def test_erf_gelu_in_the_linear_layer():
    g = torch.Generator().manual_seed(3)
    x, w = torch.randn(7, 40, generator=g, dtype=F64), torch.randn(30, 40, generator=g, dtype=F64) * 0.3
    out = torch.empty(7, 30, device=DEV)
    seqlib.linear(_dev(x), _dev(w), out, act=seqlib.ACT_GELU_ERF)
    assert torch.allclose(out.double().cpu(), O.gelu_erf(x.float().double() @ w.float().double().T), atol=1e-5, rtol=1e-5)


def test_combine_with_the_next_sublayers_norm():
    g = torch.Generator().manual_seed(5)
    T, C, top, eps = 6, 72, 2, 1e-5
    ys, ysh = torch.randn(16, C, generator=g, dtype=F64), torch.randn(T, C, generator=g, dtype=F64)
    slot_of = torch.randperm(16, generator=g)[:T * top].view(T, top).to(torch.int32)
    w, gate = torch.rand(T, top, generator=g, dtype=F64), torch.rand(T, generator=g, dtype=F64)
    nw, wn = torch.randn(C, generator=g, dtype=F64) * 0.2, torch.randn(C, generator=g, dtype=F64) * 0.2
    h = torch.randn(T, C, generator=g, dtype=F64)
    y = sum(w[:, j:j + 1] * ys[slot_of[:, j].long()] for j in range(top)) + gate[:, None] * ysh
    want_h = h + O.norm_zero_centred(y, nw, eps)
    hd, xb = _dev(h), torch.empty(T, C, device=DEV)
    seqlib.moe_combine_norm(_dev(ys), slot_of.to(DEV), _dev(w), top, _dev(gate), _dev(ysh), _dev(nw), eps, hd, xb, w_next=_dev(wn))
    assert torch.allclose(hd.double().cpu(), want_h, atol=1e-5, rtol=1e-5)
    assert torch.allclose(xb.double().cpu(), O.norm_zero_centred(want_h, wn, eps), atol=1e-5, rtol=1e-5)


# ------------------------------------------------------------------------------------------------------------- whole prompts
@pytest.mark.parametrize("cfgf", [config_a, config_b, config_c])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_against_the_plain_model_layer_by_layer(cfgf, dtype):
    cd = cfgf()
    model, sd = build(cd, dtype, seed=1)
    toks = tokens_for(cd, 97, 2)
    want_layers = []
    want = O.forward(sd, cd, toks, want_layers)
    sched = StepScheduler(model, max_tokens=256, slots=2)
    got = sched.run_step([("a", toks, list(range(len(toks))))], ["a"])
    assert close(got, want, dtype), row_errors(got, want).max()
    # the residual stream after every layer run (fp32 only: it pins the layer that differs)
    if dtype == torch.float32:
        T = len(toks)
        cache = model.decoder.new_cache(8, 1)
        cache.set_pages(0, 0, list(range(1, 8)))
        cache.sync()
        col = []
        model.step(_i32(toks), _i32(list(range(T))), _i32([0] * T), cache, None, collect=col, portions=[(0, T, 0, 0)])
        assert len(col) == len(want_layers) == len(model.config.layer_runs())
        for r, (a, b) in enumerate(zip(col, want_layers)):
            assert torch.allclose(a.double().cpu(), b, atol=2e-4 * float(b.abs().max()), rtol=0), f"layer run {r}"


def test_wide_layers_on_the_tensor_core_gemms():
    cd = config_d()
    model, sd = build(cd, torch.bfloat16, seed=21)
    toks = tokens_for(cd, 200, 22)
    want = O.forward(sd, cd, toks)
    # a long portion (tensor-core GEMMs with 128-row tiles), a short one, then single tokens (skinny GEMMs, graph replay)
    steps = [([("w", toks[:150], list(range(150)))], []), ([("w", toks[150:170], list(range(20)))], [])]
    steps += [([("w", [t], [0])], []) for t in toks[170:]]
    out, _ = run_schedule(model, steps, 256)
    got = torch.stack(out["w"])
    assert close(got, want, torch.bfloat16), row_errors(got, want).max()


def test_trace_replay_from_a_checkpoint_folder(tmp_path):
    """The command-line runner on a saved checkpoint: the model class comes from config.json, steps arrive on standard input,
    logits leave as files; requests pause, end and hand their slots and pages on."""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    from omchat_b200.model.checkpoint import save_checkpoint
    cd = config_a(page=64)
    del cd["kv_page_size"]
    cfg = FofisunConfig.from_dict(cd)
    sd = random_state_dict(cfg, seed=23)
    save_checkpoint(sd, cfg, str(tmp_path / "model"))
    toks = {k: tokens_for(cd, n, 40 + n) for k, n in (("x", 90), ("y", 70), ("z", 30), ("u", 65), ("v", 5))}
    plan = [[("x", 50), ("y", 3)], [("x", 1), ("y", 60)], [("y", 7), ("z", 30)], [("x", 39), ("u", 2), ("v", 5)], [("u", 63)]]
    fed, lines, rows = {k: 0 for k in toks}, [], []
    for n, step in enumerate(plan):
        entries, end = [], []
        for k, c in step:
            want = [c - 1] if c > 1 else [0]
            entries.append({"id": k, "tokens": toks[k][fed[k]:fed[k] + c], "want": want})
            rows.append((n, k, fed[k] + want[0]))
            fed[k] += c
            if fed[k] == len(toks[k]):
                end.append(k)
        lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    # four slots, and pages for three requests of two pages each: the later requests take over what the earlier ones give back
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path / "model"), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "384"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {n}" for n in range(len(plan))]
    want = {k: O.forward(sd, cd, toks[k]) for k in toks}
    at = {}
    for n, k, p in rows:
        data = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cd["vocab"])
        i = at.get(n, 0)
        at[n] = i + 1
        assert rel_err(torch.from_numpy(data[i:i + 1].copy()), want[k][p:p + 1]) < TOL[torch.float32], (n, k, p)


def test_fused_and_separate_convolution_paths_agree_in_the_model():
    cd = config_a()
    model, sd = build(cd, torch.float32, seed=3)
    toks = tokens_for(cd, 70, 6)
    outs = []
    for fused in (True, False):
        model.decoder.fused_conv_store = fused
        steps = [([("a", toks[:40], list(range(40)))], [])] + [([("a", [t], [0])], []) for t in toks[40:]]
        out, _ = run_schedule(model, steps, 128)
        outs.append(torch.stack(out["a"]))
    assert rel_err(outs[0], outs[1].double()) < 1e-5
    assert close(outs[0], O.forward(sd, cd, toks), torch.float32)


def test_plain_and_tensor_core_attention_agree_in_the_model():
    cd = config_c()
    model, sd = build(cd, torch.bfloat16, seed=4)
    toks = tokens_for(cd, 180, 5)
    want = O.forward(sd, cd, toks)
    for tc, fused in ((True, True), (True, False), (False, False)):
        model.decoder.tensor_attention, model.decoder.fused_maps = tc, fused
        got = StepScheduler(model, max_tokens=256, slots=1).run_step([("a", toks, list(range(len(toks))))], ["a"])
        assert close(got, want, torch.bfloat16), row_errors(got, want).max()


# ---------------------------------------------------------------------------------------- decoding, portions, batches, reuse
@pytest.mark.parametrize("cfgf", [config_a, config_b, config_c])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prefill_against_token_by_token_decoding(cfgf, dtype):
    cd = cfgf()
    model, sd = build(cd, dtype, seed=7)
    toks = tokens_for(cd, 90, 8)
    want = O.forward(sd, cd, toks)
    # 30 tokens as a prompt, then one by one (the decode-only steps go through the captured graph)
    steps = [([("r", toks[:30], [29])], [])] + [([("r", [toks[i]], [0])], []) for i in range(30, 90)]
    out, _ = run_schedule(model, steps, 128)
    got = torch.stack(out["r"])
    assert close(got, want[29:], dtype), row_errors(got, want[29:]).max()
    # and from the very first token on, without the graph
    model.decoder.use_graph = False
    model.decoder._graphs.clear()
    out, _ = run_schedule(model, [([("r", [toks[i]], [0])], []) for i in range(40)], 64)
    assert close(torch.stack(out["r"]), want[:40], dtype)


@pytest.mark.parametrize("cfgf", [config_a, config_c])
@pytest.mark.parametrize("sizes", [[2] * 30, [1, 2, 3, 5, 8, 13, 21, 7], [16, 16, 16, 12], [59, 1], [3, 57]])
def test_portions_of_several_sizes(cfgf, sizes):
    cd = cfgf()
    model, sd = build(cd, torch.float32, seed=9)
    toks = tokens_for(cd, 60, 10)
    want = O.forward(sd, cd, toks)
    steps, at = [], 0
    for n in sizes:
        steps.append(([("p", toks[at:at + n], list(range(n)))], []))
        at += n
    assert at == 60
    out, _ = run_schedule(model, steps, 64)
    assert rel_err(torch.stack(out["p"]), want) < TOL[torch.float32]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batches_of_unequal_requests_and_reuse_of_pages_and_slots(dtype):
    """Five requests over three slots and a pool that holds far less than their sum: portions of some beside single tokens of others,
    requests that pause, slots and pages that change hands (poisoned with NaN in between)."""
    cd = config_a(page=16)
    model, sd = build(cd, dtype, seed=11)
    lens = {"a": 70, "b": 9, "c": 41, "d": 33, "e": 18}
    toks = {k: tokens_for(cd, n, 20 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: O.forward(sd, cd, toks[k]) for k in lens}
    sched = StepScheduler(model, max_tokens=160, slots=3)
    fed = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    plan = [[("a", 17), ("b", 2)], [("a", 1), ("b", 7), ("c", 30)], [("a", 20), ("c", 1)], [("c", 1), ("a", 1)], [("c", 9), ("d", 5)],
            [("a", 31), ("d", 1)], [("d", 27), ("e", 2)], [("e", 1)], [("e", 15)]]
    for step in plan:
        entries, end = [], []
        for k, n in step:
            entries.append((k, toks[k][fed[k]:fed[k] + n], list(range(n))))
            fed[k] += n
            if fed[k] == lens[k]:
                end.append(k)
        lg = sched.run_step(entries, [])
        at = 0
        for k, n in step:
            got[k] += [lg[at + i].float().cpu() for i in range(n)]
            at += n
        for k in end:   # what the request leaves behind must never be read by the next owner
            r = sched.live[k]
            for pool in sched.cache.pools:
                pool[torch.tensor(r.pages, device=DEV)] = float("nan")
            sched.cache.poison_slot(r.slot)
            sched.release(k)
    assert all(fed[k] == lens[k] for k in lens)
    for k in lens:
        assert close(torch.stack(got[k]), want[k], dtype), (k, row_errors(torch.stack(got[k]), want[k]).max())


def test_long_decoding_through_windows_and_pages():
    """Hundreds of single-token steps: the window slides off the prompt and over decoded tokens, the kept first keys fall tiles
    behind it, pages fill and new ones are taken; two requests of different lengths decode together."""
    cd = config_c(page=16)
    model, sd = build(cd, torch.float32, seed=13)
    ta, tb = tokens_for(cd, 330, 14), tokens_for(cd, 250, 15)
    wa, wb = O.forward(sd, cd, ta), O.forward(sd, cd, tb)
    steps = [([("a", ta[:80], [79])], [])]
    for i in range(250):
        steps.append(([("a", [ta[80 + i]], [0]), ("b", [tb[i]], [0])], []))
    out, _ = run_schedule(model, steps, 640)
    assert rel_err(torch.stack(out["a"]), wa[79:]) < TOL[torch.float32]
    assert rel_err(torch.stack(out["b"]), wb) < TOL[torch.float32]


# --------------------------------------------------------------------------------------------------------- greedy generation
def test_greedy_generation_through_the_scheduler():
    cd = config_a()
    model, sd = build(cd, torch.float32, seed=17)
    prompts = [tokens_for(cd, n, 30 + n) for n in (5, 23, 1, 40, 12, 17)]   # six prompts over four slots: slots are used again
    outs = model.generate(prompts, max_new_tokens=12, slots=4, chunk=16)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for _ in range(12):
            lg = O.forward(sd, cd, seq)[-1]
            top2 = torch.topk(lg, 2).values
            nxt = int(lg.argmax())
            if float(top2[0] - top2[1]) < 1e-3:     # a near tie: follow the model, the next comparison starts from its choice
                nxt = int(o[len(seq)])
            assert int(o[len(seq)]) == nxt
            seq.append(nxt)
        assert o.tolist() == seq
