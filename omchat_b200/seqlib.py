"""ctypes binding of libomchat_b200_seq.so (include/omchat_b200_seq.h): the sequence-step kernels, with torch-tensor wrappers.

Like `lib`, there is no fallback: CPU tensors are refused and a failing call raises. The library is built on first use when a
fresh checkout has none yet (`build.ensure("seq")`, a few seconds of nvcc).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import lib as _core
from .lib import OmcError, _need_cuda, _ptr, _stream

_P, _I, _L, _F = c_void_p, c_int, c_longlong, c_float
DT_F32, DT_BF16 = 0, 1
ACT_NONE, ACT_RELU2, ACT_GELU_TANH, ACT_GELU_ERF, ACT_CLAMP_SWISH, ACT_SILU = 0, 1, 2, 3, 4, 5
ROUTER_SOFTMAX, ROUTER_SIGMOID = 0, 1
CONV_LINEAR, CONV_SILU = 0, 1
LINEAR_TILE = 64  # rows per tile of omc_linear's tile -> group table

SIGNATURES = {
    "omc_last_error": (c_char_p, []),
    "omc_linear": (_I, [_P, _I, _L, _L, _P, _I, _L, _L, _P, _I, _L, _L, _I, _I, _I, _I, _F, _I, _P, _L, _P]),
    "omc_linear_bias": (_I, [_P, _I, _L, _L, _P, _I, _L, _L, _P, _I, _L, _L, _I, _I, _I, _I, _F, _I, _P, _L, _P, _L, _P]),
    "omc_post_norm_residual": (_I, [_P, _L, _P, _P, _L, _P, _P, _I, _F, _F, _P, _L, _P, _P, _I, _L, _I, _I, _P]),
    "omc_glu_mul": (_I, [_P, _I, _L, _I, _I, _I, _F, _F, _F, _P, _I, _L, _P]),
    "omc_embed_sinusoid": (_I, [_P, _P, _I, _P, _I, _I, _I, _F, _P, _P, _L, _P]),
    "omc_diff_heads_gate": (_I, [_P, _L, _I, _I, _I, _F, _F, _F, _P, _L, _I, _P, _I, _L, _P]),
    "omc_causal_conv": (_I, [_P, _L, _I, _I, _P, _P, _I, _I, _P, _P, _P, _P, _I, _L, _I, _I, _I, _F, _I, _F, _I, _P]),
    "omc_dyt_conv": (_I, [_P, _L, _P, _L, _F, _P, _L, _F, _P, _L, _P, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _L, _I, _I, _I, _P]),
    "omc_dyt_rows": (_I, [_P, _L, _P, _P, _P, _I, _P, _I, _L, _I, _I, _P]),
    "omc_tanh_cap_rows": (_I, [_P, _L, _I, _I, _F, _P]),
    "omc_selective_scan": (_I, [_P, _I, _L, _P, _L, _P, _P, _L, _P, _L, _P, _P, _P, _L, _P, _P, _I, _L, _P, _I, _P, _P, _I, _I, _P]),
    "omc_pos_qkv_store": (_I, [_P, _L, _I, _P, _L, _I, _I, _P, _L, _I, _P, _I, _F, _I, _I, _F, _I, _P, _P, _P, _I, _I, _P, _P, _L, _I, _P]),
    "omc_moe_combine_depth": (_I, [_P, _L, _P, _P, _I, _P, _L, _P, _L, _F, _P, _L, _F, _F, _P, _L, _L, _I, _P, _I, _P, _L, _I, _I, _P]),
    "omc_conv_qk_norm_kv_store": (_I, [_P, _L, _I, _I, _P, _I, _I, _P, _P, _P, _I, _I, _I, _P, _P, _F, _P, _I, _I, _P, _P, _L, _I, _I, _P]),
    "omc_linear_state_scan": (_I, [_P, _L, _P, _L, _P, _L, _I, _I, _P, _P, _L, _P, _P, _P, _L, _P, _P, _L, _P, _I, _P, _P, _I, _I, _I, _I, _F, _F, _P]),
    "omc_map_rows": (_I, [_P, _L, _I, _I, _I, _P, _P, _I, _F, _P]),
    "omc_gated_rms_rows": (_I, [_P, _L, _I, _I, _I, _P, _I, _F, _P, _L, _I, _P, _I, _L, _P]),
    "omc_qk_norm_kv_store": (_I, [_P, _L, _I, _I, _P, _P, _L, _I, _I, _P, _I, _P, _L, _I, _F, _I, _P, _P, _P, _I, _I, _P, _P, _L, _I, _P]),
    "omc_window_attn": (_I, [_P, _L, _I, _I, _I, _I, _I, _I, _P, _I, _P, _I, _I, _P, _P, _I, _I, _F, _F, _P, _P, _P, _L, _I, _P, _I, _L, _P]),
    "omc_window_attn_mma_ok": (_I, [_I, _I, _I, _I]),
    "omc_window_attn_mma": (_I, [_P, _L, _I, _I, _I, _I, _I, _I, _P, _P, _I, _I, _P, _I, _P, _P, _I, _I, _F, _F, _P, _P, _P, _L, _I, _P, _I, _L, _P]),
    "omc_diff_attn_pair_ok": (_I, [_I, _I, _I, _I]),
    "omc_diff_attn_pair": (_I, [_P, _L, _I, _I, _I, _I, _I, _P, _P, _I, _I, _P, _I, _I, _I, _F, _F, _F, _F, _P, _L, _I, _P, _I, _L, _P]),
    "omc_embed_scale": (_I, [_P, _I, _P, _I, _I, _I, _F, _P, _L, _P, _I, _L, _P]),
    "omc_rms_rows": (_I, [_P, _L, _P, _I, _I, _F, _P, _I, _L, _I, _I, _P]),
    "omc_norm_residual": (_I, [_P, _L, _P, _I, _F, _P, _L, _P, _I, _L, _I, _I, _P]),
    "omc_latent_kv_store": (_I, [_P, _L, _I, _I, _I, _P, _I, _F, _P, _I, _P, _P, _P, _I, _I, _P, _I, _P]),
    "omc_latent_rope_store": (_I, [_P, _L, _I, _I, _I, _P, _F, _P, _I, _P, _P, _P, _I, _I, _P, _P, _L, _I, _I, _P, _I, _P]),
    "omc_moe_plan_scatter_small": (_I, [_P, _I, _I, _I, _P, _P, _P, _I, _L, _I, _I, _P, _I, _P, _P, _L, _P, _P]),
    "omc_rotary_q": (_I, [_P, _I, _L, _I, _I, _I, _I, _P, _I, _P, _P, _I, _I, _P]),
    "omc_latent_attn": (_I, [_P, _I, _I, _I, _I, _I, _P, _I, _P, _I, _I, _P, _P, _P, _F, _P, _P]),
    "omc_latent_attn_mma": (_I, [_P, _I, _I, _I, _I, _P, _P, _I, _I, _P, _I, _P, _I, _P, _F, _P, _I, _P, _P, _P]),
    "omc_latent_decode_items": (_I, [_P, _P, _I, _I, _I, _P, _P, _P]),
    "omc_router_topk": (_I, [_P, _L, _I, _I, _I, _I, _P, _P, _I, _I, _I, _P, _P, _P, _P, _P]),
    "omc_moe_plan_tiles": (_I, [_P, _I, _I, _I, _P, _P, _P, _P]),
    "omc_moe_scatter_rows": (_I, [_P, _I, _L, _I, _I, _P, _I, _I, _P, _P, _P, _P, _L, _P, _P]),
    "omc_moe_combine_norm": (_I, [_P, _L, _P, _P, _I, _P, _P, _L, _P, _I, _F, _P, _L, _P, _P, _I, _L, _I, _I, _P]),
}

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("OMCHAT_B200_SEQ_LIB")
    if path is None:
        from . import build
        path = str(build.ensure("seq"))
    if not os.path.exists(path):
        raise OmcError(f"{path} not found (there is no CPU fallback)")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _check(rc: int, what: str):
    _core.add_launches(1)
    if rc != 0:
        raise OmcError(f"{what} failed ({rc}): {load().omc_last_error().decode(errors='replace')}")


def dt_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return DT_F32
    if dtype == torch.bfloat16:
        return DT_BF16
    raise OmcError(f"the sequence-step kernels store float32 or bfloat16, not {dtype}")


def _dt(t: Optional[torch.Tensor]) -> int:
    return DT_F32 if t is None else dt_code(t.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, M: Optional[int] = None, N: Optional[int] = None,
           K: Optional[int] = None, ldx: Optional[int] = None, ldw: Optional[int] = None, ldy: Optional[int] = None,
           batch: int = 1, sx: int = 0, sw: int = 0, sy: int = 0, alpha: float = 1.0, act: int = ACT_NONE,
           tile_group: Optional[torch.Tensor] = None, group_stride: int = 0, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = act(alpha * x @ w^T (+ bias)). With the defaults x [M, K], w [N, K], out [M, N] are 2-D row-strided tensors; the keyword
    overrides describe batched column slices (heads) or a grouped product over expert-sorted row tiles (see the header)."""
    _need_cuda(x, w, out, tile_group)
    M = x.shape[0] if M is None else M
    K = x.shape[-1] if K is None else K
    N = w.shape[-2] if N is None else N
    ldx = x.stride(0) if ldx is None else ldx
    ldw = w.stride(-2) if ldw is None else ldw
    ldy = out.stride(0) if ldy is None else ldy
    if bias is not None:
        _need_cuda(bias)
        assert bias.dtype == w.dtype and bias.numel() == N and batch == 1
        rc = load().omc_linear_bias(_ptr(x), _dt(x), ldx, sx, _ptr(w), _dt(w), ldw, sw, _ptr(out), _dt(out), ldy, sy, M, N, K, batch,
                                    alpha, act, _ptr(tile_group), group_stride, _ptr(bias), 0, _stream())
    else:
        rc = load().omc_linear(_ptr(x), _dt(x), ldx, sx, _ptr(w), _dt(w), ldw, sw, _ptr(out), _dt(out), ldy, sy, M, N, K, batch,
                               alpha, act, _ptr(tile_group), group_stride, _stream())
    _check(rc, "omc_linear")
    return out


def embed_scale(ids: torch.Tensor, table: torch.Tensor, scale: float, h32: torch.Tensor, xb: Optional[torch.Tensor]):
    _need_cuda(ids, table, h32, xb)
    assert ids.dtype == torch.int32 and h32.dtype == torch.float32 and table.is_contiguous()
    T, C = ids.numel(), table.shape[1]
    rc = load().omc_embed_scale(_ptr(ids), T, _ptr(table), _dt(table), C, table.shape[0], scale, _ptr(h32), h32.stride(0),
                                _ptr(xb), _dt(xb), xb.stride(0) if xb is not None else 0, _stream())
    _check(rc, "omc_embed_scale")


def sinusoid_frequencies(C: int, base: float, device) -> torch.Tensor:
    """float64 [ceil(C / 2)] on the device: f_i = base^(-2i / C), the table omc_embed_sinusoid reads."""
    n = (C + 1) // 2
    return torch.tensor([base ** (-2.0 * i / C) for i in range(n)], dtype=torch.float64).to(device)


def embed_sinusoid(ids: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, scale: float, freq: torch.Tensor, h32: torch.Tensor):
    """h32[t] = table[ids[t]] * scale + (sin, cos)(pos[t] * freq) interleaved (entry 2i: sin, 2i + 1: cos)."""
    _need_cuda(ids, pos, table, freq, h32)
    T, C = ids.numel(), table.shape[1]
    assert ids.dtype == torch.int32 and pos.dtype == torch.int32 and h32.dtype == torch.float32 and table.is_contiguous()
    assert freq.dtype == torch.float64 and freq.is_contiguous() and freq.numel() >= (C + 1) // 2
    rc = load().omc_embed_sinusoid(_ptr(ids), _ptr(pos), T, _ptr(table), _dt(table), C, table.shape[0], scale, _ptr(freq), _ptr(h32),
                                   h32.stride(0), _stream())
    _check(rc, "omc_embed_sinusoid")


def rms_rows(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, out: torch.Tensor, one_plus: bool = False, n: Optional[int] = None):
    """out[t] = x[t, :n] / rms * (w | 1 + w); x fp32 [rows, >= n]."""
    _need_cuda(x, w, out)
    assert x.dtype == torch.float32 and x.stride(1) == 1 and out.stride(1) == 1
    n = x.shape[1] if n is None else n
    rc = load().omc_rms_rows(_ptr(x), x.stride(0), _ptr(w), _dt(w), 1 if one_plus else 0, eps, _ptr(out), _dt(out), out.stride(0),
                             x.shape[0], n, _stream())
    _check(rc, "omc_rms_rows")
    return out


def norm_residual(y: torch.Tensor, w: torch.Tensor, eps: float, h32: torch.Tensor, xb: Optional[torch.Tensor]):
    """h32 += y / rms(y) * (1 + w); xb = round(h32)."""
    _need_cuda(y, w, h32, xb)
    assert y.dtype == torch.float32 and h32.dtype == torch.float32
    rc = load().omc_norm_residual(_ptr(y), y.stride(0), _ptr(w), _dt(w), eps, _ptr(h32), h32.stride(0), _ptr(xb), _dt(xb),
                                  xb.stride(0) if xb is not None else 0, y.shape[0], y.shape[1], _stream())
    _check(rc, "omc_norm_residual")


def latent_kv_store(dkv: torch.Tensor, r: int, dr: int, w: torch.Tensor, eps: float, cs: torch.Tensor, rot_dims: int,
                    pos: torch.Tensor, slot: torch.Tensor, block_table: torch.Tensor, page_size: int, pool: torch.Tensor):
    _need_cuda(dkv, w, cs, pos, slot, block_table, pool)
    assert dkv.dtype == torch.float32 and cs.dtype == torch.float32 and pos.dtype == torch.int32 and slot.dtype == torch.int32
    assert block_table.dtype == torch.int32 and block_table.is_contiguous() and pool.is_contiguous() and pool.shape[-1] == r + dr
    rc = load().omc_latent_kv_store(_ptr(dkv), dkv.stride(0), dkv.shape[0], r, dr, _ptr(w), _dt(w), eps, _ptr(cs), rot_dims,
                                    _ptr(pos), _ptr(slot), _ptr(block_table), block_table.shape[1], page_size, _ptr(pool),
                                    _dt(pool), _stream())
    _check(rc, "omc_latent_kv_store")


def latent_rope_store(dkv, r: int, dr: int, w, eps: float, cs, rot_dims: int, pos, slot, block_table, page_size: int, pool, q, H: int,
                      dn: int, qcat):
    """latent_kv_store + rotary_q in one launch (w, pool, q, qcat of one dtype)."""
    _need_cuda(dkv, w, cs, pos, slot, block_table, pool, q, qcat)
    assert dkv.dtype == torch.float32 and w.dtype == pool.dtype == q.dtype == qcat.dtype and q.stride(1) == 1
    assert block_table.is_contiguous() and pool.is_contiguous() and qcat.is_contiguous() and pool.shape[-1] == r + dr
    rc = load().omc_latent_rope_store(_ptr(dkv), dkv.stride(0), dkv.shape[0], r, dr, _ptr(w), eps, _ptr(cs), rot_dims, _ptr(pos), _ptr(slot),
                                      _ptr(block_table), block_table.shape[1], page_size, _ptr(pool), _ptr(q), q.stride(0), H, dn,
                                      _ptr(qcat), _dt(pool), _stream())
    _check(rc, "omc_latent_rope_store")


def moe_plan_scatter_small(counts, experts: int, tile: int, max_tiles: int, seg_start, tile_group, x, ids, top: int, slot_of, xs,
                           row_w: Optional[torch.Tensor] = None):
    """moe_plan_tiles + moe_scatter_rows as one single-CTA launch (steps of a few rows). row_w as in moe_scatter_rows."""
    _need_cuda(counts, seg_start, tile_group, x, ids, slot_of, xs, row_w)
    assert x.dtype == xs.dtype
    rc = load().omc_moe_plan_scatter_small(_ptr(counts), experts, tile, max_tiles, _ptr(seg_start), _ptr(tile_group), _ptr(x), _dt(x),
                                           x.stride(0), x.shape[0], x.shape[1], _ptr(ids), top, _ptr(slot_of), _ptr(xs), xs.stride(0),
                                           _ptr(row_w), _stream())
    _check(rc, "omc_moe_plan_scatter_small")


def rotary_q(q32: torch.Tensor, H: int, dn: int, dr: int, cs: torch.Tensor, rot_dims: int, pos: torch.Tensor, qcat: torch.Tensor,
             r: int):
    _need_cuda(q32, cs, pos, qcat)
    assert qcat.is_contiguous() and qcat.shape[-1] == r + dr and q32.stride(1) == 1
    rc = load().omc_rotary_q(_ptr(q32), _dt(q32), q32.stride(0), q32.shape[0], H, dn, dr, _ptr(cs), rot_dims, _ptr(pos), _ptr(qcat),
                             _dt(qcat), r, _stream())
    _check(rc, "omc_rotary_q")


def latent_attn(qcat: torch.Tensor, r: int, dr: int, pool: torch.Tensor, block_table: torch.Tensor, page_size: int,
                pos: torch.Tensor, slot: torch.Tensor, sink: Optional[torch.Tensor], scale: float, out: torch.Tensor):
    """qcat [T, H, r + dr] -> out fp32 [T, H, r] (weighted sums of cached latents)."""
    _need_cuda(qcat, pool, block_table, pos, slot, sink, out)
    T, H = qcat.shape[0], qcat.shape[1]
    assert out.dtype == torch.float32 and out.is_contiguous() and qcat.is_contiguous()
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == H)
    rc = load().omc_latent_attn(_ptr(qcat), _dt(qcat), T, H, r, dr, _ptr(pool), _dt(pool), _ptr(block_table), block_table.shape[1],
                                page_size, _ptr(pos), _ptr(slot), _ptr(sink), scale, _ptr(out), _stream())
    _check(rc, "omc_latent_attn")
    return out


MMA_ROWS = 64  # rows ((token, head) pairs) and keys per tile of the tensor-core latent attention


def latent_attn_mma_ok(H: int, r: int, dr: int, dtype: torch.dtype) -> bool:
    """Shapes the tensor-core kernel takes; everything else runs on the plain kernel."""
    exchange = (MMA_ROWS * (MMA_ROWS + 8) * 2 + 4 * MMA_ROWS * 4) if r > 128 else 0   # probabilities / row statistics of a row group
    return (dtype == torch.bfloat16 and H <= MMA_ROWS and r % 16 == 0 and 0 < r <= 512 and dr % 16 == 0
            and 2 * MMA_ROWS * (r + dr + 8) * 2 + exchange <= 227 * 1024)


class LatentAttnPlan:
    """Work list of one step for one head count (omc_latent_attn_mma): items, merge groups and the partial-result workspace.
    portions: host list of (first_row, n_rows, slot, first_pos) - the consecutive rows of each request in the packed batch.
    Contexts are cut into key ranges (multiples of 64 keys, at least `min_keys` each) while the step has fewer CTAs than
    `target_ctas`, so that a few decode rows over a long context still fill the device."""

    MAX_PARTS = 64  # key ranges one merge group may have (csrc/latent_attention.cu: kMergeMaxParts)

    def __init__(self, portions, H: int, device, target_ctas: int = 296, min_keys: int = 128):
        import numpy as np
        tok = max(1, MMA_ROWS // H)
        base = sum(-(-n // tok) for _, n, _, _ in portions)
        items, merges, part = [], [], 0
        for first_row, n, slot, p0 in portions:
            starts = np.arange(0, n, tok, dtype=np.int64)
            ntok = np.minimum(tok, n - starts)
            keys = p0 + starts + ntok                                  # keys the tile's last row sees
            parts = np.ones_like(starts)
            if base < target_ctas // 2:
                parts = np.clip(np.minimum(-(-keys // min_keys), -(-target_ctas // max(base, 1))), 1, self.MAX_PARTS)
            for i in range(len(starts)):
                np_i, k = int(parts[i]), int(keys[i])
                fr, nt = first_row + int(starts[i]), int(ntok[i])
                if np_i == 1:
                    items.append((fr, nt, slot, p0 + int(starts[i]), 0, k, -1, 0))
                    continue
                span = -(-(-(-k // np_i)) // MMA_ROWS) * MMA_ROWS       # keys per part, a multiple of 64
                np_i = -(-k // span)
                merges.append((fr * H, nt * H, part, np_i))
                for j in range(np_i):
                    items.append((fr, nt, slot, p0 + int(starts[i]), j * span, min(k, (j + 1) * span), part, 0))
                    part += 1
        self.n_items, self.n_merges, self.n_parts = len(items), len(merges), part
        flat = torch.tensor(items, dtype=torch.int32).view(-1)
        flat = torch.cat([flat, torch.tensor(merges, dtype=torch.int32).view(-1)]) if merges else flat
        buf = flat.pin_memory().to(device, non_blocking=True)
        self.items = buf[:self.n_items * 8]
        self.merges = buf[self.n_items * 8:] if merges else None


class DecodeAttnPlan:
    """Work list of a decode-only step of B rows with static device buffers: `fill(pos, slot)` rewrites it on the device each step
    (omc_latent_decode_items), so a captured CUDA graph stays valid while the contexts grow. parts: key ranges per row."""

    def __init__(self, B: int, H: int, parts: int, device):
        self.B, self.H, self.parts = B, H, parts
        self.items = torch.zeros(B * parts * 8, device=device, dtype=torch.int32)
        self.merges = torch.zeros(B * 4, device=device, dtype=torch.int32) if parts > 1 else None
        self.n_items = B * parts
        self.n_merges = B if parts > 1 else 0
        self.n_parts = B * parts if parts > 1 else 0

    @staticmethod
    def parts_for(B: int, max_keys: int, target_ctas: int = 296, min_keys: int = 128) -> int:
        """Key ranges per row for contexts up to max_keys (rounded up to a power of two, so that a growing context changes the
        answer - and with it the captured graph - only a few times)."""
        bucket = 1 << max(max_keys - 1, 0).bit_length()
        return max(1, min(bucket // min_keys, -(-target_ctas // B), LatentAttnPlan.MAX_PARTS))

    def fill(self, pos: torch.Tensor, slot: torch.Tensor):
        rc = load().omc_latent_decode_items(_ptr(pos), _ptr(slot), self.B, self.H, self.parts, _ptr(self.items), _ptr(self.merges),
                                            _stream())
        _check(rc, "omc_latent_decode_items")


_mma_ws = {}


def latent_attn_mma(qcat: torch.Tensor, r: int, dr: int, pool: torch.Tensor, block_table: torch.Tensor, page_size: int,
                    plan: LatentAttnPlan, sink: Optional[torch.Tensor], scale: float, out: torch.Tensor):
    _need_cuda(qcat, pool, block_table, plan.items, sink, out)
    T, H = qcat.shape[0], qcat.shape[1]
    assert qcat.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16
    assert qcat.is_contiguous() and out.is_contiguous() and pool.is_contiguous()
    ws_o = ws_ml = None
    if plan.n_parts:
        key = (str(qcat.device), torch.cuda.current_stream().cuda_stream)
        need = plan.n_parts * MMA_ROWS * (r + 2)
        ws = _mma_ws.get(key)
        if ws is None or ws.numel() < need:
            ws = torch.empty(need, device=qcat.device, dtype=torch.float32)
            _mma_ws[key] = ws
        ws_o, ws_ml = ws[:plan.n_parts * MMA_ROWS * r], ws[plan.n_parts * MMA_ROWS * r:]
    rc = load().omc_latent_attn_mma(_ptr(qcat), T, H, r, dr, _ptr(pool), _ptr(block_table), block_table.shape[1], page_size,
                                    _ptr(plan.items), plan.n_items, _ptr(plan.merges), plan.n_merges, _ptr(sink), scale, _ptr(out),
                                    _dt(out), _ptr(ws_o), _ptr(ws_ml), _stream())
    _check(rc, "omc_latent_attn_mma")
    if plan.n_merges:
        _core.add_launches(1)
    return out


def router_topk(z: torch.Tensor, e_tot: int, experts: int, top: int, correction: Optional[torch.Tensor], has_gate: bool,
                ids: torch.Tensor, w: torch.Tensor, gate: Optional[torch.Tensor], counts: torch.Tensor,
                bias: Optional[torch.Tensor] = None, renorm: bool = False, score: int = ROUTER_SOFTMAX):
    """bias: fp32 [e_tot] added to the logits; renorm: the weights of the chosen are divided by their sum (softmax over the chosen);
    score ROUTER_SIGMOID: every output is scored by a sigmoid of its own instead of the softmax over all."""
    _need_cuda(z, correction, bias, ids, w, gate, counts)
    assert z.dtype == torch.float32 and ids.dtype == torch.int32 and w.dtype == torch.float32 and counts.dtype == torch.int32
    assert correction is None or correction.dtype == torch.float32
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == e_tot)
    rc = load().omc_router_topk(_ptr(z), z.stride(0), z.shape[0], e_tot, experts, top, _ptr(correction), _ptr(bias), 1 if renorm else 0, score,
                                1 if has_gate else 0, _ptr(ids), _ptr(w), _ptr(gate), _ptr(counts), _stream())
    _check(rc, "omc_router_topk")


def moe_max_tiles(T: int, top: int, experts: int, tile: int = LINEAR_TILE) -> int:
    """Upper bound of the row tiles of the expert-sorted layout: every (row, choice) pair plus one partly filled tile per expert."""
    return (T * top + tile - 1) // tile + experts


def moe_plan_tiles(counts, experts: int, tile: int, max_tiles: int, seg_start, cursor, tile_group):
    _need_cuda(counts, seg_start, cursor, tile_group)
    rc = load().omc_moe_plan_tiles(_ptr(counts), experts, tile, max_tiles, _ptr(seg_start), _ptr(cursor), _ptr(tile_group), _stream())
    _check(rc, "omc_moe_plan_tiles")


def moe_scatter_rows(x, ids, top: int, experts: int, seg_start, cursor, slot_of, xs, row_w: Optional[torch.Tensor] = None):
    """row_w fp32 [T, top]: the copy of a row for its j-th choice is multiplied by row_w[t, j] (weights on the experts' input)."""
    _need_cuda(x, ids, seg_start, cursor, slot_of, xs, row_w)
    assert row_w is None or (row_w.dtype == torch.float32 and row_w.is_contiguous())
    assert x.dtype == xs.dtype
    rc = load().omc_moe_scatter_rows(_ptr(x), _dt(x), x.stride(0), x.shape[0], x.shape[1], _ptr(ids), top, experts, _ptr(seg_start),
                                     _ptr(cursor), _ptr(slot_of), _ptr(xs), xs.stride(0), _ptr(row_w), _stream())
    _check(rc, "omc_moe_scatter_rows")


def moe_combine_depth(ys: Optional[torch.Tensor], slot_of, w: Optional[torch.Tensor], top: int, x: torch.Tensor, mult: float,
                      streams: Optional[torch.Tensor], n_streams: int, coef: Optional[torch.Tensor], out: torch.Tensor,
                      y1: Optional[torch.Tensor] = None, a1: float = 0.0, y2: Optional[torch.Tensor] = None, a2: float = 0.0):
    """xn = x + a1 y1 + a2 y2 + mult * sum_j (w[t, j] | 1) ys[slot_of[t, j]] (absent terms are zero) -> streams[n_streams - 1];
    out = sum_j coef[j] streams[j] over the first n_streams of streams fp32 [>= n_streams, T, C] (coef None: out = xn)."""
    _need_cuda(ys, slot_of, w, x, streams, coef, out, y1, y2)
    for t in (y1, y2):
        assert t is None or (t.dtype == torch.float32 and t.stride(1) == 1)
    assert x.dtype == torch.float32 and out.dtype == torch.float32 and x.stride(1) == 1 and out.stride(1) == 1
    assert streams is None or (streams.dtype == torch.float32 and streams.stride(2) == 1 and streams.shape[0] >= n_streams)
    assert coef is None or (coef.is_contiguous() and coef.numel() >= n_streams)
    rc = load().omc_moe_combine_depth(_ptr(ys), ys.stride(0) if ys is not None else 0, _ptr(slot_of), _ptr(w), top, _ptr(x), x.stride(0),
                                      _ptr(y1), y1.stride(0) if y1 is not None else 0, a1, _ptr(y2), y2.stride(0) if y2 is not None else 0, a2,
                                      mult, _ptr(streams), streams.stride(0) if streams is not None else 0,
                                      streams.stride(1) if streams is not None else 0, n_streams, _ptr(coef), _dt(coef), _ptr(out),
                                      out.stride(0), x.shape[0], x.shape[1], _stream())
    _check(rc, "omc_moe_combine_depth")


def moe_combine_norm(ys: Optional[torch.Tensor], slot_of, w, top: int, gate, ysh: Optional[torch.Tensor], nw, eps: float, h32, xb,
                     w_next: Optional[torch.Tensor] = None):
    """w_next: xb receives h32 / rms(h32) * (1 + w_next), the next sublayer's normed input, instead of the rounded h32."""
    _need_cuda(ys, slot_of, w, gate, ysh, nw, h32, xb, w_next)
    assert w_next is None or w_next.dtype == nw.dtype
    rc = load().omc_moe_combine_norm(_ptr(ys), ys.stride(0) if ys is not None else 0, _ptr(slot_of), _ptr(w), top, _ptr(gate),
                                     _ptr(ysh), ysh.stride(0) if ysh is not None else 0, _ptr(nw), _dt(nw), eps, _ptr(h32),
                                     h32.stride(0), _ptr(w_next), _ptr(xb), _dt(xb), xb.stride(0) if xb is not None else 0, h32.shape[0],
                                     h32.shape[1], _stream())
    _check(rc, "omc_moe_combine_norm")


# ---- pre/post norms around sublayers, gated feed-forward halves
def post_norm_residual(y1: torch.Tensor, w_post: torch.Tensor, eps: float, mult: float, h32: torch.Tensor,
                       w_next: Optional[torch.Tensor], xb: Optional[torch.Tensor], y2: Optional[torch.Tensor] = None,
                       wa: Optional[torch.Tensor] = None, wb: Optional[torch.Tensor] = None):
    """h32 += mult * N(y), N(y) = y / rms(y) * (1 + w_post), with y = y1 or the mean of y1 / rms * wa and y2 / rms * wb;
    xb = h32 / rms(h32) * (1 + w_next) (w_next None: the rounded h32)."""
    _need_cuda(y1, y2, wa, wb, w_post, h32, w_next, xb)
    assert y1.dtype == torch.float32 and h32.dtype == torch.float32 and y1.stride(1) == 1 and (y2 is None or y2.dtype == torch.float32)
    rc = load().omc_post_norm_residual(_ptr(y1), y1.stride(0), _ptr(wa), _ptr(y2), y2.stride(0) if y2 is not None else 0, _ptr(wb),
                                       _ptr(w_post), _dt(w_post), eps, mult, _ptr(h32), h32.stride(0), _ptr(w_next), _ptr(xb), _dt(xb),
                                       xb.stride(0) if xb is not None else 0, h32.shape[0], h32.shape[1], _stream())
    _check(rc, "omc_post_norm_residual")


def glu_mul(z: torch.Tensor, n: int, act: int, out: torch.Tensor, limit: float = 0.0, slope: float = 1.0, shift: float = 0.0):
    """out[:, c] = act(z[:, c]) * z[:, n + c]. ACT_CLAMP_SWISH: g = min(z[:, c], limit), u = clamp(z[:, n + c], -limit, limit),
    out = g * sigmoid(slope * g) * (u + shift)."""
    _need_cuda(z, out)
    assert z.stride(1) == 1 and out.stride(1) == 1 and z.shape[1] >= 2 * n
    rc = load().omc_glu_mul(_ptr(z), _dt(z), z.stride(0), z.shape[0], n, act, limit, slope, shift, _ptr(out), _dt(out), out.stride(0),
                            _stream())
    _check(rc, "omc_glu_mul")
    return out


# ---- state mixers
GATE_NONE, GATE_SILU, GATE_SIGMOID = 0, 1, 2
DECAY_CONST, DECAY_HEAD, DECAY_CHANNEL, DECAY_GIVEN, DECAY_SIGMOID_POW, DECAY_GIVEN_MINUS_ONE = 0, 1, 2, 3, 4, 5
MAP_SILU, MAP_DECAY, MAP_SIGMOID_POW = 1, 2, 3


def causal_conv_silu(x: torch.Tensor, w: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, state: Optional[torch.Tensor],
                     y: torch.Tensor, unit_channels: int = 0, unit_group: int = 0, unit_eps: float = 1e-6, scaled_channels: int = 0,
                     unit_mult: float = 1.0, single_rows: bool = False, act: int = CONV_SILU, bias: Optional[torch.Tensor] = None):
    """x fp32 [T, >= ch] (a column slice is fine), w [ch, taps], state fp32 [slots, taps - 1, ch] -> y [T, ch] (fp32 or bf16).
    single_rows: every row is a request of its own (one launch instead of two). act: CONV_SILU, or CONV_LINEAR for the weighted
    sum itself (`causal_conv`). bias [ch] of w's dtype: added in front of the activation."""
    _need_cuda(x, w, pos, slot, state, y, bias)
    ch, taps = w.shape
    assert x.dtype == torch.float32 and x.stride(1) == 1 and y.stride(1) == 1 and w.is_contiguous()
    assert bias is None or (bias.dtype == w.dtype and bias.numel() == ch and bias.is_contiguous())
    assert pos.dtype == torch.int32 and slot.dtype == torch.int32
    assert taps == 1 or (state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (taps - 1, ch))
    rc = load().omc_causal_conv(_ptr(x), x.stride(0), x.shape[0], ch, _ptr(w), _ptr(bias), _dt(w), taps, _ptr(pos), _ptr(slot), _ptr(state),
                                _ptr(y), _dt(y), y.stride(0), act, unit_channels, unit_group, unit_eps, scaled_channels, unit_mult,
                                1 if single_rows else 0, _stream())
    _check(rc, "omc_causal_conv")
    if taps > 1 and not single_rows:
        _core.add_launches(1)
    return y


def causal_conv(x, w, pos, slot, state, y, single_rows: bool = False):
    """The causal convolution alone (no activation, no unit vectors)."""
    return causal_conv_silu(x, w, pos, slot, state, y, single_rows=single_rows, act=CONV_LINEAR)


def conv_qk_norm_kv_store(x: torch.Tensor, w: torch.Tensor, pos, slot, state: Optional[torch.Tensor], nq: int, nk: int, group: int,
                          wq: torch.Tensor, wk: torch.Tensor, eps: float, block_table: torch.Tensor, page_size: int, pool: torch.Tensor,
                          q_out: torch.Tensor, single_rows: bool = False):
    """causal_conv (no activation) over x fp32 [T, nq + nk + nv], then qk_norm_kv_store with norms per `group` channels, in one launch:
    q_out [T, nq] and the cache rows [k | v] receive the results; the convolved rows are never written."""
    _need_cuda(x, w, pos, slot, state, wq, wk, block_table, pool, q_out)
    ch, taps = w.shape
    assert x.dtype == torch.float32 and x.stride(1) == 1 and x.shape[1] >= ch and w.is_contiguous() and q_out.stride(1) == 1
    assert pos.dtype == torch.int32 and slot.dtype == torch.int32 and block_table.dtype == torch.int32 and block_table.is_contiguous()
    assert taps == 1 or (state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (taps - 1, ch))
    assert pool.is_contiguous() and pool.shape[-1] == ch - nq and pool.dtype == q_out.dtype
    assert wq.dtype == wk.dtype == w.dtype and wq.numel() == group and wk.numel() == group
    rc = load().omc_conv_qk_norm_kv_store(_ptr(x), x.stride(0), x.shape[0], ch, _ptr(w), _dt(w), taps, _ptr(pos), _ptr(slot), _ptr(state),
                                          nq, nk, group, _ptr(wq), _ptr(wk), eps, _ptr(block_table), block_table.shape[1], page_size,
                                          _ptr(pool), _ptr(q_out), q_out.stride(0), _dt(pool), 1 if single_rows else 0, _stream())
    _check(rc, "omc_conv_qk_norm_kv_store")
    if taps > 1 and not single_rows:
        _core.add_launches(1)


def linear_state_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, out: torch.Tensor, row_begin: torch.Tensor,
                      portions: int, pos: torch.Tensor, slot: torch.Tensor, H: int, G: int, dim: int, vdim: int, *, silu_in: bool = False,
                      decay_const: Optional[torch.Tensor] = None, a: Optional[torch.Tensor] = None, A_log: Optional[torch.Tensor] = None,
                      dt_bias: Optional[torch.Tensor] = None, channel_decay: bool = False, beta: Optional[torch.Tensor] = None,
                      decay_given: bool = False, sigmoid_pow: Optional[float] = None, out_scale: float = 1.0):
    """The recurrence of omc_linear_state_scan; q / k / v / a / beta are fp32 2-D tensors or column slices of one.
    decay_given: `a` [T, H * dim] already holds the per-channel decays (map_rows(..., MAP_DECAY / MAP_SIGMOID_POW)).
    sigmoid_pow: the decay of key channel i is sigmoid(a[t, i] + dt_bias[i])^sigmoid_pow (with decay_given: `a` holds that decay
    minus one). out_scale multiplies the read-out."""
    _need_cuda(q, k, v, state, out, row_begin, pos, slot, decay_const, a, A_log, dt_bias, beta)
    for t in (q, k, v, out, a, beta):
        assert t is None or (t.dtype == torch.float32 and t.stride(1) == 1)
    for t in (decay_const, A_log, dt_bias):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (H, dim, vdim) and row_begin.dtype == torch.int32
    mode = DECAY_CONST if decay_const is not None else (DECAY_GIVEN if decay_given else (DECAY_CHANNEL if channel_decay else DECAY_HEAD))
    if sigmoid_pow is not None:   # given: by map_rows(..., MAP_SIGMOID_POW), which leaves the decay minus one
        mode = DECAY_GIVEN_MINUS_ONE if decay_given else DECAY_SIGMOID_POW
    rc = load().omc_linear_state_scan(_ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), 1 if silu_in else 0, mode,
                                      _ptr(decay_const), _ptr(a), a.stride(0) if a is not None else 0, _ptr(A_log), _ptr(dt_bias),
                                      _ptr(beta), beta.stride(0) if beta is not None else 0, _ptr(state), _ptr(out), out.stride(0),
                                      _ptr(row_begin), portions, _ptr(pos), _ptr(slot), H, G, dim, vdim,
                                      float(sigmoid_pow or 0.0), out_scale, _stream())
    _check(rc, "omc_linear_state_scan")
    return out


def gated_rms_rows(x: torch.Tensor, groups: int, n: int, w: torch.Tensor, eps: float, gate: Optional[torch.Tensor], gate_act: int,
                   out: torch.Tensor):
    _need_cuda(x, w, gate, out)
    assert x.dtype == torch.float32 and x.stride(1) == 1 and out.stride(1) == 1 and w.numel() == n
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1)
    rc = load().omc_gated_rms_rows(_ptr(x), x.stride(0), x.shape[0], groups, n, _ptr(w), _dt(w), eps, _ptr(gate),
                                   gate.stride(0) if gate is not None else 0, gate_act, _ptr(out), _dt(out), out.stride(0), _stream())
    _check(rc, "omc_gated_rms_rows")
    return out


# ---- windowed attention over a paged key/value cache
def qk_norm_kv_store(q: torch.Tensor, wq: torch.Tensor, k: torch.Tensor, wk: torch.Tensor, v: torch.Tensor, eps: float, pos, slot,
                     block_table: torch.Tensor, page_size: int, pool: torch.Tensor, q_out: torch.Tensor, group: int = 0):
    """group 0: one norm over all query (key) columns, weights as wide as the projections; group > 0: one norm per `group` columns
    with weights [group] shared by the groups (q and k are then given with their true widths)."""
    _need_cuda(q, wq, k, wk, v, pos, slot, block_table, pool, q_out)
    nq, nk, nv = (wq.numel(), wk.numel(), v.shape[1]) if group == 0 else (q.shape[1], k.shape[1], v.shape[1])
    assert group == 0 or (wq.numel() == group and wk.numel() == group)
    assert q.dtype == k.dtype == v.dtype == torch.float32 and q.stride(1) == k.stride(1) == v.stride(1) == 1
    assert pool.is_contiguous() and pool.shape[-1] == nk + nv and pool.dtype == q_out.dtype and wq.dtype == wk.dtype
    assert block_table.dtype == torch.int32 and block_table.is_contiguous() and q_out.stride(1) == 1
    rc = load().omc_qk_norm_kv_store(_ptr(q), q.stride(0), nq, group, _ptr(wq), _ptr(k), k.stride(0), nk, group, _ptr(wk), _dt(wq), _ptr(v), v.stride(0),
                                     nv, eps, q.shape[0], _ptr(pos), _ptr(slot), _ptr(block_table), block_table.shape[1], page_size,
                                     _ptr(pool), _ptr(q_out), q_out.stride(0), _dt(pool), _stream())
    _check(rc, "omc_qk_norm_kv_store")


WINDOW_ALL = 1 << 30   # a window that never ends: plain causal attention


def window_attn(q: torch.Tensor, H: int, G: int, d: int, dv: int, pool: torch.Tensor, block_table: torch.Tensor, page_size: int, pos, slot,
                window: int, scale: float, softcap: float, dist_bias: Optional[torch.Tensor], out: torch.Tensor, maps: int = 1,
                keep_first: int = 0, sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, gate_act: int = 0):
    """q [T, H * maps * d] and pool of one dtype -> out [T, H * maps * dv]. maps: score maps per head (queries and keys of their
    own, shared values); keep_first: the first keys of a sequence stay visible behind the window; sink fp32 [H]: one more
    denominator term exp(sink[h]); gate fp32 [T, H * maps * dv] with gate_act (GATE_*): the output is multiplied by act(gate)."""
    _need_cuda(q, pool, block_table, pos, slot, dist_bias, out, sink, gate)
    assert sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == H)
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1)
    assert q.dtype == pool.dtype and q.stride(1) == 1 and out.stride(1) == 1 and pool.is_contiguous()
    assert pool.shape[-1] == G * (maps * d + dv)
    assert dist_bias is None or (dist_bias.dtype == torch.float32 and dist_bias.is_contiguous() and dist_bias.shape == (window, H))
    rc = load().omc_window_attn(_ptr(q), q.stride(0), q.shape[0], H, G, d, dv, maps, _ptr(pool), _dt(pool), _ptr(block_table),
                                block_table.shape[1], page_size, _ptr(pos), _ptr(slot), window, keep_first, scale, softcap,
                                _ptr(dist_bias), _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0, gate_act, _ptr(out),
                                _dt(out), out.stride(0), _stream())
    _check(rc, "omc_window_attn")
    return out


def window_attn_mma_ok(H: int, G: int, d: int, dv: int, dtype: torch.dtype) -> bool:
    """Shapes the tensor-core kernel takes; everything else runs on the plain kernel."""
    return dtype == torch.bfloat16 and bool(load().omc_window_attn_mma_ok(H, G, d, dv))


def window_attn_items(portions, rep: int, device) -> torch.Tensor:
    """Work list of omc_window_attn_mma for one step: portions [(first_row, n_rows, slot, first_pos)] cut into tiles of 64 // rep
    tokens (rep = query heads per key/value head) -> int32 [n_items, 4] on the device."""
    import numpy as np
    tok = MMA_ROWS // rep
    parts = []
    for first_row, n, slot, p0 in portions:
        st = np.arange(0, n, tok, dtype=np.int32)
        parts.append(np.stack([first_row + st, np.minimum(tok, n - st), np.full_like(st, slot), p0 + st], axis=1))
    flat = torch.from_numpy(np.concatenate(parts, axis=0).astype(np.int32))
    return flat.pin_memory().to(device, non_blocking=True) if torch.device(device).type == "cuda" else flat


def window_attn_mma(q: torch.Tensor, H: int, G: int, d: int, dv: int, pool: torch.Tensor, block_table: torch.Tensor, page_size: int,
                    items: Optional[torch.Tensor], pos, slot, window: int, scale: float, softcap: float,
                    dist_bias: Optional[torch.Tensor], out: torch.Tensor, maps: int = 1, keep_first: int = 0,
                    sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, gate_act: int = 0):
    """items None: every row of q is a request of its own at (slot[t], pos[t]). maps / keep_first / sink / gate as in window_attn."""
    _need_cuda(q, pool, block_table, items, pos, slot, dist_bias, out, sink, gate)
    assert sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == H)
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1)
    assert q.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert pool.is_contiguous() and pool.shape[-1] == G * (maps * d + dv) and block_table.is_contiguous()
    assert items is None or (items.dtype == torch.int32 and items.is_contiguous() and items.shape[1] == 4)
    assert dist_bias is None or (dist_bias.dtype == torch.float32 and dist_bias.is_contiguous() and dist_bias.shape == (window, H))
    rc = load().omc_window_attn_mma(_ptr(q), q.stride(0), q.shape[0], H, G, d, dv, maps, _ptr(pool), _ptr(block_table), block_table.shape[1],
                                    page_size, _ptr(items), items.shape[0] if items is not None else 0, _ptr(pos), _ptr(slot), window,
                                    keep_first, scale, softcap, _ptr(dist_bias), _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                    gate_act, _ptr(out), _dt(out), out.stride(0), _stream())
    _check(rc, "omc_window_attn_mma")
    return out


def diff_attn_pair_ok(H: int, G: int, d: int, dv: int, dtype: torch.dtype) -> bool:
    """Shapes the one-kernel differential attention of prompt portions takes (the tensor-core shapes whose two maps fit shared memory)."""
    return dtype == torch.bfloat16 and bool(load().omc_diff_attn_pair_ok(H, G, d, dv))


def diff_attn_pair(q: torch.Tensor, H: int, G: int, d: int, dv: int, pool: torch.Tensor, block_table: torch.Tensor, page_size: int,
                   items: torch.Tensor, window: int, keep_first: int, scale: float, lam: float, mult: float, eps: float,
                   gate: Optional[torch.Tensor], gate_act: int, out: torch.Tensor):
    """window_attn_mma(maps=2) + diff_heads_gate in one launch: q [T, H * 2 * d], gate fp32 [T, H * dv] -> out [T, H * dv]."""
    _need_cuda(q, pool, block_table, items, gate, out)
    assert q.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert pool.is_contiguous() and pool.shape[-1] == G * (2 * d + dv) and block_table.is_contiguous()
    assert items.dtype == torch.int32 and items.is_contiguous() and items.shape[1] == 4
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1)
    rc = load().omc_diff_attn_pair(_ptr(q), q.stride(0), q.shape[0], H, G, d, dv, _ptr(pool), _ptr(block_table), block_table.shape[1],
                                   page_size, _ptr(items), items.shape[0], window, keep_first, scale, lam, mult, eps, _ptr(gate),
                                   gate.stride(0) if gate is not None else 0, gate_act, _ptr(out), _dt(out), out.stride(0), _stream())
    _check(rc, "omc_diff_attn_pair")
    return out


def diff_heads_gate(a: torch.Tensor, H: int, dv: int, lam: float, mult: float, eps: float, gate: Optional[torch.Tensor], gate_act: int,
                    out: torch.Tensor):
    """a fp32 [T, H * 2 * dv] (two score maps per head, side by side) -> out [T, H * dv]:
    o = a1 - lam * a2;  o / sqrt(mean(o^2) + eps) * mult * act(gate)."""
    _need_cuda(a, gate, out)
    assert a.dtype == torch.float32 and a.stride(1) == 1 and out.stride(1) == 1 and a.shape[1] >= 2 * H * dv
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1)
    rc = load().omc_diff_heads_gate(_ptr(a), a.stride(0), a.shape[0], H, dv, lam, mult, eps, _ptr(gate),
                                    gate.stride(0) if gate is not None else 0, gate_act, _ptr(out), _dt(out), out.stride(0), _stream())
    _check(rc, "omc_diff_heads_gate")
    return out


def map_rows(x: torch.Tensor, op: int, A_log: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, group: int = 1,
             p_exp: float = 1.0):
    """In place over the fp32 rows x (a column slice is fine): MAP_SILU, MAP_DECAY: exp(-exp(A_log[c // group]) softplus(x + bias[c])),
    or MAP_SIGMOID_POW: sigmoid(x + bias[c])^p_exp - 1 (the decay as its distance from 1)."""
    _need_cuda(x, A_log, bias)
    assert x.dtype == torch.float32 and x.stride(1) == 1
    rc = load().omc_map_rows(_ptr(x), x.stride(0), x.shape[0], x.shape[1], op, _ptr(A_log), _ptr(bias), group, p_exp, _stream())
    _check(rc, "omc_map_rows")
    return x


# ---- tanh norm, input convolution, selective scan, positions in queries and keys
def dyt_conv(x: torch.Tensor, alpha: torch.Tensor, nw: torch.Tensor, nb: torch.Tensor, cw: torch.Tensor, pos, slot,
             state: Optional[torch.Tensor], u: torch.Tensor, *, y1: Optional[torch.Tensor] = None, a1: float = 0.0,
             y2: Optional[torch.Tensor] = None, a2: float = 0.0, x_out: Optional[torch.Tensor] = None, single_rows: bool = False):
    """With xv = x + a1 y1 + a2 y2 (written to x_out when an output is given): h = tanh(alpha xv) nw + nb, u = h + causal
    convolution of h with cw [C, taps]; state fp32 [slots, taps - 1, C] is the ring of the last rows h of every request."""
    _need_cuda(x, alpha, nw, nb, cw, pos, slot, state, u, y1, y2, x_out)
    T, C = x.shape
    taps = cw.shape[1]
    assert x.dtype == torch.float32 and x.stride(1) == 1 and u.stride(1) == 1 and alpha.dtype == torch.float32 and alpha.numel() == 1
    assert nw.dtype == nb.dtype == cw.dtype and nw.numel() == C and nb.numel() == C and cw.shape[0] == C and cw.is_contiguous()
    assert taps == 1 or (state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (taps - 1, C))
    for t in (y1, y2, x_out):
        assert t is None or (t.dtype == torch.float32 and t.stride(1) == 1)
    rc = load().omc_dyt_conv(_ptr(x), x.stride(0), _ptr(y1), y1.stride(0) if y1 is not None else 0, a1, _ptr(y2),
                             y2.stride(0) if y2 is not None else 0, a2, _ptr(x_out), x_out.stride(0) if x_out is not None else 0,
                             _ptr(alpha), _ptr(nw), _ptr(nb), _ptr(cw), _dt(cw), taps, _ptr(pos), _ptr(slot), _ptr(state), _ptr(u), _dt(u),
                             u.stride(0), T, C, 1 if single_rows else 0, _stream())
    _check(rc, "omc_dyt_conv")
    if taps > 1 and not single_rows:
        _core.add_launches(1)
    return u


def dyt_rows(x: torch.Tensor, alpha: torch.Tensor, w: torch.Tensor, b: torch.Tensor, out: torch.Tensor):
    """out = tanh(alpha x) w + b."""
    _need_cuda(x, alpha, w, b, out)
    assert x.dtype == torch.float32 and x.stride(1) == 1 and out.stride(1) == 1 and w.dtype == b.dtype and alpha.dtype == torch.float32
    rc = load().omc_dyt_rows(_ptr(x), x.stride(0), _ptr(alpha), _ptr(w), _ptr(b), _dt(w), _ptr(out), _dt(out), out.stride(0), x.shape[0],
                             x.shape[1], _stream())
    _check(rc, "omc_dyt_rows")
    return out


def tanh_cap_rows(x: torch.Tensor, cap: float):
    """x <- cap tanh(x / cap), in place (fp32)."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.stride(1) == 1
    rc = load().omc_tanh_cap_rows(_ptr(x), x.stride(0), x.shape[0], x.shape[1], cap, _stream())
    _check(rc, "omc_tanh_cap_rows")
    return x


def selective_scan(x: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, B: torch.Tensor, Cm: torch.Tensor, A_log: torch.Tensor,
                   D: torch.Tensor, z: Optional[torch.Tensor], state: torch.Tensor, out: torch.Tensor, row_begin: torch.Tensor, portions: int,
                   pos, slot):
    """The recurrence of omc_selective_scan: x [T, inner] (fp32 or bf16), dt / B / Cm / z fp32 rows or column slices, state fp32
    [slots, inner, N] -> out [T, inner] = (S . C + D x) silu(z)."""
    _need_cuda(x, dt, dt_bias, B, Cm, A_log, D, z, state, out, row_begin, pos, slot)
    inner, N = A_log.shape
    for t in (dt, B, Cm, z):
        assert t is None or (t.dtype == torch.float32 and t.stride(1) == 1)
    for t in (dt_bias, A_log, D):
        assert t.dtype == torch.float32 and t.is_contiguous()
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (inner, N) and row_begin.dtype == torch.int32
    assert x.stride(1) == 1 and out.stride(1) == 1 and x.shape[1] == inner and B.shape[1] == N and Cm.shape[1] == N
    rc = load().omc_selective_scan(_ptr(x), _dt(x), x.stride(0), _ptr(dt), dt.stride(0), _ptr(dt_bias), _ptr(B), B.stride(0), _ptr(Cm),
                                   Cm.stride(0), _ptr(A_log), _ptr(D), _ptr(z), z.stride(0) if z is not None else 0, _ptr(state), _ptr(out),
                                   _dt(out), out.stride(0), _ptr(row_begin), portions, _ptr(pos), _ptr(slot), inner, N, _stream())
    _check(rc, "omc_selective_scan")
    return out


def rotary_frequencies(dims: int, base: float, device) -> torch.Tensor:
    """fp32 [dims / 2] on the device: f_i = base^(-2i / dims), evaluated in double precision and rounded once."""
    return torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64).to(torch.float32).to(device)


def pos_qkv_store(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, H: int, G: int, d: int, dv: int, pos, slot, block_table: torch.Tensor,
                  page_size: int, pool: torch.Tensor, q_out: torch.Tensor, *, freq: Optional[torch.Tensor] = None, rot_dims: int = 0,
                  temp_coef: float = 0.0, temp_every: int = 1, v_unit: bool = False, eps: float = 0.0):
    """Rows of a step -> queries (rotated, with their temperature) in q_out and the cache rows [rotated k | v or unit-RMS v]."""
    _need_cuda(q, k, v, pos, slot, block_table, pool, q_out, freq)
    assert q.dtype == k.dtype == v.dtype == torch.float32 and q.stride(1) == k.stride(1) == v.stride(1) == 1
    assert pool.is_contiguous() and pool.shape[-1] == G * (d + dv) and pool.dtype == q_out.dtype and q_out.stride(1) == 1
    assert block_table.dtype == torch.int32 and block_table.is_contiguous()
    assert freq is None or (freq.dtype == torch.float32 and freq.is_contiguous() and freq.numel() >= rot_dims // 2)
    rc = load().omc_pos_qkv_store(_ptr(q), q.stride(0), H, _ptr(k), k.stride(0), G, d, _ptr(v), v.stride(0), dv, _ptr(freq), rot_dims,
                                  temp_coef, temp_every, 1 if v_unit else 0, eps, q.shape[0], _ptr(pos), _ptr(slot), _ptr(block_table),
                                  block_table.shape[1], page_size, _ptr(pool), _ptr(q_out), q_out.stride(0), _dt(pool), _stream())
    _check(rc, "omc_pos_qkv_store")
