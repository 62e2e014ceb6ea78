"""The expert-sorted feed-forward of the sequence-step decoders, host side: the per-step workspace and the chain plan -> scatter ->
grouped gate | up product -> gate * up -> grouped down product. The router in front and the combine behind differ per design and
stay with the model.

Rows are sorted by expert into tiles of 64 rows (omc_linear with a tile -> expert table) or 128 rows (the grouped tcgen05 GEMM of the
core library, for bf16 experts whose widths are multiples of 128 and large enough to matter). Nothing here synchronises with the
host: the chain can be captured in a CUDA graph.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import lib, seqlib
from .seq_linear import TENSOR_GEMM_MIN_WEIGHT

SMALL_STEP_ROWS = 4    # steps of up to this many rows sort their rows by expert in one single-CTA launch


class ExpertWorkspace:
    pass


def grouped_tensor_gemm_ok(tensor_gemm: bool, expert_ff: int, C: int) -> bool:
    """Experts on the grouped tcgen05 GEMM (128-row tiles): bf16, tile-aligned widths, matrices large enough to matter."""
    return tensor_gemm and expert_ff % 128 == 0 and C % 128 == 0 and expert_ff * C >= TENSOR_GEMM_MIN_WEIGHT // 4


def expert_workspace(store: dict, T: int, experts: int, top: int, expert_ff: int, tile: int, C: int, dtype: torch.dtype, device) -> ExpertWorkspace:
    """Buffers for steps of up to the next power of two above T rows, kept in `store` (one per shape)."""
    bucket = 1 << max(T - 1, 0).bit_length()
    key = (bucket, experts, top, expert_ff, tile)
    ws = store.get(key)
    if ws is None:
        i32 = torch.int32
        ws = ExpertWorkspace()
        ws.max_tiles = seqlib.moe_max_tiles(bucket, top, experts, tile)
        rows = ws.max_tiles * tile
        ws.ids = torch.empty(bucket, top, device=device, dtype=i32)
        ws.w = torch.empty(bucket, top, device=device, dtype=torch.float32)
        ws.gate = torch.empty(bucket, device=device, dtype=torch.float32)
        ws.counts = torch.zeros(experts, device=device, dtype=i32)
        ws.cursor = torch.zeros(experts, device=device, dtype=i32)
        ws.seg_start = torch.zeros(experts + 1, device=device, dtype=i32)
        ws.tile_group = torch.empty(ws.max_tiles, device=device, dtype=i32)
        ws.slot_of = torch.empty(bucket, top, device=device, dtype=i32)
        ws.xs = torch.zeros(rows, C, device=device, dtype=dtype)
        ws.gu = torch.zeros(rows, 2 * expert_ff, device=device, dtype=dtype)
        ws.act = torch.zeros(rows, expert_ff, device=device, dtype=dtype)
        ws.ys = torch.empty(rows, C, device=device, dtype=torch.float32)
        store[key] = ws
    return ws


def run_sorted_experts(ws: ExpertWorkspace, xb: torch.Tensor, experts: int, top: int, expert_ff: int, tile: int, gate_up: torch.Tensor,
                       down: torch.Tensor, act: int, *, grouped: bool, input_weights: Optional[torch.Tensor] = None, limit: float = 0.0,
                       slope: float = 1.0, shift: float = 0.0) -> int:
    """ws.ids / ws.counts hold the router's choice for the rows xb [T, C]. Sorts the rows (times input_weights[t, j] when the mixing
    weights act on the experts' input), runs gate | up [E, 2 ff, C], act(gate) * up, and down [E, C, ff]; the experts' outputs are
    in ws.ys at the rows ws.slot_of names. Returns the number of rows of the sorted layout."""
    T, C = xb.shape
    max_tiles = seqlib.moe_max_tiles(T, top, experts, tile)
    if T <= SMALL_STEP_ROWS:
        seqlib.moe_plan_scatter_small(ws.counts, experts, tile, max_tiles, ws.seg_start, ws.tile_group, xb, ws.ids, top, ws.slot_of, ws.xs,
                                      row_w=input_weights)
    else:
        seqlib.moe_plan_tiles(ws.counts, experts, tile, max_tiles, ws.seg_start, ws.cursor, ws.tile_group)
        seqlib.moe_scatter_rows(xb, ws.ids, top, experts, ws.seg_start, ws.cursor, ws.slot_of, ws.xs, row_w=input_weights)
    rows, ff = max_tiles * tile, expert_ff
    if grouped:
        hint = min(max_tiles, T * top)
        lib.gemm_grouped(ws.xs[:rows], gate_up, ws.tile_group, ws.gu[:rows], lib.EPI_NONE, hint)
    else:
        seqlib.linear(ws.xs, gate_up, ws.gu, M=rows, N=2 * ff, K=C, ldw=C, tile_group=ws.tile_group, group_stride=2 * ff * C)
    seqlib.glu_mul(ws.gu[:rows], ff, act, ws.act[:rows], limit=limit, slope=slope, shift=shift)
    if grouped:
        lib.gemm_grouped(ws.act[:rows], down, ws.tile_group, ws.ys[:rows], lib.EPI_NONE, hint)
    else:
        seqlib.linear(ws.act, down, ws.ys, M=rows, N=C, K=ff, ldw=ff, tile_group=ws.tile_group, group_stride=C * ff)
    return rows
