"""The linear layer of the sequence-step decoders (Voduzen, Tifisun, Fofisun): which kernel multiplies which matrix.

Matrices with at least TENSOR_GEMM_MIN_WEIGHT elements go through the tcgen05 GEMM of the core library when the operands are bf16
and the dimensions are multiples of 8; below it a launch is latency-bound either way and the kernel of the sequence-step library
(FMA pipe for fp32 or ragged shapes, mma.sync for aligned bf16) needs no second library. Steps of up to 64 rows stream the weights
through the skinny GEMM from a much smaller size on: the small-matrix kernel walks K with one row tile per CTA, which leaves a
decode step waiting on a handful of CTAs. The choice depends on widths, layout and dtypes only, never on what else is in the
batch beyond the 64-row threshold of the skinny kernel, and every kernel accumulates a row's K terms in an order of its own
that does not depend on M.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import lib, seqlib

TENSOR_GEMM_MIN_WEIGHT = 1 << 20
SKINNY_GEMM_MIN_WEIGHT = 1 << 17
_TENSOR_EPILOGUES = {seqlib.ACT_RELU2: lib.EPI_RELU2, seqlib.ACT_GELU_ERF: lib.EPI_GELU}   # activations the tensor-core GEMMs apply themselves


def dense_linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, *, tensor_gemm: bool, act: int = seqlib.ACT_NONE,
                 alpha: float = 1.0, bias: Optional[torch.Tensor] = None, min_weight: Optional[int] = None) -> torch.Tensor:
    """act(alpha * x @ w^T + bias) -> [rows, N] of out_dtype. x [rows, K] (fp32 or bf16, rows may be strided), w [N, K].
    min_weight: the caller's own size threshold for the tensor-core GEMM on steps of more than 64 rows (narrow products inside a
    mixer, which the small-matrix kernel leaves to a handful of CTAs)."""
    M, K = x.shape
    N = w.shape[0]
    big = N * K >= (SKINNY_GEMM_MIN_WEIGHT if M <= lib.SKINNY_MAX_M else (min_weight if min_weight is not None else TENSOR_GEMM_MIN_WEIGHT))
    if (tensor_gemm and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and big and N % 8 == 0 and K % 8 == 0
            and x.stride(0) % 8 == 0 and (act == seqlib.ACT_NONE or (act in _TENSOR_EPILOGUES and out_dtype == torch.bfloat16))):
        y = lib.gemm(x, w, bias=bias, out_f32=out_dtype == torch.float32, epi=_TENSOR_EPILOGUES.get(act, lib.EPI_NONE))
        return y if alpha == 1.0 else y.mul_(alpha)
    out = torch.empty(M, N, device=x.device, dtype=out_dtype)
    return seqlib.linear(x, w, out, alpha=alpha, act=act, bias=bias)
