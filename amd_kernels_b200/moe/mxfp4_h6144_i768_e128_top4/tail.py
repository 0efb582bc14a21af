"""The layer's fused tail on B200: slot sum (+ shared expert) -> residual add -> Gemma RMSNorm -> MXFP8 operands of the
next layer, in ONE pass over the slots. The reference fuses the same steps into its 4-rank reduce-scatter
(``amd_kernels/collectives/pull_collectives_ranks4/README.md:25-27`` ``slots4_reduce_scatter_add_rmsnorm_mxfp8``); this is
that tail on one rank's rows, which is also what an expert-parallel rank runs after the combine has filled its slot buffer.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from ... import _lib

H, TOPK = 6144, 4


@dataclass
class TailOutput:
    """``residual`` bf16 [M, H] (the new residual stream), ``codes`` u8 [M, H] E4M3 and ``scales`` u8 [M, H/32] E8M0
    (row-major MXFP8 of the fp32 norm output), ``normed`` bf16 [M, H] when asked for."""
    residual: torch.Tensor
    codes: torch.Tensor | None
    scales: torch.Tensor | None
    normed: torch.Tensor | None


def slots4_add_rmsnorm_mxfp8(slots: torch.Tensor, shared: torch.Tensor | None, residual: torch.Tensor,
                             weight: torch.Tensor, eps: float = 1e-6, *, mxfp8: bool = True,
                             bf16_out: bool = False) -> TailOutput:
    """``x = bf16((((s0+s1)+s2)+s3) + shared)`` in fp32 (``.../pull_collectives_ranks4/reference.py:74-91``), then steps
    2-4 of ``amd_kernels/norm/gemma_add_rmsnorm_h6144/reference.py``: ``s = x + residual`` (residual out ``bf16(s)``),
    ``y = s * rstd * (weight + 1)``, MXFP8 of the fp32 ``y``. The sum and the residual are bit-exact; ``y`` follows that
    reference's tolerances against its fp64 statement."""
    if slots.dtype != torch.bfloat16 or slots.ndim != 3 or slots.shape[1:] != (TOPK, H) or not slots.is_contiguous():
        raise ValueError("expected contiguous BF16 [M, 4, 6144] slots")
    m, dev = slots.shape[0], slots.device
    for name, t in (("shared", shared), ("residual", residual)):
        if t is None and name == "shared":
            continue
        if t is None or t.dtype != torch.bfloat16 or tuple(t.shape) != (m, H) or not t.is_contiguous() or t.device != dev:
            raise ValueError(f"{name}: expected contiguous BF16 [{m}, {H}] on {dev}")
    if weight.dtype != torch.bfloat16 or tuple(weight.shape) != (H,) or not weight.is_contiguous() or weight.device != dev:
        raise ValueError(f"weight: expected contiguous BF16 [{H}] on {dev}")
    res = torch.empty((m, H), dtype=torch.bfloat16, device=dev)
    normed = torch.empty((m, H), dtype=torch.bfloat16, device=dev) if bf16_out else None
    codes = torch.empty((m, H), dtype=torch.uint8, device=dev) if mxfp8 else None
    scales = torch.empty((m, H // 32), dtype=torch.uint8, device=dev) if mxfp8 else None
    p = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())  # noqa: E731
    _lib.check(_lib.load().b200moe_reduce_slots_add_rmsnorm_quant(
        p(slots), p(shared), p(residual), p(weight), float(eps), m, p(res), p(normed), p(codes), p(scales),
        ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)), "reduce_slots_add_rmsnorm_quant")
    return TailOutput(res, codes, scales, normed)
