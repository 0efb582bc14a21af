"""The entry's prepared (sequence-parallel) input on B200, mirroring the reference's
``amd_kernels/moe/mxfp4_h6144_i768_e128_top4/prepared_input.py``: ``prepare_mxfp4_moe`` quantises and routes a local
bf16 shard; the caller concatenates the row-major payloads of every rank in rank order and builds the matching input type
from them; ``mxfp4_moe`` takes either type in place of the bf16 rows. The compact form carries the FP4 scales and one
correction bit per value instead of the FP4 codes and is rebuilt bit for bit.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from ... import _lib

H, I, TOPK = 6144, 768, 4  # noqa: E741


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


# Every payload field of the two input types: (row width, dtype). A payload is valid when each of its fields is a
# contiguous [M, width] tensor of that dtype on the layer's device, with one M for all of them.
_FIELDS = {
    "routed_codes": (H // 2, torch.uint8), "routed_scales": (H // 32, torch.uint8),
    "topk_weights": (TOPK, torch.float32), "topk_ids": (TOPK, torch.int32),
    "shared_codes": (H, torch.uint8), "shared_scales": (H // 32, torch.uint8),
    "correction_mask": (H // 8, torch.uint8),
}


def _rows_of(obj, anchor):
    """Token count of a payload, read from its ``anchor`` field; ValueError when that field is no [M, width] tensor or M is
    outside the range the entry serves."""
    from .chain import variant_for
    t = getattr(obj, anchor)
    if not isinstance(t, torch.Tensor) or t.ndim != 2:
        raise ValueError(f"{anchor}: expected a row-major [M, {_FIELDS[anchor][0]}] tensor")
    variant_for(t.shape[0])
    return t.shape[0]


def _require(obj, names, rows, device):
    for name in names:
        width, dtype = _FIELDS[name]
        t = getattr(obj, name)
        if (not isinstance(t, torch.Tensor) or tuple(t.shape) != (rows, width) or t.dtype != dtype
                or not t.is_contiguous() or t.device != device):
            raise ValueError(f"{name}: expected contiguous {dtype} [{rows}, {width}] on {device}")


@dataclass(frozen=True)
class MoeInput:
    """What the routed experts and the shared expert need from a token, and nothing else: its MXFP4 codes and scales, its
    top-4 routing (weights already times the routed scaling factor) and, for a layer with a shared expert, its MXFP8 codes
    and scales. Field order is the schema of the reference's type (prepared_input.py:15-36) so payloads interchange;
    ``tensors()`` hands the fields out in that order without copying."""
    routed_codes: torch.Tensor
    routed_scales: torch.Tensor
    topk_weights: torch.Tensor
    topk_ids: torch.Tensor
    shared_codes: torch.Tensor | None = None
    shared_scales: torch.Tensor | None = None

    def tensors(self):
        return (self.routed_codes, self.routed_scales, self.topk_weights, self.topk_ids, self.shared_codes,
                self.shared_scales)

    def compact(self):
        """Drops the 3072 bytes of FP4 codes per token in favour of a 768-byte correction mask (one kernel launch):
        7328 bytes per token to gather instead of 9632. Needs the shared expert's operands, from which the codes are
        rebuilt (reference prepared_input.py:38-51)."""
        if self.shared_codes is None or self.shared_scales is None:
            raise ValueError("compact input requires shared MXFP8 operands")
        n = _rows_of(self, "routed_codes")
        dev = self.routed_codes.device
        if dev.type != "cuda":
            raise ValueError("compact input requires CUDA operands")
        _require(self, ("routed_codes", "routed_scales", "topk_weights", "topk_ids", "shared_codes", "shared_scales"), n, dev)
        mask = torch.empty((n, _FIELDS["correction_mask"][0]), dtype=torch.uint8, device=dev)
        _lib.check(_lib.load().b200moe_sidecar_pack(_ptr(self.routed_codes), _ptr(self.routed_scales),
                                                    _ptr(self.shared_codes), _ptr(self.shared_scales), n, _ptr(mask),
                                                    _stream(dev)), "sidecar_pack")
        return MoeInputCompact(self.routed_scales, self.topk_weights, self.topk_ids, self.shared_codes, self.shared_scales,
                               mask)

    def validate(self, w):
        """ValueError unless every field the layer ``w`` reads is present with the right shape, dtype and device."""
        n = _rows_of(self, "routed_codes")
        names = ["routed_codes", "routed_scales", "topk_weights", "topk_ids"]
        if w.shared_weights is not None:
            names += ["shared_codes", "shared_scales"]
        _require(self, names, n, w.w13.device)


@dataclass(frozen=True)
class MoeInputCompact:
    """``MoeInput`` without the FP4 codes: the FP4 scales plus one bit per value say how each FP4 code differs from the
    one the FP8 code would give, so ``expand`` restores the codes exactly, signed zeros included. Same field order as the
    reference's type (prepared_input.py:79-96); 2304 bytes per token smaller on the wire."""
    routed_scales: torch.Tensor
    topk_weights: torch.Tensor
    topk_ids: torch.Tensor
    shared_codes: torch.Tensor
    shared_scales: torch.Tensor
    correction_mask: torch.Tensor | None

    def tensors(self):
        return (self.routed_scales, self.topk_weights, self.topk_ids, self.shared_codes, self.shared_scales,
                self.correction_mask)

    def expand(self) -> MoeInput:
        """The full ``MoeInput`` again (one kernel launch writes the FP4 codes; every other field is shared, not copied)."""
        n = _rows_of(self, "shared_codes")
        dev = self.shared_codes.device
        if dev.type != "cuda":
            raise ValueError("compact input requires CUDA operands")
        _require(self, ("routed_scales", "topk_weights", "topk_ids", "shared_codes", "shared_scales", "correction_mask"), n, dev)
        codes = torch.empty((n, _FIELDS["routed_codes"][0]), dtype=torch.uint8, device=dev)
        _lib.check(_lib.load().b200moe_sidecar_unpack(_ptr(self.correction_mask), _ptr(self.routed_scales),
                                                      _ptr(self.shared_codes), _ptr(self.shared_scales), n, _ptr(codes),
                                                      _stream(dev)), "sidecar_unpack")
        return MoeInput(codes, self.routed_scales, self.topk_weights, self.topk_ids, self.shared_codes, self.shared_scales)


def prepare_mxfp4_moe(x, w) -> MoeInput:
    """One local bf16 [M, 6144] shard prepared before the caller's all-gather (reference prepared_input.py:117-136):
    routing from ``w.router_weight`` (split-K partials added in split order), the routed experts' MXFP4 operands and, with
    a shared expert, its MXFP8 operands, every scale row-major: below 128 tokens from ONE pass over x (the router GEMM fused
    with both quantisers), from 128 tokens on with the router on the tensor cores. The payload carries exactly the routing
    and codes ``mxfp4_moe(x, w)`` computes. Returns only tensor payloads; the caller owns the gather."""
    from .chain import router_gemm_quant, topk_route, variant_for
    if (not isinstance(x, torch.Tensor) or x.ndim != 2 or x.shape[1] != H or x.dtype != torch.bfloat16
            or not x.is_contiguous()):
        raise ValueError("expected contiguous BF16 [M,6144]")
    variant_for(x.shape[0])
    if w.router_weight is None:
        raise ValueError("needs MoeWeights with router_weight: MoeWeights.from_row_major(router_weight, ...)")
    w.abi()  # makes the gate's bf16 terms on first use
    parts, (q, s), (q8, s8) = router_gemm_quant(x, w.router_weight, shared=w.shared_weights is not None,
                                                split=w.router_split)
    wt, ids = topk_route(parts, w.correction_bias, w.routed_scaling_factor, w.routing_mode)
    return MoeInput(q, s, wt, ids, q8, s8)


def mxfp4_moe_prepared(x, w, *, return_partials):
    """``mxfp4_moe`` on a prepared input (reference prepared_input.py:159-187): the routed experts on the MXFP4 operands,
    the shared expert on the MXFP8 ones on the side stream, summed in slot order then shared."""
    from .chain import mxfp4_moe_experts, reduce_slots
    from .shared_expert import shared_expert_parallel
    if isinstance(x, MoeInputCompact):
        x = x.expand()
    x.validate(w)
    dev = x.routed_codes.device
    sw = w.shared_weights
    shared = None
    current = torch.cuda.current_stream(dev)
    if sw is not None:
        shared = shared_expert_parallel(None, sw, current, x_quant=(x.shared_codes, x.shared_scales))
    parts = mxfp4_moe_experts((x.routed_codes, x.routed_scales), x.topk_weights, x.topk_ids, w)
    if sw is not None:
        current.wait_stream(sw.stream)
        shared.record_stream(current)
    return (parts, shared) if return_partials else reduce_slots(parts, shared)


def gather_mxfp4_moe(local: MoeInput, comm) -> MoeInputCompact:
    """All ranks of ``comm`` (a ``torch.distributed`` process group over NCCL) contribute their prepared shard and receive
    every rank's rows, rank 0's first, in the compact form (the role of reference prepared_input.py:190-209). Each rank
    brings the same number of rows (pad with zero rows where needed); a layer without a shared expert cannot use the compact
    form and is refused."""
    import torch.distributed as dist
    if not isinstance(local, MoeInput):
        raise ValueError("expected an explicit prepared MoeInput")
    if local.shared_codes is None or local.shared_scales is None:
        raise ValueError("lossless mixed-format gather requires shared MXFP8 operands")
    fields = local.compact().tensors()
    ranks = dist.get_world_size(comm)
    gathered = [f.new_empty((ranks * f.shape[0],) + tuple(f.shape[1:])) for f in fields]
    for dst, src in zip(gathered, fields):
        dist.all_gather_into_tensor(dst, src, group=comm)
    return MoeInputCompact(*gathered)
