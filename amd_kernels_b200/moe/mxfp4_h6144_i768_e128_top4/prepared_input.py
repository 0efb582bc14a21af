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


def _check(fields, device):
    for tensor, shape, dtype in fields:
        if (not isinstance(tensor, torch.Tensor) or tuple(tensor.shape) != shape or tensor.dtype != dtype
                or not tensor.is_contiguous() or tensor.device != device):
            raise ValueError(f"expected contiguous {dtype} {shape} on {device}")


@dataclass(frozen=True)
class MoeInput:
    """Quantised operands and routing, no bf16 activations or expert weights (reference prepared_input.py:15-76).

    ``tensors()`` returns the gather payload in constructor order, without copies. The scales are e8m0 bytes per 32
    values, the routing weights include the routed scaling factor; the shared payloads are the shared expert's MXFP8
    input (None for a layer without one)."""
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
        """The 7328 B/token payload (packing costs a launch); release this object's FP4 codes after packing."""
        if self.shared_codes is None or self.shared_scales is None:
            raise ValueError("compact input requires shared MXFP8 operands")
        if not isinstance(self.routed_codes, torch.Tensor) or self.routed_codes.ndim != 2:
            raise ValueError("expected routed codes [M,3072]")
        n = self.routed_codes.shape[0]
        partial = MoeInputCompact(self.routed_scales, self.topk_weights, self.topk_ids, self.shared_codes,
                                  self.shared_scales, None)
        partial._validate(check_mask=False)
        dev = self.shared_codes.device
        _check(((self.routed_codes, (n, H // 2), torch.uint8),), dev)
        mask = torch.empty((n, H // 8), dtype=torch.uint8, device=dev)
        _lib.check(_lib.load().b200moe_sidecar_pack(_ptr(self.routed_codes), _ptr(self.routed_scales),
                                                    _ptr(self.shared_codes), _ptr(self.shared_scales), n, _ptr(mask),
                                                    _stream(dev)), "sidecar_pack")
        return MoeInputCompact(*partial.tensors()[:-1], mask)

    def validate(self, w):
        from .chain import variant_for
        if not isinstance(self.routed_codes, torch.Tensor) or self.routed_codes.ndim != 2:
            raise ValueError("routed_codes must be row-major [M,3072]")
        n = self.routed_codes.shape[0]
        variant_for(n)
        dev = w.w13.device
        fields = [(self.routed_codes, (n, H // 2), torch.uint8), (self.routed_scales, (n, H // 32), torch.uint8),
                  (self.topk_weights, (n, TOPK), torch.float32), (self.topk_ids, (n, TOPK), torch.int32)]
        if w.shared_weights is not None:
            fields += [(self.shared_codes, (n, H), torch.uint8), (self.shared_scales, (n, H // 32), torch.uint8)]
        _check(fields, dev)


@dataclass(frozen=True)
class MoeInputCompact:
    """The lossless gather payload, in ``tensors()`` order, all row-major (reference prepared_input.py:79-114): the FP4
    scales and one correction bit per value rebuild the direct FP4 codes from the shared FP8 ones (signed zero and the
    quantisation kept): 2304 B/token less than ``MoeInput`` with a shared expert, at one launch to pack and one to
    rebuild."""
    routed_scales: torch.Tensor
    topk_weights: torch.Tensor
    topk_ids: torch.Tensor
    shared_codes: torch.Tensor
    shared_scales: torch.Tensor
    correction_mask: torch.Tensor | None

    def tensors(self):
        return (self.routed_scales, self.topk_weights, self.topk_ids, self.shared_codes, self.shared_scales,
                self.correction_mask)

    def _validate(self, *, check_mask=True):
        from .chain import variant_for
        if not isinstance(self.shared_codes, torch.Tensor) or self.shared_codes.ndim != 2:
            raise ValueError("expected shared codes [M,6144]")
        n = self.shared_codes.shape[0]
        if self.shared_codes.device.type != "cuda":
            raise ValueError("compact input requires CUDA operands")
        variant_for(n)
        specs = (((n, H // 32), torch.uint8), ((n, TOPK), torch.float32), ((n, TOPK), torch.int32), ((n, H), torch.uint8),
                 ((n, H // 32), torch.uint8), ((n, H // 8), torch.uint8))
        tensors = self.tensors() if check_mask else self.tensors()[:-1]
        _check([(t, shape, dtype) for t, (shape, dtype) in zip(tensors, specs)], self.shared_codes.device)

    def expand(self) -> MoeInput:
        """Reconstruct the FP4 codes bit for bit; keep routing, scales and shared codes."""
        self._validate()
        n, dev = self.shared_codes.shape[0], self.shared_codes.device
        q = torch.empty((n, H // 2), dtype=torch.uint8, device=dev)
        _lib.check(_lib.load().b200moe_sidecar_unpack(_ptr(self.correction_mask), _ptr(self.routed_scales),
                                                      _ptr(self.shared_codes), _ptr(self.shared_scales), n, _ptr(q),
                                                      _stream(dev)), "sidecar_unpack")
        return MoeInput(q, self.routed_scales, self.topk_weights, self.topk_ids, self.shared_codes, self.shared_scales)


def prepare_mxfp4_moe(x, w) -> MoeInput:
    """One local bf16 [M, 6144] shard prepared before the caller's all-gather (reference prepared_input.py:117-136):
    routing from ``w.router_weight`` (split-K partials added in split order), the routed experts' MXFP4 operands and, with
    a shared expert, its MXFP8 operands, every scale row-major, all from ONE pass over x (the router GEMM fused with both
    quantisers). Returns only tensor payloads; the caller owns the gather."""
    from .chain import router_gemm_quant, topk_route, variant_for
    if (not isinstance(x, torch.Tensor) or x.ndim != 2 or x.shape[1] != H or x.dtype != torch.bfloat16
            or not x.is_contiguous()):
        raise ValueError("expected contiguous BF16 [M,6144]")
    variant_for(x.shape[0])
    if w.router_weight is None:
        raise ValueError("needs MoeWeights with router_weight: MoeWeights.from_row_major(router_weight, ...)")
    parts, (q, s), (q8, s8) = router_gemm_quant(x, w.router_weight, shared=w.shared_weights is not None)
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
    """A prepared shard gathered losslessly (compact) for the same public MoE entry (reference prepared_input.py:190-209).
    ``comm``: the ``torch.distributed`` process group (NCCL) of the ranks that share the sequence; every rank supplies the
    same positive row count, zero padding included. The result holds the rows of all ranks in rank order."""
    import torch.distributed as dist
    if not isinstance(local, MoeInput):
        raise ValueError("expected an explicit prepared MoeInput")
    if local.shared_codes is None or local.shared_scales is None:
        raise ValueError("lossless mixed-format gather requires shared MXFP8 operands")
    compact = local.compact()
    world = dist.get_world_size(comm)
    rows = local.routed_codes.shape[0]
    outs = []
    for t in compact.tensors():
        out = torch.empty((world * rows, *t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=comm)
        outs.append(out)
    return MoeInputCompact(*outs)
