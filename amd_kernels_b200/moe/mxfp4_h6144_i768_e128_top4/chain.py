"""Routed MXFP4 H6144 I768 E128 top4 on B200: the host side of the entry, mirroring the reference's
``amd_kernels/moe/mxfp4_h6144_i768_e128_top4/chain.py`` (names, argument meaning and error behaviour), on top of the
C ABI of libb200moe.so. PyTorch is used for device memory and streams only; every computation is a kernel of the library.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch

from ... import _lib

H, I, E, TOPK = 6144, 768, 128, 4  # noqa: E741
MAX_TOKENS = 87381  # reference chain.py:13-18: variant_for raises above
ROUTING_MODES = {"sigmoid_bias": _lib.ROUTE_SIGMOID_BIAS, "softmax": _lib.ROUTE_SOFTMAX}


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


_status: dict = {}


def status_word(device) -> torch.Tensor:
    """The per-device int32 word kernels write device-side conditions to (0 = none, 1 = a bounded wait ran out)."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _status:
        with torch.inference_mode(False):  # a normal tensor even when first used under inference_mode
            _status[key] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
    return _status[key]


def last_status(device=None) -> int:
    """Synchronises and returns the device status word (and clears it)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = status_word(dev)
    value = int(word.item())
    word.zero_()
    return value


def variant_for(n_tokens: int) -> int:
    """The block height (sorted rows per expert block) served at ``n_tokens``; ValueError outside 1..87381, the range
    the reference's ``variant_for`` accepts (chain.py:53-57)."""
    if not 0 < n_tokens <= MAX_TOKENS:
        raise ValueError(f"unsupported token count {n_tokens}")
    return int(_lib.load().b200moe_block_rows(n_tokens))


@dataclass
class MoeWeights:
    """The router (fp32 [E, H]) and bias (fp32 [E]), and the experts in the kernels' layouts, built once by
    ``from_row_major`` before graph capture (reference chain.py:23-50).

    ``w13`` [E, 12, 24, 17408] u8 and ``w2`` [E, 48, 3, 17408] u8 are streams of tile records: 128 rows x 256
    K-elements of codes in the 128-byte-swizzled shared-memory image followed by the tile's scale atoms, so a pipeline
    stage is one contiguous bulk copy. A W13 tile holds 64 gate rows and the matching 64 up rows in 32-row groups.
    ``w13_scale`` / ``w2_scale`` stay None: the scales travel inside the records."""
    router_weight: torch.Tensor | None
    correction_bias: torch.Tensor | None
    w13: torch.Tensor
    w13_scale: torch.Tensor | None
    w2: torch.Tensor
    w2_scale: torch.Tensor | None
    routed_scaling_factor: float = 2.0
    routing_mode: str = "sigmoid_bias"
    shared_weights: object | None = None
    row_major: tuple | None = None  # the checkpoint tensors, kept only on request (the CUDA-core cross-check reads them)
    router_split: torch.Tensor | None = None  # the gate as three bf16 terms [3, 128, H] for the tensor-core router
    _abi: object = field(default=None, repr=False)
    INTERMEDIATE = I  # the served shape's intermediate size; the i1536 sibling package pins 1536

    @property
    def intermediate(self) -> int:
        return self.w13.shape[1] * 64  # 128-row tiles of 64 gate + 64 up rows

    def lib(self):
        """The library built for this shape's intermediate size."""
        return _lib.load(self.intermediate)

    @classmethod
    def from_row_major(cls, router_weight, correction_bias, w13, w13_scale, w2, w2_scale, *, shared=None,
                       routed_scaling_factor=2.0, routing_mode="sigmoid_bias", keep_row_major=False):
        """Checkpoint layout (row-major uint8 MXFP4 codes / e8m0 scales, gate rows then up rows) -> the kernels'
        layouts. ``routing_mode``: "sigmoid_bias" (the reference's rule) or "softmax" (top-4 of the softmax,
        renormalised). ``shared``: the MXFP8 shared expert's ``SharedWeights`` (or None: routed experts only)."""
        inter = cls.INTERMEDIATE
        reason = unsupported_reason(w13, w13_scale, w2, w2_scale, None, None, None, None, routed_only=True, inter=inter)
        if reason is not None:
            raise ValueError(reason)
        if shared is not None and not hasattr(shared, "stream"):
            raise ValueError("shared= takes SharedWeights.from_row_major(...)")
        if routing_mode not in ROUTING_MODES:
            raise ValueError(f"routing_mode must be one of {sorted(ROUTING_MODES)}")
        if not w13.is_cuda:
            raise ValueError("weights must be CUDA tensors")
        lib = _lib.load(inter)
        n_exp = w13.shape[0]
        dev = w13.device
        w13, w13_scale, w2, w2_scale = (t.contiguous() for t in (w13, w13_scale, w2, w2_scale))
        w13t = torch.empty((n_exp, 2 * inter // 128, 24, 17408), dtype=torch.uint8, device=dev)
        w2t = torch.empty((n_exp, 48, inter // 256, 17408), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.b200moe_preshuffle_w13(_ptr(w13), _ptr(w13_scale), n_exp, _ptr(w13t), _stream(dev)),
                       "preshuffle_w13")
            _lib.check(lib.b200moe_preshuffle_w2(_ptr(w2), _ptr(w2_scale), n_exp, _ptr(w2t), _stream(dev)),
                       "preshuffle_w2")
        bias = None if correction_bias is None else correction_bias.to(device=dev, dtype=torch.float32).contiguous()
        if router_weight is not None:
            if tuple(router_weight.shape) != (n_exp, H):
                raise ValueError(f"router_weight: needs ({n_exp}, {H}), got {tuple(router_weight.shape)}")
            router_weight = router_weight.to(device=dev, dtype=torch.float32).contiguous()
        return cls(router_weight, bias, w13t, None, w2t, None, float(routed_scaling_factor), routing_mode,
                   shared_weights=shared, row_major=(w13, w13_scale, w2, w2_scale) if keep_row_major else None)

    @property
    def num_experts(self) -> int:
        return self.w13.shape[0]

    def abi(self) -> _lib.Weights:
        """``struct b200moe_weights`` over this object's tensors."""
        if self._abi is None:
            gate = self.router_weight
            if gate is not None and (gate.dtype != torch.float32 or not gate.is_contiguous() or gate.device != self.w13.device
                                     or tuple(gate.shape) != (self.num_experts, H)):
                raise ValueError(f"router_weight: expected contiguous fp32 [{self.num_experts}, {H}] on {self.w13.device}")
            if gate is not None and self.router_split is None:
                self.router_split = split_gate(gate)
            self._abi = _lib.Weights(self.w13.data_ptr(), self.w2.data_ptr(),
                                     None if self.correction_bias is None else self.correction_bias.data_ptr(),
                                     self.num_experts, ROUTING_MODES[self.routing_mode],
                                     self.routed_scaling_factor, None if gate is None else gate.data_ptr(),
                                     None if gate is None else self.router_split.data_ptr())
        return self._abi


def unsupported_reason(w13, w13_scale, w2, w2_scale, shared_w13, shared_s13, shared_w2, shared_s2,
                       swiglu=(1.702, 7.0, 1.0), *, routed_only=False, inter=I) -> str | None:
    """None when ``MoeWeights.from_row_major`` takes these checkpoint-layout tensors, else the reason
    (reference __init__.py:19-35). ``routed_only`` skips the shared-expert tensors (a layer without one); ``inter``: the
    intermediate size of the served shape."""
    I = inter  # noqa: E741,N806
    ref = (1.702, 7.0, 1.0)
    if any(abs(a - b) > 1e-6 for a, b in zip(swiglu, ref)):
        return f"needs SwiGLU-OAI (alpha, limit, beta) {ref}, got {tuple(swiglu)}"
    n_exp = w13.shape[0] if w13 is not None and w13.ndim == 3 and routed_only else E
    spec = [("w13", w13, (n_exp, 2 * I, H // 2), torch.uint8), ("w13_scale", w13_scale, (n_exp, 2 * I, H // 32), torch.uint8),
            ("w2", w2, (n_exp, H, I // 2), torch.uint8), ("w2_scale", w2_scale, (n_exp, H, I // 32), torch.uint8)]
    if not routed_only:
        spec += [("shared w13", shared_w13, (2 * I, H), torch.float8_e4m3fn), ("shared w13 scale", shared_s13, (2 * I, H // 32), None),
                 ("shared w2", shared_w2, (H, I), torch.float8_e4m3fn), ("shared w2 scale", shared_s2, (H, I // 32), None)]
    for name, t, shape, dtype in spec:
        if t is None or tuple(t.shape) != shape or (dtype is not None and t.dtype != dtype):
            got = None if t is None else (tuple(t.shape), t.dtype)
            return f"{name}: needs {shape} {dtype or 'e8m0'}, got {got}"
    if not 1 <= n_exp <= E:
        return f"w13: needs 1..{E} experts, got {n_exp}"
    return None


# ------------------------------------------------------------------------------------------------ single kernels
def mxfp4_quant(x: torch.Tensor):
    """bf16 [M, K] -> (codes u8 [M, K/2], e8m0 u8 [M, K/32]) row-major (reference quant.py:32 ``mxfp4_quant``)."""
    if x.ndim != 2 or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.shape[1] % 256:
        raise ValueError("expected contiguous BF16 [M, K] with K a multiple of 256")
    m, k = x.shape
    codes = torch.empty((m, k // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty((m, k // 32), dtype=torch.uint8, device=x.device)
    _lib.check(_lib.load().b200moe_quant_mxfp4(_ptr(x), m, k, _ptr(codes), _ptr(scales), _stream(x.device)), "quant_mxfp4")
    return codes, scales


def topk_route(logits: torch.Tensor, bias, scale: float, mode: str = "sigmoid_bias"):
    """fp32 logits [M, E] or split-K partials [M, S, E] (any strides on M and S) -> (weights fp32 [M, 4], ids int32
    [M, 4]) (reference router_topk.py:239 ``splitk_biased_topk``)."""
    if logits.dtype != torch.float32 or logits.ndim not in (2, 3) or logits.stride(-1) != 1:
        raise ValueError("expected fp32 [M, E] logits or [M, S, E] partials, unit stride on E")
    m, n_exp = logits.shape[0], logits.shape[-1]
    splits, stride_s = (1, 0) if logits.ndim == 2 else (logits.shape[1], logits.stride(1))
    wt = torch.empty((m, TOPK), dtype=torch.float32, device=logits.device)
    ids = torch.empty((m, TOPK), dtype=torch.int32, device=logits.device)
    _lib.check(_lib.load().b200moe_route_topk(_ptr(logits), logits.stride(0), stride_s, splits, _ptr(bias), m, n_exp,
                                              ROUTING_MODES[mode], scale, _ptr(wt), _ptr(ids), _stream(logits.device)),
               "route_topk")
    return wt, ids


@dataclass
class SortBuffers:
    """The routing sort's outputs (reference common/sort.py:19-65)."""
    sorted_ids: torch.Tensor
    sorted_weights: torch.Tensor
    block_expert: torch.Tensor
    num_valid: torch.Tensor
    bm: int
    tokens: int

    @property
    def max_rows(self) -> int:
        return self.sorted_ids.shape[0]


def moe_sort(topk_ids: torch.Tensor, topk_weights: torch.Tensor, bm: int, num_experts: int = E,
             live_pairs: torch.Tensor | None = None) -> SortBuffers:
    """ids int32 [M, 4], weights fp32 [M, 4] -> expert-sorted, block-padded rows in pair order. ``live_pairs`` (a device
    int32 scalar): only the first that many pairs count, whatever the ids behind them say."""
    if topk_ids.dtype != torch.int32 or topk_weights.dtype != torch.float32 or topk_ids.shape != topk_weights.shape \
            or topk_ids.ndim != 2 or topk_ids.shape[1] != TOPK:
        raise ValueError("expected int32 ids and fp32 weights of shape [M, 4]")
    lib = _lib.load()
    m, dev = topk_ids.shape[0], topk_ids.device
    variant_for(m)
    rows = int(lib.b200moe_max_sorted_rows(m, bm, num_experts))
    buf = SortBuffers(torch.empty(rows, dtype=torch.int32, device=dev), torch.empty(rows, dtype=torch.float32, device=dev),
                      torch.empty(rows // bm, dtype=torch.int32, device=dev), torch.empty(2, dtype=torch.int32, device=dev),
                      bm, m)
    scratch_bytes = int(lib.b200moe_permute_scratch_bytes(m, num_experts))
    scratch = torch.empty(max(scratch_bytes // 4, 1), dtype=torch.int32, device=dev)
    _lib.check(lib.b200moe_permute_live(_ptr(topk_ids.contiguous()), _ptr(topk_weights.contiguous()), m, num_experts, bm,
                                        _ptr(live_pairs), _ptr(buf.sorted_ids), _ptr(buf.sorted_weights),
                                        _ptr(buf.block_expert), _ptr(buf.num_valid), _ptr(scratch), _stream(dev)), "permute")
    return buf


def dispatch_rows(x_quant, sort: SortBuffers, by_pair: bool = False):
    """Row-major (codes, scales) -> (codes in sorted-row order [rows, 3072], scale atoms [rows/bm, 48, 512]).
    ``by_pair``: the input holds one row per (token, slot) pair instead of one per token."""
    codes, scales = x_quant
    dev = codes.device
    xq = torch.empty((sort.max_rows, H // 2), dtype=torch.uint8, device=dev)
    sfx = torch.empty((sort.max_rows // sort.bm, H // 128, 512), dtype=torch.uint8, device=dev)
    _lib.check(_lib.load().b200moe_dispatch_rows(_ptr(codes), _ptr(scales), _ptr(sort.sorted_ids), _ptr(sort.num_valid),
                                                 sort.tokens, sort.bm, int(by_pair), sort.max_rows, _ptr(xq), _ptr(sfx),
                                                 _stream(dev)), "dispatch_rows")
    return xq, sfx


def quant_dispatch(x: torch.Tensor, sort: SortBuffers):
    """bf16 x [M, 6144] -> (codes in sorted-row order, scale atoms): quantisation fused with the gather."""
    if x.ndim != 2 or x.shape[1] != H or x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("expected contiguous BF16 [M,6144]")
    dev = x.device
    xq = torch.empty((sort.max_rows, H // 2), dtype=torch.uint8, device=dev)
    sfx = torch.empty((sort.max_rows // sort.bm, H // 128, 512), dtype=torch.uint8, device=dev)
    _lib.check(_lib.load().b200moe_quant_dispatch(_ptr(x), _ptr(sort.sorted_ids), _ptr(sort.num_valid), sort.tokens,
                                                  sort.bm, sort.max_rows, _ptr(xq), _ptr(sfx), None, _stream(dev)),
               "quant_dispatch")
    return xq, sfx


def route_sort(logits: torch.Tensor, w: "MoeWeights", bm: int | None = None):
    """fp32 logits [M, E] -> (weights, ids, SortBuffers): the router top-4 and the routing sort (one kernel up to 256
    tokens)."""
    if logits.dtype != torch.float32 or logits.ndim != 2 or not logits.is_contiguous():
        raise ValueError("expected contiguous fp32 [M, E] logits")
    lib = _lib.load()
    m, n_exp = logits.shape
    bm = variant_for(m) if bm is None else bm
    dev = logits.device
    rows = int(lib.b200moe_max_sorted_rows(m, bm, n_exp))
    wt = torch.empty((m, TOPK), dtype=torch.float32, device=dev)
    ids = torch.empty((m, TOPK), dtype=torch.int32, device=dev)
    buf = SortBuffers(torch.empty(rows, dtype=torch.int32, device=dev), torch.empty(rows, dtype=torch.float32, device=dev),
                      torch.empty(rows // bm, dtype=torch.int32, device=dev), torch.empty(2, dtype=torch.int32, device=dev),
                      bm, m)
    scratch = torch.empty(max(int(lib.b200moe_permute_scratch_bytes(m, n_exp)) // 4, 1), dtype=torch.int32, device=dev)
    _lib.check(lib.b200moe_route_sort(_ptr(logits), _ptr(w.correction_bias), m, n_exp, ROUTING_MODES[w.routing_mode],
                                      w.routed_scaling_factor, bm, _ptr(wt), _ptr(ids), _ptr(buf.sorted_ids),
                                      _ptr(buf.sorted_weights), _ptr(buf.block_expert), _ptr(buf.num_valid),
                                      _ptr(scratch), _stream(dev)), "route_sort")
    return wt, ids, buf


def grouped_gemm1(xq_sorted, sfx, sort: SortBuffers, w: MoeWeights, prefetch_next: bool = False):
    """GEMM1 + SwiGLU-OAI + MXFP4 requantisation on tcgen05 -> (h codes [rows, 384], h scale atoms [rows/bm, 6, 512]).
    ``prefetch_next``: also ask L2 for the W2 tiles the following GEMM2 reads first. (From about 3000 tokens' worth of rows
    the library runs the 256-column kernel of ``grouped_gemm1_wide``; same bits.)"""
    dev = xq_sorted.device
    hq = torch.empty((sort.max_rows, w.intermediate // 2), dtype=torch.uint8, device=dev)
    sfh = torch.empty((sort.max_rows // sort.bm, w.intermediate // 128, 512), dtype=torch.uint8, device=dev)
    _lib.check(w.lib().b200moe_gemm1_swiglu_quant(_ptr(w.w13), w.num_experts, _ptr(xq_sorted),
                                                      _ptr(sfx), _ptr(sort.block_expert), _ptr(sort.num_valid),
                                                      sort.max_rows, sort.bm, _ptr(hq), _ptr(sfh),
                                                      _ptr(w.w2) if prefetch_next else None,
                                                      _ptr(status_word(dev)), _stream(dev)), "gemm1_swiglu_quant")
    return hq, sfh


def grouped_gemm1_pair(xq_sorted, sfx, sort: SortBuffers, w: MoeWeights):
    """``grouped_gemm1`` at block height 128 on CTA pairs (``tcgen05.mma.cta_group::2``, 256 token rows x 256 weight rows
    per instruction): the same h codes and scale atoms."""
    if sort.bm != 128:
        raise ValueError("the CTA-pair GEMM1 serves block height 128")
    dev = xq_sorted.device
    hq = torch.empty((sort.max_rows, w.intermediate // 2), dtype=torch.uint8, device=dev)
    sfh = torch.empty((sort.max_rows // sort.bm, w.intermediate // 128, 512), dtype=torch.uint8, device=dev)
    _lib.check(w.lib().b200moe_gemm1_swiglu_quant_pair(_ptr(w.w13), w.num_experts, _ptr(xq_sorted), _ptr(sfx),
                                                           _ptr(sort.block_expert), _ptr(sort.num_valid), sort.max_rows,
                                                           _ptr(hq), _ptr(sfh), _ptr(status_word(dev)), _stream(dev)),
               "gemm1_swiglu_quant_pair")
    return hq, sfh


def grouped_gemm1_wide(xq_sorted, sfx, sort: SortBuffers, w: MoeWeights):
    """``grouped_gemm1`` at block height 128 with 256 weight rows per MMA on one CTA (128 token rows x 256 weight rows x 64):
    the same h codes and scale atoms."""
    if sort.bm != 128:
        raise ValueError("the wide GEMM1 serves block height 128")
    dev = xq_sorted.device
    hq = torch.empty((sort.max_rows, w.intermediate // 2), dtype=torch.uint8, device=dev)
    sfh = torch.empty((sort.max_rows // sort.bm, w.intermediate // 128, 512), dtype=torch.uint8, device=dev)
    _lib.check(w.lib().b200moe_gemm1_swiglu_quant_wide(_ptr(w.w13), w.num_experts, _ptr(xq_sorted), _ptr(sfx),
                                                       _ptr(sort.block_expert), _ptr(sort.num_valid), sort.max_rows,
                                                       _ptr(hq), _ptr(sfh), _ptr(status_word(dev)), _stream(dev)),
               "gemm1_swiglu_quant_wide")
    return hq, sfh


def block_chunks(sort: SortBuffers, chunks: int) -> torch.Tensor:
    """int32 [chunks, 2] on the device: the sorted row blocks in ``chunks`` runs of nearly equal length (first block, one past
    the last), for ``grouped_gemm1_gather`` / ``grouped_gemm2_peer`` with ``block_range``. Nothing reaches the host."""
    ranges = torch.empty((chunks, 2), dtype=torch.int32, device=sort.num_valid.device)
    _lib.check(_lib.load().b200moe_block_chunks(_ptr(sort.num_valid), sort.bm, chunks, _ptr(ranges),
                                                _stream(ranges.device)), "block_chunks")
    return ranges


def grouped_gemm1_gather(codes, scales, sort: SortBuffers, w: MoeWeights, by_pair: bool = False, block_range=None,
                         max_ctas: int = 0, out=None):
    """``grouped_gemm1`` at block height 128 straight from the UNSORTED row-major quantised tokens (``quant_mxfp4``'s codes
    [T, 3072] and scales [T, 192]): the kernel gathers each block's rows by ``sort.sorted_ids`` itself, the way the
    reference's prefill GEMM1 reads through sorted_token_ids (gemm1_prefill_h6144_i768.py:560-598). The same h codes and
    scale atoms as ``quant_dispatch`` + ``grouped_gemm1``. ``by_pair``: the input holds one row per (token, slot) pair
    instead of one per token (rows that arrived from other ranks). ``block_range`` (a row of ``block_chunks``): only those
    row blocks; ``max_ctas``: at most that many CTAs; ``out``: the (hq, sfh) buffers of an earlier call on the same sort."""
    if sort.bm != 128:
        raise ValueError("the gathering GEMM1 serves block height 128")
    dev = codes.device
    tokens = sort.tokens
    if out is None:
        out = (torch.empty((sort.max_rows, w.intermediate // 2), dtype=torch.uint8, device=dev),
               torch.empty((sort.max_rows // sort.bm, w.intermediate // 128, 512), dtype=torch.uint8, device=dev))
    hq, sfh = out
    _lib.check(w.lib().b200moe_gemm1_swiglu_quant_gather_range(
        _ptr(w.w13), w.num_experts, _ptr(codes), _ptr(scales), tokens, int(by_pair), _ptr(sort.sorted_ids),
        _ptr(sort.block_expert), _ptr(sort.num_valid), sort.max_rows, _ptr(hq), _ptr(sfh),
        None if block_range is None else _ptr(block_range), int(max_ctas), _ptr(status_word(dev)), _stream(dev)),
        "gemm1_swiglu_quant_gather")
    return hq, sfh


def grouped_gemm12(xq_sorted, sfx, sort: SortBuffers, w: MoeWeights, slots=None, done=None):
    """Both grouped GEMMs in one persistent launch (block heights 16 / 32 / 64): -> (slots, h codes, h scale atoms), the
    same bits as ``grouped_gemm1`` followed by ``grouped_gemm2`` (reference gemm12_a4w4.py:24). ``done``: the per-block
    completion counts, int32 [rows / bm], zero on entry (allocated when not given)."""
    dev = xq_sorted.device
    hq = torch.empty((sort.max_rows, w.intermediate // 2), dtype=torch.uint8, device=dev)
    sfh = torch.empty((sort.max_rows // sort.bm, w.intermediate // 128, 512), dtype=torch.uint8, device=dev)
    if done is None:
        done = torch.zeros(sort.max_rows // sort.bm, dtype=torch.int32, device=dev)
    if slots is None:
        slots = torch.empty((sort.tokens, TOPK, H), dtype=torch.bfloat16, device=dev)
    _lib.check(w.lib().b200moe_gemm12(_ptr(w.w13), _ptr(w.w2), w.num_experts, _ptr(xq_sorted), _ptr(sfx),
                                          _ptr(sort.block_expert), _ptr(sort.num_valid), _ptr(sort.sorted_ids),
                                          _ptr(sort.sorted_weights), sort.max_rows, sort.bm, sort.tokens, _ptr(hq),
                                          _ptr(sfh), _ptr(done), _ptr(slots), _ptr(status_word(dev)), _stream(dev)),
               "gemm12")
    return slots, hq, sfh


def grouped_gemm2(hq, sfh, sort: SortBuffers, w: MoeWeights, slots=None):
    """GEMM2 x routing weight -> bf16 slots [M, 4, 6144] (rows of padded or absent pairs are left untouched)."""
    dev = hq.device
    if slots is None:
        slots = torch.empty((sort.tokens, TOPK, H), dtype=torch.bfloat16, device=dev)
    _lib.check(w.lib().b200moe_gemm2_weighted(_ptr(w.w2), w.num_experts, _ptr(hq), _ptr(sfh),
                                                  _ptr(sort.block_expert), _ptr(sort.num_valid), _ptr(sort.sorted_ids),
                                                  _ptr(sort.sorted_weights), sort.max_rows, sort.bm, sort.tokens,
                                                  _ptr(slots), _ptr(status_word(dev)), _stream(dev)), "gemm2_weighted")
    return slots


def grouped_gemm2_peer(hq, sfh, sort: SortBuffers, w: MoeWeights, row_rank, row_pair, peer_ptrs, world: int,
                       peer_rows: int, block_range=None, max_ctas: int = 0):
    """GEMM2 whose result rows go straight into the slot buffers of the ranks that own the pairs (expert parallel):
    ``row_rank`` / ``row_pair`` int32 [4 * sort.tokens], ``peer_ptrs`` a ctypes array of ``world`` device pointers.
    ``block_range`` / ``max_ctas`` as in ``grouped_gemm1_gather``."""
    dev = hq.device
    _lib.check(w.lib().b200moe_gemm2_weighted_peer_range(
        _ptr(w.w2), w.num_experts, _ptr(hq), _ptr(sfh), _ptr(sort.block_expert), _ptr(sort.num_valid),
        _ptr(sort.sorted_ids), _ptr(sort.sorted_weights), sort.max_rows, sort.bm, sort.tokens, _ptr(row_rank),
        _ptr(row_pair), peer_ptrs, world, peer_rows, None if block_range is None else _ptr(block_range), int(max_ctas),
        _ptr(status_word(dev)), _stream(dev)), "gemm2_weighted_peer")


def simt_gemm1(x_quant, sort: SortBuffers, w: MoeWeights, rows=None):
    """The CUDA-core cross-check of ``grouped_gemm1`` on the checkpoint-layout weights (``keep_row_major=True``)."""
    if w.row_major is None:
        raise ValueError("needs MoeWeights.from_row_major(..., keep_row_major=True)")
    codes, scales = x_quant
    dev = codes.device
    hq = torch.zeros((sort.max_rows, w.intermediate // 2), dtype=torch.uint8, device=dev)
    sfh = torch.zeros((sort.max_rows // sort.bm, w.intermediate // 128, 512), dtype=torch.uint8, device=dev)
    _lib.check(w.lib().b200moe_gemm1_simt(_ptr(w.row_major[0]), _ptr(w.row_major[1]), _ptr(codes), _ptr(scales),
                                              _ptr(sort.sorted_ids), _ptr(sort.block_expert), _ptr(sort.num_valid),
                                              _ptr(rows), 0 if rows is None else rows.numel(), sort.max_rows, sort.bm,
                                              sort.tokens, _ptr(hq), _ptr(sfh), _stream(dev)), "gemm1_simt")
    return hq, sfh


def simt_gemm2(hq, sfh, sort: SortBuffers, w: MoeWeights, rows=None, slots=None):
    """The CUDA-core cross-check of ``grouped_gemm2``."""
    if w.row_major is None:
        raise ValueError("needs MoeWeights.from_row_major(..., keep_row_major=True)")
    dev = hq.device
    if slots is None:
        slots = torch.zeros((sort.tokens, TOPK, H), dtype=torch.bfloat16, device=dev)
    _lib.check(w.lib().b200moe_gemm2_simt(_ptr(w.row_major[2]), _ptr(w.row_major[3]), _ptr(hq), _ptr(sfh),
                                              _ptr(sort.sorted_ids), _ptr(sort.sorted_weights), _ptr(sort.block_expert),
                                              _ptr(sort.num_valid), _ptr(rows), 0 if rows is None else rows.numel(),
                                              sort.max_rows, sort.bm, sort.tokens, _ptr(slots), _stream(dev)), "gemm2_simt")
    return slots


def reduce_slots(slots: torch.Tensor, shared: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 [M, 4, H] (+ bf16 [M, H]) -> bf16 [M, H], slots 0..3 then shared in fp32, one rounding
    (reference common/reduce_slots_shared.py:37-41)."""
    if slots.dtype != torch.bfloat16 or slots.ndim != 3 or slots.shape[1:] != (TOPK, H) or not slots.is_contiguous():
        raise ValueError("expected contiguous BF16 [M, 4, 6144]")
    out = torch.empty((slots.shape[0], H), dtype=torch.bfloat16, device=slots.device)
    _lib.check(_lib.load().b200moe_reduce_slots(_ptr(slots), _ptr(shared), slots.shape[0], _ptr(out),
                                                _stream(slots.device)), "reduce_slots")
    return out


def reduce_rows(rows: torch.Tensor, index: torch.Tensor, tokens: int) -> torch.Tensor:
    """bf16 rows [N, 6144] + int32 index [M, 4] (row of pair 4*token+slot) -> bf16 [M, 6144], slots 0..3 in fp32."""
    if rows.dtype != torch.bfloat16 or rows.ndim != 2 or rows.shape[1] != H or not rows.is_contiguous():
        raise ValueError("expected contiguous BF16 [N, 6144]")
    if index.dtype != torch.int32 or index.numel() != tokens * TOPK or not index.is_contiguous():
        raise ValueError("expected a contiguous int32 index of 4 entries per token")
    out = torch.empty((tokens, H), dtype=torch.bfloat16, device=rows.device)
    _lib.check(_lib.load().b200moe_reduce_rows(_ptr(rows), _ptr(index), None, tokens, _ptr(out), _stream(rows.device)),
               "reduce_rows")
    return out


# ------------------------------------------------------------------------------------------------ the entry
def _logits(x, w, router_logits):
    if router_logits is not None:
        if router_logits.shape != (x.shape[0], w.num_experts) or router_logits.dtype != torch.float32:
            raise ValueError(f"router_logits: expected fp32 [{x.shape[0]}, {w.num_experts}]")
        return router_logits.contiguous()
    if w.router_weight is None:
        raise ValueError("needs router_logits= or MoeWeights with router_weight")
    w.abi()  # makes the gate's bf16 terms on first use
    return router_gemm_partials(x, w.router_weight, w.router_split)


def split_gate(gate: torch.Tensor) -> torch.Tensor:
    """fp32 gate [E, 6144] -> its three bf16 terms RN(w), RN(w - w0), RN(w - w0 - w1) as bf16 [3, 128, 6144] (rows from E on
    zero): the tensor-core router's B operand (reference router_gemm.py:32-44 ``_split3``). Once, at load time."""
    if gate.dtype != torch.float32 or gate.ndim != 2 or gate.shape[1] != H or not gate.is_contiguous() or gate.shape[0] > E:
        raise ValueError("expected a contiguous fp32 gate [E <= 128, 6144]")
    out = torch.empty((3, E, H), dtype=torch.bfloat16, device=gate.device)
    with torch.cuda.device(gate.device):
        _lib.check(_lib.load().b200moe_router_split_gate(_ptr(gate), gate.shape[0], _ptr(out), _stream(gate.device)),
                   "router_split_gate")
    return out


def router_gemm_partials(x: torch.Tensor, gate: torch.Tensor, split: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 x [M, 6144] times the fp32 gate [E, 6144] -> split-K partials as an [M, S, E] view of [S, M, E] (the layout
    the reference's routers write, router_gemm.py:390-467); ``topk_route`` adds them in split order. With ``split``
    (``split_gate(gate)``) and 128 tokens or more the product runs on the tensor cores, else on the CUDA cores."""
    if x.ndim != 2 or x.shape[1] != H or x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("expected contiguous BF16 [M,6144]")
    if gate.dtype != torch.float32 or gate.ndim != 2 or gate.shape[1] != H or not gate.is_contiguous():
        raise ValueError("expected a contiguous fp32 gate [E, 6144]")
    lib = _lib.load()
    m, n_exp = x.shape[0], gate.shape[0]
    splits = int(lib.b200moe_router_splits(m))
    parts = torch.empty((splits, m, n_exp), dtype=torch.float32, device=x.device)
    if split is not None and m >= 128:
        _lib.check(lib.b200moe_router_gemm_tc(_ptr(x), _ptr(split), m, n_exp, splits, _ptr(parts),
                                              _ptr(status_word(x.device)), _stream(x.device)), "router_gemm_tc")
    else:
        _lib.check(lib.b200moe_router_gemm(_ptr(x), _ptr(gate), m, n_exp, splits, _ptr(parts), _stream(x.device)),
                   "router_gemm")
    return parts.permute(1, 0, 2)


def router_gemm_quant(x: torch.Tensor, gate: torch.Tensor, shared: bool = False, split: torch.Tensor | None = None):
    """The split-K logit partials of ``router_gemm_partials``, the row-major MXFP4 operands of ``mxfp4_quant`` and, with
    ``shared``, the row-major MXFP8 operands of ``shared_quant_rows`` (else None), all with those kernels' bits (reference
    router_mxfp4_mxfp8_quant_row_scales.py). Below 128 tokens (or without ``split``) ONE kernel makes one pass over x; from
    128 tokens on the router runs on the tensor cores (``split`` = ``split_gate(gate)``) with the quantisers beside it."""
    if x.ndim != 2 or x.shape[1] != H or x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("expected contiguous BF16 [M,6144]")
    if gate.dtype != torch.float32 or gate.ndim != 2 or gate.shape[1] != H or not gate.is_contiguous():
        raise ValueError("expected a contiguous fp32 gate [E, 6144]")
    lib = _lib.load()
    m, n_exp, dev = x.shape[0], gate.shape[0], x.device
    if split is not None and m >= 128:
        from .shared_expert import shared_quant_rows
        return router_gemm_partials(x, gate, split), mxfp4_quant(x), (shared_quant_rows(x) if shared else (None, None))
    splits = int(lib.b200moe_router_splits(m))
    parts = torch.empty((splits, m, n_exp), dtype=torch.float32, device=dev)
    q4 = torch.empty((m, H // 2), dtype=torch.uint8, device=dev)
    s4 = torch.empty((m, H // 32), dtype=torch.uint8, device=dev)
    q8 = torch.empty((m, H), dtype=torch.uint8, device=dev) if shared else None
    s8 = torch.empty((m, H // 32), dtype=torch.uint8, device=dev) if shared else None
    _lib.check(lib.b200moe_router_gemm_quant(_ptr(x), _ptr(gate), m, n_exp, splits, _ptr(parts), _ptr(q4), _ptr(s4),
                                             _ptr(q8), _ptr(s8), _stream(dev)), "router_gemm_quant")
    return parts.permute(1, 0, 2), (q4, s4), (q8, s8)


def route(x, w, router_logits=None):
    """The entry's routing (topk weights incl. the routed scale, topk ids), exposed for numerical checks
    (reference chain.py:106-110)."""
    logits = _logits(x, w, router_logits)
    return topk_route(logits, w.correction_bias, w.routed_scaling_factor, w.routing_mode)


def mxfp4_moe_experts(x_quant, topk_weights, topk_ids, w):
    """The routed experts on the MXFP4 input ``x_quant`` = (codes, scales), already routed (``topk_weights`` include
    the routed scale) -> the BF16 [M, 4, H] slots (reference chain.py:113-124). Served at every M here."""
    n = x_quant[0].shape[0]
    bm = variant_for(n)
    sort = moe_sort(topk_ids, topk_weights, bm, w.num_experts)
    xq, sfx = dispatch_rows(x_quant, sort)
    hq, sfh = grouped_gemm1(xq, sfx, sort, w)
    return grouped_gemm2(hq, sfh, sort, w)


def mxfp4_moe(x, w, *, return_partials=False, router_logits=None):
    """Normed BF16 [M, 6144] -> the routed experts' output (reference chain.py:127-197).

    Reduced mode returns BF16 [M, 6144] = slots 0..3, then the shared expert's output, summed in fp32; partials mode
    returns (slots BF16 [M, 4, H], shared BF16 [M, H]); without ``w.shared_weights`` the shared term is absent (None).
    ``router_logits`` fp32 [M, E] skips the router GEMM. The routed part is one ``b200moe_forward`` on the current
    stream; the shared expert runs on the device's side stream beside it and the current stream joins it before the
    reduce. Without ``router_logits`` the router runs inside the same call (``b200moe_forward_x``). Scratch and outputs come
    from ``torch.empty``."""
    if not isinstance(x, torch.Tensor):
        from .prepared_input import MoeInput, MoeInputCompact, mxfp4_moe_prepared
        if not isinstance(x, (MoeInput, MoeInputCompact)):
            raise ValueError("expected BF16 [M,6144] rows, a MoeInput or a MoeInputCompact")
        return mxfp4_moe_prepared(x, w, return_partials=return_partials)
    variant_for(x.shape[0])
    if x.ndim != 2 or x.shape[1] != H or x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("expected contiguous BF16 [M,6144]")
    n, dev = x.shape[0], x.device
    sw = w.shared_weights
    shared = None
    if sw is not None:
        from .shared_expert import shared_expert_parallel
        current = torch.cuda.current_stream(dev)
        shared = shared_expert_parallel(x, sw, current)
    slots = torch.empty((n, TOPK, H), dtype=torch.bfloat16, device=dev)
    out = None if (return_partials or sw is not None) else torch.empty((n, H), dtype=torch.bfloat16, device=dev)
    _routed_layer(x, w, router_logits, slots, out)
    if sw is None:
        return (slots, None) if return_partials else out
    current = torch.cuda.current_stream(dev)
    current.wait_stream(sw.stream)
    shared.record_stream(current)
    return (slots, shared) if return_partials else reduce_slots(slots, shared)


def _routed_layer(x, w, router_logits, slots, out):
    """One C-ABI call for the routed layer on the current stream: ``b200moe_forward`` when the caller hands fp32 logits,
    ``b200moe_forward_x`` (router GEMM fused with the input quantiser inside the call) when it hands only ``x``."""
    lib = w.lib()
    n, dev = x.shape[0], x.device
    if router_logits is not None:
        if router_logits.shape != (n, w.num_experts) or router_logits.dtype != torch.float32:
            raise ValueError(f"router_logits: expected fp32 [{n}, {w.num_experts}]")
        logits = router_logits.contiguous()
        ws_bytes = int(lib.b200moe_workspace_bytes(n, w.num_experts))
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        _lib.check(lib.b200moe_forward(ctypes.byref(w.abi()), _ptr(x), _ptr(logits), n, _ptr(workspace), ws_bytes,
                                       _ptr(slots), _ptr(out), _ptr(status_word(dev)), _stream(dev)), "forward")
        return
    if w.router_weight is None:
        raise ValueError("needs router_logits= or MoeWeights with router_weight")
    ws_bytes = int(lib.b200moe_workspace_bytes_x(n, w.num_experts))
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    _lib.check(lib.b200moe_forward_x(ctypes.byref(w.abi()), _ptr(x), n, _ptr(workspace), ws_bytes, _ptr(slots), _ptr(out),
                                     _ptr(status_word(dev)), _stream(dev)), "forward_x")


def set_wait_limit_ns(ns: int) -> None:
    """How long a device-side wait may last on the current device before the kernel gives up with status 1 (default 2 s)."""
    for inter in (768, 1536):  # every build of the library this process has loaded keeps its own limit
        if inter == 768 or inter in _lib._libs:
            _lib.check(_lib.load(inter).b200moe_set_wait_limit_ns(int(ns)), "set_wait_limit_ns")


WARM_UP_TOKENS = (1, 64, 481, 513, 5000)  # one-launch GEMMs, one size per block height the entry uses


def warm_up_mxfp4_moe(w, *, partials=False, workers=None):
    """Loads the library and runs one call per kernel variant before serving, so that the first served call (or a CUDA
    graph capture) does no one-time set-up (reference chain.py:239-258; there is nothing to compile here, ``workers``
    is accepted and ignored)."""
    dev = w.w13.device
    with torch.inference_mode():
        for m in WARM_UP_TOKENS:
            x = torch.zeros((m, H), device=dev, dtype=torch.bfloat16)
            lg = torch.zeros((m, w.num_experts), device=dev, dtype=torch.float32)
            mxfp4_moe(x, w, return_partials=False, router_logits=lg)
            if w.router_weight is not None:
                mxfp4_moe(x, w, return_partials=False)
            if partials:
                mxfp4_moe(x, w, return_partials=True, router_logits=lg)
    torch.cuda.synchronize(dev)
    if last_status(dev):
        raise RuntimeError("a kernel reported a device-side timeout during warm-up")
