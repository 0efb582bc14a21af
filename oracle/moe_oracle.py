"""CPU restatement (numpy) of the reference's MXFP4 MoE hot path. TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA kernels: only the tests, the smoke check and the benchmark's CPU-baseline leg
may import it. Nothing in the product package imports it, and the product has no CPU fallback.

Every function restates one function of the reference's torch oracle
``amd_kernels/moe/mxfp4_h6144_i768_e128_top4/reference.py`` (cited per function as ``reference.py:LINES``) or one of the
test-local references under ``tests/moe/mxfp4_h6144_i768_e128_top4``. Parity is pinned: ``tests/golden/make_golden.py``
ran the reference's own ``reference.py`` in the build container and stored its outputs; ``tests/test_oracle_golden.py``
checks this module against those files bit for bit (quant, routing ids, reduce) or to fp32 round-off (the MoE sums).

Conventions: bf16 tensors are carried as ``uint16`` bit patterns; "codes" are E2M1 nibbles packed two per byte with the
even element in the low nibble; "scales" are E8M0 bytes (value 2**(byte-127)), one per 32 elements along K.
"""
from __future__ import annotations

import numpy as np

H, I, E, TOPK = 6144, 768, 128, 4  # noqa: E741
ALPHA, LIMIT = 1.702, 7.0
GRID = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
LUT = np.concatenate([GRID, -GRID]).astype(np.float32)
TIE_EPS = 1e-6
WEIGHT_RTOL = 2.0 ** -20


# ----------------------------------------------------------------------------------------------- bf16 helpers
def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> float32 (exact)."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> uint16 bf16 bit patterns, round to nearest even (what ``tensor.bfloat16()`` does for finite values)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))) >> 16
    nan = (u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    return np.where(nan, (u >> 16) | np.uint32(0x40), rounded).astype(np.uint16)


# ----------------------------------------------------------------------------------------------- MXFP4
def dequant_mxfp4(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """[.., K/2] u8 codes + [.., K/32] u8 scales -> float32 [.., K]  (reference.py:23-29)."""
    lo = LUT[codes & 0xF]
    hi = LUT[codes >> 4]
    v = np.stack([lo, hi], axis=-1).reshape(*codes.shape[:-1], codes.shape[-1] * 2)
    s = np.exp2(scales.astype(np.float32) - 127.0).astype(np.float32)
    return v * np.repeat(s, 32, axis=-1)


def quant_mxfp4(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """float32 [M, K] -> (codes u8 [M, K/2], scales u8 [M, K/32]); the "Quark even" rule (reference.py:32-46).

    scale byte e = max(1, (bits(amax) - 0x00E00000) >> 23) with an arithmetic shift; a = |v| / 2**(e-127); the code is
    the number of midpoints {.25 .75 1.25 1.75 2.5 3.5 5} below a, a tie going to the even code; bit 3 = signbit(v)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    v = x.reshape(m, k // 32, 32)
    a_abs = np.abs(v)
    amax = a_abs.max(axis=-1)
    e = np.maximum((amax.view(np.int32) - np.int32(0xE00000)) >> 23, 1)
    a = a_abs / np.exp2(e.astype(np.float32) - 127.0)[..., None].astype(np.float32)
    code = np.zeros(a.shape, dtype=np.uint8)
    for i, mid in enumerate((0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)):
        code += (a >= np.float32(mid)) if i % 2 else (a > np.float32(mid))
    code = (code | (np.signbit(v).astype(np.uint8) << 3)).reshape(m, k)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return np.ascontiguousarray(packed), np.ascontiguousarray(e.astype(np.uint8))


def swiglu_oai(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    """SwiGLU-OAI in float32: min(g,7) * sigmoid(1.702*g) * (clamp(u,-7,7) + 1)  (reference.py:49-52)."""
    g = np.minimum(g, np.float32(LIMIT)).astype(np.float32)
    u = np.clip(u, np.float32(-LIMIT), np.float32(LIMIT)).astype(np.float32)
    sig = (np.float32(1.0) / (np.float32(1.0) + np.exp(-(np.float32(ALPHA) * g)))).astype(np.float32)
    return (g * sig * (u + np.float32(1.0))).astype(np.float32)


# ----------------------------------------------------------------------------------------------- routing
def splitk_logits(partials: np.ndarray) -> np.ndarray:
    """fp32 partials [M, S, E] -> logits [M, E], summed from 0.0 in split order (reference.py:118-124)."""
    out = np.zeros((partials.shape[0], partials.shape[2]), dtype=np.float32)
    for k in range(partials.shape[1]):
        out = out + partials[:, k].astype(np.float32)
    return out


def _topk_lowest_id(choice: np.ndarray, k: int) -> np.ndarray:
    """Indices of the k largest entries per row, descending; exactly equal values resolve to the LOWER index (this
    build's tie rule; the reference leaves exact ties to its ``decided`` mask, reference.py:143-148)."""
    order = np.argsort(-choice, axis=-1, kind="stable")
    return order[:, :k]


def route_sigmoid_bias(logits: np.ndarray, bias: np.ndarray, scale: float, topk: int = TOPK):
    """The reference's routing (reference.py:127-140) in float64: s = sigmoid(logit); choice = s + bias; top-k of choice
    descending; weight = s * scale / sum(s over the chosen). Returns (weights f64 [M,k], ids i64 [M,k], the k+1 largest
    choice values f64 [M,k+1])."""
    s = 1.0 / (1.0 + np.exp(-logits.astype(np.float64)))
    choice = s + bias.astype(np.float64)
    ids = _topk_lowest_id(choice, topk + 1)
    vals = np.take_along_axis(choice, ids, axis=1)
    chosen = np.take_along_axis(s, ids[:, :topk], axis=1)
    weights = chosen * scale / chosen.sum(-1, keepdims=True)
    return weights, ids[:, :topk], vals


def route_softmax(logits: np.ndarray, scale: float = 1.0, topk: int = TOPK):
    """Softmax over the experts, top-k, renormalised over the picks (the benchmark configurations' routing):
    ids = top-k of the fp32 logits (ties to the lower id, exact compares), weight_k = exp(l_k - m) / sum_sel exp(l_j - m)
    times ``scale``, m the row maximum. Float64 arithmetic on the fp32 logits."""
    lg = logits.astype(np.float32)
    ids = _topk_lowest_id(lg.astype(np.float64), topk + 1)
    vals = np.take_along_axis(lg.astype(np.float64), ids, axis=1)
    sel = vals[:, :topk]
    p = np.exp(sel - sel[:, :1])
    return p * scale / p.sum(-1, keepdims=True), ids[:, :topk], vals


def decided(vals: np.ndarray, eps: float = TIE_EPS) -> np.ndarray:
    """[M, k] bool: position j's id is decided when its choice is more than ``eps`` from both neighbours
    (reference.py:143-148)."""
    gaps = vals[:, :-1] - vals[:, 1:]
    above = np.concatenate([np.full_like(gaps[:, :1], np.inf), gaps[:, :-1]], axis=1)
    return (gaps > eps) & (above > eps)


# ----------------------------------------------------------------------------------------------- permutation
def max_sorted_rows(tokens: int, bm: int, topk: int = TOPK, experts: int = E) -> int:
    """Upper bound of the padded row count (amd_kernels/moe/.../common/sort.py:19-23)."""
    pairs = tokens * topk
    return -(-(pairs + min(experts, pairs) * (bm - 1)) // bm) * bm


def permute(ids: np.ndarray, weights: np.ndarray, bm: int, experts: int = E):
    """Group the (token, slot) pairs by expert ascending, pair order q = 4*token + slot inside an expert, each expert
    padded to a multiple of ``bm`` rows with (token = M, weight 0) — the canonical order of
    tests/moe/.../test_id_rows_experts.py:20-31 and the padding convention of test_sort_a16w4.py:43-59.

    Returns (sorted_ids i32 [rows] = token | slot << 24, sorted_w f32 [rows], block_expert i32 [rows / bm],
    num_valid i32 [2] = [padded rows, first row of the last non-empty expert])."""
    m, k = ids.shape
    flat = ids.reshape(-1)
    rows, wts, blocks = [], [], []
    last_start = 0
    for e in range(experts):
        q = np.nonzero(flat == e)[0]
        if q.size == 0:
            continue
        last_start = len(rows)
        pairs = ((q // k) | ((q % k) << 24)).astype(np.int64).tolist()
        w = weights.reshape(-1)[q].astype(np.float32).tolist()
        pad = -len(pairs) % bm
        rows += pairs + [m] * pad
        wts += w + [0.0] * pad
        blocks += [e] * ((len(pairs) + pad) // bm)
    return (np.array(rows, dtype=np.int32), np.array(wts, dtype=np.float32), np.array(blocks, dtype=np.int32),
            np.array([len(rows), last_start], dtype=np.int32))


# ----------------------------------------------------------------------------------------------- experts
def w4a4_moe(xq, xs, w13, w13_scale, w2, w2_scale, topk_weights, topk_ids, *, return_slots=False):
    """One MoE call on dequantized operands in float32 (reference.py:55-75): per expert e with rows (t, s):
    gu = x[t] @ W13[e]^T; h = dequant(quant(swiglu_oai(gu[:, :I], gu[:, I:]))); y = h @ W2[e]^T; out[t] += y * w[t, s].

    ``return_slots``: also the per-(token, slot) products y * w as float32 [M, k, H] (what the kernels round to bf16)."""
    x = dequant_mxfp4(xq, xs)
    m = x.shape[0]
    inter = w13.shape[1] // 2
    hdim = w2.shape[1]
    out = np.zeros((m, hdim), dtype=np.float32)
    slots = np.zeros((m, topk_ids.shape[1], hdim), dtype=np.float32) if return_slots else None
    for e in np.unique(topk_ids).tolist():
        t, s = np.nonzero(topk_ids == e)
        gu = x[t] @ dequant_mxfp4(w13[e], w13_scale[e]).T
        h = dequant_mxfp4(*quant_mxfp4(swiglu_oai(gu[:, :inter], gu[:, inter:])))
        y = (h @ dequant_mxfp4(w2[e], w2_scale[e]).T).astype(np.float32)
        yw = y * topk_weights[t, s].astype(np.float32)[:, None]
        np.add.at(out, t, yw)
        if return_slots:
            slots[t, s] = yw
    return (out, slots) if return_slots else out


def reduce_slots_bf16(slots_bits: np.ndarray, shared_bits: np.ndarray | None = None) -> np.ndarray:
    """bf16 bits [M, k, H] -> bf16 bits [M, H]: +0, then slots 0..k-1 in float32, (then the shared output), one rounding
    (reference.py:151-159; shared order: amd_kernels/moe/.../common/reduce_slots_shared.py:17-30)."""
    acc = np.zeros(slots_bits[:, 0].shape, dtype=np.float32)
    for k in range(slots_bits.shape[1]):
        acc = acc + bf16_to_f32(slots_bits[:, k])
    if shared_bits is not None:
        acc = acc + bf16_to_f32(shared_bits)
    return f32_to_bf16(acc)


def moe_layer(x_bits, logits, w13, w13_scale, w2, w2_scale, *, mode="softmax", bias=None, scale=1.0):
    """The whole routed layer as the product computes it: quantize x, route, experts, per-slot bf16 rounding, fixed-order
    reduce. Returns dict(out bf16 bits [M,H], slots bf16 bits [M,4,H], ids, weights f32, xq, xs)."""
    xq, xs = quant_mxfp4(bf16_to_f32(x_bits))
    if mode == "softmax":
        w, ids, _ = route_softmax(logits, scale)
    else:
        w, ids, _ = route_sigmoid_bias(logits, np.zeros(logits.shape[1]) if bias is None else bias, scale)
    w32 = w.astype(np.float32)
    _, slots = w4a4_moe(xq, xs, w13, w13_scale, w2, w2_scale, w32, ids, return_slots=True)
    slot_bits = f32_to_bf16(slots)
    return dict(out=reduce_slots_bf16(slot_bits), slots=slot_bits, ids=ids.astype(np.int32), weights=w32, xq=xq, xs=xs)


# ----------------------------------------------------------------------------------------------- fused tail
# Restates amd_kernels/collectives/pull_collectives_ranks4/reference.py:74-91 (the local slot sum of
# slots4_reduce_scatter_reference, = amd_kernels/norm/gemma_add_rmsnorm_h6144/reference.py slots4_local_reference) and
# steps 2-4 of amd_kernels/norm/gemma_add_rmsnorm_h6144/reference.py (add_rmsnorm_reference, mxfp8_scale_reference,
# mxfp8_codes); pinned by tests/golden/tail.npz, which those functions wrote.
TAIL_FP8_MAX, TAIL_TINY = 448.0, 2.0 ** -126
TAIL_OUT_ULPS, TAIL_OUT_MISMATCH, TAIL_OUT_COS = 1, 1e-3, 0.99999       # the norm reference's tolerances
TAIL_SCALE_MISMATCH, TAIL_CODE_MISMATCH, TAIL_MXFP8_COS = 1e-3, 1e-3, 0.999


def slots4_local(slots_bits: np.ndarray, shared_bits: np.ndarray | None = None) -> np.ndarray:
    """bf16 bits [M, 4, H] (+ [M, H]) -> bf16 bits [M, H]: (((s0 + s1) + s2) + s3) + shared in float32 starting FROM s0
    (not from +0: a row of -0.0 stays -0.0), one rounding."""
    acc = bf16_to_f32(slots_bits[:, 0])
    for k in range(1, slots_bits.shape[1]):
        acc = acc + bf16_to_f32(slots_bits[:, k])
    if shared_bits is not None:
        acc = acc + bf16_to_f32(shared_bits)
    return f32_to_bf16(acc)


def add_rmsnorm(x_bits: np.ndarray, residual_bits: np.ndarray, weight_bits: np.ndarray, eps: float):
    """-> (y float64 [M, H], residual out bf16 bits): s = fp32(x) + fp32(residual) (one float32 rounding), residual out =
    bf16(s), y = s * rsqrt(sum(s^2) / H + fp32(eps)) * (weight + 1) in float64; a sum of squares above the float32
    maximum counts as +inf."""
    s = (bf16_to_f32(x_bits) + bf16_to_f32(residual_bits)).astype(np.float32)
    s64 = s.astype(np.float64)
    with np.errstate(over="ignore", invalid="ignore"):
        ss = (s64 * s64).sum(-1, keepdims=True)
        ss = np.where(ss > np.finfo(np.float32).max, np.inf, ss)
        y = s64 / np.sqrt(ss / s.shape[-1] + np.float64(np.float32(eps))) * (bf16_to_f32(weight_bits).astype(np.float64) + 1.0)
    return y, f32_to_bf16(s)


def tail_mxfp8_scale(y64: np.ndarray) -> np.ndarray:
    """[M, H/32] E8M0 bytes: a = max(max|y|, 2^-126) per 32 columns (NaNs skipped), byte = clamp(ceil(log2(fp32(a) / 448))
    + 127, 0, 254), the division rounded to float32; 254 for an infinite a."""
    m, h = y64.shape
    mag = np.abs(y64)
    mag = np.where(np.isnan(mag), 0.0, mag)
    with np.errstate(over="ignore"):
        a = np.maximum(mag.reshape(m, h // 32, 32).max(-1).astype(np.float32), np.float32(TAIL_TINY))
        d = (a / np.float32(TAIL_FP8_MAX)).astype(np.float32).astype(np.float64)
    man, ex = np.frexp(np.where(np.isinf(d), 1.0, d))
    ceil_log2 = ex.astype(np.int64) - (man == 0.5)
    sb = np.clip(ceil_log2 + 127, 0, 254)
    return np.where(np.isinf(a), 254, sb).astype(np.uint8)


def tail_mxfp8_codes(y64: np.ndarray, scale_bytes: np.ndarray) -> np.ndarray:
    """[M, H] E4M3 bytes of y at the given scale bytes: y * 2^(127 - byte) rounded to float32, clamped to +-448, round to
    nearest even (finite inputs)."""
    m, h = y64.shape
    q = (y64.reshape(m, h // 32, 32) * np.exp2(127.0 - scale_bytes.astype(np.float64))[:, :, None]).astype(np.float32)
    return f32_to_e4m3(np.clip(q, -TAIL_FP8_MAX, TAIL_FP8_MAX)).reshape(m, h)


def tail_dequant(codes: np.ndarray, scale_bytes: np.ndarray) -> np.ndarray:
    m, h = codes.shape
    v = e4m3_to_f32(codes).astype(np.float64).reshape(m, h // 32, 32)
    return (v * np.exp2(scale_bytes.astype(np.float64) - 127.0)[:, :, None]).reshape(m, h)


def bf16_ulp(v: np.ndarray) -> np.ndarray:
    """The bf16 spacing at |v| (2^-133 at zero and among the subnormals)."""
    _, e = np.frexp(np.asarray(v, dtype=np.float64))
    e = np.where(v == 0, -125, e)
    return np.exp2(np.maximum(e.astype(np.float64) - 8.0, -133.0))


def compare_tail(out_bits, codes, scale_bytes, y64) -> dict:
    """The norm reference's acceptance statistics (its compare_out / compare_mxfp8) of a bf16 ``out`` and row-major
    MXFP8 ``codes`` / ``scale_bytes`` against the float64 y, finite y assumed. Any of the three may be None."""
    stats = {}
    if out_bits is not None:
        o = bf16_to_f32(out_bits).astype(np.float64)
        err = np.abs(o - y64)
        ulp = np.maximum(bf16_ulp(y64), bf16_ulp(o))
        yb = bf16_to_f32(f32_to_bf16(y64.astype(np.float32))).astype(np.float64)
        stats.update(bad_ulp=int((err > TAIL_OUT_ULPS * ulp).sum()), mismatch=float((o != yb).mean()),
                     cos=float((o * y64).sum() / np.linalg.norm(o) / np.linalg.norm(y64)))
    if codes is not None:
        ref_sb = tail_mxfp8_scale(y64)
        sd = np.abs(scale_bytes.astype(np.int64) - ref_sb.astype(np.int64))
        ref_codes = tail_mxfp8_codes(y64, scale_bytes)
        diff = codes != ref_codes
        mag = lambda c: (c & 0x7F).astype(np.int64)  # noqa: E731
        near = (np.abs(mag(codes) - mag(ref_codes)) <= 1) & (((codes & 0x80) == (ref_codes & 0x80)) | (mag(codes) == 0)
                                                             | (mag(ref_codes) == 0))
        deq = tail_dequant(codes, scale_bytes)
        stats.update(scale_max_diff=int(sd.max()), scale_mismatch=float((sd != 0).mean()),
                     code_mismatch=float(diff.mean()), code_far=int((diff & ~near).sum()),
                     mxfp8_cos=float((deq * y64).sum() / np.linalg.norm(deq) / np.linalg.norm(y64)))
    return stats


# ----------------------------------------------------------------------------------------------- shared expert (MXFP8)
def _e4m3_table() -> np.ndarray:
    """float32 value of every E4M3 (fn) byte; 0x7f / 0xff are NaN."""
    codes = np.arange(256, dtype=np.uint32)
    sign = np.where(codes & 0x80, -1.0, 1.0)
    exp = (codes >> 3) & 0xF
    man = codes & 7
    val = np.where(exp == 0, man / 8.0 * 2.0 ** -6, (1.0 + man / 8.0) * np.exp2(exp.astype(np.float64) - 7.0))
    val = np.where((codes & 0x7F) == 0x7F, np.nan, val)
    return (sign * val).astype(np.float32)


E4M3 = _e4m3_table()


def e4m3_to_f32(codes: np.ndarray) -> np.ndarray:
    return E4M3[codes]


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """float32 -> E4M3 bytes, round to nearest, ties to the even code, |x| <= 448 (what ``.to(torch.float8_e4m3fn)``
    does for in-range values; the quantiser below never leaves the range)."""
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    pos = E4M3[:127].astype(np.float64)  # codes 0..126 ascend with their values
    hi = np.clip(np.searchsorted(pos, a, side="left"), 1, 126)
    lo = hi - 1
    d_lo, d_hi = a - pos[lo], pos[hi] - a
    code = np.where(d_lo < d_hi, lo, np.where(d_hi < d_lo, hi, np.where(lo % 2 == 0, lo, hi)))
    code = np.where(a >= 448.0, 126, code)
    return (code.astype(np.uint8) | (np.signbit(x).astype(np.uint8) << 7)).astype(np.uint8)


def shared_mxfp8_quant(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """float32 [.., K] -> (E4M3 codes u8 [.., K], E8M0 u8 [.., K/32]); scale = ceil_pow2(amax / 448), exponent >= 1, no
    bf16 rounding first (reference.py:162-171)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    v = x.reshape(*x.shape[:-1], x.shape[-1] // 32, 32)
    u = (np.abs(v).max(-1) / np.float32(448.0)).astype(np.float32).view(np.int32)
    e = (u >> 23) & 255
    e = np.maximum(e + (((u & 0x7FFFFF) != 0) & (e < 255)), 1)
    q = f32_to_e4m3((v / np.exp2(e.astype(np.float32) - 127.0)[..., None]).astype(np.float32))
    return q.reshape(x.shape), e.astype(np.uint8)


def dequant_shared_mxfp8(q: np.ndarray, s: np.ndarray) -> np.ndarray:
    """(reference.py:174-175)"""
    return e4m3_to_f32(q) * np.repeat(np.exp2(s.astype(np.float32) - 127.0), 32, axis=-1)


def shared_mxfp8(x: np.ndarray, w13, s13, w2, s2) -> np.ndarray:
    """The shared expert in float32 (reference.py:178-189, quantized=True): x and the SwiGLU output go through the
    MXFP8 quantiser, both GEMMs and SwiGLU-OAI run in float32."""
    xq = dequant_shared_mxfp8(*shared_mxfp8_quant(x))
    gu = xq @ dequant_shared_mxfp8(w13, s13).T
    inter = w13.shape[0] // 2
    h = dequant_shared_mxfp8(*shared_mxfp8_quant(swiglu_oai(gu[:, :inter], gu[:, inter:])))
    return (h @ dequant_shared_mxfp8(w2, s2).T).astype(np.float32)


def _mxfp4_via_shared_codes(s4: np.ndarray, q8: np.ndarray, s8: np.ndarray):
    """The FP4 codes (one per byte, sign in bit 3) of the FP8 values re-read at the FP4 scales, and the magnitudes they
    were rounded from (reference.py:198-207): magnitude = |e4m3| / 2**(s4 - s8); thresholds .25 .75 1.25 1.75 2.5 3.5 5
    with ties to the even code."""
    ratio = np.repeat(np.exp2((s4.astype(np.int32) - s8.astype(np.int32)).astype(np.float32)), 32, axis=-1)
    magnitude = (np.abs(e4m3_to_f32(q8)) / ratio).astype(np.float32)
    codes = np.zeros(q8.shape, dtype=np.uint8)
    for j, mid in enumerate((0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)):
        codes += ((magnitude >= mid) if j % 2 else (magnitude > mid)).astype(np.uint8)
    return codes | ((q8 >> 7) << 3), magnitude


def sidecar_pack(q4: np.ndarray, s4: np.ndarray, q8: np.ndarray, s8: np.ndarray) -> np.ndarray:
    """The correction mask u8 [M, K/8] (bit i % 8 is value i): set where the direct FP4 code differs from the FP4 rounding
    of the shared FP8 code (reference.py:210-220). q4 [M, K/2] packed codes, q8 [M, K] E4M3 bytes, scales [M, K/32]."""
    candidate, _ = _mxfp4_via_shared_codes(s4, q8, s8)
    direct = np.stack((q4 & 15, q4 >> 4), axis=-1).reshape(q4.shape[0], -1)
    bits = (candidate != direct).reshape(q8.shape[0], -1, 8).astype(np.uint32)
    return (bits << np.arange(8, dtype=np.uint32)).sum(-1).astype(np.uint8)


def sidecar_unpack(mask: np.ndarray, s4: np.ndarray, q8: np.ndarray, s8: np.ndarray) -> np.ndarray:
    """The direct FP4 bytes [M, K/2] back from the mask (reference.py:223-235): a set bit takes the other neighbour of
    the candidate code, the lower one when the magnitude is a midpoint that rounds up (.75, 1.75, 3.5), else the upper."""
    candidate, magnitude = _mxfp4_via_shared_codes(s4, q8, s8)
    bits = ((mask[..., None].astype(np.int32) >> np.arange(8)) & 1).reshape(mask.shape[0], -1).astype(bool)
    down = (magnitude == 0.75) | (magnitude == 1.75) | (magnitude == 3.5)
    other = (candidate & 8) | (((candidate & 7).astype(np.int32) + np.where(down, -1, 1)) & 7).astype(np.uint8)
    codes = np.where(bits, other, candidate).astype(np.uint8)
    return np.ascontiguousarray(codes[:, ::2] | (codes[:, 1::2] << 4))


def make_shared_weights(seed: int = 607, hidden: int = H, inter: int = I):
    """Random MXFP8 shared-expert weights, the recipe of the reference's tests/moe/.../workload.py:48-61 with a CPU
    generator: E4M3 codes of 20*N(0,1), E8M0 bytes uniform in [118, 124)."""
    import torch
    g = torch.Generator().manual_seed(seed)

    def weight(n, k):
        q = f32_to_e4m3((torch.randn((n, k), generator=g) * 20).numpy())
        s = torch.randint(118, 124, (n, k // 32), dtype=torch.uint8, generator=g).numpy()
        return q, s

    return (*weight(2 * inter, hidden), *weight(hidden, inter))


# ----------------------------------------------------------------------------------------------- input recipes
def make_weights(seed: int = 0, experts: int = E, hidden: int = H, inter: int = I, scale_lo: int = 120,
                 scale_hi: int = 125):
    """The benchmark's synthetic checkpoint: E2M1 codes uniform over all 16 values, E8M0 bytes uniform in
    [scale_lo, scale_hi) (2**-7 .. 2**-3 by default), drawn from one CPU torch generator in the order w13, w13_scale, w2,
    w2_scale (the recipe of tests/moe/.../workload.py:25-35 with the benchmark's scale span). Returns numpy arrays and
    the generator for the draws that follow (activations, logits)."""
    import torch
    g = torch.Generator().manual_seed(seed)

    def rnd(lo, hi, shape):
        return torch.randint(lo, hi, shape, dtype=torch.uint8, generator=g).numpy()

    w13 = rnd(0, 256, (experts, 2 * inter, hidden // 2))
    s13 = rnd(scale_lo, scale_hi, (experts, 2 * inter, hidden // 32))
    w2 = rnd(0, 256, (experts, hidden, inter // 2))
    s2 = rnd(scale_lo, scale_hi, (experts, hidden, inter // 32))
    return (w13, s13, w2, s2), g


def make_inputs(gen, tokens: int, hidden: int = H, experts: int = E, pad_rows: int = 0):
    """x bf16 bits [T, hidden] ~ N(0,1) (the last ``pad_rows`` rows zero: CUDA-graph padding) and fp32 logits [T, experts]
    ~ N(0,1), drawn in that order from ``gen``."""
    import torch
    x = torch.randn((tokens, hidden), generator=gen).bfloat16()
    logits = torch.randn((tokens, experts), generator=gen)
    if pad_rows:
        x[tokens - pad_rows:] = 0
    return x.view(torch.int16).numpy().view(np.uint16).copy(), logits.numpy().copy()
