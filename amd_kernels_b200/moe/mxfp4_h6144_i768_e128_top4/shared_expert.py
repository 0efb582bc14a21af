"""The MXFP8 shared expert on B200: the host side, mirroring the reference's
``amd_kernels/moe/mxfp4_h6144_i768_e128_top4/shared_expert.py`` (``SharedWeights``, ``shared_quant``, ``shared_expert``,
``shared_expert_parallel``), on top of the C ABI of libb200moe.so. A dense SwiGLU-OAI MLP on every token: E4M3 codes with
one E8M0 scale per 32 elements for the weights, the input and the SwiGLU output, fp32 accumulation in tensor memory.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from ... import _lib

H, I = 6144, 768  # noqa: E741
RECORD_BYTES = 17408

_side_streams: dict = {}

# Inside a dual-batch-overlap microbatch the shared expert stays on the caller's stream (the server already overlaps one
# microbatch's compute with the other's collectives). A server hands over its query with ``set_dbo_query``; without one
# the module constant ``DBO`` answers (reference shared_expert.py:30-44).
DBO = False
_dbo_query = None


def set_dbo_query(query) -> None:
    """``query()`` tells whether the current call runs inside a DBO microbatch; ``None`` goes back to ``DBO``."""
    global _dbo_query
    _dbo_query = query


def in_dbo() -> bool:
    return bool(_dbo_query()) if _dbo_query is not None else DBO


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def side_stream(device) -> torch.cuda.Stream:
    """The device's side stream for the shared expert, one per device (reference shared_expert.py ``side_stream``)."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=key)
    return _side_streams[key]


@dataclass
class SharedWeights:
    """The shared expert's MXFP8 weights in the kernels' layout, and the device's side stream (reference
    shared_expert.py:48-67). ``w13`` [12, 48, 17408] u8 and ``w2`` [48, 6, 17408] u8 are tile records: 128 rows x 128
    K-elements of E4M3 codes in the 128-byte-swizzled shared-memory image, then the tile's scale atom; the scales travel
    inside the records, so ``s13`` / ``s2`` stay None."""
    w13: torch.Tensor
    s13: torch.Tensor | None
    w2: torch.Tensor
    s2: torch.Tensor | None
    stream: object
    INTERMEDIATE = I  # the i1536 sibling package pins 1536

    @property
    def intermediate(self) -> int:
        return self.w13.shape[0] * 64

    @classmethod
    def from_row_major(cls, w13, s13, w2, s2):
        """From row-major e4m3 [N, K] weights and e8m0 [N, K / 32] scales (gate rows, then up rows in ``w13``)."""
        I = cls.INTERMEDIATE  # noqa: E741,N806
        if tuple(w13.shape) != (2 * I, H) or tuple(w2.shape) != (H, I):
            raise ValueError(f"shared weights: needs [{2 * I}, {H}] and [{H}, {I}]")
        if tuple(s13.shape) != (2 * I, H // 32) or tuple(s2.shape) != (H, I // 32):
            raise ValueError(f"shared scales: needs [{2 * I}, {H // 32}] and [{H}, {I // 32}]")
        if not w13.is_cuda:
            raise ValueError("weights must be CUDA tensors")
        if w13.element_size() != 1 or w2.element_size() != 1 or s13.element_size() != 1 or s2.element_size() != 1:
            raise ValueError("shared weights and scales must be 1-byte types (e4m3 codes, e8m0 scales)")
        dev = w13.device
        c13, b13, c2, b2 = (t.contiguous().view(torch.uint8) for t in (w13, s13, w2, s2))
        w13t = torch.empty((2 * I // 128, 48, RECORD_BYTES), dtype=torch.uint8, device=dev)
        w2t = torch.empty((48, I // 128, RECORD_BYTES), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            st = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
            _lib.check(_lib.load(I).b200moe_preshuffle_shared(_ptr(c13), _ptr(b13), _ptr(c2), _ptr(b2), _ptr(w13t),
                                                             _ptr(w2t), st), "preshuffle_shared")
        return cls(w13t, None, w2t, None, side_stream(dev))


def _check_x(x):
    if x.ndim != 2 or x.shape[1] != H or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.shape[0] < 1:
        raise ValueError("expected contiguous BF16 [M,6144], M >= 1")


def shared_quant(x: torch.Tensor, bm: int | None = None, *, stream=None):
    """bf16 [M, 6144] -> (E4M3 codes u8 [ceil(M/bm)*bm, 6144], scale atoms u8 [ceil(M/bm), 48, 512]), the layout the
    first GEMM loads (reference shared_expert.py ``shared_quant``; rule: reference.py:162-171). ``atoms_to_rows`` turns
    the atoms back into [M, 192]."""
    _check_x(x)
    lib = _lib.load()
    m = x.shape[0]
    bm = int(lib.b200moe_shared_block_rows(m)) if bm is None else bm
    rows = (m + bm - 1) // bm * bm
    codes = torch.empty((rows, H), dtype=torch.uint8, device=x.device)
    atoms = torch.empty((rows // bm, H // 128, 512), dtype=torch.uint8, device=x.device)
    st = torch.cuda.current_stream(x.device) if stream is None else stream
    _lib.check(lib.b200moe_shared_quant(_ptr(x), m, bm, _ptr(codes), _ptr(atoms), ctypes.c_void_p(st.cuda_stream)),
               "shared_quant")
    return codes, atoms


def shared_quant_rows(x: torch.Tensor, *, stream=None):
    """bf16 [M, 6144] -> (E4M3 codes u8 [M, 6144], E8M0 scales u8 [M, 192]) row-major: the prepared-input payload
    (reference prepared_input.py:16-36); same bits as ``shared_quant``."""
    _check_x(x)
    m = x.shape[0]
    codes = torch.empty((m, H), dtype=torch.uint8, device=x.device)
    scales = torch.empty((m, H // 32), dtype=torch.uint8, device=x.device)
    st = torch.cuda.current_stream(x.device) if stream is None else stream
    _lib.check(_lib.load().b200moe_shared_quant_rows(_ptr(x), m, _ptr(codes), _ptr(scales),
                                                     ctypes.c_void_p(st.cuda_stream)), "shared_quant_rows")
    return codes, scales


def atoms_to_rows(atoms: torch.Tensor, bm: int, m: int) -> torch.Tensor:
    """Scale atoms [B, A, 512] of ``bm``-row blocks -> row-major scales [m, 4*A] (an index permutation, for checks)."""
    b, a, _ = atoms.shape
    r = torch.arange(bm, device=atoms.device)
    base = (r % 32) * 16 + (r // 32) * 4
    idx = base[:, None] + torch.arange(4, device=atoms.device)[None, :]  # [bm, 4]
    rows = atoms[:, :, idx.reshape(-1)].reshape(b, a, bm, 4).permute(0, 2, 1, 3).reshape(b * bm, a * 4)
    return rows[:m].contiguous()


def shared_expert(x: torch.Tensor | None, w: SharedWeights, *, x_quant=None, stream=None) -> torch.Tensor:
    """The shared expert of bf16 ``x`` [n, 6144] -> bf16 [n, 6144] (reference shared_expert.py:70-84; served at every n
    here). ``x_quant``: ``shared_quant_rows(x)``'s (codes, scales) if already computed (then ``x`` is not read).
    ``stream``: launch there instead of on the current stream; the buffers still come from the current stream's
    allocator pool and are recorded on ``stream``."""
    from .chain import status_word, variant_for
    lib = _lib.load(w.intermediate)
    if x_quant is None:
        _check_x(x)
        n, dev = x.shape[0], x.device
    else:
        q, s = x_quant
        n, dev = q.shape[0], q.device
        if (q.shape != (n, H) or q.dtype != torch.uint8 or not q.is_contiguous() or s.shape != (n, H // 32)
                or s.dtype != torch.uint8 or not s.is_contiguous()):
            raise ValueError("x_quant: expected contiguous uint8 codes [M,6144] and scales [M,192]")
    variant_for(n)
    ws_bytes = int(lib.b200moe_shared_workspace_bytes(n))
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    out = torch.empty((n, H), dtype=torch.bfloat16, device=dev)
    st = torch.cuda.current_stream(dev) if stream is None else stream
    if x_quant is None:
        _lib.check(lib.b200moe_shared_expert(_ptr(w.w13), _ptr(w.w2), _ptr(x), n, _ptr(workspace), ws_bytes, _ptr(out),
                                             _ptr(status_word(dev)), ctypes.c_void_p(st.cuda_stream)), "shared_expert")
        used = (workspace, out, x)
    else:
        _lib.check(lib.b200moe_shared_expert_quantized(_ptr(w.w13), _ptr(w.w2), _ptr(q), _ptr(s), n, _ptr(workspace),
                                                       ws_bytes, _ptr(out), _ptr(status_word(dev)),
                                                       ctypes.c_void_p(st.cuda_stream)), "shared_expert_quantized")
        used = (workspace, out, q, s)
    if stream is not None and stream != torch.cuda.current_stream(dev):
        for t in used:
            t.record_stream(stream)
    return out


def shared_expert_parallel(x, w: SharedWeights, current, **kwargs):
    """``shared_expert`` on ``w.stream`` (the device's side stream) after the work queued on ``current`` so far
    (reference shared_expert.py:94-101). The caller makes ``current`` wait for ``w.stream`` before reading the result."""
    if in_dbo():  # a DBO microbatch: no side stream (``current.wait_stream(w.stream)`` afterwards is then a no-op)
        return shared_expert(x, w, stream=current, **kwargs)
    w.stream.wait_stream(current)
    return shared_expert(x, w, stream=w.stream, **kwargs)
