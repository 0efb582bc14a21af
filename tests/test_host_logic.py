"""CPU-only checks: the C-ABI library loads and exports what include/b200_moe.h declares, and the host-side mirror of
the reference interface validates its arguments the way the reference does."""
import ctypes
import os
import re

import pytest
import torch

from amd_kernels_b200 import _lib
from amd_kernels_b200.moe import mxfp4_h6144_i768_e128_top4 as P
from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain
from oracle import moe_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "b200_moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert len(names) >= 18
    for inter in (768, 1536):  # both builds of the sources: the i768 package's library and its i1536 sibling's
        lib = ctypes.CDLL(_lib.lib_path(inter))
        for name in names:
            assert hasattr(lib, name), (inter, name)
    assert set(_lib.SIGNATURES) == set(names), "the ctypes table and the header disagree"
    # the builds differ where the intermediate size enters: scratch for h (codes + scale atoms per sorted row)
    assert _lib.load(1536).b200moe_workspace_bytes(4096, 128) > _lib.load(768).b200moe_workspace_bytes(4096, 128)
    lib = _lib.load()
    assert lib.b200moe_arch() == b"sm_100a" and lib.b200moe_version() >= 1


def test_sizes_match_oracle_and_reference_bounds():
    lib = _lib.load()
    for tokens in (1, 2, 15, 16, 17, 300, 4097, 87381):
        for bm in (16, 32, 64, 128):
            assert lib.b200moe_max_sorted_rows(tokens, bm, 128) == orc.max_sorted_rows(tokens, bm)
        assert lib.b200moe_workspace_bytes(tokens, 128) > tokens * 3264
    assert [lib.b200moe_block_rows(t) for t in (1, 480, 481, 512, 513, 1024, 1729, 87381)] == [16, 16, 32, 32, 128, 128, 128, 128]
    assert lib.b200moe_workspace_bytes(0, 128) == 0 and lib.b200moe_workspace_bytes(87382, 128) == 0
    # the shared expert's dense blocks: the widest block the token count fills
    assert [lib.b200moe_shared_block_rows(t) for t in (1, 16, 17, 32, 33, 64, 65, 87381)] == [16, 16, 32, 32, 64, 64, 128, 128]
    assert lib.b200moe_shared_block_rows(0) == 0 and lib.b200moe_shared_workspace_bytes(0) == 0
    assert lib.b200moe_shared_workspace_bytes(100) >= 128 * (6144 + 768)
    assert lib.b200moe_permute_scratch_bytes(256, 128) == 0 and lib.b200moe_permute_scratch_bytes(257, 128) == 2 * 128 * 4


def test_dispatch_range():
    # the reference's variant_for: 1..87381, ValueError outside (tests/moe/.../test_entry.py:107-114)
    for m in (1, 8, 512, 513, 4097, 87381):
        assert chain.variant_for(m) in (16, 32, 64, 128)
    for m in (0, -1, 87382):
        with pytest.raises(ValueError):
            chain.variant_for(m)


def _weights(**override):
    m = dict(device="meta")
    w = dict(
        w13=torch.empty((P.E, 2 * P.I, P.H // 2), dtype=torch.uint8, **m),
        w13_scale=torch.empty((P.E, 2 * P.I, P.H // 32), dtype=torch.uint8, **m),
        w2=torch.empty((P.E, P.H, P.I // 2), dtype=torch.uint8, **m),
        w2_scale=torch.empty((P.E, P.H, P.I // 32), dtype=torch.uint8, **m),
        shared_w13=torch.empty((2 * P.I, P.H), dtype=torch.float8_e4m3fn, **m),
        shared_s13=torch.empty((2 * P.I, P.H // 32), dtype=torch.uint8, **m),
        shared_w2=torch.empty((P.H, P.I), dtype=torch.float8_e4m3fn, **m),
        shared_s2=torch.empty((P.H, P.I // 32), dtype=torch.uint8, **m),
    )
    w.update(override)
    return w


def test_unsupported_reason_like_the_reference():
    # tests/moe/.../test_unsupported_reason.py:29-37
    assert P.unsupported_reason(**_weights()) is None
    assert "w2:" in P.unsupported_reason(**_weights(w2=torch.empty((P.E, P.H, P.I), dtype=torch.uint8, device="meta")))
    bf16 = torch.empty((2 * P.I, P.H), dtype=torch.bfloat16, device="meta")
    assert "shared w13:" in P.unsupported_reason(**_weights(shared_w13=bf16))
    assert "SwiGLU" in P.unsupported_reason(**_weights(), swiglu=(1.0, 7.0, 1.0))
    assert "w13:" in P.unsupported_reason(**_weights(w13=None))
    assert P.SWIGLU_OAI == (1.702, 7.0, 1.0) and (P.H, P.I, P.E, P.TOPK) == (6144, 768, 128, 4)


def test_entry_rejects_bad_inputs_without_a_gpu():
    w = object()
    with pytest.raises(ValueError):
        P.mxfp4_moe(torch.zeros((0, 6144), dtype=torch.bfloat16), w)
    with pytest.raises(ValueError):
        P.mxfp4_moe(torch.zeros((4, 6144), dtype=torch.float32), w)
    with pytest.raises(ValueError):
        P.mxfp4_moe(torch.zeros((4, 6000), dtype=torch.bfloat16), w)
    with pytest.raises(ValueError):
        P.mxfp4_moe(torch.zeros((8, 6144), dtype=torch.bfloat16)[::2], w)
    with pytest.raises(ValueError):
        P.MoeWeights.from_row_major(None, None, *(_weights()[k] for k in ("w13", "w13_scale", "w2")), None)


def test_c_abi_rejects_null_and_bad_sizes():
    lib = _lib.load()
    assert lib.b200moe_quant_mxfp4(None, 4, 6144, None, None, None) == _lib.E_ARG
    assert lib.b200moe_permute(None, None, 4, 128, 16, None, None, None, None, None, None) == _lib.E_ARG
    assert lib.b200moe_reduce_slots(None, None, 4, None, None) == _lib.E_ARG
    one = ctypes.c_void_p(16)
    assert lib.b200moe_permute(one, one, 4, 128, 24, one, one, one, one, one, None) == _lib.E_ARG  # bm not 16/32/64/128
    assert lib.b200moe_permute(one, one, 87382, 128, 16, one, one, one, one, one, None) == _lib.E_ARG
    assert lib.b200moe_quant_mxfp4(ctypes.c_void_p(8), 4, 6144, one, one, None) == _lib.E_ALIGN
    with pytest.raises(ValueError):
        _lib.check(_lib.E_ARG, "x")
    with pytest.raises(RuntimeError):
        _lib.check(700, "x")
