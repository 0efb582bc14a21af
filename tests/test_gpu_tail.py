"""GPU parity of the fused tail (slot sum + shared -> residual add -> Gemma RMSNorm -> MXFP8), through the C ABI.

Bit-exact: the slot sum and the residual out (against the reference-made golden and the numpy oracle). The norm output
and its MXFP8 form follow the tolerances of the reference's norm contract
(amd_kernels/norm/gemma_add_rmsnorm_h6144/reference.py: out within 1 bf16 ulp of the fp64 y and != bf16(y) at <= 1e-3 of the
elements, cosine >= 0.99999; scale bytes within 1 and different at <= 1e-3 of the groups; codes different from the fp64 y
requantised at the kernel's own scales at <= 1e-3 of the elements, never further than the neighbouring magnitude;
dequantised cosine >= 0.999)."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.conftest import golden
from tests.util import bf16_dev, bits_of

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import tail
    return tail


def check_norm(out_bits, codes, scales, y64):
    st = orc.compare_tail(out_bits, codes, scales, y64)
    assert st["bad_ulp"] == 0 and st["mismatch"] <= orc.TAIL_OUT_MISMATCH and st["cos"] >= orc.TAIL_OUT_COS, st
    assert st["scale_max_diff"] <= 1 and st["scale_mismatch"] <= orc.TAIL_SCALE_MISMATCH, st
    assert st["code_mismatch"] <= orc.TAIL_CODE_MISMATCH and st["code_far"] == 0 and st["mxfp8_cos"] >= orc.TAIL_MXFP8_COS, st


def test_tail_against_reference_golden(T):
    g = golden("tail.npz")
    slots, shared, resid, weight = (bf16_dev(g[k]) for k in ("slots", "shared", "residual", "weight"))
    r = T.slots4_add_rmsnorm_mxfp8(slots, shared, resid, weight, float(g["eps"]), bf16_out=True)
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(r.residual), g["residual_out"])
    check_norm(bits_of(r.normed), r.codes.cpu().numpy(), r.scales.cpu().numpy(), g["y64"])
    again = T.slots4_add_rmsnorm_mxfp8(slots, shared, resid, weight, float(g["eps"]), bf16_out=True)
    assert all(torch.equal(a, b) for a, b in zip((r.residual, r.codes, r.scales, r.normed),
                                                 (again.residual, again.codes, again.scales, again.normed)))


@pytest.mark.parametrize("tokens,with_shared", [(1, True), (37, False), (2048, True)])
def test_tail_against_the_oracle(T, tokens, with_shared):
    gen = torch.Generator().manual_seed(tokens)
    slots = (torch.randn((tokens, 4, 6144), generator=gen) * torch.exp2(torch.randint(-4, 3, (tokens, 4, 1), generator=gen).float())).bfloat16()
    shared = torch.randn((tokens, 6144), generator=gen).bfloat16() if with_shared else None
    resid = (torch.randn((tokens, 6144), generator=gen) * 3).bfloat16()
    weight = (torch.randn((6144,), generator=gen) * 0.2).bfloat16()
    r = T.slots4_add_rmsnorm_mxfp8(slots.cuda(), None if shared is None else shared.cuda(), resid.cuda(), weight.cuda(), 1e-6,
                                   bf16_out=True)
    b = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    x = orc.slots4_local(b(slots), None if shared is None else b(shared))
    y64, res = orc.add_rmsnorm(x, b(resid), b(weight), 1e-6)
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(r.residual), res)
    check_norm(bits_of(r.normed), r.codes.cpu().numpy(), r.scales.cpu().numpy(), y64)


def test_tail_equals_reduce_then_norm_on_the_layer_output(T):
    """Without the norm outputs the tail's residual equals bf16(reduce(slots, shared) + residual) built from the
    library's own slot reduce (whose sum starts from +0: equal here, no row sums to -0)."""
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain
    gen = torch.Generator().manual_seed(3)
    slots = torch.randn((64, 4, 6144), generator=gen).bfloat16().cuda()
    shared = torch.randn((64, 6144), generator=gen).bfloat16().cuda()
    resid = torch.randn((64, 6144), generator=gen).bfloat16().cuda()
    weight = torch.zeros(6144, dtype=torch.bfloat16).cuda()
    r = T.slots4_add_rmsnorm_mxfp8(slots, shared, resid, weight, mxfp8=False)
    x = chain.reduce_slots(slots, shared)
    assert r.codes is None and torch.equal(r.residual, (x.float() + resid.float()).bfloat16())
    with pytest.raises(ValueError):
        T.slots4_add_rmsnorm_mxfp8(slots, shared, resid[:8], weight)
