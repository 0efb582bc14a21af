"""GPU parity tests of the prepared (sequence-parallel) input and its compact form, through the C ABI.

Everything here is bit-exact: the correction mask against the reference's golden mask and the CPU oracle, the FP4 codes
rebuilt from it, the payloads of ``prepare_mxfp4_moe`` against the single kernels, and ``mxfp4_moe`` on a prepared or a
compact input against ``mxfp4_moe`` on the bf16 rows.
"""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.conftest import golden
from tests.util import H, bf16_dev, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def P():
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import prepared_input
    return prepared_input


@pytest.fixture(scope="module")
def full_layer(config0):
    """Configuration 0's routed weights, a router gate, a bias and the shared expert: the reference's full entry."""
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain as C, shared_expert as S
    raw, _, _ = config0
    sw = S.SharedWeights.from_row_major(*(dev(a) for a in orc.make_shared_weights()))
    g = torch.Generator().manual_seed(12)
    gate = (torch.randn((128, H), generator=g) * 0.02).cuda()
    bias = (torch.randn((128,), generator=g) * 0.1).cuda()
    w = C.MoeWeights.from_row_major(gate, bias, *(dev(a) for a in raw), shared=sw)
    return C, S, w


def rows(m, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn((m, H), generator=g) * torch.exp2(torch.randint(-3, 4, (m, H // 32), generator=g).float()
                                                           ).repeat_interleave(32, 1)).bfloat16()


def test_sidecar_kernels_match_golden_and_oracle(P):
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain as C, shared_expert as S
    g = golden("sidecar.npz")
    x = bf16_dev(g["x_bits"])
    q4, s4 = C.mxfp4_quant(x)
    q8, s8 = S.shared_quant_rows(x)
    for got, want in ((q4, "q4"), (s4, "s4"), (q8, "q8"), (s8, "s8")):
        assert (got.cpu().numpy() == g[want]).all(), want
    n = x.shape[0]
    inp = P.MoeInput(q4, s4, torch.zeros((n, 4), device="cuda"), torch.zeros((n, 4), dtype=torch.int32, device="cuda"), q8, s8)
    compact = inp.compact()
    assert (compact.correction_mask.cpu().numpy() == g["mask"]).all()
    assert torch.equal(compact.expand().routed_codes, q4)
    # more rows, against the oracle
    xr = rows(70, 3)
    q4, s4 = C.mxfp4_quant(xr.cuda())
    q8, s8 = S.shared_quant_rows(xr.cuda())
    inp = P.MoeInput(q4, s4, torch.zeros((70, 4), device="cuda"), torch.zeros((70, 4), dtype=torch.int32, device="cuda"), q8, s8)
    compact = inp.compact()
    want = orc.sidecar_pack(q4.cpu().numpy(), s4.cpu().numpy(), q8.cpu().numpy(), s8.cpu().numpy())
    assert (compact.correction_mask.cpu().numpy() == want).all()
    assert torch.equal(compact.expand().routed_codes, q4)


@pytest.mark.parametrize("m", [1, 5, 48, 300, 1600])
def test_prepared_and_compact_inputs_give_the_entry_bits(P, full_layer, m):
    C, S, w = full_layer
    x = rows(m, 20 + m).cuda()
    inp = P.prepare_mxfp4_moe(x, w)
    q, s = C.mxfp4_quant(x)
    wt, ids = C.route(x, w)
    q8, s8 = S.shared_quant_rows(x)
    for got, want in zip(inp.tensors(), (q, s, wt, ids, q8, s8)):
        assert torch.equal(got, want)
    assert torch.equal(S.shared_expert(None, w.shared_weights, x_quant=(q8, s8)), S.shared_expert(x, w.shared_weights))
    out = C.mxfp4_moe(x, w)
    slots, shared = C.mxfp4_moe(x, w, return_partials=True)
    assert torch.equal(C.mxfp4_moe(inp, w), out)
    p_slots, p_shared = C.mxfp4_moe(inp, w, return_partials=True)
    assert torch.equal(p_slots, slots) and torch.equal(p_shared, shared)
    compact = inp.compact()
    assert sum(t.numel() * t.element_size() for t in compact.tensors()) == m * 7328
    assert torch.equal(C.mxfp4_moe(compact, w), out)
    assert C.last_status() == 0


def test_gather_on_one_rank_and_argument_errors(P, full_layer):
    from tests.test_gpu_moe import _single_rank_group
    C, S, w = full_layer
    dist = _single_rank_group()
    x = rows(32, 9).cuda()
    inp = P.prepare_mxfp4_moe(x, w)
    gathered = P.gather_mxfp4_moe(inp, dist.group.WORLD)
    assert isinstance(gathered, P.MoeInputCompact)
    assert torch.equal(C.mxfp4_moe(gathered, w), C.mxfp4_moe(x, w))
    with pytest.raises(ValueError):
        P.gather_mxfp4_moe(x, dist.group.WORLD)
    with pytest.raises(ValueError):
        P.MoeInput(inp.routed_codes, inp.routed_scales, inp.topk_weights, inp.topk_ids).compact()
    with pytest.raises(ValueError):
        P.prepare_mxfp4_moe(x.float(), w)
    with pytest.raises(ValueError):
        C.mxfp4_moe(P.MoeInput(inp.routed_codes[:, :100].contiguous(), inp.routed_scales, inp.topk_weights, inp.topk_ids,
                               inp.shared_codes, inp.shared_scales), w)
    with pytest.raises(ValueError):
        C.mxfp4_moe([1, 2, 3], w)
    routed_only = C.MoeWeights(None, None, w.w13, None, w.w2, None)
    with pytest.raises(ValueError):
        P.prepare_mxfp4_moe(x, routed_only)


@pytest.mark.parametrize("m", [1, 17, 300, 2100])
def test_router_gemm_fused_with_the_quantisers(full_layer, m):
    """One pass over x gives the router GEMM's partials and both quantisers' payloads, bit for bit."""
    C, S, w = full_layer
    x = rows(m, 60 + m).cuda()
    parts, (q4, s4), (q8, s8) = C.router_gemm_quant(x, w.router_weight, shared=True)
    assert torch.equal(parts, C.router_gemm_partials(x, w.router_weight))
    want4, want8 = C.mxfp4_quant(x), S.shared_quant_rows(x)
    assert torch.equal(q4, want4[0]) and torch.equal(s4, want4[1])
    assert torch.equal(q8, want8[0]) and torch.equal(s8, want8[1])
    _, _, (n8, ns8) = C.router_gemm_quant(x, w.router_weight)
    assert n8 is None and ns8 is None
