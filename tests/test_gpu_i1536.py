"""The TP2 sibling shape (intermediate 1536; reference package amd_kernels/moe/mxfp4_h6144_i1536_e128_top4, same entry as the
i768 package): the same kernels built with the other intermediate size, checked the same way -- tensor-core GEMMs against
the CUDA-core cross-check kernels, the entry against the CPU oracle (same tolerances as tests/test_gpu_moe.py), the
router-inside call, the shared expert, bit-equal reruns."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.test_gpu_moe import check_against_oracle
from tests.util import H, atoms_to_rowmajor, bf16_dev, bits_of, dev, make_routing, oracle_slots

pytestmark = pytest.mark.gpu
I2, EXPERTS = 1536, 8  # noqa: E741


@pytest.fixture(scope="module")
def P():
    import amd_kernels_b200.moe.mxfp4_h6144_i1536_e128_top4 as pkg
    return pkg


@pytest.fixture(scope="module")
def C():
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain
    return chain


@pytest.fixture(scope="module")
def sibling(P):
    raw, gen = orc.make_weights(seed=15, experts=EXPERTS, inter=I2)
    gate = torch.randn((EXPERTS, H), generator=gen) / H ** 0.5
    w = P.MoeWeights.from_row_major(gate.cuda(), None, *(dev(a) for a in raw), routing_mode="softmax",
                                    routed_scaling_factor=1.0, keep_row_major=True)
    return raw, w, gate


def test_shape_contract(P, C, sibling):
    raw, w, _ = sibling
    assert P.I == I2 and w.intermediate == I2 and tuple(w.w13.shape[1:]) == (24, 24, 17408) and tuple(w.w2.shape[1:]) == (48, 6, 17408)
    t = [dev(a) for a in raw]
    assert P.unsupported_reason(*t, None, None, None, None, routed_only=True) is None
    small, _ = orc.make_weights(seed=1, experts=2)  # the i768 shape is not this package's
    with pytest.raises(ValueError):
        P.MoeWeights.from_row_major(None, None, *(dev(a) for a in small))
    with pytest.raises(ValueError):
        C.MoeWeights.from_row_major(None, None, *t)


@pytest.mark.parametrize("tokens,bm", [(3, 16), (40, 32), (100, 64), (300, 128), (900, 128)])
def test_tensor_core_gemms_equal_cuda_core_gemms(C, sibling, tokens, bm):
    raw, w, _ = sibling
    gen = torch.Generator().manual_seed(tokens)
    xb, _ = orc.make_inputs(gen, tokens, experts=EXPERTS)
    ids, wts = make_routing(tokens, "uniform", seed=tokens, experts=EXPERTS)
    xq = C.mxfp4_quant(bf16_dev(xb))
    sb = C.moe_sort(dev(ids), dev(wts), bm, EXPERTS)
    xs, sfx = C.dispatch_rows(xq, sb)
    hq, sfh = C.grouped_gemm1(xs, sfx, sb, w)
    slots = C.grouped_gemm2(hq, sfh, sb, w, slots=torch.zeros((tokens, 4, H), dtype=torch.bfloat16, device="cuda"))
    hq_r, sfh_r = C.simt_gemm1(xq, sb, w)
    slots_r = C.simt_gemm2(hq_r, sfh_r, sb, w)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    nv = int(sb.num_valid[0])
    live = ((sb.sorted_ids[:nv] & 0xFFFFFF) < tokens).cpu().numpy()
    a, b = hq[:nv].cpu().numpy()[live], hq_r[:nv].cpu().numpy()[live]
    assert a.shape[1] == I2 // 2 and (a != b).mean() < 1e-4
    sa, sr = (atoms_to_rowmajor(t.cpu().numpy(), bm)[:nv][live] for t in (sfh, sfh_r))
    assert (sa != sr).mean() < 1e-4
    check_against_oracle(slots.float().cpu().numpy().sum(1), slots_r.float().cpu().numpy().sum(1))
    # and against the CPU oracle directly, so the two GPU paths cannot be wrong together
    pick = np.unique(np.linspace(0, tokens - 1, 4).astype(int))
    xq_np, xs_np = orc.quant_mxfp4(orc.bf16_to_f32(xb))
    check_against_oracle(slots.float().cpu().numpy()[pick].sum(1), oracle_slots(xq_np, xs_np, raw, ids, wts, tokens=pick).sum(1))
    if bm == 128 and C._lib.load(I2).b200moe_gemm1_pair_supported():
        p_h, p_s = C.grouped_gemm1_pair(xs, sfx, sb, w)
        torch.cuda.synchronize()
        assert torch.equal(p_h[:nv][torch.from_numpy(live).cuda()], hq[:nv][torch.from_numpy(live).cuda()]) and C.last_status() == 0
    if bm < 128:
        one, _, _ = C.grouped_gemm12(xs, sfx, sb, w)
        torch.cuda.synchronize()
        assert torch.equal(one, slots) and C.last_status() == 0


@pytest.mark.parametrize("tokens", [1, 16, 200, 2048])
def test_entry_against_the_oracle(P, C, sibling, tokens):
    raw, w, gate = sibling
    gen = torch.Generator().manual_seed(50 + tokens)
    xb, lg = orc.make_inputs(gen, tokens, experts=EXPERTS)
    x, logits = bf16_dev(xb), dev(lg)
    out = P.mxfp4_moe(x, w, router_logits=logits)
    slots, _ = P.mxfp4_moe(x, w, router_logits=logits, return_partials=True)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    pick = np.unique(np.linspace(0, tokens - 1, 8).astype(int))
    ref = orc.moe_layer(xb[pick], lg[pick], *raw)
    check_against_oracle(out.float().cpu().numpy()[pick], orc.bf16_to_f32(ref["out"]))
    assert np.array_equal(bits_of(out), orc.reduce_slots_bf16(bits_of(slots)))
    assert torch.equal(out, P.mxfp4_moe(x, w, router_logits=logits))
    # the router inside the call: same slots as the staged kernels on the entry's own routing
    x_only, _ = P.mxfp4_moe(x, w, return_partials=True)
    wt, ids = P.route(x, w)
    assert torch.equal(x_only, P.mxfp4_moe_experts(C.mxfp4_quant(x), wt, ids, w))
    got = oracle_slots(ref["xq"], ref["xs"], raw, ids.cpu().numpy()[pick], wt.cpu().numpy()[pick])
    check_against_oracle(x_only.float().cpu().numpy()[pick].sum(1), got.sum(1))
    torch.cuda.synchronize()
    assert C.last_status() == 0


@pytest.mark.parametrize("tokens", [5, 300])
def test_shared_expert_of_the_sibling_shape(P, C, tokens):
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import shared_expert as S
    sw_np = orc.make_shared_weights(seed=611, inter=I2)
    sw = P.SharedWeights.from_row_major(*(dev(a) for a in sw_np))
    assert sw.intermediate == I2
    gen = torch.Generator().manual_seed(tokens)
    x = (torch.randn((tokens, H), generator=gen) * 0.5).bfloat16()
    out = S.shared_expert(x.cuda(), sw)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    ref = orc.shared_mxfp8(x.float().numpy(), *sw_np)
    got = out.float().cpu().numpy()
    cos = (got * ref).sum(1) / np.linalg.norm(got, axis=1) / np.linalg.norm(ref, axis=1)
    assert cos.min() >= 0.9999 and np.linalg.norm(got - ref) / np.linalg.norm(ref) < 4e-3
