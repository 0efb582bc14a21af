"""GPU parity tests of the grouped GEMMs and the whole entry, through the C ABI.

Tolerances (the reference's, its tests/moe/.../test_entry.py:45-58,131-141 and reference.py:78-83): slot sums against
the fp32 oracle on the same MXFP4 operands: cosine >= 0.9999 over the output, relative L2 < 4e-3, and max-abs error
below MAX_ABS (stated here: 2% of the output's largest magnitude). Bit-exact: routing ids, the permutation, h codes and
scales against the CUDA-core cross-check, repeated calls, CUDA-graph replays, and one token's slots whatever the batch.
"""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.conftest import golden
from tests.util import (H, atoms_to_rowmajor, bf16_dev, bits_of, cosine, dev, make_routing, oracle_slots, rel_l2)

pytestmark = pytest.mark.gpu
COS_MIN, REL_L2_MAX, MAX_ABS_FRACTION = 0.9999, 4e-3, 0.02


@pytest.fixture(scope="module")
def C():
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain
    return chain


@pytest.fixture(scope="module")
def layer(C, config0):
    """Configuration 0's weights on the GPU in both layouts, softmax routing (scale 1)."""
    raw, xb, lg = config0
    w = C.MoeWeights.from_row_major(None, None, *(dev(a) for a in raw), routing_mode="softmax",
                                    routed_scaling_factor=1.0, keep_row_major=True)
    return raw, w, xb, lg


def check_against_oracle(got, ref):
    assert np.isfinite(got).all()
    assert cosine(got, ref) >= COS_MIN, cosine(got, ref)
    assert rel_l2(got, ref) < REL_L2_MAX, rel_l2(got, ref)
    assert np.abs(got - ref).max() <= MAX_ABS_FRACTION * np.abs(ref).max(), np.abs(got - ref).max()


def run_stages(C, w, xq, ids, wts, bm, tc=True, rows=None):
    sb = C.moe_sort(ids, wts, bm, w.num_experts)
    if tc:
        hq, sfh = C.grouped_gemm1(*C.dispatch_rows(xq, sb), sb, w)
        slots = C.grouped_gemm2(hq, sfh, sb, w, slots=torch.zeros((sb.tokens, 4, H), dtype=torch.bfloat16, device="cuda"))
    else:
        hq, sfh = C.simt_gemm1(xq, sb, w, rows)
        slots = C.simt_gemm2(hq, sfh, sb, w, rows)
    return sb, hq, sfh, slots


@pytest.mark.parametrize("tokens,bm", [(1, 16), (16, 16), (40, 32), (100, 64), (200, 128), (300, 16)])
@pytest.mark.parametrize("kind", ["uniform", "one", "dup"])
def test_tensor_core_gemms_equal_cuda_core_gemms(C, tokens, bm, kind):
    """4 experts, every block height, against the CUDA-core kernels. Both accumulate exact products in fp32 but in a
    different order, so an h value that lands next to a rounding boundary may take the neighbouring code: fewer than
    1e-4 of the h codes and scale bytes may differ; where none differs the bf16 slots are equal bit for bit, and the
    slot sums always meet the oracle tolerances."""
    (w13, s13, w2, s2), gen = orc.make_weights(seed=tokens, experts=4)
    xb, _ = orc.make_inputs(gen, tokens, experts=4)
    w = C.MoeWeights.from_row_major(None, None, dev(w13), dev(s13), dev(w2), dev(s2), keep_row_major=True)
    ids, wts = make_routing(tokens, kind, seed=tokens, experts=4)
    xq = C.mxfp4_quant(bf16_dev(xb))
    sb, hq, sfh, slots = run_stages(C, w, xq, dev(ids), dev(wts), bm)
    _, hq_r, sfh_r, slots_r = run_stages(C, w, xq, dev(ids), dev(wts), bm, tc=False)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    nv = int(sb.num_valid[0])
    live = ((sb.sorted_ids[:nv] & 0xFFFFFF) < tokens).cpu().numpy()
    a, b = hq[:nv].cpu().numpy()[live], hq_r[:nv].cpu().numpy()[live]
    assert (a != b).mean() < 1e-4
    sa, sr = (atoms_to_rowmajor(t.cpu().numpy(), bm)[:nv][live] for t in (sfh, sfh_r))
    assert (sa != sr).mean() < 1e-4
    if np.array_equal(a, b):
        assert torch.equal(slots, slots_r)
    check_against_oracle(slots.float().cpu().numpy().sum(1), slots_r.float().cpu().numpy().sum(1))


@pytest.mark.parametrize("tokens,kind", [(300, "uniform"), (2048, "uniform"), (3000, "hot"), (700, "one"), (5, "dup")])
def test_cta_pair_gemm1_equals_single_cta_gemm1(C, layer, tokens, kind):
    """GEMM1 on CTA pairs (tcgen05.mma.cta_group::2, two row blocks of an expert x two W13 tiles per unit, odd last blocks
    alone) and GEMM1 with 256 weight rows per MMA on one CTA write the h codes and scales of the 128 x 128 kernel bit for bit: experts with one, an even and an odd number of
    128-row blocks, and one expert holding every row."""
    from amd_kernels_b200 import _lib
    if not _lib.load().b200moe_gemm1_pair_supported():
        pytest.skip("the device cannot launch CTA pairs")
    raw, w, _, _ = layer
    gen = torch.Generator().manual_seed(31 + tokens)
    xb, _ = orc.make_inputs(gen, tokens)
    ids, wts = make_routing(tokens, kind, seed=tokens)
    sb = C.moe_sort(dev(ids), dev(wts), 128, w.num_experts)
    xq, sfx = C.quant_dispatch(bf16_dev(xb), sb)
    a_h, a_s = C.grouped_gemm1(xq, sfx, sb, w)
    b_h, b_s = C.grouped_gemm1_pair(xq, sfx, sb, w)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    nv = int(sb.num_valid[0])
    live = ((sb.sorted_ids[:nv] & 0xFFFFFF) < tokens)
    assert torch.equal(a_h[:nv][live], b_h[:nv][live])
    sa, sp = (atoms_to_rowmajor(t.cpu().numpy(), 128)[:nv][live.cpu().numpy()] for t in (a_s, b_s))
    assert np.array_equal(sa, sp)
    assert torch.equal(b_h[:nv], C.grouped_gemm1_pair(xq, sfx, sb, w)[0][:nv])
    # the same 256-column unit on one CTA (128 token rows x 256 weight rows per MMA)
    c_h, c_s = C.grouped_gemm1_wide(xq, sfx, sb, w)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    assert torch.equal(a_h[:nv][live], c_h[:nv][live])
    assert np.array_equal(sa, atoms_to_rowmajor(c_s.cpu().numpy(), 128)[:nv][live.cpu().numpy()])
    # the same kernel gathering its rows from the unsorted row-major quantised tokens (no sorted copy of the activations)
    q, s = C.mxfp4_quant(bf16_dev(xb))
    d_h, d_s = C.grouped_gemm1_gather(q, s, sb, w)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    assert torch.equal(a_h[:nv][live], d_h[:nv][live])
    assert np.array_equal(sa, atoms_to_rowmajor(d_s.cpu().numpy(), 128)[:nv][live.cpu().numpy()])
    assert torch.equal(d_h[:nv], C.grouped_gemm1_gather(q, s, sb, w)[0][:nv])
    # one input row per (token, slot) pair (rows that arrived from other ranks): row 4 * token + slot, all different
    pick = (torch.arange(4 * tokens, device="cuda") * 7 + 3) % tokens
    qp, sp_ = q[pick].contiguous(), s[pick].contiguous()
    e_h, e_s = C.grouped_gemm1(*C.dispatch_rows((qp, sp_), sb, by_pair=True), sb, w)
    f_h, f_s = C.grouped_gemm1_gather(qp, sp_, sb, w, by_pair=True)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    assert torch.equal(e_h[:nv][live], f_h[:nv][live])
    assert np.array_equal(atoms_to_rowmajor(e_s.cpu().numpy(), 128)[:nv][live.cpu().numpy()],
                          atoms_to_rowmajor(f_s.cpu().numpy(), 128)[:nv][live.cpu().numpy()])


@pytest.mark.parametrize("tokens,chunks", [(2048, 4), (3000, 3), (700, 5)])
def test_grouped_gemms_by_block_ranges_equal_one_launch(C, layer, tokens, chunks):
    """The gathering GEMM1 and the peer-storing GEMM2 restricted to runs of row blocks (device-side ranges from
    ``block_chunks``), on capped grids, one run after the other: the same bits as one launch over all blocks."""
    import ctypes
    raw, w, _, _ = layer
    gen = torch.Generator().manual_seed(91 + tokens)
    xb, _ = orc.make_inputs(gen, tokens)
    ids, wts = make_routing(tokens, "uniform" if tokens != 700 else "hot", seed=tokens)
    sb = C.moe_sort(dev(ids), dev(wts), 128, w.num_experts)
    q, s = C.mxfp4_quant(bf16_dev(xb))
    nv = int(sb.num_valid[0])
    ranges = C.block_chunks(sb, chunks)
    r = ranges.cpu().numpy()
    assert r[0, 0] == 0 and r[-1, 1] == nv // 128 and (r[1:, 0] == r[:-1, 1]).all() and (r[:, 1] >= r[:, 0]).all()
    full_h, full_s = C.grouped_gemm1_gather(q, s, sb, w)
    out = None
    for c in range(chunks):
        out = C.grouped_gemm1_gather(q, s, sb, w, block_range=ranges[c], max_ctas=0 if c == 0 else 84, out=out)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    assert torch.equal(out[0][:nv], full_h[:nv]) and torch.equal(out[1][:nv // 128], full_s[:nv // 128])
    want = C.grouped_gemm2(full_h, full_s, sb, w)
    got = torch.zeros_like(want)
    pairs = tokens * 4
    rank0 = torch.zeros(pairs, dtype=torch.int32, device="cuda")
    ident = torch.arange(pairs, dtype=torch.int32, device="cuda")
    one = (ctypes.c_void_p * 1)(got.data_ptr())
    for c in range(chunks):
        C.grouped_gemm2_peer(full_h, full_s, sb, w, rank0, ident, one, 1, pairs, block_range=ranges[c], max_ctas=64)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    assert torch.equal(got, want)


def test_config0_against_reference_golden(C, layer):
    """Configuration 0 (T=16) end to end against the output of the reference's own w4a4_moe_ref."""
    raw, w, xb, lg = layer
    g = golden("moe_config0.npz")
    x, logits = bf16_dev(xb), dev(lg)
    wt, ids = C.route(x, w, router_logits=logits)
    assert np.array_equal(ids.cpu().numpy(), g["ids_softmax"])
    np.testing.assert_allclose(wt.cpu().numpy(), g["weights_softmax"], rtol=orc.WEIGHT_RTOL)
    q, s = C.mxfp4_quant(x)
    assert np.array_equal(q.cpu().numpy(), g["xq"]) and np.array_equal(s.cpu().numpy(), g["xs"])
    out = C.mxfp4_moe(x, w, router_logits=logits)
    slots, shared = C.mxfp4_moe(x, w, router_logits=logits, return_partials=True)
    torch.cuda.synchronize()
    assert C.last_status() == 0 and shared is None
    check_against_oracle(out.float().cpu().numpy(), g["out_softmax"])
    check_against_oracle(slots.float().sum(1).cpu().numpy(), g["out_softmax"])
    assert np.array_equal(bits_of(out), orc.reduce_slots_bf16(bits_of(slots)))
    for _ in range(3):
        assert torch.equal(out, C.mxfp4_moe(x, w, router_logits=logits))


def test_reference_routing_rule_and_distributions(C):
    """The reference's own test distributions: scale bytes 118..123, activations 0.5*N(0,1), sigmoid + bias routing
    with the routed scale 2 (tests/moe/.../workload.py:34-35,88-90; test_entry.py:18-25)."""
    (w13, s13, w2, s2), gen = orc.make_weights(seed=9, scale_lo=118, scale_hi=124)
    tokens = 12
    x = (torch.randn((tokens, H), generator=gen) * 0.5).bfloat16()
    gate = torch.randn((128, H), generator=gen) / H ** 0.5
    bias = torch.randn((128,), generator=gen) * 0.01
    w = C.MoeWeights.from_row_major(gate.cuda(), bias.cuda(), dev(w13), dev(s13), dev(w2), dev(s2))
    xd = x.cuda()
    wt, ids = C.route(xd, w)
    logits = (x.double() @ gate.double().t())
    wr, ir, vals = orc.route_sigmoid_bias(logits.numpy(), bias.numpy(), 2.0)
    dec = orc.decided(vals, eps=1e-4)  # logits come from an fp32 library GEMM here, not from the fp64 product
    assert np.array_equal(ids.cpu().numpy()[dec], ir[dec]) and dec.mean() > 0.95
    np.testing.assert_allclose(wt.cpu().numpy()[dec.all(1)], wr[dec.all(1)], atol=1e-3, rtol=0)
    out = C.mxfp4_moe(xd, w)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    xq, xs = orc.quant_mxfp4(x.float().numpy())
    ref = orc.w4a4_moe(xq, xs, w13, s13, w2, s2, wt.cpu().numpy(), ids.cpu().numpy())
    check_against_oracle(out.float().cpu().numpy(), ref)


@pytest.mark.parametrize("mode", ["sigmoid_bias", "softmax"])
@pytest.mark.parametrize("tokens", [1, 5, 32, 33, 256, 2048])
def test_entry_with_the_router_inside(C, layer, tokens, mode):
    """``mxfp4_moe(x, w)`` WITHOUT ``router_logits`` -- the call a server makes (reference chain.py:127-197; its test
    tests/moe/.../test_entry.py:94-104): the router GEMM fused with the input quantiser, top-4, sort, gather, GEMMs and
    reduce in one C-ABI call (b200moe_forward_x). Routing ids against the fp64 logits on decided rows (reference.py:127-148),
    weights to 1e-3; the slots bit for bit against the staged kernels on the same routing; sampled tokens against the CPU
    oracle; graph replay into poisoned buffers."""
    raw, w0, _, _ = layer
    sigmoid = mode == "sigmoid_bias"
    gen = torch.Generator().manual_seed(7000 + tokens)
    x = torch.randn((tokens, H), generator=gen).bfloat16()
    gate = torch.randn((128, H), generator=gen) / H ** 0.5
    bias = torch.randn((128,), generator=gen) * 0.01 if sigmoid else None
    scale = 2.0 if sigmoid else 1.0
    w = C.MoeWeights(gate.cuda(), None if bias is None else bias.cuda(), w0.w13, None, w0.w2, None, scale, mode)
    xd = x.cuda()
    out = C.mxfp4_moe(xd, w)
    slots, shared = C.mxfp4_moe(xd, w, return_partials=True)
    wt, ids = C.route(xd, w)
    torch.cuda.synchronize()
    assert C.last_status() == 0 and shared is None
    logits64 = (x.double() @ gate.double().t()).numpy()
    if sigmoid:
        wr, ir, vals = orc.route_sigmoid_bias(logits64, bias.numpy(), scale)
    else:
        wr, ir, vals = orc.route_softmax(logits64, scale)
    dec = orc.decided(vals, eps=5e-4)  # the router's partials are within 2^-18 * sum|x||w| ~ 1.5e-4 of the fp64 logits
    assert dec.mean() > 0.9
    assert np.array_equal(ids.cpu().numpy()[dec], ir[dec])
    np.testing.assert_allclose(wt.cpu().numpy()[dec.all(1)], wr[dec.all(1)], atol=1e-3, rtol=0)
    staged = C.mxfp4_moe_experts(C.mxfp4_quant(xd), wt, ids, w)
    assert torch.equal(slots, staged), "the one-call entry and the staged kernels disagree"
    assert np.array_equal(bits_of(out), orc.reduce_slots_bf16(bits_of(slots)))
    pick = np.unique(np.linspace(0, tokens - 1, 6).astype(int))
    xq, xs = orc.quant_mxfp4(x.float().numpy())
    ref = oracle_slots(xq, xs, raw, ids.cpu().numpy(), wt.cpu().numpy(), tokens=pick)
    check_against_oracle(slots.float().cpu().numpy()[pick].sum(1), ref.sum(1))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        replayed = C.mxfp4_moe(xd, w)
    replayed.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(replayed, out) and C.last_status() == 0


@pytest.mark.parametrize("tokens", [1, 2, 4, 8, 16, 32, 64, 128, 256])
def test_decode_sweep_with_graph_padding_rows(C, layer, tokens):
    """The decode sizes; the last quarter of the rows are CUDA-graph padding (zero rows, ordinary logits). Checked
    against the CUDA-core kernels on every row, against the CPU oracle on four tokens, replayed from a CUDA graph."""
    raw, w, _, _ = layer
    gen = torch.Generator().manual_seed(1000 + tokens)
    xb, lg = orc.make_inputs(gen, tokens, pad_rows=tokens // 4)
    x, logits = bf16_dev(xb), dev(lg)
    out = C.mxfp4_moe(x, w, router_logits=logits)
    slots, _ = C.mxfp4_moe(x, w, router_logits=logits, return_partials=True)
    wt, ids = C.route(x, w, router_logits=logits)
    xq = C.mxfp4_quant(x)
    _, _, _, slots_r = run_stages(C, w, xq, ids, wt, C.variant_for(tokens), tc=False)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    got, ref = slots.float().cpu().numpy(), slots_r.float().cpu().numpy()
    assert np.isfinite(got).all()
    if tokens // 4:
        assert not got[tokens - tokens // 4:].any() and not bits_of(out)[tokens - tokens // 4:].any()
    assert cosine(got, ref) >= 0.99999 and rel_l2(got, ref) < 2e-3
    pick = np.unique(np.linspace(0, tokens - 1, 4).astype(int))
    cpu = oracle_slots(xq[0].cpu().numpy(), xq[1].cpu().numpy(), raw, ids.cpu().numpy(), wt.cpu().numpy(), pick)
    if np.abs(cpu).max() > 0:
        check_against_oracle(got[pick].sum(1), cpu.sum(1))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = C.mxfp4_moe(x, w, router_logits=logits)
    captured.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, out) and C.last_status() == 0


@pytest.mark.parametrize("tokens,kind", [(2048, "softmax"), (8192, "softmax"), (4096, "zipf")])
def test_full_size_properties(C, layer, tokens, kind):
    """Prefill sizes, where the CPU oracle is out of reach: (1) sampled sorted rows equal the CUDA-core kernels,
    (2) sixteen tokens agree with the CPU oracle, (3) a token's slots are bit-identical whether it runs in this batch or
    in a batch of 16 (each token is its own accumulator column), (4) two runs are bit-identical, (5) the reduce of the
    slots reproduces the reduced output. "zipf": the skewed-routing configuration (logit bias -2.2*ln(rank))."""
    raw, w, _, _ = layer
    gen = torch.Generator().manual_seed(tokens)
    xb, lg = orc.make_inputs(gen, tokens)
    if kind == "zipf":
        lg = lg - 2.2 * np.log(np.arange(1, 129, dtype=np.float32))[None, :]
    x, logits = bf16_dev(xb), dev(lg)
    slots, _ = C.mxfp4_moe(x, w, router_logits=logits, return_partials=True)
    out = C.mxfp4_moe(x, w, router_logits=logits)
    wt, ids = C.route(x, w, router_logits=logits)
    xq = C.mxfp4_quant(x)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    assert np.array_equal(ids.cpu().numpy(), orc.route_softmax(lg)[1])
    assert np.array_equal(bits_of(out), orc.reduce_slots_bf16(bits_of(slots)))
    assert torch.equal(slots, C.mxfp4_moe(x, w, router_logits=logits, return_partials=True)[0])
    # (1) sampled rows through the CUDA-core path
    bm = C.variant_for(tokens)
    sb = C.moe_sort(ids, wt, bm)
    nv = int(sb.num_valid[0])
    rows = torch.from_numpy(np.unique(np.random.default_rng(0).integers(0, nv, 96)).astype(np.int32)).cuda()
    hq_r, sfh_r = C.simt_gemm1(xq, sb, w, rows)
    slots_r = C.simt_gemm2(hq_r, sfh_r, sb, w, rows)
    sid = sb.sorted_ids[rows.long()]
    live = (sid & 0xFFFFFF) < tokens
    tok, slot = (sid[live] & 0xFFFFFF).long(), (sid[live] >> 24).long()
    a, b = slots[tok, slot].float().cpu().numpy(), slots_r[tok, slot].float().cpu().numpy()
    assert cosine(a, b) >= 0.99999 and rel_l2(a, b) < 2e-3
    # (2) CPU oracle on 16 tokens
    pick = np.linspace(0, tokens - 1, 16).astype(int)
    cpu = oracle_slots(xq[0].cpu().numpy(), xq[1].cpu().numpy(), raw, ids.cpu().numpy(), wt.cpu().numpy(), pick)
    check_against_oracle(slots[torch.from_numpy(pick).cuda()].float().sum(1).cpu().numpy(), cpu.sum(1))
    # (3) batch invariance
    sel = torch.from_numpy(pick).cuda()
    small, _ = C.mxfp4_moe(x[sel].contiguous(), w, router_logits=logits[sel].contiguous(), return_partials=True)
    torch.cuda.synchronize()
    assert torch.equal(small, slots[sel])


def test_guard_bands_around_every_allocation(C, layer, monkeypatch):
    """Every torch.empty of a call gets 128-byte guard bands and NaN / sentinel payloads (the reference's fixture,
    tests/moe/.../test_entry.py:144-174): no kernel writes outside its buffers, and the outputs are fully written."""
    import math
    raw, w, _, _ = layer
    for tokens in (1, 17, 129, 600):
        gen = torch.Generator().manual_seed(tokens)
        xb, lg = orc.make_inputs(gen, tokens)
        x, logits = bf16_dev(xb), dev(lg)
        real, guards = torch.empty, []

        def guarded(*size, **kw):
            dims = tuple(size[0]) if isinstance(size[0], (tuple, list, torch.Size)) else size
            dtype = kw.get("dtype", torch.float32)
            g = 512 // torch.tensor([], dtype=dtype).element_size()  # keeps the payload 512-byte aligned
            store = real((math.prod(dims) + 2 * g,), **kw)
            store.view(torch.uint8).fill_(17)
            payload = store[g:-g].view(dims)
            if dtype == torch.bfloat16:
                payload.fill_(float("nan"))
            guards.append((store, g))
            return payload

        with monkeypatch.context() as p:
            p.setattr(torch, "empty", guarded)
            out = C.mxfp4_moe(x, w, router_logits=logits)
            slots, _ = C.mxfp4_moe(x, w, router_logits=logits, return_partials=True)
        torch.cuda.synchronize()
        assert guards and torch.isfinite(out).all() and torch.isfinite(slots).all()
        for store, g in guards:
            raw_bytes = store.view(torch.uint8)
            n = g * store.element_size()
            assert bool((raw_bytes[:n] == 17).all()) and bool((raw_bytes[-n:] == 17).all())


def test_results_identical_next_to_a_concurrent_kernel(C, layer):
    raw, w, xb, lg = layer
    x, logits = bf16_dev(xb), dev(lg)
    expected = C.mxfp4_moe(x, w, router_logits=logits)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    a = torch.randn((4096, 4096), device="cuda", dtype=torch.bfloat16)
    with torch.cuda.stream(side):
        for _ in range(20):
            a @ a
    actual = C.mxfp4_moe(x, w, router_logits=logits)
    torch.cuda.synchronize()
    assert torch.equal(actual, expected) and C.last_status() == 0


def test_entry_errors_and_warm_up(C, layer):
    raw, w, xb, lg = layer
    with pytest.raises(ValueError):
        C.mxfp4_moe(torch.zeros((4, 6144), device="cuda"), w)
    with pytest.raises(ValueError):
        C.mxfp4_moe(torch.zeros((4, 6144), device="cuda", dtype=torch.bfloat16), w, router_logits=torch.zeros((4, 64), device="cuda"))
    with pytest.raises(ValueError):
        C.mxfp4_moe(torch.zeros((4, 6144), device="cuda", dtype=torch.bfloat16), w)  # no router weight, no logits
    with pytest.raises(ValueError):
        C.mxfp4_moe_experts((torch.zeros((0, 3072), dtype=torch.uint8, device="cuda"), None), None, None, w)
    C.warm_up_mxfp4_moe(w, partials=True)


def _single_rank_group():
    import socket
    import torch.distributed as dist
    if not dist.is_initialized():
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    return dist


@pytest.mark.parametrize("tokens", [3, 300])
def test_expert_parallel_path_equals_the_layer_bit_for_bit(C, layer, tokens):
    """The expert-parallel code path (plan, all-to-all, grouped GEMMs on received rows, combine) with every expert on
    one rank gives the single-GPU layer's bits: a (token, slot) row does not depend on the batch it is computed in."""
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import ep
    _single_rank_group()
    raw, w, _, _ = layer
    gen = torch.Generator().manual_seed(77 + tokens)
    xb, lg = orc.make_inputs(gen, tokens)
    x, logits = bf16_dev(xb), dev(lg)
    par = ep.ExpertParallelMoe(w, None, routing_mode="softmax", scale=1.0)
    out = par.forward(x, logits)
    slots = par.forward(x, logits, return_partials=True)
    ref_slots, _ = C.mxfp4_moe(x, w, router_logits=logits, return_partials=True)
    torch.cuda.synchronize()
    assert C.last_status() == 0 and par.recv_rows == 4 * tokens
    assert torch.equal(slots, ref_slots) and torch.equal(out, C.mxfp4_moe(x, w, router_logits=logits))
    # the combine fused into GEMM2 (result rows stored through the rank/pair tables into the owner's slot buffer)
    fused = ep.ExpertParallelMoe(w, None, routing_mode="softmax", scale=1.0, peer_pairs=4 * tokens)
    assert fused.peer is not None
    for _ in range(2):
        assert torch.equal(fused.forward(x, logits), out)
    assert torch.equal(fused.forward(x, logits, return_partials=True), ref_slots)
    torch.cuda.synchronize()
    assert C.last_status() == 0


def test_largest_sizes_cross_int32_byte_offsets(C, layer):
    """65536 and 87381 tokens (the slot tensor is 3.2 / 4.3 GB: byte offsets exceed int32, as in the reference's
    tests/moe/.../test_gemm_half_rows.py:28-30): the last tokens of the big batch equal, bit for bit, the same tokens run
    as a batch of 16; outputs are finite; the reduce identity holds on the tail."""
    raw, w, _, _ = layer
    for tokens in (65536, 87381):
        gen = torch.Generator(device="cuda").manual_seed(tokens)
        x = torch.randn((tokens, H), device="cuda", generator=gen).bfloat16()
        logits = torch.randn((tokens, 128), device="cuda", generator=gen)
        slots, _ = C.mxfp4_moe(x, w, router_logits=logits, return_partials=True)
        tail = slice(tokens - 16, tokens)
        small, _ = C.mxfp4_moe(x[tail].contiguous(), w, router_logits=logits[tail].contiguous(), return_partials=True)
        torch.cuda.synchronize()
        assert C.last_status() == 0
        assert torch.equal(slots[tail], small)
        assert bool(torch.isfinite(slots[::997].float()).all())
        out = C.mxfp4_moe(x, w, router_logits=logits)
        assert np.array_equal(bits_of(out[tail]), orc.reduce_slots_bf16(bits_of(slots[tail])))
        del slots, out, x, logits
        torch.cuda.empty_cache()
    with pytest.raises(ValueError):
        C.mxfp4_moe(torch.zeros((87382, H), device="cuda", dtype=torch.bfloat16), w, router_logits=torch.zeros((87382, 128), device="cuda"))


@pytest.mark.parametrize("tokens,bm,kind", [(1, 16, "uniform"), (16, 16, "uniform"), (100, 32, "hot"), (256, 32, "uniform"),
                                            (700, 64, "uniform"), (300, 16, "one")])
def test_one_launch_gemm12_equals_two_launches(C, layer, tokens, bm, kind):
    """GEMM1 and GEMM2 in one persistent launch (the decode path of the entry) against the two separate launches: h codes,
    h scales and slots bit for bit (the reference's tests/moe/.../test_gemm12_a4w4.py:65-77), three runs in a row."""
    raw, w, _, _ = layer
    gen = torch.Generator().manual_seed(500 + tokens)
    xb, _ = orc.make_inputs(gen, tokens)
    ids, wts = make_routing(tokens, kind, seed=tokens)
    x = bf16_dev(xb)
    sb = C.moe_sort(dev(ids), dev(wts), bm)
    xq, sfx = C.quant_dispatch(x, sb)
    hq, sfh = C.grouped_gemm1(xq, sfx, sb, w)
    ref = C.grouped_gemm2(hq, sfh, sb, w, slots=torch.zeros((tokens, 4, H), dtype=torch.bfloat16, device="cuda"))
    nv = int(sb.num_valid[0])
    for _ in range(3):
        slots, hq2, sfh2 = C.grouped_gemm12(xq, sfx, sb, w, slots=torch.zeros((tokens, 4, H), dtype=torch.bfloat16, device="cuda"))
        torch.cuda.synchronize()
        assert C.last_status() == 0
        assert torch.equal(hq2[:nv], hq[:nv])
        assert np.array_equal(atoms_to_rowmajor(sfh2.cpu().numpy(), bm)[:nv], atoms_to_rowmajor(sfh.cpu().numpy(), bm)[:nv])
        assert torch.equal(slots, ref)
