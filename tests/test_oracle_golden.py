"""The CPU oracle against the golden outputs of the reference's own ``reference.py`` (made by tests/golden/make_golden.py)."""
import zlib

import numpy as np

from oracle import moe_oracle as orc
from tests.conftest import golden


def test_quant_bit_exact_bf16_and_fp32_inputs():
    g = golden("quant.npz")
    q, s = orc.quant_mxfp4(orc.bf16_to_f32(g["x_bits"]))
    assert np.array_equal(s, g["scales"]) and np.array_equal(q, g["codes"])
    q, s = orc.quant_mxfp4(g["f32"])
    assert np.array_equal(s, g["scales32"]) and np.array_equal(q, g["codes32"])
    assert np.array_equal(orc.dequant_mxfp4(g["codes"], g["scales"]), g["deq"])


def test_quant_known_answers():
    # amax -> scale byte, and the midpoint / sign rules, as listed in the reference's docstring (reference.py:5-9)
    for amax, byte in ((7.0, 128), (6.0, 127), (4.0, 127), (3.5, 127), (3.4999, 126), (1.0, 125), (1e-30, 25), (0.0, 1)):
        x = np.zeros((1, 32), np.float32)
        x[0, 0] = amax
        assert orc.quant_mxfp4(x)[1][0, 0] == byte, amax
    x = np.zeros((1, 32), np.float32)
    x[0, :8] = [4.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, -0.0]
    q, s = orc.quant_mxfp4(x)
    codes = np.stack([q[0] & 15, q[0] >> 4], -1).reshape(-1)[:8].tolist()
    assert s[0, 0] == 127 and codes == [6, 0, 2, 2, 4, 4, 6, 8]


def test_routing_matches_reference_on_decided_rows():
    g = golden("routing.npz")
    assert np.array_equal(orc.splitk_logits(g["partials"]), g["logits"])
    w, ids, vals = orc.route_sigmoid_bias(g["logits"], g["bias"], 2.0)
    dec = g["decided"]
    assert np.array_equal(orc.decided(vals), dec)
    assert dec.mean() > 0.9
    assert np.array_equal(ids[dec], g["ids"][dec])
    np.testing.assert_allclose(vals, g["vals"], rtol=0, atol=1e-12)
    rows = dec.all(1)
    np.testing.assert_allclose(w[rows], g["weights"][rows], rtol=1e-12)


def test_tie_rule_lowest_id():
    logits = np.full((1, 128), 0.25, np.float32)
    assert orc.route_softmax(logits)[1].tolist() == [[0, 1, 2, 3]]
    assert orc.route_sigmoid_bias(logits, np.zeros(128), 2.0)[1].tolist() == [[0, 1, 2, 3]]
    w = orc.route_softmax(np.random.default_rng(0).standard_normal((64, 128)).astype(np.float32), scale=1.0)[0]
    np.testing.assert_allclose(w.sum(1), 1.0, rtol=1e-12)


def test_swiglu_and_reduce():
    g = golden("swiglu.npz")
    np.testing.assert_allclose(orc.swiglu_oai(g["gate"], g["up"]), g["out"], rtol=2e-6, atol=1e-7)
    g = golden("reduce.npz")
    assert np.array_equal(orc.reduce_slots_bf16(g["slots"]), g["out"])


def test_permute_canonical_order_and_padding():
    rng = np.random.default_rng(1)
    for m, bm in ((1, 16), (5, 16), (33, 32), (300, 128)):
        ids = np.stack([rng.permutation(128)[:4] for _ in range(m)]).astype(np.int32)
        if m > 4:
            ids[3] = [7, 7, 9, 7]  # one expert in several slots of a token is accepted
        w = rng.random((m, 4)).astype(np.float32)
        rows, wt, blocks, nv = orc.permute(ids, w, bm)
        assert nv[0] == rows.size == blocks.size * bm and rows.size <= orc.max_sorted_rows(m, bm)
        assert np.all(np.diff(blocks) >= 0)
        for b, e in enumerate(blocks):
            chunk = rows[b * bm:(b + 1) * bm]
            live = chunk[chunk != m]
            tok, slot = live & 0xFFFFFF, live >> 24
            assert np.all(ids[tok, slot] == e)
            assert np.all(wt[b * bm:(b + 1) * bm][chunk == m] == 0)
        live = rows[rows != m]
        assert live.size == 4 * m and np.unique(live).size == 4 * m
        # pair order inside each expert
        q = (live & 0xFFFFFF) * 4 + (live >> 24)
        e_of = ids.reshape(-1)[q]
        assert np.all(np.diff(e_of) >= 0)
        assert all(np.all(np.diff(q[e_of == e]) > 0) for e in np.unique(e_of))


def test_moe_small_matches_reference():
    g = golden("moe_small.npz")
    xq, xs = orc.quant_mxfp4(orc.bf16_to_f32(g["x_bits"]))
    w, ids, _ = orc.route_softmax(g["logits"])
    assert np.array_equal(ids, g["ids"])
    out = orc.w4a4_moe(xq, xs, g["w13"], g["s13"], g["w2"], g["s2"], g["weights"], g["ids"])
    rel = np.linalg.norm(out - g["out"]) / np.linalg.norm(g["out"])
    assert rel < 1e-5, rel


def test_moe_config0_matches_reference(config0):
    (w13, s13, w2, s2), xb, lg = config0
    g = golden("moe_config0.npz")
    crc = [zlib.crc32(a.tobytes()) for a in (w13, s13, w2, s2, xb, lg)]
    assert crc == g["crc"].tolist(), "seeded inputs differ from the ones the golden outputs were made from"
    xq, xs = orc.quant_mxfp4(orc.bf16_to_f32(xb))
    assert np.array_equal(xq, g["xq"]) and np.array_equal(xs, g["xs"])
    w, ids, _ = orc.route_softmax(lg)
    assert np.array_equal(ids, g["ids_softmax"])
    out = orc.w4a4_moe(xq, xs, w13, s13, w2, s2, g["weights_softmax"], g["ids_softmax"])
    rel = np.linalg.norm(out - g["out_softmax"]) / np.linalg.norm(g["out_softmax"])
    # the few-1e-4 budget covers h codes that flip on fp32 summation order (the reference's own note, reference.py:14-16)
    assert rel < 5e-4, rel
    wsig, isig, vals = orc.route_sigmoid_bias(lg, np.zeros(128), 2.0)
    dec = orc.decided(vals)
    assert np.array_equal(isig[dec], g["ids_sigmoid"][dec])
    np.testing.assert_allclose(wsig, g["weights_sigmoid"], rtol=1e-12)


def test_shared_expert_quant_cast_and_mlp_match_reference():
    g = golden("shared.npz")
    assert np.array_equal(orc.f32_to_e4m3(g["cast_in"]), g["cast_codes"])           # torch's E4M3 cast, ties included
    q, s = orc.shared_mxfp8_quant(orc.bf16_to_f32(g["x_bits"]))
    assert np.array_equal(s, g["scales"]) and np.array_equal(q, g["codes"])
    weights = orc.make_shared_weights()
    assert [zlib.crc32(a.tobytes()) for a in weights] == g["weight_crc"].tolist()
    out = orc.shared_mxfp8(orc.bf16_to_f32(g["x_bits"]), *weights)
    rel = np.linalg.norm(out - g["out"]) / np.linalg.norm(g["out"])
    assert rel < 2e-3, rel  # FP8 codes of h that flip on fp32 summation order


def test_sidecar_pack_and_unpack_match_reference():
    """mask == mxfp4_sidecar_pack_ref, and the FP4 codes come back bit for bit (reference.py:210-235)."""
    g = golden("sidecar.npz")
    x = orc.bf16_to_f32(g["x_bits"])
    q4, s4 = orc.quant_mxfp4(x)
    q8, s8 = orc.shared_mxfp8_quant(x)
    assert (q4 == g["q4"]).all() and (s4 == g["s4"]).all() and (q8 == g["q8"]).all() and (s8 == g["s8"]).all()
    mask = orc.sidecar_pack(q4, s4, q8, s8)
    assert mask.shape == (x.shape[0], 768) and (mask == g["mask"]).all()
    assert mask.any()
    assert (orc.sidecar_unpack(mask, s4, q8, s8) == q4).all()


def test_fused_tail_matches_reference():
    """Slot sum + shared, residual add, Gemma RMSNorm and the MXFP8 of the fp32 norm against the reference's
    slots4_local_reference / add_rmsnorm_reference / mxfp8_scale_reference / mxfp8_codes
    (amd_kernels/norm/gemma_add_rmsnorm_h6144/reference.py): the sum, residual, scale bytes and codes bit for bit, y to
    fp64 round-off."""
    g = golden("tail.npz")
    x = orc.slots4_local(g["slots"], g["shared"])
    assert np.array_equal(x, g["x"])
    y, res = orc.add_rmsnorm(x, g["residual"], g["weight"], float(g["eps"]))
    assert np.array_equal(res, g["residual_out"])
    np.testing.assert_allclose(y, g["y64"], rtol=1e-14, atol=0)
    assert np.array_equal(orc.tail_mxfp8_scale(g["y64"]), g["scales"])
    assert np.array_equal(orc.tail_mxfp8_codes(g["y64"], g["scales"]), g["codes"])
    st = orc.compare_tail(g["out"], g["codes"], g["scales"], g["y64"])
    assert st["bad_ulp"] == 0 and st["code_mismatch"] == 0 and st["scale_mismatch"] == 0
    # -0.0 runs survive the slot sum (it starts from s0, not from +0) but not the library's plain slot reduce
    assert (x[0, :64] == 0x8000).all() and (orc.reduce_slots_bf16(g["slots"])[0, :64] == 0).all()
