"""GPU parity tests of the MXFP8 shared expert, through the C ABI.

Bit-exact: the input quantiser (E4M3 codes and E8M0 scales) against the golden fixture and the CPU oracle; one token's
output whatever the batch it sits in (every block height); repeated calls and CUDA-graph replays; the reduce with the
shared term. Floating point: the output against the fp32 oracle on the same MXFP8 operands, per-token cosine >= 0.9999
(the reference's tests/moe/.../test_shared_expert.py:39-40 asks 0.999 against its fp32 reference), relative L2 < 4e-3.
"""
import zlib

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.conftest import golden
from tests.util import H, I, bf16_dev, bits_of, cosine, dev, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def S():
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import shared_expert
    return shared_expert


@pytest.fixture(scope="module")
def shared_layer(S):
    raw = orc.make_shared_weights()
    crc = np.array([zlib.crc32(a.tobytes()) for a in raw], dtype=np.uint32)
    assert (crc == golden("shared.npz")["weight_crc"]).all()
    w13, s13, w2, s2 = (dev(a) for a in raw)
    sw = S.SharedWeights.from_row_major(w13.view(torch.float8_e4m3fn), s13, w2.view(torch.float8_e4m3fn), s2)
    return raw, sw


def random_rows(m, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((m, H), generator=g) * torch.exp2(torch.randint(-4, 5, (m, H // 32), generator=g).float()
                                                       ).repeat_interleave(32, 1)
    return x.bfloat16()


@pytest.mark.parametrize("bm", [16, 32, 64, 128])
def test_input_quantiser_is_bit_exact(S, bm):
    g = golden("shared.npz")
    x = bf16_dev(g["x_bits"])
    codes, atoms = S.shared_quant(x, bm)
    m = x.shape[0]
    assert codes.shape[0] % bm == 0 and (codes[m:] == 0).all()
    assert (codes[:m].cpu().numpy() == g["codes"]).all()
    assert (S.atoms_to_rows(atoms, bm, m).cpu().numpy() == g["scales"]).all()
    # a ragged row count, against the oracle
    xr = random_rows(bm + 5, 11)
    codes, atoms = S.shared_quant(xr.cuda(), bm)
    q, s = orc.shared_mxfp8_quant(xr.float().numpy())
    assert (codes[:bm + 5].cpu().numpy() == q).all()
    assert (S.atoms_to_rows(atoms, bm, bm + 5).cpu().numpy() == s).all()


def test_golden_rows_match_the_reference_output(S, shared_layer):
    _, sw = shared_layer
    g = golden("shared.npz")
    out = S.shared_expert(bf16_dev(g["x_bits"]), sw).float().cpu().numpy()
    ref = g["out"]
    assert np.isfinite(out).all()
    for t in range(ref.shape[0]):
        assert cosine(out[t], ref[t]) >= 0.9999, (t, cosine(out[t], ref[t]))
    assert rel_l2(out, ref) < 4e-3, rel_l2(out, ref)


@pytest.mark.parametrize("m", [1, 7, 16, 100, 257, 900, 1600])
def test_output_matches_oracle_and_is_batch_invariant(S, shared_layer, m):
    raw, sw = shared_layer
    x = random_rows(m, 100 + m)
    xd = x.cuda()
    out = S.shared_expert(xd, sw)
    again = S.shared_expert(xd, sw)
    assert torch.equal(out, again)
    pick = np.unique(np.concatenate([np.arange(min(m, 4)), np.arange(max(0, m - 4), m)]))
    ref = orc.shared_mxfp8(x[pick].float().numpy(), *raw)
    got = out[pick].float().cpu().numpy()
    for j in range(len(pick)):
        assert cosine(got[j], ref[j]) >= 0.9999, (m, pick[j], cosine(got[j], ref[j]))
    assert rel_l2(got, ref) < 4e-3
    # the same rows alone (another block height unless m is small): the same bits
    alone = S.shared_expert(xd[pick].contiguous(), sw)
    assert torch.equal(alone, out[pick])


def test_graph_replay_and_side_stream(S, shared_layer):
    _, sw = shared_layer
    x = random_rows(48, 5).cuda()
    eager = S.shared_expert(x, sw)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = S.shared_expert(x, sw)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    cur = torch.cuda.current_stream()
    par = S.shared_expert_parallel(x, sw, cur)
    cur.wait_stream(sw.stream)
    torch.cuda.synchronize()
    assert torch.equal(par, eager)


@pytest.mark.parametrize("m", [3, 64, 300])
def test_entry_with_shared_expert(S, shared_layer, config0, m):
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain as C
    _, sw = shared_layer
    raw, _, _ = config0
    on_gpu = [dev(a) for a in raw]
    w0 = C.MoeWeights.from_row_major(None, None, *on_gpu, routing_mode="softmax", routed_scaling_factor=1.0)
    w1 = C.MoeWeights.from_row_major(None, None, *on_gpu, shared=sw, routing_mode="softmax", routed_scaling_factor=1.0)
    x = random_rows(m, 40 + m).cuda()
    lg = torch.randn((m, 128), generator=torch.Generator().manual_seed(m)).cuda()
    slots0, none = C.mxfp4_moe(x, w0, return_partials=True, router_logits=lg)
    assert none is None
    slots, shared = C.mxfp4_moe(x, w1, return_partials=True, router_logits=lg)
    assert torch.equal(slots, slots0)
    assert torch.equal(shared, S.shared_expert(x, sw))
    out = C.mxfp4_moe(x, w1, router_logits=lg)
    want = orc.reduce_slots_bf16(bits_of(slots), bits_of(shared))
    assert (bits_of(out) == want).all()
    assert C.last_status() == 0


def test_argument_errors(S, shared_layer):
    _, sw = shared_layer
    with pytest.raises(ValueError):
        S.shared_expert(torch.zeros((4, H - 32), dtype=torch.bfloat16, device="cuda"), sw)
    with pytest.raises(ValueError):
        S.shared_expert(torch.zeros((4, H), dtype=torch.float16, device="cuda"), sw)
    with pytest.raises(ValueError):
        S.SharedWeights.from_row_major(torch.zeros((2 * I, H), dtype=torch.uint8, device="cuda"),
                                       torch.zeros((2 * I, H // 32 - 1), dtype=torch.uint8, device="cuda"),
                                       torch.zeros((H, I), dtype=torch.uint8, device="cuda"),
                                       torch.zeros((H, I // 32), dtype=torch.uint8, device="cuda"))
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain as C
    e4 = torch.float8_e4m3fn
    z = lambda *s, dt=torch.uint8: torch.zeros(s, dtype=dt, device="cuda")  # noqa: E731
    ok = C.unsupported_reason(z(128, 2 * I, H // 2), z(128, 2 * I, H // 32), z(128, H, I // 2), z(128, H, I // 32),
                              z(2 * I, H, dt=e4), z(2 * I, H // 32), z(H, I, dt=e4), z(H, I // 32))
    assert ok is None
    bad = C.unsupported_reason(z(128, 2 * I, H // 2), z(128, 2 * I, H // 32), z(128, H, I // 2), z(128, H, I // 32),
                               z(2 * I, H), z(2 * I, H // 32), z(H, I, dt=e4), z(H, I // 32))
    assert bad is not None and "shared w13" in bad
