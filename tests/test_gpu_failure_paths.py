"""The device-side failure paths, exercised without faulting or hanging the GPU: a bounded wait that is made to run out
(nothing ever satisfies it) and routing tables with out-of-range entries. In both cases the kernels return, the status word
says what happened, and the next ordinary call on the same context is correct."""
import ctypes
import time

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.util import bf16_dev, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C():
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain
    return chain


@pytest.fixture(scope="module")
def small(C):
    (w13, s13, w2, s2), gen = orc.make_weights(seed=11, experts=8)
    xb, lg = orc.make_inputs(gen, 24, experts=8)
    w = C.MoeWeights.from_row_major(None, None, dev(w13), dev(s13), dev(w2), dev(s2), routing_mode="softmax",
                                    routed_scaling_factor=1.0)
    x, logits = bf16_dev(xb), dev(lg)
    wt, ids = C.topk_route(logits, None, 1.0, "softmax")
    return w, x, wt, ids


def test_a_wait_that_cannot_be_satisfied_times_out_and_the_context_survives(C, small):
    """b200moe_gemm12 with the per-block completion counts preset to -100: no GEMM2 unit can ever see 12 finished GEMM1
    tiles, so every CTA's wait runs out (limit lowered to 20 ms), the roles wind down, tensor memory is freed and the call
    returns with status B200MOE_DEV_TIMEOUT."""
    from amd_kernels_b200 import _lib
    w, x, wt, ids = small
    sort = C.moe_sort(ids, wt, 16, w.num_experts)
    xq, sfx = C.quant_dispatch(x, sort)
    good, _, _ = C.grouped_gemm12(xq, sfx, sort, w)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    C.set_wait_limit_ns(20_000_000)
    try:
        stuck = torch.full((sort.max_rows // sort.bm,), -100, dtype=torch.int32, device="cuda")
        t0 = time.perf_counter()
        C.grouped_gemm12(xq, sfx, sort, w, done=stuck)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
    finally:
        C.set_wait_limit_ns(2_000_000_000)
    assert C.last_status() == _lib.DEV_TIMEOUT
    assert elapsed < 5.0, f"the kernel took {elapsed:.2f} s to give up"
    again, _, _ = C.grouped_gemm12(xq, sfx, sort, w)
    torch.cuda.synchronize()
    assert C.last_status() == 0 and torch.equal(again, good)


def test_out_of_range_routing_tables_set_the_status_and_touch_nothing_outside(C, small):
    """An expert id outside the weights and a row count beyond the buffers: the kernels substitute safe values or do
    nothing, record B200MOE_DEV_BAD_INDEX, and never form an address from the bad entry."""
    from amd_kernels_b200 import _lib
    w, x, wt, ids = small
    sort = C.moe_sort(ids, wt, 16, w.num_experts)
    xq, sfx = C.quant_dispatch(x, sort)
    good = C.grouped_gemm2(*C.grouped_gemm1(xq, sfx, sort, w), sort, w)
    torch.cuda.synchronize()
    assert C.last_status() == 0
    bad = C.SortBuffers(sort.sorted_ids, sort.sorted_weights, sort.block_expert.clone(), sort.num_valid, sort.bm, sort.tokens)
    bad.block_expert[0] = 9999
    C.grouped_gemm1(xq, sfx, bad, w)
    torch.cuda.synchronize()
    assert C.last_status() == _lib.DEV_BAD_INDEX
    bad = C.SortBuffers(sort.sorted_ids, sort.sorted_weights, sort.block_expert, sort.num_valid.clone(), sort.bm, sort.tokens)
    bad.num_valid[0] = sort.max_rows + 16 * 1000
    slots = torch.full((sort.tokens, 4, 6144), 7.0, dtype=torch.bfloat16, device="cuda")
    hq, sfh = C.grouped_gemm1(xq, sfx, bad, w)
    C.grouped_gemm2(hq, sfh, bad, w, slots=slots)
    torch.cuda.synchronize()
    assert C.last_status() == _lib.DEV_BAD_INDEX
    assert bool((slots == 7.0).all()), "a launch with an impossible row count must not write"
    after = C.grouped_gemm2(*C.grouped_gemm1(xq, sfx, sort, w), sort, w)
    torch.cuda.synchronize()
    assert C.last_status() == 0 and torch.equal(after, good)


def test_the_gathering_gemm1_never_reads_outside_the_tokens(C, small):
    """The GEMM1 that gathers its own rows: an expert id outside the weights is replaced and reported; a sorted entry
    whose token index is not below the token count (whatever its bits) is a padding row and reads as zeros, so a corrupt
    list cannot form an address outside the quantised tokens."""
    from amd_kernels_b200 import _lib
    w, x, wt, ids = small
    sort = C.moe_sort(ids, wt, 128, w.num_experts)
    q, s = C.mxfp4_quant(x)
    xq, sfx = C.quant_dispatch(x, sort)
    nv = int(sort.num_valid[0])
    good = C.grouped_gemm1(xq, sfx, sort, w)[0][:nv]
    assert torch.equal(C.grouped_gemm1_gather(q, s, sort, w)[0][:nv], good)
    assert C.last_status() == 0
    bad = C.SortBuffers(sort.sorted_ids, sort.sorted_weights, sort.block_expert.clone(), sort.num_valid, sort.bm, sort.tokens)
    bad.block_expert[0] = -3
    C.grouped_gemm1_gather(q, s, bad, w)
    torch.cuda.synchronize()
    assert C.last_status() == _lib.DEV_BAD_INDEX
    wild = sort.sorted_ids.clone()
    wild[::3] = torch.randint(sort.tokens, 1 << 24, (wild[::3].numel(),), device="cuda", dtype=torch.int32) | (0x7F << 24)
    wild[1::3] = -1
    odd = C.SortBuffers(wild, sort.sorted_weights, sort.block_expert, sort.num_valid, sort.bm, sort.tokens)
    h = C.grouped_gemm1_gather(q, s, odd, w)[0][:nv]
    torch.cuda.synchronize()
    assert C.last_status() == 0
    kept = torch.arange(nv, device="cuda") % 3 == 2
    assert torch.equal(h[kept], good[kept])  # rows whose entry was left alone are unchanged
    assert not bool(h[~kept].any())  # a padding row's h is zero (codes of 0.0)
    assert torch.equal(C.grouped_gemm1_gather(q, s, sort, w)[0][:nv], good)


def test_an_ordering_point_whose_peer_never_arrives_times_out(C):
    """b200moe_ep_sync with a second rank that does not exist (its flag array is this rank's own, so nobody ever raises
    slot 1): the launch gives up after the lowered limit with B200MOE_DEV_TIMEOUT, the context stays usable and a
    one-rank ordering point passes at once. No second GPU, no collective library, nothing traps."""
    import ctypes
    from amd_kernels_b200 import _lib
    lib = _lib.load()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    matrix = torch.zeros((2, 2), dtype=torch.int64, device="cuda")
    counts = torch.tensor([5, 7], dtype=torch.int64, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = C.status_word(flags.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    two = (ctypes.c_void_p * 2)(flags.data_ptr(), flags.data_ptr())
    two_m = (ctypes.c_void_p * 2)(matrix.data_ptr(), matrix.data_ptr())
    C.set_wait_limit_ns(20_000_000)
    try:
        t0 = time.perf_counter()
        _lib.check(lib.b200moe_ep_sync(two, two_m, p(counts), 2, 0, p(epoch), p(status), stream), "ep_sync")
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
    finally:
        C.set_wait_limit_ns(2_000_000_000)
    assert C.last_status() == _lib.DEV_TIMEOUT
    assert elapsed < 5.0
    assert int(epoch.item()) == 1 and matrix[0].tolist() == [5, 7]  # the payload and the epoch were still written
    one = (ctypes.c_void_p * 1)(flags.data_ptr())
    status.zero_()
    for expect in (2, 3):
        _lib.check(lib.b200moe_ep_sync(one, None, None, 1, 0, p(epoch), p(status), stream), "ep_sync")
        torch.cuda.synchronize()
        assert C.last_status() == 0 and int(epoch.item()) == expect and int(flags[0].item()) == expect

