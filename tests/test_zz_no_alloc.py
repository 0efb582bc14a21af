"""The allocation-free routing sort (b200moe_permute_static), called through the C ABI.

It exists for hosts that may not allocate device memory around a call (a fixed memory budget handed out at start-up, or
a stream that is being captured); its scratch is an array inside the library. This file is collected last so that a run
that stops at the first failure has already run every other test. The check: on two calls in a row, with different
routing, every output equals the ordinary entry point's bit for bit (the sort is integer work), the second call is not
disturbed by what the first left in the shared array, and sizes beyond the built-in limit are refused."""
import ctypes

import numpy as np
import pytest
import torch

from tests.util import dev, make_routing

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _outputs(rows, bm):
    return (torch.full((rows,), -7, dtype=torch.int32, device="cuda"), torch.full((rows,), -1.0, device="cuda"),
            torch.full((rows // bm,), -7, dtype=torch.int32, device="cuda"), torch.full((2,), -7, dtype=torch.int32, device="cuda"))


def test_static_scratch_sort_equals_the_ordinary_sort_twice_in_a_row():
    from amd_kernels_b200 import _lib
    from amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4 import chain
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # 3000 and 8192 tokens use 12 and 32 chunks of the built-in scratch; the second call reuses what the first left there
    for tokens, kind, bm in ((8192, "uniform", 128), (3000, "hot", 32)):
        ids, w = make_routing(tokens, kind, seed=tokens)
        ids_d, w_d = dev(ids), dev(w)
        ref = chain.moe_sort(ids_d, w_d, bm)
        outs = _outputs(ref.max_rows, bm)
        code = lib.b200moe_permute_static(_ptr(ids_d), _ptr(w_d), tokens, 128, bm, *(_ptr(t) for t in outs), stream)
        assert code == 0
        torch.cuda.synchronize()
        n = int(ref.num_valid[0])
        assert torch.equal(outs[3], ref.num_valid)
        assert torch.equal(outs[0][:n], ref.sorted_ids[:n])
        assert torch.equal(outs[1][:n].view(torch.int32), ref.sorted_weights[:n].view(torch.int32))
        assert torch.equal(outs[2][:n // bm], ref.block_expert[:n // bm])
        assert bool((outs[0][n:] == -7).all())  # nothing written past the padded rows


def test_static_scratch_sort_refuses_sizes_beyond_its_limit():
    from amd_kernels_b200 import _lib
    lib = _lib.load()
    one = ctypes.c_void_p(256)
    assert lib.b200moe_permute_static(one, one, 8193, 128, 128, one, one, one, one, None) == _lib.E_TOO_LARGE
    with pytest.raises(ValueError):
        _lib.check(_lib.E_TOO_LARGE, "permute_static")
